"""Parity of the CUDA path, called through the C ABI, against the committed golden vectors (TensorFlow fp64 and the
reference CPU drivers), the numpy oracle and - where it travelled - the compiled reference; plus the size-independent
properties the domain offers (symmetries, energy conservation of the forces, replication)."""
import numpy as np
import pytest

from conftest import (EXTRA_CELLS, F32_MODELS, REF_TOL, TF_CELLS, TF_MODELS, TOL_E, TOL_F, TOL_S, compare_tf, model_path,
                      stress_of)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(backend):
    return {}


def _model(backend, models, name):
    if name not in models:
        models[name] = backend.Model(model_path(name))
    return models[name]


def _compute(backend, model, c, **kw):
    s = backend.System(model, c["species"], skin=kw.pop("skin", 0.5), chunksize=kw.pop("chunksize", -1))
    return s.compute(c["types"], c["positions"], c["cell"], c["pbc"], energies=True, **kw)


@pytest.mark.parametrize("cell", TF_CELLS)
@pytest.mark.parametrize("name", TF_MODELS)
def test_matches_tf_fp64_golden(backend, models, cells, tf_golden, name, cell):
    """the reference's own golden test (python/tests/test_order3_tf.py) with its thresholds"""
    c = cells.get(cell)
    r = _compute(backend, _model(backend, models, name), c)
    d = compare_tf(r, tf_golden, f"{name}/{cell}", c)
    for q, v in d.items():
        assert v < (2e-6 if q == "energy" and c["n"] < 10 else REF_TOL[q]), (q, v)


@pytest.mark.parametrize("cell", TF_CELLS + EXTRA_CELLS)
@pytest.mark.parametrize("name", TF_MODELS + F32_MODELS)
def test_matches_reference_cpu_golden(backend, models, cells, ref_golden, name, cell):
    """against frozen outputs of the reference CPU drivers: thresholds the reference accepts between its GPU and CPU
    calculators (python/tests/test_gpu_calculator.py:74-76)"""
    c = cells.get(cell)
    r = _compute(backend, _model(backend, models, name), c)
    k = f"{name}/{cell}"
    assert abs(r["energy"] - ref_golden[f"{k}/energy"]) / c["n"] < 1e-5
    assert np.abs(r["forces"] - ref_golden[f"{k}/forces"]).max() < 5e-5
    assert np.abs(r["energies"] - ref_golden[f"{k}/energies"]).max() < 1e-5
    ds = np.abs(stress_of(r["virial"], c["volume"]) - stress_of(ref_golden[f"{k}/virial"], c["volume"])).max()
    assert ds < 1e-6


def _config_case(tmp_path_factory, cfg, lattice, a, reps, nsp, sigma, seed):
    from grace_runtime_b200 import modelgen, structures
    els = modelgen._subset(11, nsp)
    path = str(tmp_path_factory.mktemp("cfg") / f"{cfg}.npz")
    modelgen.write_config_model(path, cfg, els, seed=seed)
    types, pos, cell, pbc = structures.crystal(lattice, a, reps, n_species=nsp, sigma=sigma, seed=seed + 1)
    return path, els, dict(species=els, types=types, positions=pos, cell=cell, pbc=pbc, n=len(types),
                           volume=abs(np.linalg.det(cell)))


@pytest.mark.parametrize("cfg,lattice,a,reps,nsp,sigma", [("1l", "bcc", 3.165, (4, 4, 4), 1, 0.05),
                                                           ("1l", "bcc", 3.2, (4, 4, 5), 4, 0.05),
                                                           ("2l", "fcc", 3.6, (3, 3, 3), 3, 0.08)])
def test_benchmark_architectures_match_oracle(backend, tmp_path_factory, cfg, lattice, a, reps, nsp, sigma):
    """scaled-down copies of the benchmark configurations (same architecture, lattice, displacements) against the
    numpy oracle (exact radial MLP, fp64) within the stated tolerances"""
    from oracle.grace_oracle import GraceOracle
    path, els, c = _config_case(tmp_path_factory, cfg, lattice, a, reps, nsp, sigma, seed=5)
    r = _compute(backend, backend.Model(path), c)
    o = GraceOracle(path).compute(els, c["types"], c["positions"], c["cell"], c["pbc"])
    assert abs(r["energy"] - o["energy"]) / c["n"] < TOL_E
    assert np.abs(r["forces"] - o["forces"]).max() < TOL_F
    assert np.abs(r["virial"] - o["virial"]).max() / c["volume"] < TOL_S
    assert np.abs(r["energies"] - o["energies"]).max() < TOL_E


def test_matches_compiled_reference_live(backend, tmp_path_factory):
    """the reference's own CPU drivers (oracle/_ref), when the prebuilt library is present, on a 2L benchmark-shaped
    case with larger displacements"""
    from oracle import refcpu
    if not refcpu.available():
        pytest.skip("oracle/_ref is not built")
    path, els, c = _config_case(tmp_path_factory, "2l", "fcc", 3.6, (3, 3, 4), 3, 0.15, seed=9)
    r = _compute(backend, backend.Model(path), c)
    ref = refcpu.RefModel(path, els).compute(c["types"], c["positions"], c["cell"], c["pbc"])
    assert abs(r["energy"] - ref["energy"]) / c["n"] < TOL_E
    assert np.abs(r["forces"] - ref["forces"]).max() < TOL_F
    assert np.abs(r["virial"] - ref["virial"]).max() / c["volume"] < TOL_S


@pytest.mark.parametrize("name", ["grace_1l_order3", "grace_2l_order3"])
def test_chunked_equals_one_pass(backend, models, cells, name):
    """python/tests/test_gpu_chunk.py:49,101-102: 2e-6 eV/atom, 2e-5 eV/A"""
    c = cells.get("WMo54")
    m = _model(backend, models, name)
    a = _compute(backend, m, c, chunksize=0)
    b = _compute(backend, m, c, chunksize=16)
    assert abs(a["energy"] - b["energy"]) / c["n"] < 2e-6
    assert np.abs(a["forces"] - b["forces"]).max() < 2e-5
    assert np.abs(a["virial"] - b["virial"]).max() < 2e-5 * c["n"]


@pytest.mark.parametrize("name", ["grace_1l_order3", "grace_2l_order3"])
def test_energy_only(backend, models, cells, name):
    c = cells.get("W54")
    m = _model(backend, models, name)
    a = _compute(backend, m, c)
    s = backend.System(m, c["species"])
    b = s.compute(c["types"], c["positions"], c["cell"], c["pbc"], energy_only=True)
    assert "forces" not in b and "virial" not in b
    assert abs(a["energy"] - b["energy"]) < 1e-9 * max(1.0, abs(a["energy"]))


@pytest.mark.parametrize("name", ["grace_1l_order3", "grace_2l_order3"])
def test_deterministic_and_symmetric(backend, models, cells, name):
    c = cells.get("slab36")
    m = _model(backend, models, name)
    a = _compute(backend, m, c)
    b = _compute(backend, m, c)
    assert a["energy"] == b["energy"]
    assert np.array_equal(a["forces"], b["forces"])      # no atomics on either path: bit-identical forces
    assert np.abs(a["forces"].sum(0)).max() < 1e-5          # Newton's third law
    # translation along a periodic direction and permutation of the atoms
    shift = np.array([1.234, -7.5, 0.0])
    perm = np.random.default_rng(1).permutation(c["n"])
    c2 = dict(c, positions=(c["positions"] + shift)[perm], types=c["types"][perm])
    p = _compute(backend, m, c2)
    assert abs(p["energy"] - a["energy"]) / c["n"] < 2e-6
    assert np.abs(p["forces"] - a["forces"][perm]).max() < 2e-5
    # rotation of the whole structure (cell and positions)
    th = 0.7
    R = np.array([[np.cos(th), -np.sin(th), 0], [np.sin(th), np.cos(th), 0], [0, 0, 1.0]])
    c3 = dict(c, positions=c["positions"] @ R.T, cell=c["cell"] @ R.T)
    q = _compute(backend, m, c3)
    assert abs(q["energy"] - a["energy"]) / c["n"] < 2e-6
    assert np.abs(q["forces"] - a["forces"] @ R.T).max() < 2e-5


@pytest.mark.parametrize("name", ["grace_1l_small", "grace_2l_l3"])
def test_forces_are_minus_energy_gradient(backend, models, cells, name):
    c = cells.get("tri9")
    m = _model(backend, models, name)
    s = backend.System(m, c["species"], skin=0.5)
    f = s.compute(c["types"], c["positions"], c["cell"], c["pbc"])["forces"]
    h = 2e-3
    for (i, d) in [(0, 0), (4, 1), (8, 2)]:
        p = c["positions"].copy(); p[i, d] += h
        q = c["positions"].copy(); q[i, d] -= h
        ep = s.compute(c["types"], p, c["cell"], c["pbc"], energy_only=True)["energy"]
        em = s.compute(c["types"], q, c["cell"], c["pbc"], energy_only=True)["energy"]
        assert abs(-(ep - em) / (2 * h) - f[i, d]) < 2e-3 * max(1.0, abs(f[i, d]))


def test_neighbor_list_reuse_and_rebuild(backend, models, cells):
    """Verlet skin: reused while no atom moved more than skin / 2, rebuilt when one did or the types / cell change
    (python/kk/kk_core.cpp:691-708); results do not depend on it"""
    c = cells.get("WMo54")
    m = _model(backend, models, "grace_1l_order3")
    s = backend.System(m, c["species"], skin=0.5)
    r0 = s.compute(c["types"], c["positions"], c["cell"], c["pbc"])
    assert s.rebuilds == 1
    rng = np.random.default_rng(3)
    p1 = c["positions"] + 0.1 * (rng.random(c["positions"].shape) - 0.5)       # < skin / 2
    r1 = s.compute(c["types"], p1, c["cell"], c["pbc"])
    assert s.rebuilds == 1
    fresh = backend.System(m, c["species"], skin=0.0).compute(c["types"], p1, c["cell"], c["pbc"])
    assert abs(r1["energy"] - fresh["energy"]) / c["n"] < 2e-6
    assert np.abs(r1["forces"] - fresh["forces"]).max() < 2e-5
    p2 = p1.copy(); p2[5] += [0.4, 0.0, 0.0]                                   # > skin / 2
    s.compute(c["types"], p2, c["cell"], c["pbc"])
    assert s.rebuilds == 2
    t2 = c["types"].copy(); t2[0] = 3 - t2[0]
    s.compute(t2, p2, c["cell"], c["pbc"])
    assert s.rebuilds == 3
    s.compute(t2, p2, c["cell"] * 1.01, c["pbc"])
    assert s.rebuilds == 4
    assert r0["energy"] != r1["energy"]


def test_batch_equals_single(backend, models, cells):
    """python/tests/test_gpu_batch.py:85-92: 2e-6 eV/atom, 2e-5 eV/A, virial / n 2e-5"""
    for name in ["grace_1l_order3", "grace_2l_order3"]:
        m = _model(backend, models, name)
        cs = [cells.get(k) for k in ["W54", "tri9", "WMo54", "slab36", "atom1", "W2tri"]]
        species = ["Mo", "W"]
        def tt(c):   # types of the two-species batch
            return np.array([species.index(c["species"][t - 1]) + 1 for t in c["types"]], dtype=np.int32)
        natoms = np.array([c["n"] for c in cs], dtype=np.int32)
        types = np.concatenate([tt(c) for c in cs])
        pos = np.concatenate([c["positions"] for c in cs])
        cell = np.stack([c["cell"] for c in cs])
        pbc = np.stack([c["pbc"] for c in cs])
        b = backend.Batch(m, species)
        for max_nall in (1 << 21, 60):       # one pass; several passes of whole structures
            r = b.compute(natoms, types, pos, cell, pbc, energies=True, max_nall=max_nall)
            assert b.passes == (1 if max_nall > 1000 else 4)      # [W54] [tri9] [WMo54] [slab36 atom1 W2tri]
            at = 0
            for q, c in enumerate(cs):
                one = _compute(backend, m, c, skin=0.0)
                assert abs(r["energy"][q] - one["energy"]) / c["n"] < 2e-6
                assert np.abs(r["forces"][at:at + c["n"]] - one["forces"]).max() < 2e-5
                assert np.abs(r["virial"][q] - one["virial"]).max() / c["n"] < 2e-5
                assert np.abs(r["energies"][at:at + c["n"]] - one["energies"]).max() < 2e-6
                at += c["n"]


def test_replicated_cell_scales(backend, models, cells):
    """2 x 2 x 2 copies of a cell give 8 x the energy and the same forces (tests/kk/test_kk_large.cpp:1-8)"""
    c = cells.get("WMo54")
    for name in ["grace_1l_order3", "grace_2l_order3"]:
        m = _model(backend, models, name)
        a = _compute(backend, m, c)
        reps = [(i, j, k) for i in range(2) for j in range(2) for k in range(2)]
        pos = np.concatenate([c["positions"] + np.array(r) @ c["cell"] for r in reps])
        big = dict(c, positions=pos, types=np.tile(c["types"], 8), cell=2 * c["cell"], n=8 * c["n"])
        b = _compute(backend, m, big, chunksize=100)
        assert abs(b["energy"] - 8 * a["energy"]) / big["n"] < 2e-6
        assert np.abs(b["forces"] - np.tile(a["forces"], (8, 1))).max() < 2e-5
        assert np.abs(b["virial"] - 8 * a["virial"]).max() / big["n"] < 2e-5


def test_errors(backend, models, cells):
    c = cells.get("W54")
    m = _model(backend, models, "grace_1l_order3")
    with pytest.raises(ValueError, match="not in the model"):
        backend.System(m, ["Xx"])
    s = backend.System(m, ["W"])
    with pytest.raises(ValueError, match="types must be"):
        s.compute(c["types"] + 1, c["positions"], c["cell"], c["pbc"])
    with pytest.raises(ValueError, match="full-rank"):
        s.compute(c["types"], c["positions"], np.zeros((3, 3)), c["pbc"])
    p = c["positions"].copy(); p[1] = p[0]
    with pytest.raises(ValueError, match="same position"):
        s.compute(c["types"], p, c["cell"], c["pbc"])
    with pytest.raises(ValueError, match="no usable UQ head"):     # python/kk/kk_core.cpp:826-827
        s.compute(c["types"], c["positions"], c["cell"], c["pbc"], uq=True)
    r = s.compute(c["types"], c["positions"], c["cell"], c["pbc"])       # usable after the failures
    assert np.isfinite(r["energy"])
    e = s.compute(np.zeros(0, dtype=np.int32), np.zeros((0, 3)), c["cell"], c["pbc"])
    assert e["energy"] == 0.0 and e["forces"].shape == (0, 3)


def test_injected_failures_recover(backend, models, cells, tmp_path_factory):
    """host-side fault injection (python/kk/kk_core.cpp:128-141,187-195; python/tests/test_gpu_alloc_failure.py): a
    failed allocation or launch is a RuntimeError that leaves the System usable; with the automatic chunk size a large
    enough structure is retried with half the pass.  Nothing here faults the GPU."""
    c = cells.get("WMo54")
    m = _model(backend, models, "grace_2l_order3")
    ok = _compute(backend, m, c)
    s = backend.System(m, c["species"], chunksize=-1)
    s.compute(c["types"], c["positions"], c["cell"], c["pbc"])
    s.release_buffers()
    backend._debug_fail_alloc("work:", 1)
    try:
        with pytest.raises(RuntimeError, match="does not fit|allocat"):
            s.compute(c["types"], c["positions"], c["cell"], c["pbc"])     # 54 atoms: no smaller pass to try
    finally:
        backend._debug_fail_alloc("", 0)
    r = s.compute(c["types"], c["positions"], c["cell"], c["pbc"])
    assert abs(r["energy"] - ok["energy"]) / c["n"] < 2e-6
    backend._debug_fail_launch(3)
    try:
        with pytest.raises(RuntimeError):
            s.compute(c["types"], c["positions"], c["cell"], c["pbc"])
    finally:
        backend._debug_fail_launch(0)
    r = s.compute(c["types"], c["positions"], c["cell"], c["pbc"])
    assert np.abs(r["forces"] - ok["forces"]).max() < 2e-5
    # automatic chunk: 2000 atoms in one pass -> retried with the power of two below n / 2 = 512 atoms per pass
    path, els, big = _config_case(tmp_path_factory, "1l", "bcc", 3.165, (10, 10, 10), 1, 0.05, seed=2)
    mb = backend.Model(path)
    ref = _compute(backend, mb, big)
    sb = backend.System(mb, els, chunksize=-1)
    sb.release_buffers()           # the work buffers are shared by the Systems of a model: grown again below
    backend._debug_fail_alloc("work:", 1)
    try:
        rb = sb.compute(big["types"], big["positions"], big["cell"], big["pbc"])
    finally:
        backend._debug_fail_alloc("", 0)
    assert sb.chunksize == 512
    assert abs(rb["energy"] - ref["energy"]) / big["n"] < 2e-6
    assert np.abs(rb["forces"] - ref["forces"]).max() < 2e-5
    # fixed chunk: the failure is reported, the System works afterwards
    sf = backend.System(mb, els, chunksize=512)
    sf.release_buffers()
    backend._debug_fail_alloc("work:", 1)
    try:
        with pytest.raises(RuntimeError, match="failed to allocate"):
            sf.compute(big["types"], big["positions"], big["cell"], big["pbc"])
    finally:
        backend._debug_fail_alloc("", 0)
    rf = sf.compute(big["types"], big["positions"], big["cell"], big["pbc"])
    assert np.abs(rf["forces"] - ref["forces"]).max() < 2e-5


# ---- the benchmark configurations at (or near) their stated sizes, against the compiled reference live -----------
@pytest.mark.parametrize("cfg,lattice,a,reps,nsp,sigma,full", [
    ("1l", "bcc", 3.165, (10, 10, 10), 1, 0.05, False),     # configuration 1 as stated: 2,000 atoms of bcc W
    ("1l", "bcc", 3.2, (20, 20, 20), 4, 0.05, True),        # a 16,000-atom block of configuration 2 (89-element model)
    ("2l", "fcc", 3.6, (13, 13, 13), 3, 0.08, True),        # an 8,788-atom block of configuration 3 (89-element model)
])
def test_stated_configurations_match_compiled_reference(backend, tmp_path_factory, cfg, lattice, a, reps, nsp, sigma, full):
    """energy, forces, stress and per-atom energies of the benchmark workloads themselves (same model generator, same
    structure generator, same seeds as bench.py) against the reference's CPU drivers, within the stated tolerances"""
    from grace_runtime_b200 import modelgen, structures
    from oracle import refcpu
    if not refcpu.available():
        pytest.skip("oracle/_ref is not built")
    species = modelgen._subset(2024, nsp) if full else ["W"]
    elements = modelgen.ELEMENTS if full else species
    path = modelgen.write_config_model(str(tmp_path_factory.mktemp("stated") / f"{cfg}.npz"), cfg, elements, seed=0)
    types, pos, cell, pbc = structures.crystal(lattice, a, reps, n_species=nsp, sigma=sigma, seed=1)
    n, vol = len(types), abs(np.linalg.det(cell))
    r = backend.System(backend.Model(path), species).compute(types, pos, cell, pbc, energies=True)
    ref = refcpu.RefModel(path, species).compute(types, pos, cell, pbc, nthreads=0)
    assert abs(r["energy"] - ref["energy"]) / n < TOL_E
    assert np.abs(r["forces"] - ref["forces"]).max() < TOL_F
    assert np.abs(r["virial"] - ref["virial"]).max() / vol < TOL_S
    assert np.abs(r["energies"] - ref["energies"]).max() < TOL_E


@pytest.mark.parametrize("cell", TF_CELLS + ["slab36", "tri9", "cluster13"])
def test_device_neighbor_list_equals_cpu_search(backend, models, cells, cell):
    """the device list bond for bond against the CPU cell-list search, as the reference checks its own device list
    (tests/kk/test_kk_neighbors.cpp:1-6): same (i, j, cell shift) multiset at radius cutoff + skin"""
    from oracle.grace_oracle import neighbor_list
    c = cells.get(cell)
    s = backend.System(_model(backend, models, "grace_1l_order3"), c["species"], skin=0.5)
    s.compute(c["types"], c["positions"], c["cell"], c["pbc"])
    bi, bj, bs = s.neighbor_list()
    a = neighbor_list(c["positions"], c["cell"], c["pbc"], s.cutoff + 0.5)
    got = sorted(zip(bi.tolist(), bj.tolist(), map(tuple, bs.tolist())))
    want = sorted(zip(a[0].tolist(), a[1].tolist(), map(tuple, a[2].tolist())))
    assert len(got) == len(want) and got == want


def test_device_neighbor_list_equals_reference_search_large(backend, tmp_path_factory):
    """the same on 2,000 displaced bcc atoms against the reference's own search (python/src/neighbors.cpp)"""
    from oracle import refcpu
    if not refcpu.available():
        pytest.skip("oracle/_ref is not built")
    path, els, c = _config_case(tmp_path_factory, "1l", "bcc", 3.165, (10, 10, 10), 1, 0.05, seed=3)
    s = backend.System(backend.Model(path), els, skin=0.5)
    s.compute(c["types"], c["positions"], c["cell"], c["pbc"])
    bi, bj, bs = s.neighbor_list()
    ri, rj, rs = refcpu.neighbors(c["positions"], c["cell"], c["pbc"], s.cutoff + 0.5)
    key = lambda i, j, S: np.lexsort((S[:, 2], S[:, 1], S[:, 0], j, i))
    ka, kb = key(bi, bj, bs), key(ri, rj, rs)
    assert len(bi) == len(ri)
    assert np.array_equal(bi[ka], ri[kb]) and np.array_equal(bj[ka], rj[kb]) and np.array_equal(bs[ka], rs[kb])


def test_one_engine_per_spline(backend, cells):
    """Systems of one model share an engine per radial mode (python/kk/kk_core.cpp:232,268-300; engine_setups counts
    them): the same spline reuses it, another resolution builds a second one whose energy differs at table-error
    level"""
    c = cells.get("WMo54")
    m = backend.Model(model_path("grace_1l_order3"))
    a = backend.System(m, c["species"], spline=1024).compute(c["types"], c["positions"], c["cell"], c["pbc"])
    assert m.engine_setups == 1
    a2 = backend.System(m, c["species"], spline=1024).compute(c["types"], c["positions"], c["cell"], c["pbc"])
    assert m.engine_setups == 1 and a2["energy"] == a["energy"]
    b = backend.System(m, c["species"], spline=64).compute(c["types"], c["positions"], c["cell"], c["pbc"])
    assert m.engine_setups == 2
    d = abs(a["energy"] - b["energy"]) / c["n"]
    assert 0.0 < d < 1e-3, d
    with pytest.raises(ValueError):
        backend.System(m, c["species"], spline=8)


def test_calls_from_a_second_host_thread(backend, models, cells):
    """any host thread may call (python/kk/kk_core.cpp:58-63): the current CUDA device is a per-thread setting, which
    the library sets itself"""
    import threading
    import torch
    c = cells.get("W54")
    m = _model(backend, models, "grace_2l_order3")
    want = _compute(backend, m, c)
    got = {}

    def work():
        try:
            got["r"] = _compute(backend, m, c)
            v = torch.arange(12, dtype=torch.float64, device="cuda:0").reshape(4, 3)
            out = torch.zeros(3, dtype=torch.float64, device="cuda:0")
            backend.sum_rows_static(v.data_ptr(), 4, 3, out.data_ptr())
            got["s"] = out.cpu().numpy()
        except Exception as e:      # surfaced by the assert below
            got["err"] = e

    t = threading.Thread(target=work)
    t.start()
    t.join()
    assert "err" not in got, got.get("err")
    assert got["r"]["energy"] == want["energy"]
    assert np.abs(got["r"]["forces"] - want["forces"]).max() < 1e-6
    assert np.array_equal(got["s"], np.array([18.0, 22.0, 26.0]))


def test_compute_device_takes_device_arrays_without_conversion(backend, models, cells):
    """Batch.compute_device with torch tensors of the GPU (python/kk/kk_module.cpp:142-197): results equal compute();
    host arrays, wrong dtypes and wrong shapes are ValueErrors, nothing is converted"""
    import torch
    c = cells.get("WMo54")
    m = _model(backend, models, "grace_2l_order3")
    b = backend.Batch(m, c["species"])
    natoms = np.array([c["n"], c["n"]], dtype=np.int32)
    types = np.concatenate([c["types"], c["types"]]).astype(np.int32)
    pos = np.concatenate([c["positions"], c["positions"] + 0.01])
    cells2 = np.stack([c["cell"], c["cell"]])
    pbc2 = np.stack([c["pbc"], c["pbc"]])
    want = b.compute(natoms, types, pos, cells2, pbc2, energies=True)
    dev = torch.device("cuda", 0)
    d_t, d_x = torch.from_numpy(types).to(dev), torch.from_numpy(pos).to(dev)
    e = torch.zeros(2, dtype=torch.float64, device=dev)
    f = torch.zeros((2 * c["n"], 3), dtype=torch.float64, device=dev)
    v = torch.zeros((2, 6), dtype=torch.float64, device=dev)
    ea = torch.zeros(2 * c["n"], dtype=torch.float64, device=dev)
    b.compute_device(natoms, d_t, d_x, cells2, pbc2, e, forces=f, virial=v, energies=ea)
    assert np.abs(e.cpu().numpy() - want["energy"]).max() < 1e-9
    assert np.abs(f.cpu().numpy() - want["forces"]).max() < 1e-6
    assert np.abs(v.cpu().numpy() - want["virial"]).max() < 1e-6
    assert np.abs(ea.cpu().numpy() - want["energies"]).max() < 1e-9
    with pytest.raises(ValueError):
        b.compute_device(natoms, types, d_x, cells2, pbc2, e)                       # host types
    with pytest.raises(ValueError):
        b.compute_device(natoms, d_t, d_x.float(), cells2, pbc2, e)                 # float32 positions
    with pytest.raises(ValueError):
        b.compute_device(natoms, d_t, d_x, cells2, pbc2, e, forces=f[:, :2])        # wrong shape / not contiguous
    with pytest.raises(ValueError):
        b.compute_device(natoms, d_t, d_x, cells2, pbc2, e.cpu())                   # host output
    with pytest.raises(ValueError, match="no usable UQ head"):
        b.compute_device(natoms, d_t, d_x, cells2, pbc2, e, gamma=ea)               # no UQ head


def test_allocation_tracking(backend, models, cells):
    """_debug_track_alloc / _debug_peak_alloc / _debug_live_alloc (python/kk/kk_core.cpp:143-184)"""
    c = cells.get("W54")
    m = _model(backend, models, "grace_1l_order3")
    s = backend.System(m, c["species"])
    s.compute(c["types"], c["positions"], c["cell"], c["pbc"])
    s.release_buffers()
    backend._debug_track_alloc(True)
    try:
        s.compute(c["types"], c["positions"], c["cell"], c["pbc"])
        peak = backend._debug_peak_alloc()
        live = backend._debug_live_alloc()
    finally:
        backend._debug_track_alloc(False)
    assert peak > 0 and live and sum(b for _, b in live) <= peak
    assert backend._debug_peak_alloc() == 0
