"""UQ head (extrapolation grade gamma, Mahalanobis distance sigma, nearest mixture component per atom; schema 6).
The reference tree has no model with a head, so the order-4 fixture models get a seeded random one
(modelgen.add_uq_head); the golden vectors tests/golden/uq_ref.npz are the outputs of the reference's own CPU drivers on
exactly these files (tests/golden/make_uq_golden.py).  CPU: numpy restatement against the goldens and the compiled
reference, loader checks.  GPU: the library through the C ABI against the goldens (System, Batch, device arrays, chunked
passes, tensor-core and SIMT forms of the projection), energies and forces unchanged by the flag, error behaviour of
python/kk/kk_core.cpp:826-827."""
import os
import sys

import numpy as np
import pytest

from conftest import GOLDEN, model_path

sys.path.insert(0, os.path.join(GOLDEN))
from make_uq_golden import UQ_CELLS, UQ_MODELS, uq_model  # noqa: E402

# gamma and sigma: the projection runs in fp32 (reference) / 3 x tf32 or fp32 (here) on an fp32 basis; everything after
# it is fp64.  The reference documents ~1e-5 of its own fp32 projection against fp64.
UQ_RTOL = 1e-4


@pytest.fixture(scope="module")
def uq_gold():
    return np.load(os.path.join(GOLDEN, "uq_ref.npz"))


@pytest.fixture(scope="module")
def uq_paths(tmp_path_factory):
    tmp = str(tmp_path_factory.mktemp("uq"))
    return {name: uq_model(name, seed, rp, k, tmp) for name, seed, rp, k in UQ_MODELS}


def _check(r, gold, key, n, rtol=UQ_RTOL):
    g = gold[f"{key}/gamma"]
    assert r["gamma"].shape == (n,)
    assert np.array_equal(r["gmm_cluster"] if "gmm_cluster" in r else r["cluster"], gold[f"{key}/cluster"])
    sg = r["atomic_sigma"] if "atomic_sigma" in r else r["sigma"]
    assert np.abs(r["gamma"] / g - 1.0).max() < rtol
    assert np.abs(sg / gold[f"{key}/sigma"] - 1.0).max() < rtol


@pytest.mark.parametrize("name", [m[0] for m in UQ_MODELS])
def test_oracle_uq_matches_reference_goldens(cells, uq_gold, uq_paths, name):
    from oracle.grace_oracle import GraceOracle
    o = GraceOracle(uq_paths[name], spline_n=1024)
    for cn in ["WMo54", "tri9", "atom1"]:
        c = cells.get(cn)
        r = o.compute(c["species"], c["types"], c["positions"], c["cell"], c["pbc"], uq=True)
        _check(r, uq_gold, f"{name}/{cn}", c["n"], rtol=2e-6)


def test_compiled_reference_reproduces_uq_goldens(cells, uq_gold, uq_paths):
    from oracle import refcpu
    if not refcpu.available():
        pytest.skip("oracle/_ref is not built")
    for name in ("grace_1l_small", "legacy_2l_small"):    # (legacy_1l_wide: see make_uq_golden.py)
        c = cells.get("WMo54")
        r = refcpu.RefModel(uq_paths[name], c["species"]).compute(c["types"], c["positions"], c["cell"], c["pbc"], uq=True)
        _check(r, uq_gold, f"{name}/WMo54", c["n"], rtol=1e-12)


def test_uq_head_writer_checks_the_model():
    from grace_runtime_b200 import modelgen
    with pytest.raises(ValueError, match="max_order 4"):
        modelgen.add_uq_head(model_path("grace_1l_order3"), os.devnull)


# ---- GPU ---------------------------------------------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("cn", UQ_CELLS)
@pytest.mark.parametrize("name", [m[0] for m in UQ_MODELS])
def test_system_uq_matches_reference(backend, cells, uq_gold, uq_paths, name, cn):
    c = cells.get(cn)
    m = backend.Model(uq_paths[name])
    assert m.has_uq
    m.validate_uq()
    s = backend.System(m, c["species"])
    r = s.compute(c["types"], c["positions"], c["cell"], c["pbc"], energies=True, uq=True)
    _check(r, uq_gold, f"{name}/{cn}", c["n"])
    assert abs(r["total_sigma"] - r["atomic_sigma"].sum()) < 1e-9
    assert abs(r["energy"] - float(uq_gold[f"{name}/{cn}/energy"])) / c["n"] < 1e-5
    # the flag changes nothing else (the reference's tests/test_driver_uq.cpp checks the same of its drivers)
    r0 = s.compute(c["types"], c["positions"], c["cell"], c["pbc"], energies=True)
    assert abs(r["energy"] - r0["energy"]) / c["n"] < 1e-6
    assert np.abs(r["forces"] - r0["forces"]).max() < 1e-5
    # energy_only keeps the UQ outputs
    r1 = s.compute(c["types"], c["positions"], c["cell"], c["pbc"], uq=True, energy_only=True)
    assert np.array_equal(r1["gamma"], r["gamma"]) and "forces" not in r1


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["tc", "ops"])
@pytest.mark.parametrize("name", ["grace_1l_small", "grace_2l_small"])
def test_uq_chunked_passes_and_projection_kernels(backend, cells, uq_gold, uq_paths, monkeypatch, name, mode):
    """passes of 16 atoms (GRACE-2L: the layer-1 projection rows wait for layer 2), projection as the tensor-core
    kernel or as the SIMT kernel"""
    monkeypatch.setenv("GRACE_B200_DENSE", mode)
    c = cells.get("WMo54")
    s = backend.System(backend.Model(uq_paths[name]), c["species"], chunksize=16)
    backend.profile_enable(True)
    r = s.compute(c["types"], c["positions"], c["cell"], c["pbc"], uq=True)
    kernels = backend.profile_report()
    backend.profile_enable(False)
    assert any("uq_gmm_kernel" in k for k in kernels) and any("uq_norm_kernel" in k for k in kernels)
    assert s.chunksize == 16
    _check(r, uq_gold, f"{name}/WMo54", c["n"])


@pytest.mark.gpu
@pytest.mark.parametrize("layers,lmax,lattice,a,reps", [(1, 4, "bcc", 3.2, (4, 4, 5)), (2, 2, "fcc", 3.6, (3, 3, 4))])
def test_uq_of_generated_order4_models_against_the_compiled_reference(backend, tmp_path, monkeypatch, layers, lmax, lattice, a, reps):
    """32 / 64-channel models of body order 5 (the shapes the tensor-core kernel covers): the projection runs as
    mv_tc_kernel; gamma, sigma and cluster against the reference's CPU drivers evaluated here"""
    from grace_runtime_b200 import modelgen, structures
    from oracle import refcpu
    if not refcpu.available():
        pytest.skip("oracle/_ref is not built")
    els = modelgen._subset(5, 3)
    base = str(tmp_path / "m.npz")
    modelgen.write_model(base, layers=layers, lmax=lmax, max_order=4, elements=tuple(els), c1=32, cr=16, c2=64,
                         rho_n_out=9, energy_hidden=(32,), avg_neigh=58.0 if lattice == "bcc" else 78.0, seed=3)
    path = modelgen.add_uq_head(base, str(tmp_path / "m_uq.npz"), seed=9, rp_dim=32, max_clusters=3)
    types, pos, cell, pbc = structures.crystal(lattice, a, reps, n_species=3, sigma=0.06, seed=4)
    ref = refcpu.RefModel(path, els).compute(types, pos, cell, pbc, uq=True)
    monkeypatch.setenv("GRACE_B200_DENSE", "tc")
    s = backend.System(backend.Model(path), els)
    backend.profile_enable(True)
    r = s.compute(types, pos, cell, pbc, uq=True)
    kernels = backend.profile_report()
    backend.profile_enable(False)
    assert any("mv_tc_kernel" in k for k in kernels)
    assert np.array_equal(r["gmm_cluster"], ref["cluster"])
    assert np.abs(r["gamma"] / ref["gamma"] - 1.0).max() < UQ_RTOL
    assert np.abs(r["atomic_sigma"] / ref["sigma"] - 1.0).max() < UQ_RTOL
    assert abs(r["energy"] - ref["energy"]) / len(types) < 1e-5


@pytest.mark.gpu
def test_batch_uq_and_device_arrays(backend, cells, uq_gold, uq_paths):
    torch = pytest.importorskip("torch")
    name = "grace_2l_small"
    cs = [cells.get(cn) for cn in ("WMo54", "tri9", "cluster13")]
    species = ["Mo", "W"]
    m = backend.Model(uq_paths[name])
    b = backend.Batch(m, species)
    types = np.concatenate([[species.index(c["species"][t - 1]) + 1 for t in c["types"]] for c in cs]).astype(np.int32)
    pos = np.concatenate([c["positions"] for c in cs])
    natoms = np.array([c["n"] for c in cs], dtype=np.int32)
    cellm = np.stack([c["cell"] for c in cs])
    pbc = np.stack([c["pbc"] for c in cs])
    r = b.compute(natoms, types, pos, cellm, pbc, uq=True)
    a0 = 0
    for c, cn in zip(cs, ("WMo54", "tri9", "cluster13")):
        part = {k: r[k][a0:a0 + c["n"]] for k in ("gamma", "atomic_sigma", "gmm_cluster")}
        _check(part, uq_gold, f"{name}/{cn}", c["n"])
        a0 += c["n"]
    # device arrays, no conversion (python/kk/kk_module.cpp:142-197)
    dev = torch.device("cuda:0")
    ntot = int(natoms.sum())
    t_d, x_d = torch.tensor(types, device=dev), torch.tensor(pos, device=dev)
    e_d = torch.zeros(len(cs), dtype=torch.float64, device=dev)
    g_d, s_d, c_d = (torch.zeros(ntot, dtype=torch.float64, device=dev) for _ in range(3))
    b.compute_device(natoms, t_d, x_d, cellm, pbc, e_d, gamma=g_d, atomic_sigma=s_d, gmm_cluster=c_d, energy_only=True)
    torch.cuda.synchronize()
    assert np.allclose(g_d.cpu().numpy(), r["gamma"], rtol=1e-12, atol=0)
    assert np.array_equal(c_d.cpu().numpy(), r["gmm_cluster"])
    with pytest.raises(ValueError, match="gamma, sigma and cluster"):
        b.compute_device(natoms, t_d, x_d, cellm, pbc, e_d, gamma=g_d, energy_only=True)


@pytest.mark.gpu
def test_uq_errors(backend, cells, tmp_path):
    from grace_runtime_b200 import modelgen
    c = cells.get("WMo54")
    m = backend.Model(model_path("grace_1l_small"))        # no head
    assert not m.has_uq
    with pytest.raises(ValueError, match="no UQ head"):
        m.validate_uq()
    s = backend.System(m, c["species"])
    with pytest.raises(ValueError, match="no usable UQ head"):
        s.compute(c["types"], c["positions"], c["cell"], c["pbc"], uq=True)
    s.compute(c["types"], c["positions"], c["cell"], c["pbc"])    # the System stays usable
    # a head whose projection matrix does not fit the model: loads, evaluates without UQ, refuses UQ
    z = dict(np.load(modelgen.add_uq_head(model_path("grace_1l_small"), str(tmp_path / "a.npz"), seed=1)))
    z["uq_rp_matrix"] = z["uq_rp_matrix"][:-1]
    np.savez(str(tmp_path / "short.npz"), **z)
    m2 = backend.Model(str(tmp_path / "short.npz"))
    assert m2.has_uq
    with pytest.raises(ValueError, match="rows"):
        m2.validate_uq()
    s2 = backend.System(m2, c["species"])
    r = s2.compute(c["types"], c["positions"], c["cell"], c["pbc"])
    assert np.isfinite(r["energy"])
    with pytest.raises(ValueError):
        s2.compute(c["types"], c["positions"], c["cell"], c["pbc"], uq=True)
    # an older schema
    z["uq_schema_version"] = np.array([4])
    np.savez(str(tmp_path / "old.npz"), **z)
    with pytest.raises(ValueError, match="schema"):
        backend.Model(str(tmp_path / "old.npz")).validate_uq()
