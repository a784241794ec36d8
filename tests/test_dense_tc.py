"""The dense network on the tensor cores (csrc/mv_tc.cu: FC layers and their adjoints as tcgen05 3 x tf32 grouped GEMMs
over atom tiles, operation by operation on chunk tensors) against the fused fp32 kernel, the numpy oracle, the golden
vectors and - where it travelled - the compiled reference.  The path is the default for large evaluations; here it is
forced on small ones with GRACE_B200_DENSE=tc (read when a model's engine is built)."""
import numpy as np
import pytest

from conftest import REF_TOL, TF_CELLS, TOL_E, TOL_F, TOL_S, compare_tf, model_path, stress_of

pytestmark = pytest.mark.gpu


def _run(backend, path, c, mode, monkeypatch, chunksize=-1, profile=False):
    monkeypatch.setenv("GRACE_B200_DENSE", mode)
    m = backend.Model(path)
    s = backend.System(m, c["species"], chunksize=chunksize)
    if profile:
        backend.profile_enable(True)
    r = s.compute(c["types"], c["positions"], c["cell"], c["pbc"], energies=True)
    if profile:
        r["kernels"] = backend.profile_report()
        backend.profile_enable(False)
    return r


def _case(tmp_path_factory, cfg, lattice, a, reps, nsp, sigma, seed):
    from grace_runtime_b200 import modelgen, structures
    els = modelgen._subset(11, nsp)
    path = str(tmp_path_factory.mktemp("tc") / f"{cfg}.npz")
    modelgen.write_config_model(path, cfg, els, seed=seed)
    types, pos, cell, pbc = structures.crystal(lattice, a, reps, n_species=nsp, sigma=sigma, seed=seed + 1)
    return path, dict(species=els, types=types, positions=pos, cell=cell, pbc=pbc, n=len(types),
                      volume=abs(np.linalg.det(cell)))


@pytest.mark.parametrize("cfg,lattice,a,reps,nsp,sigma", [("1l", "bcc", 3.2, (4, 4, 5), 4, 0.05),
                                                           ("2l", "fcc", 3.6, (3, 3, 4), 3, 0.08)])
def test_tensor_core_path_matches_oracle_and_fused(backend, tmp_path_factory, monkeypatch, cfg, lattice, a, reps, nsp, sigma):
    """benchmark architectures (32 / 64 channels): tensor-core operations against the numpy fp64 oracle within the
    stated tolerances and against the fused fp32 kernel at rounding level; the kernel list shows the path that ran"""
    from oracle.grace_oracle import GraceOracle
    path, c = _case(tmp_path_factory, cfg, lattice, a, reps, nsp, sigma, seed=31)
    tc = _run(backend, path, c, "tc", monkeypatch, profile=True)
    assert any("mv_tc_kernel" in k for k in tc["kernels"]), sorted(tc["kernels"])
    assert not any("chain_fused" in k for k in tc["kernels"])
    fu = _run(backend, path, c, "fused", monkeypatch)
    ops = _run(backend, path, c, "ops", monkeypatch, profile=True)    # every operation as its fp32 SIMT kernel
    assert not any("mv_tc_kernel" in k or "chain_fused" in k for k in ops["kernels"])
    o = GraceOracle(path).compute(c["species"], c["types"], c["positions"], c["cell"], c["pbc"])
    for r in (tc, fu, ops):
        assert abs(r["energy"] - o["energy"]) / c["n"] < TOL_E
        assert np.abs(r["forces"] - o["forces"]).max() < TOL_F
        assert np.abs(r["virial"] - o["virial"]).max() / c["volume"] < TOL_S
        assert np.abs(r["energies"] - o["energies"]).max() < TOL_E
    assert abs(tc["energy"] - fu["energy"]) / c["n"] < 1e-6
    assert np.abs(tc["forces"] - fu["forces"]).max() < 1e-5


@pytest.mark.parametrize("cell", TF_CELLS)
@pytest.mark.parametrize("name", ["grace_1l_order3", "grace_2l_order3", "legacy_1l_order3", "legacy_2l_order3"])
def test_tensor_core_path_on_tf_goldens(backend, cells, tf_golden, monkeypatch, name, cell):
    """the reference's TensorFlow-fp64 golden cases under its own thresholds, with every eligible operation on the
    tensor cores (models whose widths the kernel does not cover keep their fp32 kernels: same thresholds)"""
    c = cells.get(cell)
    r = _run(backend, model_path(name), c, "tc", monkeypatch)
    d = compare_tf(r, tf_golden, f"{name}/{cell}", c)
    for q, v in d.items():
        assert v < (2e-6 if q == "energy" and c["n"] < 10 else REF_TOL[q]), (q, v)


def test_tensor_core_path_passes_with_ragged_tiles(backend, tmp_path_factory, monkeypatch):
    """passes of 200 atoms over 432 atoms: atom tiles of 128 with ragged ends; equal to one pass"""
    path, c = _case(tmp_path_factory, "2l", "fcc", 3.6, (3, 6, 6), 3, 0.08, seed=33)
    a = _run(backend, path, c, "tc", monkeypatch, chunksize=0)
    b = _run(backend, path, c, "tc", monkeypatch, chunksize=200)
    assert abs(a["energy"] - b["energy"]) / c["n"] < 2e-6
    assert np.abs(a["forces"] - b["forces"]).max() < 2e-5
    ds = np.abs(stress_of(a["virial"], c["volume"]) - stress_of(b["virial"], c["volume"])).max()
    assert ds < 1e-6


def test_tensor_core_path_matches_compiled_reference(backend, tmp_path_factory, monkeypatch):
    """an 8,788-atom block of the 1,024,000-atom GRACE-2L workload (89-element model): large enough that the tensor-core
    path is the default one"""
    from grace_runtime_b200 import modelgen, structures
    from oracle import refcpu
    if not refcpu.available():
        pytest.skip("oracle/_ref is not built")
    monkeypatch.setenv("GRACE_B200_TC_MIN_ATOMS", "4096")
    monkeypatch.delenv("GRACE_B200_DENSE", raising=False)
    species = modelgen._subset(2024, 3)
    path = modelgen.write_config_model(str(tmp_path_factory.mktemp("tcref") / "2l.npz"), "2l", modelgen.ELEMENTS, seed=0)
    types, pos, cell, pbc = structures.crystal("fcc", 3.6, (13, 13, 13), n_species=3, sigma=0.08, seed=1)
    n, vol = len(types), abs(np.linalg.det(cell))
    backend.profile_enable(True)
    r = backend.System(backend.Model(path), species).compute(types, pos, cell, pbc, energies=True)
    kernels = backend.profile_report()
    backend.profile_enable(False)
    assert any("mv_tc_kernel" in k for k in kernels), sorted(kernels)
    ref = refcpu.RefModel(path, species).compute(types, pos, cell, pbc, nthreads=0)
    assert abs(r["energy"] - ref["energy"]) / n < TOL_E
    assert np.abs(r["forces"] - ref["forces"]).max() < TOL_F
    assert np.abs(r["virial"] - ref["virial"]).max() / vol < TOL_S
    assert np.abs(r["energies"] - ref["energies"]).max() < TOL_E
