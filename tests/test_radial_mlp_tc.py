"""The exact radial MLP on the tensor cores (csrc/radial_mlp_tc.cu, tcgen05) through the C ABI against the fp64 numpy
restatement of the reference's forward-mode MLP (oracle.grace_oracle.radial_basis / mlp_forward_mode; reference
libgrace/include/grace/radial_x.h:11-60), for the benchmark architectures (8 -> 64 -> 64 -> 160 and the two GRACE-2L
MLPs).  Tolerance: 2e-6 of the largest |R| (3 x tf32 products, fp32 sums and activations); 1e-5 of the largest |dR/dx|,
whose Chebyshev derivatives (up to 2 k^2 = 128) amplify the fp32 rounding of the basis the kernel evaluates per bond."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _expected(path, layer, x):
    from oracle.grace_oracle import GraceOracle, mlp_forward_mode, radial_basis
    o = GraceOracle(path)
    layers = o.rad1 if layer == 1 else o.rad2
    g, dg = radial_basis(x.astype(np.float64), o.p, o.nrb)
    R, dR = mlp_forward_mode(layers, g, dg, o.rad_act)
    nl = o.lmax + 1
    C = R.shape[1] // nl
    perm = lambda a: a.reshape(len(x), C, nl).transpose(0, 2, 1).reshape(len(x), -1)     # model order n nl + l -> [l][n]
    return perm(R), perm(dR)


@pytest.mark.parametrize("cfg,layer", [("1l", 1), ("2l", 1), ("2l", 2)])
@pytest.mark.parametrize("nb", [1, 64, 1000, 200_000])
def test_radial_mlp_matches_fp64(backend, tmp_path_factory, cfg, layer, nb):
    import torch
    from grace_runtime_b200 import modelgen
    els = modelgen._subset(11, 3)
    path = str(tmp_path_factory.mktemp("rad") / f"{cfg}.npz")
    modelgen.write_config_model(path, cfg, els, seed=3)
    m = backend.Model(path)
    w = m.radial_mlp_width(layer)
    rng = np.random.default_rng(nb)
    x = rng.uniform(0.05, 0.999, size=nb).astype(np.float32)
    dx = torch.from_numpy(x).cuda()
    R = torch.full((nb, w), float("nan"), dtype=torch.float32, device="cuda")
    dR = torch.full((nb, w), float("nan"), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    for _ in range(2):        # a second launch reuses the set-up
        m.radial_mlp_device(layer, nb, dx.data_ptr(), R.data_ptr(), dR.data_ptr())
    eR, edR = _expected(path, layer, x)
    gR, gdR = R.cpu().numpy().astype(np.float64), dR.cpu().numpy().astype(np.float64)
    assert np.isfinite(gR).all() and np.isfinite(gdR).all()
    assert np.abs(gR - eR).max() <= 2e-6 * max(1.0, np.abs(eR).max())
    assert np.abs(gdR - edR).max() <= 1e-5 * max(1.0, np.abs(edR).max())


@pytest.mark.parametrize("cfg,lattice,a,reps,nsp,sigma", [("1l", "bcc", 3.2, (4, 4, 5), 4, 0.05),
                                                           ("2l", "fcc", 3.6, (3, 3, 3), 3, 0.08)])
def test_exact_radial_mode_matches_oracle(backend, tmp_path_factory, cfg, lattice, a, reps, nsp, sigma):
    """spline = 0: energies, forces and virial with the radial MLP evaluated per bond by the tensor-core kernel, against
    the numpy oracle with its exact MLP, and against the table mode of the same library (whose interpolation error is
    the only difference)"""
    from conftest import TOL_E, TOL_F, TOL_S
    from grace_runtime_b200 import modelgen, structures
    from oracle.grace_oracle import GraceOracle
    els = modelgen._subset(11, nsp)
    path = str(tmp_path_factory.mktemp("exact") / f"{cfg}.npz")
    modelgen.write_config_model(path, cfg, els, seed=5)
    types, pos, cell, pbc = structures.crystal(lattice, a, reps, n_species=nsp, sigma=sigma, seed=6)
    n, vol = len(types), abs(np.linalg.det(cell))
    exact = backend.System(backend.Model(path, spline=0), els, spline=0)
    r = exact.compute(types, pos, cell, pbc, energies=True)
    r2 = exact.compute(types, pos, cell, pbc, energies=True)
    # (GRACE-2L adds dE/dmessage into neighbour rows with fp32 atomics: forces repeat to rounding, not to the bit)
    assert r["energy"] == r2["energy"] and np.abs(r["forces"] - r2["forces"]).max() < 1e-6
    o = GraceOracle(path).compute(els, types, pos, cell, pbc)
    assert abs(r["energy"] - o["energy"]) / n < TOL_E * 0.1
    assert np.abs(r["forces"] - o["forces"]).max() < TOL_F
    assert np.abs(r["virial"] - o["virial"]).max() / vol < TOL_S
    assert np.abs(r["energies"] - o["energies"]).max() < TOL_E
    t = backend.System(backend.Model(path), els).compute(types, pos, cell, pbc)
    assert abs(r["energy"] - t["energy"]) / n < TOL_E
    assert np.abs(r["forces"] - t["forces"]).max() < TOL_F
