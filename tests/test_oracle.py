"""The oracle pinned: the numpy restatement (oracle/grace_oracle.py) against the reference's own golden vectors
(TensorFlow fp64, python/tests/test_order3_tf.py) and against frozen outputs of the reference CPU drivers; the
compiled reference (oracle/_ref) against the same goldens where it is built."""
import numpy as np
import pytest

from conftest import EXTRA_CELLS, F32_MODELS, REF_TOL, TF_CELLS, TF_MODELS, compare_tf, model_path
from oracle import refcpu
from oracle.grace_oracle import GraceOracle, neighbor_list, sph_harm


@pytest.fixture(scope="module")
def oracles():
    return {}


def _oracle(oracles, name, spline=0):
    k = (name, spline)
    if k not in oracles:
        oracles[k] = GraceOracle(model_path(name), spline_n=spline)
    return oracles[k]


@pytest.mark.parametrize("cell", TF_CELLS)
@pytest.mark.parametrize("name", TF_MODELS)
def test_oracle_matches_tf_fp64(oracles, cells, tf_golden, name, cell):
    c = cells.get(cell)
    r = _oracle(oracles, name).compute(c["species"], c["types"], c["positions"], c["cell"], c["pbc"])
    d = compare_tf(r, tf_golden, f"{name}/{cell}", c)
    # exact MLP in fp64 against TensorFlow fp64: far below the reference's fp32 thresholds
    assert d["energy"] < 1e-9 and d["forces"] < 1e-9 and d["energies"] < 1e-9 and d["stress"] < 1e-8, d
    assert np.abs(tf_golden[f"{name}/{cell}/forces"]).max() > 1e-2


@pytest.mark.parametrize("cell", ["WMo54", "tri9", "slab36", "cluster13", "atom1"])
@pytest.mark.parametrize("name", TF_MODELS + F32_MODELS)
def test_oracle_matches_reference_cpu(oracles, cells, ref_golden, name, cell):
    """spline-table oracle against the frozen outputs of the reference CPU drivers (fp32 network)"""
    c = cells.get(cell)
    r = _oracle(oracles, name, 1024).compute(c["species"], c["types"], c["positions"], c["cell"], c["pbc"])
    k = f"{name}/{cell}"
    assert abs(r["energy"] - ref_golden[f"{k}/energy"]) / c["n"] < REF_TOL["energy"]
    assert np.abs(r["forces"] - ref_golden[f"{k}/forces"]).max() < REF_TOL["forces"]
    assert np.abs(r["energies"] - ref_golden[f"{k}/energies"]).max() < REF_TOL["energies"]
    assert np.abs(r["virial"] - ref_golden[f"{k}/virial"]).max() < 2e-5 * max(1.0, np.abs(ref_golden[f"{k}/virial"]).max())


@pytest.mark.skipif(not refcpu.available(), reason="oracle/_ref is not built")
@pytest.mark.parametrize("cell", TF_CELLS)
@pytest.mark.parametrize("name", TF_MODELS)
def test_compiled_reference_matches_tf_fp64(cells, tf_golden, name, cell):
    c = cells.get(cell)
    r = refcpu.RefModel(model_path(name), c["species"]).compute(c["types"], c["positions"], c["cell"], c["pbc"], nthreads=2)
    d = compare_tf(r, tf_golden, f"{name}/{cell}", c)
    for q, v in d.items():
        assert v < (2e-6 if q == "energy" and c["n"] < 10 else REF_TOL[q]), (q, v)


@pytest.mark.skipif(not refcpu.available(), reason="oracle/_ref is not built")
@pytest.mark.parametrize("cell", TF_CELLS + ["slab36", "tri9", "cluster13"])
def test_neighbor_list_matches_reference(cells, cell):
    c = cells.get(cell)
    a = neighbor_list(c["positions"], c["cell"], c["pbc"], 5.0)
    b = refcpu.neighbors(c["positions"], c["cell"], c["pbc"], 5.0)
    sa = sorted(zip(a[0].tolist(), a[1].tolist(), map(tuple, a[2].tolist())))
    sb = sorted(zip(b[0].tolist(), b[1].tolist(), map(tuple, b[2].tolist())))
    assert sa == sb


def test_sph_harm_gradient_and_norm():
    rng = np.random.default_rng(0)
    u = rng.standard_normal((20, 3))
    u /= np.linalg.norm(u, axis=1)[:, None]
    Y, G = sph_harm(u, 4)
    assert np.allclose(Y[:, 0], 1.0)
    for l in range(5):     # sum_m Y_lm^2 = 2l + 1 in this normalisation
        assert np.allclose((Y[:, l * l:(l + 1) ** 2] ** 2).sum(1), 2 * l + 1)
    h = 1e-6
    for d in range(3):     # G is the gradient of the polynomial extension
        up = u.copy(); up[:, d] += h
        um = u.copy(); um[:, d] -= h
        num = (sph_harm(up, 4)[0] - sph_harm(um, 4)[0]) / (2 * h)
        assert np.abs(num - G[:, :, d]).max() < 1e-7


def test_oracle_forces_are_energy_gradient(oracles, cells):
    c = cells.get("tri9")
    o = _oracle(oracles, "grace_2l_order3")
    r = o.compute(c["species"], c["types"], c["positions"], c["cell"], c["pbc"])
    h = 1e-5
    for (i, d) in [(0, 0), (3, 1), (8, 2)]:
        p = c["positions"].copy(); p[i, d] += h
        m = c["positions"].copy(); m[i, d] -= h
        ep = o.compute(c["species"], c["types"], p, c["cell"], c["pbc"])["energy"]
        em = o.compute(c["species"], c["types"], m, c["cell"], c["pbc"])["energy"]
        assert abs(-(ep - em) / (2 * h) - r["forces"][i, d]) < 1e-7
