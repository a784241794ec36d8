"""grace_sum_rows_static: column sums on the device with the partial sums in a static device array (no allocation).
Collected last; runs alone or after the other GPU tests.  Checked through the C ABI against the totals the existing
entry point grace_system_compute returns for the same per-atom values, twice in a row, and against fp64 numpy sums."""
import numpy as np
import pytest

from conftest import TOL_E, model_path

pytestmark = pytest.mark.gpu


def _dev(a):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float64)).to("cuda:0")
    torch.cuda.synchronize()
    return t


def _static_sum(backend, values, k):
    import torch
    v = _dev(values)
    out = torch.full((k,), np.nan, dtype=torch.float64, device="cuda:0")
    torch.cuda.synchronize()
    backend.sum_rows_static(v.data_ptr(), v.numel() // k, k, out.data_ptr())
    return out.cpu().numpy()


def test_static_sum_matches_compute_totals_twice(backend, cells):
    c = cells.get("WMo54")
    m = backend.Model(model_path("grace_2l_order3"))
    s = backend.System(m, c["species"])
    pos = c["positions"].copy()
    for call in range(2):     # two calls in a row share the static array
        r = s.compute(c["types"], pos, c["cell"], c["pbc"], energies=True)
        e = _static_sum(backend, r["energies"], 1)
        assert abs(e[0] - r["energy"]) / c["n"] < TOL_E * 1e-3, (call, e[0], r["energy"])
        assert abs(e[0] - np.sum(r["energies"])) < 1e-11 * max(1.0, np.abs(r["energies"]).sum())
        pos = pos + 0.01 * np.random.default_rng(call).standard_normal(pos.shape)


@pytest.mark.parametrize("n,k", [(0, 1), (1, 6), (255, 3), (4097, 6), (300_000, 8), (2_000_000, 6)])
def test_static_sum_sizes(backend, n, k):
    rng = np.random.default_rng(n + k)
    v = rng.standard_normal((n, k)) * 10.0 ** rng.integers(-3, 4, size=(n, 1))
    want = v.sum(axis=0)
    tol = 1e-12 * max(1.0, np.abs(v).sum())
    first = _static_sum(backend, v, k)
    second = _static_sum(backend, v, k)
    assert np.abs(first - want).max() <= tol
    assert np.array_equal(first, second)          # fixed summation tree: identical bits, counter back at zero


def test_static_sum_rejects_sizes_beyond_the_array(backend):
    import torch
    out = torch.zeros(16, dtype=torch.float64, device="cuda:0")
    v = torch.zeros(16, dtype=torch.float64, device="cuda:0")
    with pytest.raises(ValueError, match="at most 8 columns"):
        backend.sum_rows_static(v.data_ptr(), 1, 9, out.data_ptr())
    with pytest.raises(ValueError, match="at most 16777216 rows"):
        backend.sum_rows_static(v.data_ptr(), 16_777_217, 1, out.data_ptr())
    with pytest.raises(ValueError):
        backend.sum_rows_static(v.data_ptr(), -1, 1, out.data_ptr())
    # still usable afterwards
    assert _static_sum(backend, np.arange(10.0), 1)[0] == 45.0
