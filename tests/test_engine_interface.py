"""The engine interface for callers with their own neighbour list and ghost atoms (grace_engine_run; the reference's
RunInput / Exchange, libgrace/include/grace/kk/grace_2l_kk.h:87-119), tested as the reference tests its engines on CSR
bonds with ghost images (tests/kk/kk_csr_util.h:1-4): a periodic cell is unfolded into local atoms plus ghost images,
the neighbour table is built on the host, the message exchange of GRACE-2L is done by the test, and the folded forces
must equal System.compute on the periodic cell."""
import numpy as np
import pytest

from conftest import TOL_E, TOL_F, TOL_S, model_path

pytestmark = pytest.mark.gpu


def _unfold(positions, cell, pbc, cutoff):
    """local atoms + every periodic image within `cutoff` of the cell as ghost atoms; neighbour table of the local atoms"""
    n = len(positions)
    inv = np.linalg.inv(cell)
    heights = 1.0 / np.linalg.norm(inv, axis=0)
    frac = positions @ inv          # atoms need not lie inside the cell: their spread adds to the reach
    span = frac.max(axis=0) - frac.min(axis=0)
    reach = [int(np.ceil(cutoff / heights[k] + span[k])) if pbc[k] else 0 for k in range(3)]
    pos, owner = [positions], [np.arange(n)]
    for a in range(-reach[0], reach[0] + 1):
        for b in range(-reach[1], reach[1] + 1):
            for c in range(-reach[2], reach[2] + 1):
                if (a, b, c) == (0, 0, 0):
                    continue
                pos.append(positions + np.array([a, b, c]) @ cell)
                owner.append(np.arange(n))
    pos, owner = np.concatenate(pos), np.concatenate(owner)
    d = np.linalg.norm(pos[None, :, :] - positions[:, None, :], axis=2)      # [n local][all]
    near = d < cutoff
    near[np.arange(n), np.arange(n)] = False
    keep = np.zeros(len(pos), dtype=bool)
    keep[:n] = True
    keep |= near.any(axis=0)                     # ghosts nobody sees are dropped
    idx = np.nonzero(keep)[0]
    remap = -np.ones(len(pos), dtype=np.int64)
    remap[idx] = np.arange(len(idx))
    pos, owner, near = pos[idx], owner[idx], near[:, idx]
    numneigh = near.sum(axis=1).astype(np.int32)
    maxneigh = int(numneigh.max())
    table = np.zeros((n, maxneigh), dtype=np.int32)
    for i in range(n):
        js = np.nonzero(near[i])[0]
        table[i, :len(js)] = js
    return pos, owner, numneigh, table, maxneigh


class _Rows:
    """a device array made from an address, for torch.as_tensor"""

    def __init__(self, ptr, shape):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": "<f4", "data": (int(ptr), False), "strides": None,
                                         "version": 3}


@pytest.mark.parametrize("name", ["grace_1l_order3", "grace_2l_order3", "legacy_2l_order3"])
@pytest.mark.parametrize("cell", ["WMo54", "tri9", "slab36"])
def test_engine_run_with_ghost_images_equals_periodic_system(backend, cells, name, cell):
    import torch
    c = cells.get(cell)
    m = backend.Model(model_path(name))
    want = backend.System(m, c["species"]).compute(c["types"], c["positions"], c["cell"], c["pbc"], energies=True)
    eng = backend.Engine(m, c["species"])
    n = c["n"]
    pos, owner, numneigh, table, maxneigh = _unfold(c["positions"], c["cell"], c["pbc"], eng.cutoff)
    nall = len(pos)
    dev = torch.device("cuda", 0)
    d_t = torch.from_numpy(np.asarray(c["types"])[owner].astype(np.int32)).to(dev)
    d_x = torch.from_numpy(np.ascontiguousarray(pos)).to(dev)
    d_nn, d_tab = torch.from_numpy(numneigh).to(dev), torch.from_numpy(table).to(dev)
    d_f = torch.zeros((nall, 3), dtype=torch.float64, device=dev)
    d_e = torch.zeros(n, dtype=torch.float64, device=dev)
    d_owner = torch.from_numpy(owner).to(dev)
    calls = []

    def forward(rows, width, stream):        # message rows of the owners -> their ghost images
        r = torch.as_tensor(_Rows(rows, (nall, width)), device=dev)
        r[n:] = r[d_owner[n:]]
        torch.cuda.synchronize()
        calls.append("f")

    def reverse(rows, width, stream):        # dE/dmsg rows of the ghost images summed into their owners
        r = torch.as_tensor(_Rows(rows, (nall, width)), device=dev)
        r.index_add_(0, d_owner[n:], r[n:].clone())
        torch.cuda.synchronize()
        calls.append("r")

    for _ in range(2):      # forces and per-atom energies accumulate: the second run doubles them
        e, v = eng.run(n, nall, d_t, d_x, d_nn, d_tab, maxneigh, d_f, eatom=d_e, forward=forward, reverse=reverse)
    assert eng.comm_width == (0 if m.layers == 1 else eng.comm_width) and (m.layers == 1 or calls == ["f", "r"] * 2)
    f = torch.zeros((n, 3), dtype=torch.float64, device=dev).index_add_(0, d_owner, d_f).cpu().numpy() / 2.0
    assert abs(e - want["energy"]) / n < TOL_E * 0.1
    assert np.abs(f - want["forces"]).max() < TOL_F * 0.1
    assert np.abs(v - want["virial"]).max() / c["volume"] < TOL_S * 0.1
    assert np.abs(d_e.cpu().numpy() / 2.0 - want["energies"]).max() < TOL_E * 0.1


def test_engine_run_rejects_bad_tables(backend, cells):
    import torch
    c = cells.get("W54")
    m = backend.Model(model_path("grace_1l_order3"))
    eng = backend.Engine(m, c["species"])
    dev = torch.device("cuda", 0)
    n = c["n"]
    d_t = torch.ones(n, dtype=torch.int32, device=dev)
    d_x = torch.from_numpy(np.ascontiguousarray(c["positions"])).to(dev)
    d_f = torch.zeros((n, 3), dtype=torch.float64, device=dev)
    nn = torch.full((n,), 3, dtype=torch.int32, device=dev)
    tab = torch.full((n, 2), 0, dtype=torch.int32, device=dev)
    with pytest.raises(ValueError):
        eng.run(n, n, d_t, d_x, nn, tab, 2, d_f)                       # a count beyond maxneigh
    nn = torch.full((n,), 1, dtype=torch.int32, device=dev)
    tab = torch.full((n, 2), n + 5, dtype=torch.int32, device=dev)
    with pytest.raises(ValueError):
        eng.run(n, n, d_t, d_x, nn, tab, 2, d_f)                       # an index outside the atoms
