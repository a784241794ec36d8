"""Host logic of the slab decomposition (grace_runtime_b200/domain.py) on CPU: the plan, the sub-systems and the
exchange, with a small differentiable stand-in for the library whose atom energies reach one or two cutoffs far, in one
process and as two gloo ranks.  The CUDA library itself is checked against the same decomposition in the GPU tests."""
import os
import socket

import numpy as np
import pytest
import torch

from grace_runtime_b200 import domain, structures

RC = 3.0


def toy_engine(layers):
    """compute(types, positions, cell, pbc, nlocal) -> (energy of the owned atoms, virial[6], forces[n, 3]) of a
    smooth model: E_i = sum_j phi(r_ij) (1 + w rho_j) with rho_j = sum_k phi(r_jk) when layers == 2."""

    def compute(types, positions, cell, pbc, nlocal):
        x = torch.tensor(np.asarray(positions), dtype=torch.float64, requires_grad=True)
        cell_t = torch.tensor(np.asarray(cell), dtype=torch.float64)
        n = x.shape[0]
        if n == 0:
            return 0.0, np.zeros(6), np.zeros((0, 3))
        rng = [(-1, 0, 1) if p else (0,) for p in pbc]
        shifts = torch.tensor([[a, b, c] for a in rng[0] for b in rng[1] for c in rng[2]], dtype=torch.float64) @ cell_t
        d = x[None, :, None, :] + shifts[None, None, :, :] - x[:, None, None, :]       # [i, j, image, 3]
        d = d.reshape(n, -1, 3)
        d.retain_grad()
        r = torch.sqrt((d * d).sum(-1) + 1e-300)
        w = torch.tensor(1.0 + 0.1 * np.asarray(types), dtype=torch.float64)
        phi = torch.where((r < RC) & (r > 1e-9), (1.0 - r / RC) ** 3, torch.zeros_like(r))
        nimg = shifts.shape[0]
        wj = w.repeat_interleave(nimg)[None, :]
        rho = (phi * wj).sum(1)
        if layers == 1:
            e_atom = rho * w
        else:
            e_atom = (phi * wj * (1.0 + 0.3 * rho.repeat_interleave(nimg))[None, :]).sum(1) * w
        e = e_atom[:nlocal].sum()
        e.backward()
        g = d.grad
        vir = torch.einsum("bk,bl->kl", d.detach().reshape(-1, 3), g.reshape(-1, 3)).numpy()
        v6 = np.array([vir[0, 0], vir[1, 1], vir[2, 2], vir[0, 1], vir[0, 2], vir[1, 2]], dtype=np.float64)
        return float(e.detach()), v6, -x.grad.numpy()

    return compute


def _structure(seed, triclinic):
    types, pos, cell, pbc = structures.crystal("bcc", 3.0, (3, 3, 7), n_species=3, sigma=0.08, seed=seed)
    cell = np.array(cell, dtype=np.float64)
    if triclinic:
        cell[2] += 0.15 * cell[0] - 0.1 * cell[1]
        cell[0] += 0.05 * cell[1]
    pos = np.array(pos) + 40.0 * cell[2] * (seed % 2)       # unwrapped positions must work too
    return np.asarray(types), pos, cell, np.asarray(pbc)


@pytest.mark.parametrize("layers", [1, 2])
@pytest.mark.parametrize("world", [1, 2, 3])
@pytest.mark.parametrize("triclinic", [False, True])
def test_slabs_reproduce_the_whole_structure(layers, world, triclinic):
    types, pos, cell, pbc = _structure(3 + world, triclinic)
    eng = toy_engine(layers)
    e0, v0, f0 = eng(types, pos, cell, pbc, len(types))
    plan = domain.make_plan(pos, cell, pbc, world, layers, RC, 0.0)
    assert plan.axis == 2
    assert sorted(np.concatenate(plan.owned).tolist()) == list(range(len(types)))
    e, v, fs = 0.0, np.zeros(6), []
    for r in range(world):
        t, p, nlocal = plan.subsystem(r, types, pos)
        er, vr, fr = eng(t, p, plan.sub_cell, plan.sub_pbc, nlocal)
        e += er
        v += vr
        fs.append(fr)
        assert plan.send_counts(r).sum() == len(t) - nlocal
    f = plan.assemble(fs)
    assert abs(e - e0) < 1e-9 * max(1.0, abs(e0))
    assert np.abs(f - f0).max() < 1e-9
    assert np.abs(v - v0).max() < 1e-8 * max(1.0, np.abs(v0).max())
    # every row a rank sends is expected by its owner
    for r in range(world):
        assert plan.recv_counts(r).sum() == len(plan.recv_index(r))
        assert sum(plan.send_counts(q)[r] for q in range(world)) == plan.recv_counts(r).sum()


def test_open_axis_and_too_short_halo():
    types, pos, cell, _ = _structure(5, False)
    pbc = np.array([True, True, False])
    eng = toy_engine(1)
    e0, v0, f0 = eng(types, pos, cell, pbc, len(types))
    plan = domain.SlabPlan(pos, cell, pbc, 2, domain.halo_width(1, RC, 0.0))
    fs, e = [], 0.0
    for r in range(2):
        t, p, nlocal = plan.subsystem(r, types, pos)
        er, _, fr = eng(t, p, plan.sub_cell, plan.sub_pbc, nlocal)
        e += er
        fs.append(fr)
    assert abs(e - e0) < 1e-9 * abs(e0)
    assert np.abs(plan.assemble(fs) - f0).max() < 1e-9
    # a halo of half a cutoff loses neighbours: the check above is sensitive to the halo width
    short = domain.SlabPlan(pos, cell, pbc, 2, 0.5 * RC)
    e = sum(eng(*short.subsystem(r, types, pos)[:2], short.sub_cell, short.sub_pbc, short.subsystem(r, types, pos)[2])[0]
            for r in range(2))
    assert abs(e - e0) > 1e-6 * abs(e0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, layers, out):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        types, pos, cell, pbc = _structure(7, True)
        plan = domain.make_plan(pos, cell, pbc, world, layers, RC, 0.0)
        ds = domain.DistributedSystem(plan, rank, types, pos, engine=toy_engine(layers))
        for _ in range(2):       # a second step must not accumulate into the first
            ds.step()
        np.savez(os.path.join(out, f"rank{rank}.npz"), energy=ds.energy, virial=ds.virial,
                 forces=ds.owned_forces.numpy(), owned=plan.owned[rank])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("layers", [1, 2])
def test_two_gloo_ranks_exchange_ghost_forces(tmp_path, layers):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), layers, str(tmp_path)), nprocs=world, join=True)
    types, pos, cell, pbc = _structure(7, True)
    e0, v0, f0 = toy_engine(layers)(types, pos, cell, pbc, len(types))
    f = np.zeros_like(f0)
    for r in range(world):
        z = np.load(tmp_path / f"rank{r}.npz")
        assert abs(float(z["energy"]) - e0) < 1e-9 * abs(e0)          # every rank holds the total
        assert np.abs(z["virial"] - v0).max() < 1e-8 * np.abs(v0).max()
        f[z["owned"]] = z["forces"]
    assert np.abs(f - f0).max() < 1e-9
