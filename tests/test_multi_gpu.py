"""Domain decomposition against the CUDA library: the slabs of grace_runtime_b200/domain.py evaluated through the C ABI
with owned / ghost atoms (grace_system_set_owned) reproduce the single-GPU result.  On one GPU the ranks' sub-systems
run one after the other in this process (no kernel waits on another rank); with two or more GPUs the same runs as two
NCCL processes."""
import os
import socket
import sys

import numpy as np
import pytest

from conftest import TOL_E, TOL_F, TOL_S, model_path

pytestmark = pytest.mark.gpu


def _case(tmp_path_factory, cfg, lattice, a, reps, nsp, sigma, seed):
    from grace_runtime_b200 import modelgen, structures
    els = modelgen._subset(11, nsp)
    path = str(tmp_path_factory.mktemp("dd") / f"{cfg}.npz")
    modelgen.write_config_model(path, cfg, els, seed=seed)
    types, pos, cell, pbc = structures.crystal(lattice, a, reps, n_species=nsp, sigma=sigma, seed=seed + 1)
    return path, els, types, pos, cell, pbc


def _slabs(backend, model, species, types, pos, cell, pbc, world, skin=0.5):
    from grace_runtime_b200 import domain
    whole = backend.System(model, species, skin=skin)
    plan = domain.make_plan(pos, cell, pbc, world, model.layers, whole.cutoff, skin)
    e, v, fs, work = 0.0, np.zeros(6), [], []
    for r in range(world):
        t, p, nlocal = plan.subsystem(r, types, pos)
        s = backend.System(model, species, skin=skin)
        s.set_owned(nlocal, nlocal + (plan.n_inner[r] if model.layers > 1 else 0))
        for _ in range(2):         # the second call reuses the neighbour list and the active ranges
            rr = s.compute(t, p, plan.sub_cell, plan.sub_pbc, energies=True)
        assert np.all(rr["energies"][nlocal:] == 0.0)
        e += rr["energy"]
        v += rr["virial"]
        fs.append(rr["forces"])
        work.append((len(t), nlocal))
    return e, v, plan.assemble(fs), work


@pytest.mark.parametrize("name", ["grace_1l_order3", "grace_2l_order3", "legacy_2l_order3"])
@pytest.mark.parametrize("world", [2, 3])
def test_slabs_of_small_cells_with_many_images(backend, cells, name, world):
    """cells smaller than the halo: every slab sees several periodic images of every atom"""
    c = cells.get("WMo54")
    m = backend.Model(model_path(name))
    r0 = backend.System(m, c["species"]).compute(c["types"], c["positions"], c["cell"], c["pbc"])
    e, v, f, _ = _slabs(backend, m, c["species"], c["types"], c["positions"], c["cell"], c["pbc"], world)
    assert abs(e - r0["energy"]) / c["n"] < TOL_E * 0.1
    assert np.abs(f - r0["forces"]).max() < TOL_F * 0.1
    assert np.abs(v - r0["virial"]).max() / c["volume"] < TOL_S * 0.1


@pytest.mark.parametrize("cfg,lattice,a,reps,nsp,sigma", [("1l", "bcc", 3.2, (5, 5, 24), 4, 0.05),
                                                           ("2l", "fcc", 3.6, (3, 18, 3), 3, 0.08)])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_slabs_of_benchmark_shaped_cells(backend, tmp_path_factory, cfg, lattice, a, reps, nsp, sigma, world):
    """long cells: slabs wider than the halo, so that most ghosts are skipped by the active ranges"""
    path, els, types, pos, cell, pbc = _case(tmp_path_factory, cfg, lattice, a, reps, nsp, sigma, seed=21)
    m = backend.Model(path)
    r0 = backend.System(m, els).compute(types, pos, cell, pbc)
    e, v, f, work = _slabs(backend, m, els, types, pos, cell, pbc, world)
    n, vol = len(types), abs(np.linalg.det(cell))
    assert abs(e - r0["energy"]) / n < TOL_E * 0.1
    assert np.abs(f - r0["forces"]).max() < TOL_F * 0.1
    assert np.abs(v - r0["virial"]).max() / vol < TOL_S * 0.1
    assert sum(w[1] for w in work) == n


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _nccl_rank(rank, world, port, path, els, out):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from grace_runtime_b200 import backend as B, domain, structures
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        B.initialize(rank)
        domain.init_library_comm(rank, world)
        types, pos, cell, pbc = structures.crystal("bcc", 3.2, (5, 5, 24), n_species=4, sigma=0.05, seed=22)
        m = B.Model(path)
        cutoff = B.System(m, els).cutoff
        plan = domain.make_plan(pos, cell, pbc, world, m.layers, cutoff, 0.5)
        ds = domain.DistributedSystem(plan, rank, types, pos, species=els, model=m, device=torch.device("cuda", rank))
        assert ds.library_exchange
        for _ in range(2):
            ds.step()
        torch.cuda.synchronize()
        np.savez(os.path.join(out, f"rank{rank}.npz"), energy=ds.energy, virial=ds.virial,
                 forces=ds.owned_forces.cpu().numpy(), owned=plan.owned[rank])
    finally:
        dist.destroy_process_group()


def test_two_nccl_ranks(backend, tmp_path_factory, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    path, els, types, pos, cell, pbc = _case(tmp_path_factory, "1l", "bcc", 3.2, (5, 5, 24), 4, 0.05, seed=21)
    r0 = backend.System(backend.Model(path), els).compute(types, pos, cell, pbc)
    mp.spawn(_nccl_rank, args=(2, _free_port(), path, els, str(tmp_path)), nprocs=2, join=True)
    f = np.zeros_like(r0["forces"])
    for r in range(2):
        z = np.load(tmp_path / f"rank{r}.npz")
        assert abs(float(z["energy"]) - r0["energy"]) / len(types) < TOL_E * 0.1
        assert np.abs(z["virial"] - r0["virial"]).max() / abs(np.linalg.det(cell)) < TOL_S * 0.1
        f[z["owned"]] = z["forces"]
    assert np.abs(f - r0["forces"]).max() < TOL_F * 0.1
