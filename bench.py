"""Benchmark of the hot path: one energy + forces + stress evaluation per step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload: the 1,024,000-atom GRACE-2L configuration (random 3-component fcc alloy, 89-element model), which
fits one GPU in one pass; the 128,000-atom GRACE-1L configuration is reported beside it (`also`, one GPU).  Prints one
JSON line (rank 0).  `value` is the step time divided by the atoms of the structure (microseconds per atom of the whole
job: at N GPUs it falls as 1 / N under ideal strong scaling; `us_per_atom_per_gpu` = value x N) with the inputs resident
in HBM and the neighbour list reused, timed with CUDA events; `e2e` is the same through the host-buffer call (pinned
host memory, copies inside the timed region).  `parity` holds the differences between the library and the reference's
CPU drivers on the block of the workload the CPU leg is timed on.  The reference arm (--impl reference) times the
reference's own CPU drivers (oracle/_ref) on the host cores on that block.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from grace_runtime_b200 import modelgen, structures  # noqa: E402

METRIC = "us_per_atom_energy_forces_stress"
UNIT = "us/atom"

WORKLOADS = {
    # name: (config, lattice, a, reps, species, sigma)
    "grace1l_128k_bcc_alloy": dict(cfg="1l", lattice="bcc", a=3.2, reps=(40, 40, 40), nsp=4, sigma=0.05, full=True),
    "grace1l_16k_bcc_alloy": dict(cfg="1l", lattice="bcc", a=3.2, reps=(20, 20, 20), nsp=4, sigma=0.05, full=True),
    "grace1l_2k_bcc_w": dict(cfg="1l", lattice="bcc", a=3.165, reps=(10, 10, 10), nsp=1, sigma=0.05, full=False),
    "grace2l_1m_fcc_alloy": dict(cfg="2l", lattice="fcc", a=3.6, reps=(40, 80, 80), nsp=3, sigma=0.08, full=True),
    "grace2l_128k_fcc_alloy": dict(cfg="2l", lattice="fcc", a=3.6, reps=(20, 40, 40), nsp=3, sigma=0.08, full=True),
    # 4096 small periodic structures (16-256 atoms, triclinic, 0.06-0.09 atoms/A^3) through the Batch entry points
    "grace2l_batch4096": dict(cfg="2l", batch=4096, unique=128, nmin=16, nmax=256, nsp=89, full=True),
    # GRACE-3L (lmax 4, 64 channels, 89 elements) on a 5-component bcc alloy: 31,250 atoms fit one pass that keeps the
    # tensors of all three layers (1.5 MB per atom); the 500,094-atom structure runs in passes over atom chunks
    "grace3l_31k_bcc_hea": dict(cfg="3l", lattice="bcc", a=3.2, reps=(25, 25, 25), nsp=5, sigma=0.05, full=True),
    "grace3l_3k_bcc_hea": dict(cfg="3l", lattice="bcc", a=3.2, reps=(12, 12, 12), nsp=5, sigma=0.05, full=True),    # ncu-sized
    "grace3l_500k_bcc_hea": dict(cfg="3l", lattice="bcc", a=3.2, reps=(63, 63, 63), nsp=5, sigma=0.05, full=True),
}
DEFAULT = "grace2l_1m_fcc_alloy"      # the 1,024,000-atom GRACE-2L configuration the target is stated on
ALSO = "grace1l_128k_bcc_alloy"       # reported beside it at one GPU (`also`)


def make_workload(name, tmp, reps=None):
    w = WORKLOADS[name]
    species = modelgen._subset(2024, w["nsp"]) if w["full"] else ["W"]
    elements = modelgen.ELEMENTS if w["full"] else species
    if w["cfg"] == "3l":
        from grace_runtime_b200 import modelgen3l
        path = modelgen3l.write_model_3l(os.path.join(tmp, f"{name}.npz"), elements=elements, lmax=4, channels=(64, 64, 64),
                                         rho_width=32, embedding=16, radial_hidden=128, energy_hidden=64, rcut=6.0,
                                         avg_neigh=58.0, seed=0)
    else:
        path = modelgen.write_config_model(os.path.join(tmp, f"{name}.npz"), w["cfg"], elements, seed=0)
    types, pos, cell, pbc = structures.crystal(w["lattice"], w["a"], reps or w["reps"], n_species=w["nsp"],
                                               sigma=w["sigma"], seed=1)
    return path, species, types, pos, cell, pbc


def make_batch(wl, count):
    """The first `count` structures of a batch workload: `unique` generated structures (rejection sampling is slow),
    repeated with rigid shifts."""
    un, ut, up, uc, upbc = structures.random_batch(wl["unique"], wl["nmin"], wl["nmax"], wl["nsp"], seed=1)
    rng = np.random.default_rng(2)
    start = np.concatenate([[0], np.cumsum(un)])
    natoms, T, P, Cc = [], [], [], []
    for s in range(count):
        u = s % wl["unique"]
        sl = slice(start[u], start[u + 1])
        natoms.append(un[u]); T.append(ut[sl]); Cc.append(uc[u])
        P.append(up[sl] + rng.random(3) @ uc[u])
    return np.array(natoms, dtype=np.int32), T, P, Cc


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu):
        self.gpu, self.proc, self.lines = gpu, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def algorithmic_bytes(kernel, model_cfg, n_atoms, n_bonds, slots):
    """Bytes one pass of a kernel over the whole structure must move at least (fp32 network, 16-byte bond records)."""
    if model_cfg not in modelgen.CONFIGS:      # GRACE-3L: no byte model of its kernels yet
        return None
    c = modelgen.CONFIGS[model_cfg]
    nlm = (c["lmax"] + 1) ** 2
    C = c["c1"]
    if kernel == "bond_fwd_kernel":       # bond record in; A[nlm][C] out; offsets, counts, element per atom
        return 16.0 * n_bonds + (4.0 * nlm * C + 16.0) * n_atoms
    if kernel == "bond_bwd_kernel":       # bond record and slot in, bond force out; gA in, virial out
        return (16.0 + 4.0 + 12.0) * n_bonds + (4.0 * nlm * C + 48.0 + 16.0) * n_atoms
    if c["layers"] == 2:                  # the message layer: (4 message functions + the chemical one) x nlm x CR sums per atom
        CR, nq = c["cr"], 5 * nlm
        if kernel == "bond_fwd_split_kernel":    # bond record in; every atom's message row once; Q out
            return 16.0 * n_bonds + (4.0 * nq * CR + 4.0 * 4 * CR + 16.0) * n_atoms
        if kernel == "bond_bwd_split_kernel":    # as bond_bwd_kernel, plus each bond's share of dE/dmsg (4 x CR floats) out
            return (16.0 + 4.0 + 12.0 + 4.0 * 4 * CR) * n_bonds + (4.0 * nq * CR + 4.0 * 4 * CR + 48.0 + 16.0) * n_atoms
    if kernel == "nl_compact":            # list entry (j, S) and positions in, record + slot out
        return (8.0 + 16.0 + 4.0) * slots + 24.0 * n_atoms
    if kernel == "force_gather_kernel":   # bond force and reverse index in, force out
        return (12.0 + 4.0 + 12.0) * slots + 24.0 * n_atoms
    return None


def bond_flops(kernel, model_cfg, n_bonds, launches_per_step):
    """Useful fp32 flops of the bond kernels per step: 2 nlm C NIT per bond forward (Y R msg accumulated into the
    A-basis), 2 nlm C (1 + 3) NIT per bond reverse (dE/dx and the three components of the direction gradient), summed
    over the layers; NIT = message functions coupled in (layer 2: I_n_funcs + the chemical one)."""
    c = modelgen.CONFIGS[model_cfg]
    nlm = (c["lmax"] + 1) ** 2
    per = [(c["c1"], 1)] + ([(c["cr"], 5)] if c["layers"] == 2 else [])
    # message layers of at most 16 channels run as the split kernels, the others (and layer 1) as the plain ones
    split2 = c["layers"] == 2 and c["cr"] <= 16
    if kernel.startswith(("bond_bwd_split", "bond_fwd_split")):
        per = per[1:]
    elif split2:
        per = per[:1]
    if kernel.startswith("bond_bwd"):
        return n_bonds * sum(2.0 * nlm * C * 4 * nit for C, nit in per)
    if kernel.startswith("bond_fwd"):
        return n_bonds * sum(2.0 * nlm * C * nit for C, nit in per)
    return None


def run_batch(args, rank, world, local_rank):
    """Batches of small structures: sharded by structure over the ranks (greedy by atom count), no data-path
    collective; `value` = max-over-ranks time per step x n_gpus / total atoms."""
    import torch
    import torch.distributed as dist

    from grace_runtime_b200 import backend as B

    wl = WORKLOADS[args.workload]
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    B.initialize(local_rank)
    tmp = tempfile.mkdtemp(prefix="grace_bench_")
    species = list(modelgen.ELEMENTS)
    path = modelgen.write_config_model(os.path.join(tmp, "batch.npz"), wl["cfg"], modelgen.ELEMENTS, seed=0)
    natoms, T, P, Cc = make_batch(wl, wl["batch"])
    n_total = int(natoms.sum())
    # this rank's structures: greedy by atom count
    order = np.argsort(-natoms, kind="stable")
    load = np.zeros(world, dtype=np.int64)
    owner = np.zeros(len(natoms), dtype=np.int64)
    for s in order:
        r = int(np.argmin(load)); owner[s] = r; load[r] += natoms[s]
    mine = np.nonzero(owner == rank)[0]
    my_n = natoms[mine]
    my_t = np.concatenate([T[s] for s in mine]).astype(np.int32)
    my_p = np.ascontiguousarray(np.concatenate([P[s] for s in mine]))
    my_c = np.stack([Cc[s] for s in mine])
    my_pbc = np.ones((len(mine), 3), dtype=np.uint8)
    model = B.Model(path)
    batch = B.Batch(model, species, chunksize=args.chunk)
    batch.keep_buffers = True
    d_t = torch.from_numpy(my_t).to(dev); d_p = torch.from_numpy(my_p).to(dev)
    d_e = torch.zeros(len(mine), dtype=torch.float64, device=dev)
    d_v = torch.zeros((len(mine), 6), dtype=torch.float64, device=dev)
    d_f = torch.zeros((len(my_t), 3), dtype=torch.float64, device=dev)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(); torch.cuda.synchronize()

    def step_device():
        batch.compute_device(my_n, d_t.data_ptr(), d_p.data_ptr(), my_c, my_pbc, d_e.data_ptr(), d_f.data_ptr(), d_v.data_ptr())

    def step_host():
        return batch.compute(my_n, my_t, my_p, my_c, my_pbc)

    sampler = ClockSampler(local_rank); sampler.start()
    for _ in range(max(args.warmup, 1)):
        step_device()
    barrier()
    l0 = B.kernel_launches()
    B.profile_enable(True)
    ev0.record()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step_device()
    ev1.record(); ev1.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    dev_ms = ev0.elapsed_time(ev1) / args.steps
    prof = B.profile_report(); B.profile_enable(False)
    launches = B.kernel_launches() - l0
    clocks = sampler.stop()
    for _ in range(max(args.warmup, 3)):
        step_host()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step_host()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    red = torch.tensor([dev_ms, wall_ms, e2e_ms], dtype=torch.float64, device=dev)
    cnt = torch.tensor([float(launches)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(red, op=dist.ReduceOp.MAX); dist.all_reduce(cnt, op=dist.ReduceOp.SUM)
    if rank == 0:
        ms = float(red[0])
        tot = sum(v[1] for v in prof.values()) or 1.0
        kern = sorted(prof.items(), key=lambda kv: -kv[1][1])
        out = {"metric": METRIC, "value": ms * 1e3 / n_total, "unit": UNIT, "n_gpus": world, "steps": args.steps,
               "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
               "dtype": "f32", "data": "synthetic", "config": base_config(args.workload, world),
               "value_definition": "max-over-ranks time per step / atoms of the batch (whole job)",
               "details": {"atoms": n_total, "unique_structures": int(wl["unique"]), "passes": batch.passes,
                           "neighbor_list": "built every step (Batch semantics)"},
               "structures_per_s": wl["batch"] / (ms * 1e-3),
               "e2e": {"value": float(red[2]) * 1e3 / n_total, "unit": UNIT, "ms_per_step": float(red[2]),
                       "h2d_bytes_per_step": int(28 * n_total + 75 * wl["batch"]), "d2h_bytes_per_step": int(24 * n_total + 56 * wl["batch"])},
               "gpu_launches": int(cnt[0]), "clocks": clocks, "roofline": None,
               "kernels": {k: {"launches": v[0], "ms_per_step": v[1] / args.steps, "share": v[1] / tot} for k, v in kern[:8]},
               "wall_ms_per_step": float(red[1])}
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def base_config(workload, world):
    """The `config` object of the JSON line, the same for both arms (--impl ours / reference)."""
    wl = WORKLOADS[workload]
    if "batch" in wl:
        return {"workload": workload, "structures": int(wl["batch"]), "model": "GRACE-2L", "elements_in_model": 89,
                "atoms_per_structure": [int(wl["nmin"]), int(wl["nmax"])], "parallelism": f"structures over {world} rank(s)"}
    n = int(np.prod(wl["reps"])) * (2 if wl["lattice"] == "bcc" else 4)
    return {"workload": workload, "atoms": n, "model": {"1l": "GRACE-1L", "2l": "GRACE-2L", "3l": "GRACE-3L"}[wl["cfg"]],
            "elements_in_model": 89 if wl["full"] else 1, "species_in_structure": int(wl["nsp"]),
            "lattice": wl["lattice"], "lattice_constant_A": wl["a"], "cells": list(wl["reps"]),
            "displacement_sigma_A": wl["sigma"], "cutoff_A": 6.0, "skin_A": 0.5,
            "neighbor_list": "reused (built in warm-up)", "radial": "cubic Hermite tables, 1024 intervals",
            "parallelism": f"slabs{world}" if world > 1 else "single",
            "l2": "per-step working set (bond records + chunk tensors) exceeds the 126 MB L2"}


def sample_reps(wl):
    """The block of the workload the CPU legs run on (the same lattice, alloy, displacements and model; about 32,000
    atoms, so that a CPU step takes a fraction of a second): None when the workload itself is that small."""
    n = int(np.prod(wl["reps"])) * (2 if wl["lattice"] == "bcc" else 4)
    if n <= 40000:
        return None
    if wl["cfg"] == "3l":
        return (12, 12, 12)      # 3,456 atoms: a GRACE-3L step on the CPU is two orders of magnitude above GRACE-1L
    return (20, 20, 40) if wl["lattice"] == "bcc" else (16, 16, 32)


def load_traffic():
    """ncu DRAM traffic per atom of a launch, by (kernel, workload): profiles/traffic.json names the capture each
    figure came from; a kernel / workload pair without an entry gets traffic null."""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            return {(e["kernel"], e["model"]): e for e in json.load(f)["entries"]}
    except (OSError, ValueError, KeyError):
        return {}


def time_device_steps(step, steps, torch):
    """K steps between two CUDA events with a synchronize on both sides; every library call ends with a synchronize of
    its own stream, so events on torch's stream bracket all of its work.  Returns (ms per step, per-step list)."""
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    torch.cuda.synchronize()
    evs[0].record()
    for k in range(steps):
        step()
        evs[k + 1].record()
    evs[-1].synchronize()
    torch.cuda.synchronize()
    per = [evs[k].elapsed_time(evs[k + 1]) for k in range(steps)]
    return evs[0].elapsed_time(evs[-1]) / steps, per


def parity_and_cpu(args, B, model, path, species, wl):
    """The CPU legs of the bench (rank 0, one GPU): the reference's CPU drivers timed on a block of the workload, and
    the SAME block through the library (host-pointer entry) with the differences against the reference."""
    from oracle import refcpu
    reps = sample_reps(wl) or wl["reps"]
    types, pos, cell, pbc = structures.crystal(wl["lattice"], wl["a"], reps, n_species=wl["nsp"], sigma=wl["sigma"], seed=1)
    n, vol = len(types), abs(np.linalg.det(cell))
    cores = len(os.sched_getaffinity(0))
    block = f"{n} atoms ({'x'.join(str(r) for r in reps)} cells) of the same alloy, model and seeds"
    if not refcpu.available():
        from oracle.grace_oracle import GraceOracle
        types, pos, cell, pbc = structures.crystal(wl["lattice"], wl["a"], (4, 4, 4), n_species=wl["nsp"], sigma=wl["sigma"], seed=1)
        n, vol = len(types), abs(np.linalg.det(cell))
        o = GraceOracle(path)
        t0 = time.perf_counter()
        ref = o.compute(species, types, pos, cell, pbc)
        dt = time.perf_counter() - t0
        base = {"value": dt * 1e6 / n, "unit": "us/atom", "cores": 1, "kind": "port",
                "sample": f"{n} atoms, numpy fp64 restatement, one call", "neighbor_search_us_per_atom": None}
    else:
        rm = refcpu.RefModel(path, species)
        rm.compute(types, pos, cell, pbc, nthreads=cores)               # warm-up (tables, buffers)
        ref = rm.compute(types, pos, cell, pbc, nthreads=cores, repeats=3)
        base = {"value": ref["seconds_median"] * 1e6 / n, "unit": "us/atom", "cores": cores, "kind": "reference",
                "sample": block + ", median of 3 calls after the first, neighbour search not included in `value`",
                "neighbor_search_us_per_atom": ref["seconds_nlist"] * 1e6 / n,
                "energy_eV_per_atom": ref["energy"] / n}
    s = B.System(model, species, skin=0.5)
    r = s.compute(types, pos, cell, pbc)
    t0 = time.perf_counter()
    for _ in range(3):
        r = s.compute(types, pos, cell, pbc)
    gpu_us = (time.perf_counter() - t0) / 3 * 1e6 / n
    s.release_buffers()
    de = abs(r["energy"] - ref["energy"]) / n
    df = float(np.abs(r["forces"] - ref["forces"]).max())
    dv = float(np.abs(r["virial"] - ref["virial"]).max() / vol)
    parity = {"against": base["kind"], "atoms": n, "block": block, "dE_per_atom_eV": de, "dF_max_eV_per_A": df,
              "dstress_max_eV_per_A3": dv, "tolerance": {"energy": 1e-5, "forces": 1e-4, "stress": 1e-4},
              "tolerance_met": bool(de <= 1e-5 and df <= 1e-4 and dv <= 1e-4),
              "F_max_eV_per_A": float(np.abs(ref["forces"]).max()),
              "gpu_us_per_atom_on_block_e2e": gpu_us}
    return base, parity


def run_also(args, B, torch, name):
    """A second workload on the same GPU, device-resident, reported beside the headline (one GPU only)."""
    tmp = tempfile.mkdtemp(prefix="grace_bench_also_")
    path, species, types, pos, cell, pbc = make_workload(name, tmp)
    n = len(types)
    dev = torch.device("cuda", torch.cuda.current_device())
    model = B.Model(path)
    s = B.System(model, species, skin=0.5)
    d_t = torch.from_numpy(types).to(dev); d_x = torch.from_numpy(pos).to(dev)
    e = torch.zeros(1, dtype=torch.float64, device=dev); v = torch.zeros(6, dtype=torch.float64, device=dev)
    f = torch.zeros((n, 3), dtype=torch.float64, device=dev)

    def step():
        s.compute_device(d_t, d_x, cell, pbc, e, forces=f, virial=v)
    for _ in range(3):
        step()
    k = max(3, min(args.steps, 10))
    ms, per = time_device_steps(step, k, torch)
    s.release_buffers()
    return {"workload": name, "atoms": n, "model": base_config(name, 1)["model"], "value": ms * 1e3 / n, "unit": UNIT,
            "ms_per_step": ms, "steps": k, "warmup": 3, "ms_per_step_median": float(np.median(per))}


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    from grace_runtime_b200 import backend as B
    from grace_runtime_b200 import domain

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    B.initialize(local_rank)
    if world > 1:
        domain.init_library_comm(rank, world)      # the halo exchange runs inside the library, on its own NCCL communicator
    tmp = tempfile.mkdtemp(prefix="grace_bench_")
    path, species, types, pos, cell, pbc = make_workload(args.workload, tmp)     # every rank: the same seeded structure
    n = len(types)
    wl = WORKLOADS[args.workload]
    model = B.Model(path)
    skin = 0.5
    cutoff = B.System(model, species, skin=skin).cutoff

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # the denominators of the compute-bound rooflines, measured on this GPU before the warm-up
    peaks_here = {"fp32_simt_tflops": B.measure_peak("fp32"), "tf32_tensor_tflops": B.measure_peak("tf32")}

    # at N > 1, once before anything is timed: the whole structure on rank 0's GPU alone, as the check of the
    # decomposed forces (workloads that fit one GPU)
    f_single = e_single = None
    if world > 1 and rank == 0 and n <= 2_500_000:
        r1 = B.System(model, species, skin=skin)
        d_t = torch.from_numpy(types).to(dev); d_x = torch.from_numpy(pos).to(dev)
        e1 = torch.zeros(1, dtype=torch.float64, device=dev); f1 = torch.zeros((n, 3), dtype=torch.float64, device=dev)
        v1 = torch.zeros(6, dtype=torch.float64, device=dev)
        r1.compute_device(d_t, d_x, cell, pbc, e1, forces=f1, virial=v1)
        f_single, e_single = f1.cpu().numpy(), float(e1.item())
        r1.release_buffers()
        del r1, d_t, d_x, f1
        torch.cuda.empty_cache()

    # slabs across the longest cell direction, one per rank, with a ghost halo of layers x (cutoff + skin)
    plan = domain.make_plan(pos, cell, pbc, world, model.layers, cutoff, skin)
    ds = domain.DistributedSystem(plan, rank, types, pos, species=species, model=model, skin=skin,
                                  chunksize=args.chunk, device=dev)
    system = ds.system
    n_sub, n_own = ds.n, ds.nlocal

    # the clock sampler starts before the warm-up: nvidia-smi takes ~100 ms to come up and must not do that inside a
    # timed region of a few milliseconds per step; its samples cover warm-up and timed steps (the same work)
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        ds.step()
    barrier()
    l0 = B.kernel_launches()
    B.profile_enable(True)
    stages = dict(neighbor_list=0.0, bonds=0.0, forward=0.0, reverse=0.0)
    busy = [0.0]

    def step_device():
        ds.step()
        ms = system.stage_ms
        busy[0] += ms["total"]
        for k in stages:
            stages[k] += ms[k] / args.steps

    t0 = time.perf_counter()
    ms_mean, per_step = time_device_steps(step_device, args.steps, torch)
    wall_ms = (time.perf_counter() - t0) * 1e3
    barrier()
    prof = B.profile_report()
    B.profile_enable(False)
    launches = B.kernel_launches() - l0
    clocks = sampler.stop()
    times = torch.tensor([ms_mean, wall_ms / args.steps, busy[0] / args.steps, float(np.median(per_step)),
                          float(np.max(per_step))], dtype=torch.float64, device=dev)
    counts = torch.tensor([float(launches), float(n_sub), float(n_own)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(counts, op=dist.ReduceOp.SUM)
    ms_per_step, wall_ms_per_step, busy_ms_per_step = float(times[0]), float(times[1]), float(times[2])
    value = ms_per_step * 1e3 / n          # whole job: step time / atoms (the driver's strong-scaling formula v_1 / (N v_N))
    energy = ds.energy

    # the decomposed forces against the single-GPU evaluation: every rank's owned rows gathered on rank 0
    digest = None
    if world > 1:
        fo = ds.owned_forces.cpu().numpy()
        gathered = [None] * world if rank == 0 else None
        dist.gather_object((plan.owned[rank], fo), gathered, dst=0)
        if rank == 0:
            F = np.zeros((n, 3))
            for own, f in gathered:
                F[own] = f
            digest = {"F_max_abs": float(np.abs(F).max()), "F_sum_sq": float((F * F).sum()),
                      "F_net_max_abs": float(np.abs(F.sum(0)).max())}
            if f_single is not None:
                digest.update(dF_max_vs_single_gpu=float(np.abs(F - f_single).max()),
                              dE_per_atom_vs_single_gpu=abs(energy - e_single) / n,
                              tolerance_met=bool(np.abs(F - f_single).max() <= 1e-4 and abs(energy - e_single) / n <= 1e-5))

    # end to end with host buffers: every step copies its inputs from pinned host memory and its results back
    if world == 1:
        # the reference-facing host-pointer entry point
        h_types = torch.from_numpy(types).pin_memory().numpy()
        h_pos = torch.from_numpy(pos).pin_memory().numpy()
        h_f = torch.zeros((n, 3), dtype=torch.float64).pin_memory().numpy()
        lib = B.load_library()
        import ctypes as C
        e1, v6 = np.zeros(1), np.zeros(6)
        pbc8 = np.ascontiguousarray(pbc, dtype=np.uint8)
        cell64 = np.ascontiguousarray(cell, dtype=np.float64)

        def step_host():
            rc = lib.grace_system_compute(system._h, n, h_types.ctypes.data_as(C.c_void_p),
                                          h_pos.ctypes.data_as(C.c_void_p), cell64.ctypes.data_as(C.c_void_p),
                                          pbc8.ctypes.data_as(C.c_void_p), 0, e1.ctypes.data_as(C.c_void_p),
                                          v6.ctypes.data_as(C.c_void_p), h_f.ctypes.data_as(C.c_void_p), None)
            if rc:
                raise RuntimeError(lib.grace_last_error().decode())
        h2d, d2h = 28 * n, 24 * n + 56
    else:
        # every rank: its sub-system's positions from pinned host memory, its owned forces and the totals back
        h_pos = torch.from_numpy(ds.pos).pin_memory()
        h_f = torch.zeros((max(n_own, 1), 3), dtype=torch.float64).pin_memory()
        h_ev = torch.zeros(7, dtype=torch.float64).pin_memory()

        def step_host():
            ds.load_positions(h_pos)
            ds.step()
            h_f[:n_own].copy_(ds.owned_forces, non_blocking=True)
            h_ev.copy_(ds.d_ev, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        h2d, d2h = 24 * int(counts[1]), 24 * n + 56 * world

    for _ in range(max(args.warmup, 3)):     # the first host-path calls grow the staging buffers and touch the pinned pages
        step_host()
    barrier()
    e2e_steps = []
    t0 = time.perf_counter()
    for _ in range(args.steps):
        t1 = time.perf_counter()
        step_host()
        e2e_steps.append((time.perf_counter() - t1) * 1e3)
    barrier()
    e2e_t = torch.tensor([(time.perf_counter() - t0) * 1e3 / args.steps, float(np.median(e2e_steps)), float(np.max(e2e_steps))],
                         dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e_t[0])
    e2e = {"value": e2e_ms * 1e3 / n, "unit": UNIT, "ms_per_step": e2e_ms, "ms_per_step_median": float(e2e_t[1]),
           "ms_per_step_max": float(e2e_t[2]), "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)}
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # dominant kernel of rank 0 and its roofline
    peaks = {}
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    hbm_peak, peak_src = (peaks["hbm_gbs"], "measured") if "hbm_gbs" in peaks else (6650.0, "fallback")
    tot = sum(v[1] for v in prof.values()) or 1.0
    kern = sorted(prof.items(), key=lambda kv: -kv[1][1])
    shares = {k: {"launches": v[0], "ms_per_step": v[1] / args.steps, "share": v[1] / tot} for k, v in kern[:10]}
    top, (top_n, top_ms) = kern[0]
    top = top.strip("()").split("<")[0]
    # atoms this rank evaluates, their bonds inside the cutoff and list slots: from the lattice of the workload (58
    # bonds per atom in bcc at 6 A, 78 in fcc; slots with the 0.5 A skin scale as (6.5 / 6)^3)
    per_atom_bonds = 58.0 if wl["lattice"] == "bcc" else 78.0
    n_bonds = per_atom_bonds * n_own
    slots = per_atom_bonds * n_sub * (6.5 / 6.0) ** 3
    per_launch_ms = top_ms / top_n
    traffic_tab = load_traffic()

    def traffic_of(kernel, launches_per_step):
        e = traffic_tab.get((kernel, wl["cfg"]))
        return e["dram_bytes_per_atom"] * n_own / launches_per_step if e else None

    dense_names = {"mv_tc_kernel": "tensor", "prod_tile_kernel": "products"}
    if top in dense_names:
        # per-operation dense path: all launches of the kernel in a step together (one per operation of the plan; GRACE-2L
        # per pass of layer 2); flops and algorithmic bytes per atom from the plan
        lps = top_n / args.steps
        fl_atom, by_atom = model.dense_stats[dense_names[top]]
        step_ms = top_ms / args.steps
        gbs = by_atom * n_own / (step_ms * 1e-3) / 1e9
        if top == "mv_tc_kernel":
            ach = fl_atom * n_own / (step_ms * 1e-3) / 1e12
            peak_tf = peaks_here["tf32_tensor_tflops"] / 3.0
            roof = {"bound": "tensor", "kernel": top, "peak": peak_tf,
                    "peak_source": "tf32 tcgen05 microbenchmark of this run (M 128, N 256) / 3: three tf32 instructions per fp32-accurate product",
                    "unit": "TFLOP/s", "achieved": ach, "frac": ach / peak_tf, "traffic": traffic_of(top, lps),
                    "hbm_achieved_GBs": gbs, "hbm_frac_of_measured": gbs / hbm_peak,
                    "note": "FC layers and adjoints as 3 x tf32 grouped GEMMs with N = 32 / 64; the tf32 rate of an N = 32 (64) "
                            "instruction is 0.29 (0.57) of the N = 256 one (grace_measure_peak), and the kernel streams its "
                            "operands from HBM: hbm_frac_of_measured is the tighter bound"}
        else:
            roof = {"bound": "hbm", "kernel": top, "peak": hbm_peak, "peak_source": peak_src, "unit": "GB/s", "achieved": gbs,
                    "frac": gbs / hbm_peak, "traffic": traffic_of(top, lps)}
        roof.update(flop_per_atom=fl_atom, algorithmic_bytes_per_atom=by_atom, ms_per_step=step_ms, launches_per_step=lps,
                    algorithmic_bytes_per_launch=by_atom * n_own / lps)
    elif top.startswith("chain_"):
        # dense network: useful fp32 multiply-adds of the forward and reverse programs (GRACE-2L may evaluate layer 1
        # twice: counted once) per launch, against the measured peak of the unit the kernel computes on
        lps = top_n / args.steps
        flop = model.dense_flops * n_own / lps
        ach = flop / (per_launch_ms * 1e-3) / 1e12
        tensor = top.startswith("chain_tc")
        # a 3 x tf32 product issues three tensor-core instructions per useful multiply-add
        peak_tf = peaks_here["tf32_tensor_tflops"] / 3.0 if tensor else peaks_here["fp32_simt_tflops"]
        roof = {"bound": "tensor" if tensor else "fp32", "kernel": top, "peak": peak_tf,
                "peak_source": ("tf32 tcgen05 microbenchmark of this run / 3 (three tf32 instructions per fp32-accurate product)"
                                if tensor else "fp32 FFMA microbenchmark of this run (measured in this run)"),
                "unit": "TFLOP/s", "achieved": ach, "frac": ach / peak_tf, "traffic": traffic_of(top, lps),
                "algorithmic_bytes_per_launch": 2.0 * 4.0 * (modelgen.CONFIGS[wl["cfg"]]["lmax"] + 1) ** 2 * modelgen.CONFIGS[wl["cfg"]]["c1"] * n_own / lps,
                "flop_per_launch": flop, "flop_per_atom": model.dense_flops, "avg_launch_ms": per_launch_ms,
                "launches_per_step": lps,
                "note": "dense-network kernel: shared-memory resident, compute-bound (not HBM-bound); useful fp32-equivalent "
                        "flops of the plan / average launch time"}
    elif top.startswith("spbf3"):
        # GRACE-3L bond sums: per bond and coupled layer 2 flops per (Y lm, message function, channel) forward, 4 in the
        # reverse kernel (its two passes over the staged gradients); shared-memory resident, compute-bound
        lps = top_n / args.steps
        nlm, nlmi, C = 25, 25, 64
        per_bond = (4.0 if "bwd" in top else 2.0) * nlm * nlmi * C * 2 + (4.0 if "bwd" in top else 2.0) * nlm * C
        flop = per_bond * n_bonds
        ach = flop / (top_ms / args.steps * 1e-3) / 1e12
        peak_tf = peaks_here["fp32_simt_tflops"]
        roof = {"bound": "fp32", "kernel": top, "peak": peak_tf, "peak_source": "fp32 FFMA microbenchmark of this run (measured in this run)",
                "unit": "TFLOP/s", "achieved": ach, "frac": ach / peak_tf, "traffic": None, "flop_per_step": flop,
                "ms_per_step": top_ms / args.steps, "launches_per_step": lps,
                "note": "useful flops of the coupled bond sums of layers 2 and 3 (lmax 4, 25 message functions, 64 channels) x "
                        "bonds inside the cutoff / time of the kernel's launches of a step; first, untuned form of the kernel"}
    elif top.startswith("bond_"):
        # bond kernels: table look-ups from L1 / L2 and fp32 arithmetic per bond and channel - issue-bound, not HBM-bound
        # (their HBM fraction is in hbm_kernels); all launches of a step together (GRACE-2L: both layers)
        lps = top_n / args.steps
        flop = bond_flops(top, wl["cfg"], n_bonds, lps)
        ach = flop / (top_ms / args.steps * 1e-3) / 1e12
        peak_tf = peaks_here["fp32_simt_tflops"]
        roof = {"bound": "fp32", "kernel": top, "peak": peak_tf, "peak_source": "fp32 FFMA microbenchmark of this run (measured in this run)",
                "unit": "TFLOP/s", "achieved": ach, "frac": ach / peak_tf, "traffic": traffic_of(top, lps),
                "algorithmic_bytes_per_launch": (algorithmic_bytes(top, wl["cfg"], n_own, n_bonds, slots) or 0.0) / lps,
                "flop_per_step": flop, "ms_per_step": top_ms / args.steps, "launches_per_step": lps,
                "note": "useful flops per bond from the A-basis / reverse-pass formulas x bonds inside the cutoff / time of the "
                        "kernel's launches of a step"}
    else:
        roof = {"bound": "hbm", "kernel": top, "peak": hbm_peak, "peak_source": peak_src, "unit": "GB/s", "traffic": None}
        ab = algorithmic_bytes(top, wl["cfg"], n_own, n_bonds, slots)
        if ab is not None:
            lps = top_n / args.steps
            per_launch_bytes = ab / lps
            roof.update(achieved=per_launch_bytes / (per_launch_ms * 1e-3) / 1e9,
                        algorithmic_bytes_per_launch=per_launch_bytes, avg_launch_ms=per_launch_ms,
                        traffic=traffic_of(top, lps))
            roof["frac"] = roof["achieved"] / hbm_peak
        else:
            roof.update(achieved=None, frac=None)
    # the HBM-bound kernels of the step, each against the measured copy bandwidth
    hbm_kernels = {}
    for k, v in kern:
        name = k.strip("()").split("<")[0]
        ab = algorithmic_bytes(name, wl["cfg"], n_own, n_bonds, slots)
        if ab is not None and v[0] > 0:
            gbs = ab * args.steps / v[0] / (v[1] / v[0] * 1e-3) / 1e9
            hbm_kernels[name] = {"achieved_GBs": gbs, "frac_of_measured_hbm": gbs / hbm_peak, "avg_launch_ms": v[1] / v[0]}
        elif name in ("mv_tc_kernel", "prod_tile_kernel") and v[1] > 0:
            by_atom = model.dense_stats[{"mv_tc_kernel": "tensor", "prod_tile_kernel": "products"}[name]][1]
            gbs = by_atom * n_own / (v[1] / args.steps * 1e-3) / 1e9
            hbm_kernels[name] = {"achieved_GBs": gbs, "frac_of_measured_hbm": gbs / hbm_peak, "ms_per_step": v[1] / args.steps,
                                 "algorithmic_bytes_per_atom": by_atom}
    # the per-element operations run as two kernels (reduces: a thread per atom; their adjoints: a lane per output float4)
    elem_ms = sum(v[1] for k, v in kern if k.strip("()").split("<")[0] in ("mv_elem_tile_kernel", "mv_elem_wide_kernel"))
    if elem_ms > 0:
        by_atom = model.dense_stats["elementwise"][1]
        gbs = by_atom * n_own / (elem_ms / args.steps * 1e-3) / 1e9
        hbm_kernels["mv_elem_tile_kernel + mv_elem_wide_kernel"] = {
            "achieved_GBs": gbs, "frac_of_measured_hbm": gbs / hbm_peak, "ms_per_step": elem_ms / args.steps,
            "algorithmic_bytes_per_atom": by_atom}

    out = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
           "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
           "dtype": "f32", "data": "synthetic", "config": base_config(args.workload, world),
           "value_definition": "max over ranks of (CUDA-event time of the K steps / K) / atoms of the structure (whole job)",
           "us_per_atom_per_gpu": value * world,
           "ms_per_step_median": float(times[3]), "ms_per_step_max": float(times[4]),
           "ms_per_step_each_rank0": [round(float(x), 2) for x in per_step],
           "e2e": e2e, "gpu_launches": int(counts[0]), "clocks": clocks, "roofline": roof, "hbm_kernels": hbm_kernels,
           "measured_peaks": peaks_here,
           "details": {"species": species, "cutoff_A": cutoff, "chunk_atoms": system.chunksize,
                       "atoms_evaluated_all_ranks": int(counts[2]), "atoms_with_ghosts_all_ranks": int(counts[1])},
           "stages_ms_per_step": stages, "kernels": shares, "wall_ms_per_step": wall_ms_per_step,
           "device_busy_ms_per_step": busy_ms_per_step,
           "energy_eV": energy, "atoms_per_s": n / (ms_per_step * 1e-3)}
    if digest is not None:
        out["force_digest"] = digest
    if world == 1:
        ds = None
        system.release_buffers()
        if not args.no_cpu:
            out["cpu_baseline"], out["parity"] = parity_and_cpu(args, B, model, path, species, wl)
        if args.workload == DEFAULT and not args.no_also:
            out["also"] = run_also(args, B, torch, ALSO)
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def run_reference(args, rank, world):
    """The reference's own CPU drivers (oracle/_ref) on the host cores: each step one evaluation of a bounded block
    of the workload (same alloy, model and seeds), rank 0 only."""
    if rank != 0:
        return
    tmp = tempfile.mkdtemp(prefix="grace_bench_ref_")
    wl = WORKLOADS[args.workload]
    if "batch" in wl:
        run_reference_batch(args, wl, world, tmp)
        return
    reps = sample_reps(wl) or wl["reps"]
    path, species, types, pos, cell, pbc = make_workload(args.workload, tmp, reps)
    from oracle import refcpu
    cores = len(os.sched_getaffinity(0))
    n = len(types)
    nl_us = None
    if not refcpu.available():
        from oracle.grace_oracle import GraceOracle
        types, pos, cell, pbc = structures.crystal(wl["lattice"], wl["a"], (4, 4, 4), n_species=wl["nsp"], sigma=wl["sigma"], seed=1)
        n = len(types)
        o = GraceOracle(path)
        t = []
        for _ in range(max(1, min(args.steps, 3))):
            t0 = time.perf_counter()
            o.compute(species, types, pos, cell, pbc)
            t.append(time.perf_counter() - t0)
        ms, kind, cores = float(np.mean(t)) * 1e3, "port", 1
        sample = f"{n} atoms, numpy fp64 restatement of the path"
    else:
        rm = refcpu.RefModel(path, species)
        for _ in range(max(1, min(args.warmup, 2))):
            rm.compute(types, pos, cell, pbc, nthreads=cores)
        t = []
        for _ in range(args.steps):
            r = rm.compute(types, pos, cell, pbc, nthreads=cores)
            t.append(r["seconds_best"])
            nl_us = r["seconds_nlist"] * 1e6 / n
        ms, kind = float(np.mean(t)) * 1e3, "reference"
        sample = (f"{n} atoms ({'x'.join(str(r) for r in reps)} cells) of the same alloy, model and seeds per step: the "
                  "reference's CPU drivers, neighbour search excluded")
    value = ms * 1e3 / n
    out = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
           "dtype": "f32", "data": "synthetic", "config": base_config(args.workload, world),
           "sample_atoms": int(n),
           "cpu_baseline": {"value": value, "unit": "us/atom", "cores": cores, "kind": kind, "sample": sample,
                            "neighbor_search_us_per_atom": nl_us},
           "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(out))


def run_reference_batch(args, wl, world, tmp):
    """The batch workload on the reference's CPU drivers: a step evaluates the first 64 structures of the batch one after
    the other (each with all host threads), neighbour search included, as a Batch call rebuilds its lists every step."""
    from oracle import refcpu
    if not refcpu.available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref (the compiled reference) is not built on this box"}))
        return
    cores = len(os.sched_getaffinity(0))
    path = modelgen.write_config_model(os.path.join(tmp, "batch.npz"), wl["cfg"], modelgen.ELEMENTS, seed=0)
    count = 64
    natoms, T, P, Cc = make_batch(wl, count)
    n = int(natoms.sum())
    rm = refcpu.RefModel(path, list(modelgen.ELEMENTS))
    pbc = [1, 1, 1]

    def step():
        ev = nl = 0.0
        for k in range(count):
            r = rm.compute(T[k], P[k], Cc[k], pbc, nthreads=cores)
            ev += r["seconds_best"]
            nl += r["seconds_nlist"]
        return ev, nl

    for _ in range(max(1, min(args.warmup, 2))):
        step()
    t = [step() for _ in range(args.steps)]
    ev, nl = float(np.mean([a for a, _ in t])), float(np.mean([b for _, b in t]))
    ms = (ev + nl) * 1e3
    value = ms * 1e3 / n
    sample = (f"the first {count} structures of the batch ({n} atoms) per step, one call of the reference's CPU driver per "
              "structure, neighbour search included")
    out = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
           "dtype": "f32", "data": "synthetic", "config": base_config(args.workload, world), "sample_atoms": n,
           "structures_per_s": count / (ms * 1e-3),
           "cpu_baseline": {"value": value, "unit": "us/atom", "cores": cores, "kind": "reference", "sample": sample,
                            "neighbor_search_us_per_atom": nl * 1e6 / n},
           "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT, choices=sorted(WORKLOADS))
    ap.add_argument("--chunk", type=int, default=-1)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline and parity legs")
    ap.add_argument("--no-also", action="store_true", help="skip the second workload reported beside the default one")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    elif WORKLOADS[args.workload]["cfg"] == "3l" and world > 1:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "unit": UNIT, "config": base_config(args.workload, world),
                              "unavailable": "GRACE-3L runs on one GPU (no domain decomposition for three layers yet)"}))
    elif "batch" in WORKLOADS[args.workload]:
        run_batch(args, rank, world, local_rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
