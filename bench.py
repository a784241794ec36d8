"""Benchmark of the hot path: one energy + forces + stress evaluation per step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workload at one GPU: the 128,000-atom GRACE-1L configuration (random 4-component bcc alloy, 89-element model) - the
single-GPU configuration the metric is quoted on.  Prints one JSON line (rank 0).  `value` is microseconds per atom
per GPU with the inputs resident in HBM and the neighbour list reused, timed with CUDA events on the stream the
kernels are launched on; `e2e` is the same through the host-buffer C ABI call (pinned host memory, copies inside the
timed region).  The reference arm (--impl reference) times the reference's own CPU drivers (oracle/_ref) on the host
cores on a bounded sample of the same workload.
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

METRIC = "us_per_atom_per_gpu_energy_forces_stress"
UNIT = "us/atom/GPU"

WORKLOADS = {
    # name: (config, lattice, a, reps, species, sigma)
    "grace1l_128k_bcc_alloy": dict(cfg="1l", lattice="bcc", a=3.2, reps=(40, 40, 40), nsp=4, sigma=0.05, full=True),
    "grace1l_16k_bcc_alloy": dict(cfg="1l", lattice="bcc", a=3.2, reps=(20, 20, 20), nsp=4, sigma=0.05, full=True),
    "grace1l_2k_bcc_w": dict(cfg="1l", lattice="bcc", a=3.165, reps=(10, 10, 10), nsp=1, sigma=0.05, full=False),
    "grace2l_1m_fcc_alloy": dict(cfg="2l", lattice="fcc", a=3.6, reps=(40, 80, 80), nsp=3, sigma=0.08, full=True),
    "grace2l_128k_fcc_alloy": dict(cfg="2l", lattice="fcc", a=3.6, reps=(20, 40, 40), nsp=3, sigma=0.08, full=True),
    # 4096 small periodic structures (16-256 atoms, triclinic, 0.06-0.09 atoms/A^3) through the Batch entry points
    "grace2l_batch4096": dict(cfg="2l", batch=4096, unique=128, nmin=16, nmax=256, nsp=89, full=True),
}
DEFAULT = "grace1l_128k_bcc_alloy"


def make_workload(name, tmp, reps=None):
    w = WORKLOADS[name]
    species = modelgen._subset(2024, w["nsp"]) if w["full"] else ["W"]
    elements = modelgen.ELEMENTS if w["full"] else species
    path = modelgen.write_config_model(os.path.join(tmp, f"{name}.npz"), w["cfg"], elements, seed=0)
    types, pos, cell, pbc = structures.crystal(w["lattice"], w["a"], reps or w["reps"], n_species=w["nsp"],
                                               sigma=w["sigma"], seed=1)
    return path, species, types, pos, cell, pbc


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


# dram__bytes_read.sum + dram__bytes_write.sum per atom of one launch, from the ncu captures summarised in profiles/
NCU_DRAM_BYTES_PER_ATOM = {("chain_fused_kernel", "1l"): 781.5e6 / 128000, ("bond_fwd_kernel", "1l"): 488.2e6 / 128000,
                           ("bond_bwd_kernel", "1l"): 693.2e6 / 128000}


def algorithmic_bytes(kernel, model_cfg, n_atoms, n_bonds, slots):
    """Bytes one pass of a kernel over the whole structure must move at least (fp32 network, 16-byte bond records)."""
    c = modelgen.CONFIGS[model_cfg]
    nlm = (c["lmax"] + 1) ** 2
    C = c["c1"]
    if kernel == "bond_fwd_kernel":       # bond record in; A[nlm][C] out; offsets, counts, element per atom
        return 16.0 * n_bonds + (4.0 * nlm * C + 16.0) * n_atoms
    if kernel == "bond_bwd_kernel":       # bond record and slot in, bond force out; gA in, virial out
        return (16.0 + 4.0 + 12.0) * n_bonds + (4.0 * nlm * C + 48.0 + 16.0) * n_atoms
    if kernel == "nl_compact":            # list entry (j, S) and positions in, record + slot out
        return (8.0 + 16.0 + 4.0) * slots + 24.0 * n_atoms
    if kernel == "force_gather_kernel":   # bond force and reverse index in, force out
        return (12.0 + 4.0 + 12.0) * slots + 24.0 * n_atoms
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
    # `unique` generated structures (rejection sampling is slow), repeated with rigid shifts to the full batch
    un, ut, up, uc, upbc = structures.random_batch(wl["unique"], wl["nmin"], wl["nmax"], wl["nsp"], seed=1)
    rng = np.random.default_rng(2)
    start = np.concatenate([[0], np.cumsum(un)])
    natoms, T, P, Cc = [], [], [], []
    for s in range(wl["batch"]):
        u = s % wl["unique"]
        sl = slice(start[u], start[u + 1])
        natoms.append(un[u]); T.append(ut[sl]); Cc.append(uc[u])
        P.append(up[sl] + rng.random(3) @ uc[u])
    natoms = np.array(natoms, dtype=np.int32)
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
        out = {"metric": METRIC, "value": ms * 1e3 * world / n_total, "unit": UNIT, "n_gpus": world, "steps": args.steps,
               "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
               "dtype": "f32", "data": "synthetic",
               "config": {"workload": args.workload, "structures": int(wl["batch"]), "atoms": n_total, "model": "GRACE-2L",
                          "elements_in_model": 89, "atoms_per_structure": [int(wl["nmin"]), int(wl["nmax"])],
                          "unique_structures": int(wl["unique"]), "parallelism": f"structures over {world} rank(s)",
                          "passes": batch.passes, "neighbor_list": "built every step (Batch semantics)",
                          "value_definition": "max-over-ranks time per step x n_gpus / atoms"},
               "structures_per_s": wl["batch"] / (ms * 1e-3),
               "e2e": {"value": float(red[2]) * 1e3 * world / n_total, "unit": UNIT, "ms_per_step": float(red[2]),
                       "h2d_bytes_per_step": int(28 * n_total + 75 * wl["batch"]), "d2h_bytes_per_step": int(24 * n_total + 56 * wl["batch"])},
               "gpu_launches": int(cnt[0]), "clocks": clocks, "roofline": None,
               "kernels": {k: {"launches": v[0], "ms_per_step": v[1] / args.steps, "share": v[1] / tot} for k, v in kern[:8]},
               "wall_ms_per_step": float(red[1])}
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


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
    tmp = tempfile.mkdtemp(prefix="grace_bench_")
    path, species, types, pos, cell, pbc = make_workload(args.workload, tmp)     # every rank: the same seeded structure
    n = len(types)
    wl = WORKLOADS[args.workload]
    model = B.Model(path)
    skin = 0.5
    cutoff = B.System(model, species, skin=skin).cutoff
    # slabs across the longest cell direction, one per rank, with a ghost halo of layers x (cutoff + skin)
    plan = domain.make_plan(pos, cell, pbc, world, model.layers, cutoff, skin)
    ds = domain.DistributedSystem(plan, rank, types, pos, species=species, model=model, skin=skin,
                                  chunksize=args.chunk, device=dev)
    system = ds.system
    n_sub, n_own = ds.n, ds.nlocal

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def step_device():
        """device time of one step on this rank: the library's own events on its launch stream around the evaluation,
        torch events on the stream of the collectives around the exchange (the two run one after the other)"""
        ds.evaluate_local()
        ms = system.stage_ms
        t = ms["total"]
        if world > 1:
            ev0.record()
            ds.exchange()
            ev1.record()
            ev1.synchronize()
            t += ev0.elapsed_time(ev1)
        return t, ms

    # the clock sampler starts before the warm-up: nvidia-smi takes ~100 ms to come up and must not do that inside a
    # timed region of a few milliseconds per step; its samples cover warm-up and timed steps (the same work)
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(max(args.warmup, 1)):
        step_device()
    barrier()
    l0 = B.kernel_launches()
    B.profile_enable(True)
    # the K steps between two CUDA events, a synchronize on both sides (the library's stream is synchronised by every
    # call, so the events on torch's stream see all of its work); the sum of the per-step device intervals is kept as
    # `device_busy_ms_per_step`
    evA, evB = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    evA.record()
    t0 = time.perf_counter()
    dev_ms, stages = 0.0, dict(neighbor_list=0.0, bonds=0.0, forward=0.0, reverse=0.0)
    for _ in range(args.steps):
        t, ms = step_device()
        dev_ms += t
        for k in stages:
            stages[k] += ms[k] / args.steps
    torch.cuda.synchronize()
    evB.record()
    evB.synchronize()
    bracket_ms = evA.elapsed_time(evB)
    wall_ms = (time.perf_counter() - t0) * 1e3
    barrier()
    prof = B.profile_report()
    B.profile_enable(False)
    launches = B.kernel_launches() - l0
    clocks = sampler.stop()
    times = torch.tensor([bracket_ms / args.steps, wall_ms / args.steps, dev_ms / args.steps], dtype=torch.float64, device=dev)
    counts = torch.tensor([float(launches), float(n_sub), float(n_own)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(counts, op=dist.ReduceOp.SUM)
    ms_per_step, wall_ms_per_step, busy_ms_per_step = float(times[0]), float(times[1]), float(times[2])
    value = ms_per_step * 1e3 * world / n          # GPU-microseconds per atom: step time x GPUs / atoms
    energy = ds.energy

    # end to end with host buffers
    if world == 1:
        # the reference-facing host-pointer entry point, pinned host memory, copies inside the timed region
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
            torch.cuda.current_stream().synchronize()
            ds.step()
            h_f[:n_own].copy_(ds.owned_forces, non_blocking=True)
            h_ev.copy_(ds.d_ev, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        h2d, d2h = 24 * int(counts[1]), 24 * n + 56 * world

    for _ in range(max(args.warmup, 3)):     # the first host-path calls grow the staging buffers and touch the pinned pages
        step_host()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step_host()
    barrier()
    e2e_t = torch.tensor([(time.perf_counter() - t0) * 1e3 / args.steps], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e_t[0])
    e2e = {"value": e2e_ms * 1e3 * world / n, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": int(h2d),
           "d2h_bytes_per_step": int(d2h)}
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
    shares = {k: {"launches": v[0], "ms_per_step": v[1] / args.steps, "share": v[1] / tot} for k, v in kern[:8]}
    top, (top_n, top_ms) = kern[0]
    top = top.strip("()").split("<")[0]
    # atoms this rank evaluates, their bonds inside the cutoff and list slots: from the lattice of the workload (58
    # bonds per atom in bcc at 6 A, 78 in fcc; slots with the 0.5 A skin scale as (6.5 / 6)^3)
    per_atom_bonds = 58.0 if wl["lattice"] == "bcc" else 78.0
    n_bonds = per_atom_bonds * n_own
    slots = per_atom_bonds * n_sub * (6.5 / 6.0) ** 3
    per_launch_ms = top_ms / top_n
    sm_mhz = clocks.get("sm_mhz") or 1965.0
    if top == "chain_fused_kernel":
        # FMA-bound: useful fp32 multiply-adds of the dense network (forward + adjoints) against the SIMT peak of the
        # SMs at the clock sampled during the run
        # (GRACE-2L evaluates layer 1 twice, once more for the reverse pass: only one is counted as useful)
        flop = model.dense_flops * n_own * args.steps / top_n
        peak_tf = 148 * 128 * 2 * sm_mhz * 1e6 / 1e12
        ach = flop / (per_launch_ms * 1e-3) / 1e12
        roof = {"bound": "fp32", "kernel": top, "peak": peak_tf, "peak_source": "148 SMs x 128 FMA lanes x 2 flop x sampled SM clock (no measured SIMT peak in MEASURED_PEAKS.json)",
                "unit": "TFLOP/s", "achieved": ach, "frac": ach / peak_tf,
                # DRAM bytes per launch from the ncu capture of this kernel on this workload (profiles/), scaled by the
                # atoms of a launch: traffic grows in proportion to the atoms
                "traffic": (NCU_DRAM_BYTES_PER_ATOM.get((top, wl["cfg"]), 0.0) * n_own * args.steps / top_n) or None,
                "algorithmic_bytes_per_launch": 2.0 * 4.0 * (modelgen.CONFIGS[wl["cfg"]]["lmax"] + 1) ** 2 * modelgen.CONFIGS[wl["cfg"]]["c1"] * n_own * args.steps / top_n,
                "flop_per_launch": flop, "flop_per_atom": model.dense_flops, "avg_launch_ms": per_launch_ms,
                "note": "dense-network kernel: shared-memory resident fp32 SIMT work, neither HBM- nor tensor-bound; "
                        "its DRAM traffic (ncu) is in profiles/"}
    else:
        roof = {"bound": "hbm", "kernel": top, "peak": hbm_peak, "peak_source": peak_src, "unit": "GB/s", "traffic": None}
        ab = algorithmic_bytes(top, wl["cfg"], n_own, n_bonds, slots)
        if ab is not None:
            per_launch_bytes = ab * args.steps / top_n
            roof.update(achieved=per_launch_bytes / (per_launch_ms * 1e-3) / 1e9,
                        algorithmic_bytes_per_launch=per_launch_bytes, avg_launch_ms=per_launch_ms,
                        traffic=(NCU_DRAM_BYTES_PER_ATOM.get((top, wl["cfg"]), 0.0) * n_own * args.steps / top_n) or None)
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

    out = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
           "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
           "dtype": "f32", "data": "synthetic",
           "config": {"workload": args.workload, "atoms": int(n), "model": "GRACE-1L" if wl["cfg"] == "1l" else "GRACE-2L",
                      "elements_in_model": 89 if wl["full"] else 1, "species": species, "cutoff_A": cutoff, "skin_A": skin,
                      "neighbor_list": "reused (built in warm-up)", "chunk_atoms": system.chunksize,
                      "parallelism": f"slabs{world}" if world > 1 else "single",
                      "value_definition": "max over ranks of (CUDA-event time of the K steps / K) x n_gpus / atoms",
                      "atoms_evaluated_all_ranks": int(counts[2]), "atoms_with_ghosts_all_ranks": int(counts[1]),
                      "l2": "per-step working set (bond records + chunk tensors) exceeds the 126 MB L2",
                      "radial": "cubic Hermite tables, 1024 intervals"},
           "e2e": e2e, "gpu_launches": int(counts[0]), "clocks": clocks, "roofline": roof, "hbm_kernels": hbm_kernels,
           "stages_ms_per_step": stages, "kernels": shares, "wall_ms_per_step": wall_ms_per_step,
           "device_busy_ms_per_step": busy_ms_per_step,
           "energy_eV": energy, "atoms_per_s": n / (ms_per_step * 1e-3)}
    if not args.no_cpu and world == 1:
        out["cpu_baseline"] = cpu_baseline(args, path, species, types, pos, cell, pbc, bounded=True)
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def cpu_baseline(args, path, species, types, pos, cell, pbc, bounded):
    """The reference's own CPU drivers on the host cores (oracle/_ref), or the numpy port when it did not travel."""
    from oracle import refcpu
    wl = WORKLOADS[args.workload]
    cores = len(os.sched_getaffinity(0))
    if refcpu.available():
        if bounded and len(types) > 32000:      # about 10-30 s of CPU work: a smaller block of the same alloy
            reps = (20, 20, 40) if wl["lattice"] == "bcc" else (16, 16, 32)
            types, pos, cell, pbc = structures.crystal(wl["lattice"], wl["a"], reps, n_species=wl["nsp"],
                                                       sigma=wl["sigma"], seed=1)
        rm = refcpu.RefModel(path, species)
        rm.compute(types, pos, cell, pbc, nthreads=cores)               # warm-up (tables, buffers)
        r = rm.compute(types, pos, cell, pbc, nthreads=cores, repeats=3)
        return {"value": r["seconds_median"] * 1e6 / len(types), "unit": "us/atom", "cores": cores, "kind": "reference",
                "sample": f"{len(types)} atoms of the same alloy and model, median of 3 calls after the first, "
                          f"neighbour search ({r['seconds_nlist'] * 1e6 / len(types):.2f} us/atom) not included",
                "energy_eV_per_atom": r["energy"] / len(types)}
    from oracle.grace_oracle import GraceOracle
    types, pos, cell, pbc = structures.crystal(wl["lattice"], wl["a"], (4, 4, 4), n_species=wl["nsp"], sigma=wl["sigma"], seed=1)
    o = GraceOracle(path)
    t0 = time.perf_counter()
    o.compute(species, types, pos, cell, pbc)
    dt = time.perf_counter() - t0
    return {"value": dt * 1e6 / len(types), "unit": "us/atom", "cores": 1, "kind": "port",
            "sample": f"{len(types)} atoms, numpy fp64 restatement, one call"}


def run_reference(args, rank, world):
    if rank != 0:
        return
    tmp = tempfile.mkdtemp(prefix="grace_bench_ref_")
    wl = WORKLOADS[args.workload]
    if "batch" in wl:
        print(json.dumps({"impl": "reference", "unavailable": "the reference arm times single structures; not wired for the batch workload"}))
        return
    reps = wl["reps"]
    if np.prod(reps) * (2 if wl["lattice"] == "bcc" else 4) > 32000:
        reps = (20, 20, 40) if wl["lattice"] == "bcc" else (16, 16, 32)
    path, species, types, pos, cell, pbc = make_workload(args.workload, tmp, reps)
    from oracle import refcpu
    cores = len(os.sched_getaffinity(0))
    n = len(types)
    if not refcpu.available():
        base = cpu_baseline(args, path, species, types, pos, cell, pbc, bounded=True)
        value, kind, sample = base["value"], base["kind"], base["sample"]
        ms = value * n / 1e3
    else:
        rm = refcpu.RefModel(path, species)
        for _ in range(max(1, min(args.warmup, 2))):
            rm.compute(types, pos, cell, pbc, nthreads=cores)
        t = []
        for _ in range(args.steps):
            r = rm.compute(types, pos, cell, pbc, nthreads=cores)
            t.append(r["seconds_best"])
        ms = float(np.mean(t)) * 1e3
        value, kind = ms * 1e3 / n, "reference"
        sample = f"{n} atoms of the same alloy and model per step (the reference's CPU drivers, neighbour search excluded)"
    out = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
           "dtype": "f32", "data": "synthetic",
           "config": {"workload": args.workload, "atoms": int(n), "model": "GRACE-1L" if wl["cfg"] == "1l" else "GRACE-2L"},
           "cpu_baseline": {"value": value, "unit": "us/atom", "cores": cores, "kind": kind, "sample": sample},
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
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    elif "batch" in WORKLOADS[args.workload]:
        run_batch(args, rank, world, local_rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
