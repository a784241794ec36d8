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


def run_ours(args, rank, world, local_rank):
    import torch

    from grace_runtime_b200 import backend as B

    if world > 1:
        raise SystemExit("bench.py: domain-decomposed runs are not implemented in this build (N = 1 only)")
    torch.cuda.set_device(local_rank)
    B.initialize(local_rank)
    tmp = tempfile.mkdtemp(prefix="grace_bench_")
    path, species, types, pos, cell, pbc = make_workload(args.workload, tmp)
    n = len(types)
    model = B.Model(path)
    system = B.System(model, species, skin=0.5, chunksize=args.chunk)
    dev = torch.device("cuda", local_rank)
    d_types = torch.from_numpy(types).to(dev)
    d_pos = torch.from_numpy(pos).to(dev)
    d_e = torch.zeros(1, dtype=torch.float64, device=dev)
    d_v = torch.zeros(6, dtype=torch.float64, device=dev)
    d_f = torch.zeros((n, 3), dtype=torch.float64, device=dev)
    torch.cuda.synchronize()

    def step_device():
        system.compute_device(n, d_types.data_ptr(), d_pos.data_ptr(), cell, pbc, d_e.data_ptr(), d_f.data_ptr(),
                              d_v.data_ptr())
        return system.stage_ms

    for _ in range(max(args.warmup, 1)):
        step_device()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    l0 = B.kernel_launches()
    B.profile_enable(True)
    t0 = time.perf_counter()
    dev_ms, stages = 0.0, dict(neighbor_list=0.0, bonds=0.0, forward=0.0, reverse=0.0)
    for _ in range(args.steps):
        ms = step_device()
        dev_ms += ms["total"]
        for k in stages:
            stages[k] += ms[k] / args.steps
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3
    prof = B.profile_report()
    B.profile_enable(False)
    launches = B.kernel_launches() - l0
    clocks = sampler.stop()
    ms_per_step = dev_ms / args.steps
    value = ms_per_step * 1e3 / n          # us per atom on this one GPU
    energy = float(d_e.item())

    # end to end: host buffers in pinned memory through the host-pointer entry point, copies inside the timed region
    h_types = torch.from_numpy(types).pin_memory().numpy()
    h_pos = torch.from_numpy(pos).pin_memory().numpy()
    h_f = torch.zeros((n, 3), dtype=torch.float64).pin_memory().numpy()
    lib = B.load_library()
    import ctypes as C
    e1, v6 = np.zeros(1), np.zeros(6)
    pbc8 = np.ascontiguousarray(pbc, dtype=np.uint8)
    cell64 = np.ascontiguousarray(cell, dtype=np.float64)

    def step_host():
        rc = lib.grace_system_compute(system._h, n, h_types.ctypes.data_as(C.c_void_p), h_pos.ctypes.data_as(C.c_void_p),
                                      cell64.ctypes.data_as(C.c_void_p), pbc8.ctypes.data_as(C.c_void_p), 0,
                                      e1.ctypes.data_as(C.c_void_p), v6.ctypes.data_as(C.c_void_p),
                                      h_f.ctypes.data_as(C.c_void_p), None)
        if rc:
            raise RuntimeError(lib.grace_last_error().decode())

    for _ in range(max(args.warmup, 3)):     # the first host-path calls grow the staging buffers and touch the pinned pages
        step_host()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step_host()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    e2e = {"value": e2e_ms * 1e3 / n, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": int(28 * n),
           "d2h_bytes_per_step": int(24 * n + 56)}

    # dominant kernel and its roofline
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
    n_bonds = None
    roof = {"bound": "hbm", "kernel": top, "peak": hbm_peak, "peak_source": peak_src, "unit": "GB/s", "traffic": None}
    # bonds inside the cutoff and list slots: from the model of the workload (58 bonds per atom in bcc at 6 A;
    # slots with the 0.5 A skin scale as (6.5 / 6)^3)
    wl = WORKLOADS[args.workload]
    per_atom_bonds = 58.0 if wl["lattice"] == "bcc" else 78.0
    n_bonds = per_atom_bonds * n
    slots = n_bonds * (6.5 / 6.0) ** 3
    ab = algorithmic_bytes(top, wl["cfg"], n, n_bonds, slots)
    if ab is not None:
        passes_per_step = 1.0      # every bond / gather kernel covers the structure once per step (in chunks)
        per_launch_bytes = ab * passes_per_step * args.steps / top_n
        per_launch_s = top_ms / top_n * 1e-3
        roof.update(achieved=per_launch_bytes / per_launch_s / 1e9, algorithmic_bytes_per_launch=per_launch_bytes,
                    avg_launch_ms=top_ms / top_n)
        roof["frac"] = roof["achieved"] / hbm_peak
    else:
        roof.update(achieved=None, frac=None, note="dense-network kernel: compute bound on fp32 FMA, no HBM roofline")

    out = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
           "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
           "dtype": "f32", "data": "synthetic",
           "config": {"workload": args.workload, "atoms": int(n), "model": "GRACE-1L" if wl["cfg"] == "1l" else "GRACE-2L",
                      "elements_in_model": 89 if wl["full"] else 1, "species": species, "cutoff_A": 6.0, "skin_A": 0.5,
                      "neighbor_list": "reused (built in warm-up)", "chunk_atoms": system.chunksize,
                      "l2": "per-step working set (bond records + chunk tensors) exceeds the 126 MB L2",
                      "radial": "cubic Hermite tables, 1024 intervals"},
           "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "roofline": roof,
           "stages_ms_per_step": stages, "kernels": shares, "wall_ms_per_step": wall_ms / args.steps,
           "energy_eV": energy, "atoms_per_s": n / (ms_per_step * 1e-3)}
    if not args.no_cpu:
        out["cpu_baseline"] = cpu_baseline(args, path, species, types, pos, cell, pbc, bounded=True)
    print(json.dumps(out))


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
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
