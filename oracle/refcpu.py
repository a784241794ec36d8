"""TEST INFRASTRUCTURE ONLY - ctypes access to oracle/_ref/libgrace_ref_{v3,v4}.so, the reference's own CPU drivers
compiled by oracle/Makefile (entry points: oracle/ref_driver.cpp).  Used by tests/ as the second checker next to the
numpy restatement, and by the benchmark's CPU-baseline / reference arm.  Nothing of the product imports it."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None


def _cpu_flags():
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def lib_path():
    """The x86-64-v4 build when the host has AVX-512 (f, bw, cd, dq, vl), else the x86-64-v3 build; None if unbuilt."""
    fl = _cpu_flags()
    v4 = {"avx512f", "avx512bw", "avx512cd", "avx512dq", "avx512vl"} <= fl
    for tag in (["v4"] if v4 else []) + ["v3"]:
        p = os.path.join(_HERE, "_ref", f"libgrace_ref_{tag}.so")
        if os.path.exists(p):
            return p
    return None


def available():
    return lib_path() is not None


def _load():
    global _lib
    if _lib is None:
        p = lib_path()
        if p is None:
            raise RuntimeError("oracle/_ref is not built: run `make -C oracle REF=<reference checkout>`")
        L = C.CDLL(p)
        L.ref_last_error.restype = C.c_char_p
        L.ref_model_load.restype = C.c_void_p
        L.ref_model_load.argtypes = [C.c_char_p, C.c_int]
        L.ref_model_free.argtypes = [C.c_void_p]
        L.ref_model_layers.argtypes = [C.c_void_p]
        L.ref_set_species.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_char_p)]
        L.ref_cutoff.restype = C.c_double
        L.ref_cutoff.argtypes = [C.c_void_p]
        L.ref_compute.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p] * 4 + [C.c_int] * 3 + [C.c_void_p] * 5
        L.ref_compute_uq.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p] * 4 + [C.c_int] * 2 + [C.c_void_p] * 7
        L.ref_neighbors.restype = C.c_int64
        L.ref_neighbors.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_double, C.c_int, C.c_int64,
                                    C.c_void_p, C.c_void_p, C.c_void_p]
        _lib = L
    return _lib


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


class RefModel:
    """The reference CPU driver of one model file for one species set."""

    def __init__(self, path, species, spline_n=1024):
        L = _load()
        self.h = L.ref_model_load(os.fsencode(path), spline_n)
        if not self.h:
            raise RuntimeError(L.ref_last_error().decode())
        arr = (C.c_char_p * len(species))(*[s.encode() for s in species])
        if L.ref_set_species(self.h, len(species), arr):
            raise RuntimeError(L.ref_last_error().decode())
        self.layers = L.ref_model_layers(self.h)
        self.cutoff = L.ref_cutoff(self.h)

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.ref_model_free(self.h)
            self.h = None

    def compute(self, types, pos, cell, pbc, nthreads=0, energy_only=False, repeats=1, uq=False):
        """uq: also gamma, sigma, cluster per atom (the model needs a UQ head; one evaluation, no timings)."""
        L = _load()
        n = len(types)
        types = np.ascontiguousarray(types, dtype=np.int32)
        pos = np.ascontiguousarray(pos, dtype=np.float64)
        cell = np.ascontiguousarray(cell, dtype=np.float64)
        pbc = np.ascontiguousarray(pbc, dtype=np.uint8)
        nth = nthreads or len(os.sched_getaffinity(0))
        e = C.c_double(0.0)
        f = np.zeros((n, 3))
        v = np.zeros(6)
        ea = np.zeros(n)
        sec = np.zeros(3)
        if uq:
            g, sg, cl = np.zeros(n), np.zeros(n), np.zeros(n)
            rc = L.ref_compute_uq(self.h, n, _ptr(types), _ptr(pos), _ptr(cell), _ptr(pbc), nth, int(energy_only),
                                  C.addressof(e), _ptr(f), _ptr(v), _ptr(ea), _ptr(g), _ptr(sg), _ptr(cl))
            if rc:
                raise RuntimeError(L.ref_last_error().decode())
            return dict(energy=e.value, forces=f, virial=v, energies=ea, gamma=g, sigma=sg, cluster=cl, threads=nth)
        rc = L.ref_compute(self.h, n, _ptr(types), _ptr(pos), _ptr(cell), _ptr(pbc), nth, int(energy_only), repeats,
                           C.addressof(e), _ptr(f), _ptr(v), _ptr(ea), _ptr(sec))
        if rc:
            raise RuntimeError(L.ref_last_error().decode())
        return dict(energy=e.value, forces=f, virial=v, energies=ea, seconds_nlist=sec[0], seconds_best=sec[1],
                    seconds_median=sec[2], threads=nth)


def neighbors(pos, cell, pbc, cutoff, nthreads=1):
    """Reference neighbour list as (i, j, S[nb,3]) in the caller's atom order and frame."""
    L = _load()
    pos = np.ascontiguousarray(pos, dtype=np.float64)
    cell = np.ascontiguousarray(cell, dtype=np.float64)
    pbc = np.ascontiguousarray(pbc, dtype=np.uint8)
    n = len(pos)
    cap = 1024
    while True:
        bi = np.zeros(cap, dtype=np.int32)
        bj = np.zeros(cap, dtype=np.int32)
        bs = np.zeros((cap, 3), dtype=np.int32)
        nb = L.ref_neighbors(n, _ptr(pos), _ptr(cell), _ptr(pbc), cutoff, nthreads, cap, _ptr(bi), _ptr(bj), _ptr(bs))
        if nb < 0:
            raise RuntimeError(L.ref_last_error().decode())
        if nb <= cap:
            return bi[:nb].astype(np.int64), bj[:nb].astype(np.int64), bs[:nb].astype(np.int64)
        cap = int(nb)
