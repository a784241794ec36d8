"""Builds the committed golden fixtures of tests/golden/ from a checkout of the reference (run here once; the GPU
box has no reference tree, the tests read only the files written by this script).

  models/<name>.npz      random-weight model fixtures of the reference test tree (tests/fixtures/*.npz).  The four
                         *_order3 models are kept in float64 (the TensorFlow goldens belong to exactly these
                         weights); the others are re-saved with float32 weights to halve their size, and their
                         goldens below are computed from the re-saved files.
  cells.npz              the fixture cells W54, WMo54, W2tri (tests/fixtures/{W54,WMo54,W2tri}.npz) plus seeded extra
                         structures: an open-boundary cluster, a slab (pbc 1 1 0), a small triclinic cell, one atom
  order3_tf.npz          TensorFlow-fp64 energy / forces / stress / energies of the four order-3 models on the three
                         fixture cells (tests/fixtures/ref_tf/order3_tf.npz; python/tests/test_order3_tf.py:14-26)
  ref_cpu.npz            outputs of the reference's own CPU drivers (oracle/_ref, built from the reference sources by
                         oracle/Makefile) for every model x structure pair, spline N = 1024

Usage:  make -C oracle && python tests/golden/make_golden.py /path/to/grace-runtime
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from oracle import refcpu  # noqa: E402

TF_MODELS = ["legacy_1l_order3", "grace_1l_order3", "legacy_2l_order3", "grace_2l_order3"]
F32_MODELS = ["grace_1l_small", "grace_2l_small", "grace_1l_w48", "grace_2l_l3", "legacy_1l_wide", "legacy_2l_small"]
SYM = {74: "W", 42: "Mo"}


def extra_cells():
    rng = np.random.default_rng(7)
    out = {}
    # open-boundary cluster of 13 atoms, cell padded (the caller pads open directions: python/grace_runtime/
    # neighbors.py:25-43)
    g = np.array([[i, j, k] for i in range(3) for j in range(3) for k in range(2)], dtype=float)[:13] * 2.7
    out["cluster13"] = dict(numbers=np.array([74, 42] * 6 + [74], dtype=np.int32),
                            positions=g + 0.15 * rng.standard_normal(g.shape) + 5.0,
                            cell=np.diag([30.0, 30.0, 30.0]), pbc=np.array([0, 0, 0], dtype=np.uint8))
    # slab: periodic in x, y; 3 x 3 x 2 bcc cells, open along z
    a = 3.165
    b = np.array([[i, j, k] for i in range(3) for j in range(3) for k in range(2)], dtype=float)
    p = np.concatenate([b, b + 0.5]) * a
    out["slab36"] = dict(numbers=rng.choice([74, 42], size=len(p)).astype(np.int32),
                         positions=p + 0.08 * rng.standard_normal(p.shape) + np.array([0.0, 0.0, 4.0]),
                         cell=np.array([[3 * a, 0, 0], [0, 3 * a, 0], [0, 0, 20.0]]),
                         pbc=np.array([1, 1, 0], dtype=np.uint8))
    # small triclinic cell, positions outside the cell on purpose (wrapping)
    cell = np.array([[6.1, 0.0, 0.0], [1.7, 5.6, 0.0], [-1.2, 0.9, 6.4]])
    f = rng.random((9, 3)) * 2.0 - 0.5
    out["tri9"] = dict(numbers=rng.choice([74, 42], size=9).astype(np.int32), positions=f @ cell, cell=cell,
                       pbc=np.array([1, 1, 1], dtype=np.uint8))
    # one isolated atom (no bonds: finite energy, zero force; tests/test_driver.cpp:432-440)
    out["atom1"] = dict(numbers=np.array([74], dtype=np.int32), positions=np.array([[1.0, 2.0, 3.0]]),
                        cell=np.diag([40.0, 40.0, 40.0]), pbc=np.array([0, 0, 0], dtype=np.uint8))
    return out


def main(ref):
    fx = os.path.join(ref, "tests", "fixtures")
    os.makedirs(os.path.join(HERE, "models"), exist_ok=True)
    for name in TF_MODELS + F32_MODELS:
        z = np.load(os.path.join(fx, name + ".npz"))
        arrs = {}
        for k in z.files:
            a = z[k]
            if name in F32_MODELS and a.dtype == np.float64 and a.size > 64 and not k.endswith("_cg_coeff"):
                a = a.astype(np.float32)
            arrs[k] = a
        with open(os.path.join(HERE, "models", name + ".npz"), "wb") as f:
            np.savez(f, **arrs)
    cells = {}
    for c in ["W54", "WMo54", "W2tri"]:
        z = np.load(os.path.join(fx, c + ".npz"))
        cells[c] = dict(numbers=z["numbers"], positions=z["positions"], cell=z["cell"],
                        pbc=np.array([1, 1, 1], dtype=np.uint8))
    cells.update(extra_cells())
    np.savez(os.path.join(HERE, "cells.npz"), **{f"{c}/{k}": v for c, d in cells.items() for k, v in d.items()})
    tf = np.load(os.path.join(fx, "ref_tf", "order3_tf.npz"))
    np.savez(os.path.join(HERE, "order3_tf.npz"), **{k: tf[k] for k in tf.files})
    out = {}
    for name in TF_MODELS + F32_MODELS:
        for c, d in cells.items():
            species = sorted(set(SYM[int(zz)] for zz in d["numbers"]))
            types = np.array([species.index(SYM[int(zz)]) + 1 for zz in d["numbers"]], dtype=np.int32)
            rm = refcpu.RefModel(os.path.join(HERE, "models", name + ".npz"), species, spline_n=1024)
            r = rm.compute(types, d["positions"], d["cell"], d["pbc"], nthreads=2)
            for k in ("energy", "forces", "virial", "energies"):
                out[f"{name}/{c}/{k}"] = np.asarray(r[k])
            print(name, c, r["energy"])
    np.savez(os.path.join(HERE, "ref_cpu.npz"), **out)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else
         os.path.abspath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "..", "reference")))
