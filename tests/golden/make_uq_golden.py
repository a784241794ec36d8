"""Golden vectors of the UQ outputs (gamma, sigma, cluster per atom): the reference's own CPU drivers
(Grace1LFused / Grace2LFused with ComputeFlags::uq, through oracle/_ref) on the order-4 fixture models with a seeded
random UQ head of schema 6 (grace_runtime_b200.modelgen.add_uq_head: the reference tree holds no model with a head).
Writes tests/golden/uq_ref.npz; the tests regenerate the same model files from the same seeds.

legacy_1l_wide (AAA = AA1 x A, `AAA_right_A`): the reference driver's default path (products reduced row by row) rebuilds
the third-order basis block for UQ as AA1 x A1 (libgrace/src/fused_1l.cpp:600-606), which is not the model's AAA; its
path with materialised products (G2LF_NOROWRED=1, read when the driver is built) uses the model's tensor
(libgrace/src/fused_1l.cpp:598,316-320).  The goldens of that model come from the second path.

Usage:  make -C oracle && python tests/golden/make_uq_golden.py
"""
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
sys.path.insert(0, os.path.join(HERE, ".."))

from conftest import Cells, model_path  # noqa: E402
from grace_runtime_b200 import modelgen  # noqa: E402
from oracle import refcpu  # noqa: E402

# (fixture model, seed of the head, projection width, clusters)
UQ_MODELS = [("grace_1l_small", 1, 32, 3), ("grace_1l_w48", 2, 48, 2), ("legacy_1l_wide", 3, 20, 4),
             ("grace_2l_small", 4, 32, 3), ("legacy_2l_small", 5, 16, 2)]
NOROWRED = ("legacy_1l_wide",)
UQ_CELLS = ["W54", "WMo54", "W2tri", "cluster13", "slab36", "tri9", "atom1"]


def uq_model(name, seed, rp, k, folder):
    return modelgen.add_uq_head(model_path(name), os.path.join(folder, f"{name}_uq.npz"), seed=seed, rp_dim=rp,
                                max_clusters=k)


def main():
    cells = Cells()
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        for name, seed, rp, k in UQ_MODELS:
            path = uq_model(name, seed, rp, k, tmp)
            os.environ.pop("G2LF_NOROWRED", None)
            if name in NOROWRED:
                os.environ["G2LF_NOROWRED"] = "1"
            for cn in UQ_CELLS:
                c = cells.get(cn)
                r = refcpu.RefModel(path, c["species"]).compute(c["types"], c["positions"], c["cell"], c["pbc"], uq=True)
                for key in ("gamma", "sigma", "cluster"):
                    out[f"{name}/{cn}/{key}"] = r[key]
                out[f"{name}/{cn}/energy"] = np.array(r["energy"])
    np.savez(os.path.join(HERE, "uq_ref.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
