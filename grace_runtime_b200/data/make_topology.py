"""Extracts the architecture tables (function-index arrays, Clebsch-Gordan coefficients, tile maps, flags) of the
random-weight model fixtures of the reference test tree into small `topology_*.npz` files next to this script.

The tables depend only on (layers, lmax, max_order), not on channel widths or the element set, so
`grace_runtime_b200.modelgen` can write a legal kokkos.npz of any width from them with freshly drawn weights.
Every floating-point weight array is dropped here; only integer tables, CG coefficients, FC output factors and
scalar flags are kept.

Usage (needs a checkout of the reference; run once, outputs are committed):
    python grace_runtime_b200/data/make_topology.py /path/to/grace-runtime
"""
import os
import sys

import numpy as np

SOURCES = {
    "topology_1l_lmax4": "grace_1l_w48.npz",      # order 4 tables (order 3 = the same without the AAAA stage)
    "topology_1l_lmax3_o3": "grace_1l_l3.npz",
    "topology_1l_lmax2": "grace_1l_small.npz",
    "topology_2l_lmax3_o3": "grace_2l_l3.npz",
    "topology_2l_lmax2": "grace_2l_small.npz",
}
KEEP_FLOAT = ("_cg_coeff", "_norm_out_factor")
# exported by tensorpotential but never read by any loader of the reference (libgrace/src/model_{1l,2l}.cpp)
NEVER_READ = ("I_out_0_", "I_out_1_", "I_1_LN_", "rho_LN_")


def main(ref):
    here = os.path.dirname(os.path.abspath(__file__))
    for out, src in SOURCES.items():
        z = np.load(os.path.join(ref, "tests", "fixtures", src))
        keep = {}
        for k in z.files:
            a = z[k]
            if k.startswith(NEVER_READ):
                continue
            if a.dtype.kind == "f" and a.size > 1 and not k.endswith(KEEP_FLOAT):
                continue
            keep[k] = a
        np.savez(os.path.join(here, out + ".npz"), **keep)
        print(out, len(keep), "arrays")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.abspath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "..", "reference")))
