import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")
SYM = {74: "W", 42: "Mo"}
TF_MODELS = ["legacy_1l_order3", "grace_1l_order3", "legacy_2l_order3", "grace_2l_order3"]
F32_MODELS = ["grace_1l_small", "grace_2l_small", "grace_1l_w48", "grace_2l_l3", "legacy_1l_wide", "legacy_2l_small"]
TF_CELLS = ["W54", "WMo54", "W2tri"]
EXTRA_CELLS = ["cluster13", "slab36", "tri9", "atom1"]

# target tolerances of the build (energy eV/atom, forces eV/A, stress eV/A^3); the golden comparisons use
# the reference's own tighter fp32-vs-fp64 thresholds (python/tests/test_ref_tf.py:22)
TOL_E, TOL_F, TOL_S = 1e-5, 1e-4, 1e-4
REF_TOL = {"energy": 1e-6, "forces": 2e-5, "energies": 1e-5, "stress": 1e-5}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


class Cells:
    def __init__(self):
        self.z = np.load(os.path.join(GOLDEN, "cells.npz"))

    def get(self, name):
        nums = self.z[f"{name}/numbers"]
        species = sorted(set(SYM[int(q)] for q in nums))
        types = np.array([species.index(SYM[int(q)]) + 1 for q in nums], dtype=np.int32)
        return dict(species=species, types=types, positions=self.z[f"{name}/positions"], cell=self.z[f"{name}/cell"],
                    pbc=self.z[f"{name}/pbc"], n=len(nums), volume=abs(np.linalg.det(self.z[f"{name}/cell"])))


@pytest.fixture(scope="session")
def cells():
    return Cells()


@pytest.fixture(scope="session")
def tf_golden():
    return np.load(os.path.join(GOLDEN, "order3_tf.npz"))


@pytest.fixture(scope="session")
def ref_golden():
    return np.load(os.path.join(GOLDEN, "ref_cpu.npz"))


def model_path(name):
    return os.path.join(GOLDEN, "models", name + ".npz")


def stress_of(virial, volume):
    """ASE Voigt stress from the bond virial (python/grace_runtime/calculator.py:155-157)."""
    return -np.asarray(virial)[[0, 1, 2, 5, 4, 3]] / volume


def compare_tf(res, gold, key, cell):
    """The comparison of the reference's own golden test (python/tests/test_ref_tf.py:43-55)."""
    n = cell["n"]
    d = {"energy": abs(res["energy"] - gold[f"{key}/energy"]) / n,
         "forces": np.abs(res["forces"] - gold[f"{key}/forces"]).max(),
         "energies": np.abs(res["energies"] - gold[f"{key}/energies"]).max(),
         "stress": np.abs(stress_of(res["virial"], cell["volume"]) - gold[f"{key}/stress"]).max() /
         np.abs(gold[f"{key}/stress"]).max()}
    return d


@pytest.fixture(scope="session")
def backend():
    """The initialised CUDA backend (C ABI through ctypes)."""
    from grace_runtime_b200 import backend as B
    B.initialize(0)
    return B
