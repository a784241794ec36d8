"""Host-side checks that need no GPU: the shared library loads, exports every symbol the header declares, the model
loader accepts the reference's fixtures and rejects broken files with the reference's error class, and nothing
computes without a device."""
import os
import re

import numpy as np
import pytest

from conftest import F32_MODELS, ROOT, TF_MODELS, model_path


@pytest.fixture(scope="module")
def B():
    from grace_runtime_b200 import backend
    backend.load_library()
    return backend


def test_library_exports_every_declared_symbol(B):
    hdr = open(os.path.join(ROOT, "include", "grace_b200.h")).read()
    declared = set(re.findall(r"\b(grace_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations found"
    lib = B.load_library()
    for name in sorted(declared):
        assert hasattr(lib, name), name
    assert declared == set(B.SIGNATURES), declared ^ set(B.SIGNATURES)


def test_identity(B):
    assert B.arch() == "sm100" and B.platform() == "cuda" and B.blas() == "" and B.ABI == 7
    assert B.load_library().grace_abi() == 7
    assert B.archs() == ["sm100"]


@pytest.mark.parametrize("name", TF_MODELS + F32_MODELS)
def test_loads_reference_fixture_models(B, name):
    m = B.Model(model_path(name))
    assert m.layers == (2 if "_2l_" in name else 1)
    assert m.element_names == ["Mo", "W"]
    assert not m.has_uq


def test_generated_config_models_load(B, tmp_path):
    from grace_runtime_b200 import modelgen
    p1 = modelgen.write_config_model(str(tmp_path / "c1.npz"), "1l", modelgen.ELEMENTS, seed=3)
    p2 = modelgen.write_config_model(str(tmp_path / "c2.npz"), "2l", ["Al", "Cu", "Ni"], seed=4)
    m1, m2 = B.Model(p1), B.Model(p2)
    assert m1.layers == 1 and len(m1.element_names) == 89
    assert m2.layers == 2 and m2.element_names == ["Al", "Cu", "Ni"]


def test_broken_files_are_value_errors(B, tmp_path):
    with pytest.raises(ValueError):
        B.Model(str(tmp_path / "missing.npz"))
    z = dict(np.load(model_path("grace_1l_order3")))
    bad = dict(z)
    bad["prod_AA_left_ind"] = bad["prod_AA_left_ind"].copy()
    bad["prod_AA_left_ind"][0] = 10 ** 6          # index out of range
    np.savez(tmp_path / "bad_index.npz", **bad)
    with pytest.raises(ValueError, match="prod_AA_left_ind"):
        B.Model(str(tmp_path / "bad_index.npz"))
    bad = dict(z)
    bad["mlp_rad_W1"] = bad["mlp_rad_W1"][:, :-1]  # shape mismatch between layers
    np.savez(tmp_path / "bad_shape.npz", **bad)
    with pytest.raises(ValueError):
        B.Model(str(tmp_path / "bad_shape.npz"))
    bad = dict(z)
    bad["chem_embedding"] = bad["chem_embedding"].copy()
    bad["chem_embedding"][0, 0] = np.nan
    np.savez(tmp_path / "bad_nan.npz", **bad)
    with pytest.raises(ValueError, match="non-finite"):
        B.Model(str(tmp_path / "bad_nan.npz"))
    np.savez_compressed(tmp_path / "compressed.npz", **z)
    with pytest.raises(ValueError, match="compressed"):
        B.Model(str(tmp_path / "compressed.npz"))
    bad = dict(z)
    bad["grace_format_version"] = np.array([99])
    np.savez(tmp_path / "future.npz", **bad)
    with pytest.raises(ValueError, match="format"):
        B.Model(str(tmp_path / "future.npz"))
    with pytest.raises(ValueError):
        B.Model(model_path("grace_1l_order3"), spline=8)


def test_no_compute_without_a_device(B):
    """there is no CPU path: creating a System needs the initialised device"""
    from conftest import has_gpu
    if has_gpu():
        pytest.skip("a device is present")
    assert not B.initialized()
    with pytest.raises(RuntimeError):
        B.initialize(0)
    m = B.Model(model_path("grace_1l_order3"))
    with pytest.raises(RuntimeError, match="not initialised"):
        B.System(m, ["W"])


def test_order3_file_has_no_order4_arrays():
    z = np.load(model_path("grace_1l_order3"))
    assert not any("AAAA" in k for k in z.files)


class _FakeDeviceArray:
    """stands in for a torch / CuPy array: only the attributes the binding reads"""

    def __init__(self, shape, typestr, strides=None, ptr=0x7f0000000000):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False),
                                         "strides": strides, "version": 3}


def test_device_array_arguments_are_checked_not_converted(B):
    """argument rules of the reference's compute_device (python/kk/kk_module.cpp:142-197, `noconvert`): the binding
    takes the address of a device array as it is, or refuses it"""
    import torch
    ok = _FakeDeviceArray((5, 3), "<f8")
    assert B._dev_ptr(ok, "positions", np.float64, (5, 3)).value == 0x7f0000000000
    assert B._dev_ptr(_FakeDeviceArray((5, 3), "<f8", strides=(24, 8)), "positions", np.float64, (5, 3)).value
    with pytest.raises(ValueError, match="dtype"):
        B._dev_ptr(_FakeDeviceArray((5, 3), "<f4"), "positions", np.float64, (5, 3))
    with pytest.raises(ValueError, match="shape"):
        B._dev_ptr(_FakeDeviceArray((5, 2), "<f8"), "positions", np.float64, (5, 3))
    with pytest.raises(ValueError, match="contiguous"):
        B._dev_ptr(_FakeDeviceArray((5, 3), "<f8", strides=(48, 8)), "positions", np.float64, (5, 3))
    with pytest.raises(ValueError, match="device array"):
        B._dev_ptr(np.zeros((5, 3)), "positions", np.float64, (5, 3))
    with pytest.raises(ValueError, match="GPU"):       # a DLPack producer on the host
        B._dev_ptr(torch.zeros((5, 3), dtype=torch.float64), "positions", np.float64, (5, 3))
    assert B._dev_ptr(None, "forces", np.float64, (5, 3), optional=True) is None
    with pytest.raises(ValueError):
        B._dev_ptr(None, "energy", np.float64, (1,))
