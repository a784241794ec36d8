"""ctypes binding of libgrace_b200.so with the module interface of the reference's GPU plug-in `_kk_<arch>`
(python/kk/kk_module.cpp:200-275): initialize / finalize / arch / platform / memory_info, and the classes Model,
System and Batch with the same argument names, defaults, result dicts and exception classes (ValueError for
std::invalid_argument, RuntimeError otherwise; MemoryError is not used by the reference, out-of-memory is a
RuntimeError there too).

There is no CPU path: importing works anywhere (so that the symbols can be checked), but every call that needs the
device fails unless libgrace_b200.so is built and a B200 is present.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

ABI = 7
_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libgrace_b200.so")
_lib = None

FLAG_ENERGIES, FLAG_ENERGY_ONLY, FLAG_UQ = 1, 2, 4

# name -> (restype, argtypes); the symbols include/grace_b200.h declares
_P, _I, _D, _I64 = C.c_void_p, C.c_int, C.c_double, C.c_int64
SIGNATURES = {
    "grace_initialize": (_I, [_I]),
    "grace_finalize": (_I, []),
    "grace_initialized": (_I, []),
    "grace_device": (_I, []),
    "grace_arch": (C.c_char_p, []),
    "grace_platform": (C.c_char_p, []),
    "grace_blas": (C.c_char_p, []),
    "grace_abi": (_I, []),
    "grace_memory_info": (_I, [_P, _P]),
    "grace_debug_fail_alloc": (_I, [C.c_char_p, _I]),
    "grace_debug_fail_launch": (_I, [_I]),
    "grace_measure_peak": (_I, [_I, _P]),
    "grace_debug_track_alloc": (_I, [_I]),
    "grace_debug_peak_alloc": (C.c_uint64, []),
    "grace_debug_live_alloc": (_I, [_P, C.c_size_t]),
    "grace_last_error": (C.c_char_p, []),
    "grace_kernel_launches": (C.c_uint64, []),
    "grace_profile_enable": (_I, [_I]),
    "grace_profile_report": (_I, [_P, C.c_size_t]),
    "grace_sum_rows_static": (_I, [_P, _I64, _I, _P]),
    "grace_model_load": (_I, [C.c_char_p, _I, _P]),
    "grace_model_layers": (_I, [_P]),
    "grace_model_has_uq": (_I, [_P]),
    "grace_model_validate_uq": (_I, [_P]),
    "grace_system_set_uq_outputs": (_I, [_P, _P, _P, _P]),
    "grace_batch_set_uq_outputs": (_I, [_P, _P, _P, _P]),
    "grace_model_n_elements": (_I, [_P]),
    "grace_model_element_name": (C.c_char_p, [_P, _I]),
    "grace_model_engine_setups": (_I64, [_P]),
    "grace_model_dense_flops": (_D, [_P]),
    "grace_model_dense_stats": (_I, [_P, _P]),
    "grace_model_radial_mlp_device": (_I, [_P, _I, _I64, _P, _P, _P]),
    "grace_model_radial_mlp_width": (_I, [_P, _I]),
    "grace_model_free": (None, [_P]),
    "grace_system_create": (_I, [_P, _P, _I, _D, _I, _I, _P]),
    "grace_system_cutoff": (_D, [_P]),
    "grace_system_compute": (_I, [_P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _P]),
    "grace_system_compute_device": (_I, [_P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _P]),
    "grace_system_set_owned": (_I, [_P, _I, _I]),
    "grace_system_set_exchange": (_I, [_P, _I, _I, _I, _P, _P, _P, _P]),
    "grace_comm_unique_id": (_I, [_P]),
    "grace_comm_init": (_I, [_P, _I, _I]),
    "grace_comm_finalize": (_I, []),
    "grace_comm_rank": (_I, []),
    "grace_comm_size": (_I, []),
    "grace_system_neighbor_list": (_I, [_P, _I64, _P, _P, _P, _P]),
    "grace_system_rebuilds": (_I64, [_P]),
    "grace_system_chunksize": (_I, [_P]),
    "grace_system_release_buffers": (_I, [_P]),
    "grace_system_stage_ms": (_I, [_P, _P]),
    "grace_system_free": (None, [_P]),
    "grace_engine_create": (_I, [_P, _P, _I, _I, _I, _P]),
    "grace_engine_cutoff": (_D, [_P]),
    "grace_engine_comm_width": (_I, [_P]),
    "grace_engine_run": (_I, [_P, _P, _P, _P, _P, _P]),
    "grace_engine_free": (None, [_P]),
    "grace_batch_create": (_I, [_P, _P, _I, _I, _I, _P]),
    "grace_batch_cutoff": (_D, [_P]),
    "grace_batch_compute": (_I, [_P, _I, _P, _I64, _P, _P, _P, _P, _I, _I64, _P, _P, _P, _P]),
    "grace_batch_compute_device": (_I, [_P, _I, _P, _I64, _P, _P, _P, _P, _I, _I64, _P, _P, _P, _P]),
    "grace_batch_passes": (_I, [_P]),
    "grace_batch_host_seconds": (_D, [_P]),
    "grace_batch_set_keep_buffers": (_I, [_P, _I]),
    "grace_batch_release_buffers": (_I, [_P]),
    "grace_batch_free": (None, [_P]),
}


def load_library(path=None):
    """Loads libgrace_b200.so (built by grace_runtime_b200/build.py) and declares every entry point; raises
    RuntimeError if the library is missing - there is nothing to fall back to."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise RuntimeError(f"{p} is not built: run `python -m grace_runtime_b200.build` (needs nvcc); this backend "
                           "has no CPU path")
    lib = C.CDLL(p)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)    # AttributeError: a symbol of the header is missing from the library
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def _check(rc):
    if rc == 0:
        return
    msg = _lib.grace_last_error().decode(errors="replace")
    if rc == 1:
        raise ValueError(msg)
    raise RuntimeError(msg)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _len_of(a, name):
    cai = getattr(a, "__cuda_array_interface__", None)
    if cai is not None:
        return int(cai["shape"][0])
    if hasattr(a, "shape"):
        return int(a.shape[0])
    raise ValueError(f"{name}: the atom count must be given with raw device addresses")


def _names(species):
    arr = (C.c_char_p * len(species))(*[str(s).encode() for s in species])
    return arr


# ---- module-level functions of the plug-in -----------------------------------------------------------------------
def initialize(device=0):
    _check(load_library().grace_initialize(int(device)))


def finalize():
    _check(load_library().grace_finalize())


def initialized():
    return bool(load_library().grace_initialized())


def device():
    return load_library().grace_device()


def arch():
    return load_library().grace_arch().decode()


def archs():
    return ["sm100"]


def platform():
    return load_library().grace_platform().decode()


def blas():
    return load_library().grace_blas().decode()


def cublas():
    return False


def memory_info():
    f, t = C.c_size_t(0), C.c_size_t(0)
    _check(load_library().grace_memory_info(C.addressof(f), C.addressof(t)))
    return f.value, t.value


def kernel_launches():
    return int(load_library().grace_kernel_launches())


def sum_rows_static(d_values, n, k, d_out):
    """Column sums of the device matrix values[n][k] (doubles, row-major; device addresses as integers) into the
    device array out[k], with no device allocation: the partial sums use a static device array shared by all calls
    (k <= 8, n <= 16,777,216; beyond that ValueError).  No counterpart in the reference."""
    _check(load_library().grace_sum_rows_static(C.c_void_p(int(d_values)), int(n), int(k), C.c_void_p(int(d_out))))


def profile_enable(on=True):
    """CUDA events around every kernel launch of the library from now on (off: drop them)."""
    _check(load_library().grace_profile_enable(int(bool(on))))


def profile_report():
    """{kernel name: (launches, total device ms)} since profile_enable(True)."""
    buf = C.create_string_buffer(1 << 16)
    _check(load_library().grace_profile_report(buf, len(buf)))
    out = {}
    for line in buf.value.decode().splitlines():
        name, n, ms = line.rsplit(" ", 2)
        out[name] = (int(n), float(ms))
    return out


def _debug_fail_alloc(label, nth):
    _check(load_library().grace_debug_fail_alloc(str(label).encode(), int(nth)))


def _debug_fail_launch(nth):
    _check(load_library().grace_debug_fail_launch(int(nth)))


def comm_unique_id():
    """128 bytes made by rank 0 that every rank passes to comm_init (send them with any transport)."""
    buf = C.create_string_buffer(128)
    _check(load_library().grace_comm_unique_id(buf))
    return buf.raw


def comm_init(unique_id, rank, world):
    """Joins the library's NCCL communicator (collective; after initialize(device))."""
    if len(unique_id) != 128:
        raise ValueError("the unique id has 128 bytes")
    _check(load_library().grace_comm_init(C.c_char_p(bytes(unique_id)), int(rank), int(world)))


def comm_finalize():
    _check(load_library().grace_comm_finalize())


def comm_rank():
    return load_library().grace_comm_rank()


def comm_size():
    return load_library().grace_comm_size()


def measure_peak(kind):
    """TFLOP/s of a microbenchmark on the module's GPU: "fp32" (SIMT FMA lanes), "tf32" (tcgen05 tensor cores, M = 128,
    N = 256) or an int N (the tf32 one with that N)."""
    v = C.c_double(0.0)
    _check(load_library().grace_measure_peak({"fp32": 0, "tf32": 1}.get(kind, kind), C.addressof(v)))
    return v.value


def _debug_track_alloc(on):
    """From now on (True) every device allocation of the library is recorded by label; False stops and forgets."""
    _check(load_library().grace_debug_track_alloc(int(bool(on))))


def _debug_peak_alloc():
    """High-water mark in bytes of the device allocations made since _debug_track_alloc(True)."""
    return int(load_library().grace_debug_peak_alloc())


def _debug_live_alloc():
    """[(label, bytes)] of the tracked allocations still alive, largest first."""
    buf = C.create_string_buffer(1 << 16)
    _check(load_library().grace_debug_live_alloc(buf, len(buf)))
    out = []
    for line in buf.value.decode().splitlines():
        name, b = line.rsplit("\t", 1)
        out.append((name, int(b)))
    return out


# ---- device arrays -----------------------------------------------------------------------------------------------
# The reference's compute_device takes DLPack arrays of the module's GPU "without implicit conversion: a converted
# output would be a temporary copy (results lost), a converted input a hidden host -> device copy per call"
# (python/kk/kk_module.cpp:142-197,258-266).  Here an argument may be an object with __cuda_array_interface__ (torch,
# CuPy, numba), an object with __dlpack__ (its capsule is read with ctypes), or - an extension - a raw device address
# as int.  Host arrays are refused with ValueError; nothing is ever copied or cast.
_KDLCUDA = 2
_TYPESTR = {np.dtype(np.float64): "<f8", np.dtype(np.int32): "<i4"}


class _DLDevice(C.Structure):
    _fields_ = [("device_type", C.c_int), ("device_id", C.c_int)]


class _DLDataType(C.Structure):
    _fields_ = [("code", C.c_uint8), ("bits", C.c_uint8), ("lanes", C.c_uint16)]


class _DLTensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("device", _DLDevice), ("ndim", C.c_int), ("dtype", _DLDataType),
                ("shape", C.POINTER(C.c_int64)), ("strides", C.POINTER(C.c_int64)), ("byte_offset", C.c_uint64)]


class _DLManagedTensor(C.Structure):
    pass


_DLManagedTensor._fields_ = [("dl_tensor", _DLTensor), ("manager_ctx", C.c_void_p),
                             ("deleter", C.CFUNCTYPE(None, C.POINTER(_DLManagedTensor)))]


def _c_contiguous(shape, strides, itemsize, in_bytes):
    if strides is None:
        return True
    want = itemsize if in_bytes else 1
    for n, st in zip(reversed(shape), reversed(strides)):
        if n > 1 and st != want:
            return False
        want *= max(n, 1)
    return True


def _from_dlpack(a, name, dtype, shape):
    cap = a.__dlpack__()
    api = C.pythonapi
    api.PyCapsule_GetPointer.restype = C.c_void_p
    api.PyCapsule_GetPointer.argtypes = [C.py_object, C.c_char_p]
    api.PyCapsule_SetName.argtypes = [C.py_object, C.c_char_p]
    p = api.PyCapsule_GetPointer(cap, b"dltensor")
    if not p:
        raise ValueError(f"{name}: not a DLPack capsule")
    mt = C.cast(p, C.POINTER(_DLManagedTensor))
    t = mt.contents.dl_tensor
    try:
        if t.device.device_type != _KDLCUDA or t.device.device_id != device():
            raise ValueError(f"{name} must be on the module's GPU (cuda:{device()})")
        code = {np.dtype(np.float64): (2, 64), np.dtype(np.int32): (0, 32)}[np.dtype(dtype)]
        if (t.dtype.code, t.dtype.bits, t.dtype.lanes) != (code[0], code[1], 1):
            raise ValueError(f"{name} must have dtype {np.dtype(dtype).name} (no conversion is made)")
        shp = tuple(int(t.shape[k]) for k in range(t.ndim))
        if shp != tuple(shape):
            raise ValueError(f"{name}: wrong shape {shp}, expected {tuple(shape)}")
        strides = None if not t.strides else tuple(int(t.strides[k]) for k in range(t.ndim))
        if not _c_contiguous(shp, strides, 1, False):
            raise ValueError(f"{name} must be C-contiguous")
        return int(t.data or 0) + int(t.byte_offset)
    finally:    # the capsule was consumed: run its deleter now; the producer `a` stays alive in the caller
        api.PyCapsule_SetName(cap, b"used_dltensor")
        if mt.contents.deleter:
            mt.contents.deleter(mt)


def _dev_ptr(a, name, dtype, shape, optional=False):
    """Device address of `a` after the checks of the reference binding (device, dtype, shape, contiguity)."""
    if a is None:
        if optional:
            return None
        raise ValueError(f"{name} must be given")
    if isinstance(a, (int, np.integer)):
        if int(a) == 0 and optional:
            return None
        return C.c_void_p(int(a))
    cai = getattr(a, "__cuda_array_interface__", None)
    if cai is not None:
        if cai.get("typestr") != _TYPESTR[np.dtype(dtype)]:
            raise ValueError(f"{name} must have dtype {np.dtype(dtype).name} (no conversion is made)")
        if tuple(cai["shape"]) != tuple(shape):
            raise ValueError(f"{name}: wrong shape {tuple(cai['shape'])}, expected {tuple(shape)}")
        if not _c_contiguous(tuple(cai["shape"]), cai.get("strides"), np.dtype(dtype).itemsize, True):
            raise ValueError(f"{name} must be C-contiguous")
        dv = getattr(a, "device", None)
        idx = getattr(dv, "index", getattr(dv, "id", None))
        if idx is not None and int(idx) != device():
            raise ValueError(f"{name} must be on the module's GPU (cuda:{device()})")
        return C.c_void_p(int(cai["data"][0]))
    if hasattr(a, "__dlpack__") and not isinstance(a, np.ndarray):
        return C.c_void_p(_from_dlpack(a, name, dtype, shape))
    raise ValueError(f"{name} must be a device array of the module's GPU (DLPack / __cuda_array_interface__); host "
                     "arrays are not converted")


# ---- classes -----------------------------------------------------------------------------------------------------
class Model:
    """A loaded GRACE-1L / GRACE-2L kokkos.npz (kk_api.h:51-64)."""

    def __init__(self, path, spline=1024, asi=""):
        if asi:
            raise ValueError("active-set files belong to PACE models, which this backend does not evaluate")
        lib = load_library()
        h = C.c_void_p()
        _check(lib.grace_model_load(os.fsencode(path), int(spline), C.addressof(h)))
        self._h = h
        self.spline = int(spline)

    def __del__(self):
        if getattr(self, "_h", None) and _lib is not None:
            _lib.grace_model_free(self._h)
            self._h = None

    @property
    def layers(self):
        return _lib.grace_model_layers(self._h)

    @property
    def has_uq(self):
        return bool(_lib.grace_model_has_uq(self._h))

    @property
    def slow_notice(self):
        return ""

    @property
    def needs_generic(self):
        return False

    @property
    def element_names(self):
        return [_lib.grace_model_element_name(self._h, i).decode() for i in range(_lib.grace_model_n_elements(self._h))]

    @property
    def engine_setups(self):
        return int(_lib.grace_model_engine_setups(self._h))

    @property
    def dense_stats(self):
        """per atom on the per-operation path: dict of (flops, bytes) for the tensor-core operations, the products and
        the per-element operations (see grace_model_dense_stats)"""
        v = np.zeros(6)
        _check(_lib.grace_model_dense_stats(self._h, _ptr(v)))
        return {"tensor": (v[0], v[1]), "products": (v[2], v[3]), "elementwise": (v[4], v[5])}

    @property
    def dense_flops(self):
        """fp32 flops per atom of the dense network (forward + reverse) in the engine's plan; 0 before the first System"""
        return float(_lib.grace_model_dense_flops(self._h))

    def radial_mlp_width(self, layer=1):
        return int(_lib.grace_model_radial_mlp_width(self._h, int(layer)))

    def radial_mlp_device(self, layer, nb, x_ptr, R_ptr, dR_ptr):
        """Exact radial MLP of a layer on the tensor cores: device pointers to x [nb] and the outputs [nb, width]."""
        _check(_lib.grace_model_radial_mlp_device(self._h, int(layer), int(nb), C.c_void_p(x_ptr), C.c_void_p(R_ptr),
                                                  C.c_void_p(dR_ptr)))

    def validate_uq(self):
        """ValueError unless the UQ head of the file can be evaluated (python/kk/kk_api.h:59)."""
        _check(_lib.grace_model_validate_uq(self._h))


def _as(a, dtype, shape=None):
    a = np.ascontiguousarray(a, dtype=dtype)
    if shape is not None and a.shape != shape:
        raise ValueError(f"array of shape {a.shape}, expected {shape}")
    return a


class System:
    """One structure on the device with a Verlet-skin neighbour list (kk_api.h:68-90)."""

    def __init__(self, model, species, skin=0.5, spline=1024, chunksize=-1):
        lib = load_library()
        h = C.c_void_p()
        self._model = model
        _check(lib.grace_system_create(model._h, _names(species), len(species), float(skin), int(spline),
                                       int(chunksize), C.addressof(h)))
        self._h = h

    def __del__(self):
        if getattr(self, "_h", None) and _lib is not None:
            _lib.grace_system_free(self._h)
            self._h = None

    @property
    def cutoff(self):
        return _lib.grace_system_cutoff(self._h)

    @property
    def rebuilds(self):
        return int(_lib.grace_system_rebuilds(self._h))

    @property
    def chunksize(self):
        return _lib.grace_system_chunksize(self._h)

    @property
    def stage_ms(self):
        ms = np.zeros(5)
        _lib.grace_system_stage_ms(self._h, _ptr(ms))
        return dict(neighbor_list=ms[0], bonds=ms[1], forward=ms[2], reverse=ms[3], total=ms[4])

    def release_buffers(self):
        _check(_lib.grace_system_release_buffers(self._h))

    def set_owned(self, nlocal, ninner=-1):
        """Atoms [0, nlocal) are owned, the rest are ghosts of a domain decomposition (-1: all owned); ghosts behind
        ninner only serve as neighbours (GRACE-2L: ghosts no owned atom has inside cutoff + skin)."""
        _check(_lib.grace_system_set_owned(self._h, int(nlocal), int(ninner)))

    def set_exchange(self, n, nlocal, ninner, send_counts, send_index, recv_counts, recv_index):
        """Domain decomposition over the library's communicator (comm_init): as set_owned, and every compute returns
        the ghost force rows to their owners and sums energy and virial over the ranks (collective)."""
        sc, si = _as(send_counts, np.int32), _as(send_index, np.int32)
        rc, ri = _as(recv_counts, np.int32), _as(recv_index, np.int32)
        _check(_lib.grace_system_set_exchange(self._h, int(n), int(nlocal), int(ninner), _ptr(sc), _ptr(si), _ptr(rc), _ptr(ri)))

    def compute(self, types, positions, cell, pbc, energies=False, uq=False, energy_only=False):
        """Result dict as python/kk/kk_module.cpp `compute`: energy, virial [6], forces [n, 3] (not with energy_only),
        energies [n] (when asked), gamma / total_sigma / atomic_sigma / gmm_cluster (with uq)."""
        types = _as(types, np.int32)
        n = len(types)
        positions = _as(positions, np.float64, (n, 3))
        cell = _as(cell, np.float64, (3, 3))
        pbc = _as(np.asarray(pbc).astype(bool), np.uint8, (3,))
        flags = (FLAG_ENERGIES if energies else 0) | (FLAG_ENERGY_ONLY if energy_only else 0) | (FLAG_UQ if uq else 0)
        e = np.zeros(1)
        v = np.zeros(6)
        f = None if energy_only else np.zeros((n, 3))
        ea = np.zeros(n) if energies else None
        if uq:
            g, sg, cl = np.zeros(n), np.zeros(n), np.zeros(n)
            _check(_lib.grace_system_set_uq_outputs(self._h, _ptr(g), _ptr(sg), _ptr(cl)))
        try:
            _check(_lib.grace_system_compute(self._h, n, _ptr(types), _ptr(positions), _ptr(cell), _ptr(pbc), flags,
                                             _ptr(e), None if energy_only else _ptr(v), _ptr(f), _ptr(ea)))
        finally:
            if uq:
                _lib.grace_system_set_uq_outputs(self._h, None, None, None)
        r = {"energy": float(e[0])}
        if uq:      # keys of python/kk/kk_module.cpp:72-78
            r.update(gamma=g, total_sigma=float(sg.sum()), atomic_sigma=sg, gmm_cluster=cl)
        if not energy_only:
            r["forces"] = f
            r["virial"] = v
        if energies:
            r["energies"] = ea
        return r

    def compute_device(self, types, positions, cell, pbc, energy, forces=None, virial=None, energies=None,
                       energy_only=False, n=None, gamma=None, atomic_sigma=None, gmm_cluster=None):
        """Device inputs and outputs, no copies (an extension: the reference has compute_device on Batch only; same
        argument rules): types int32 [n], positions float64 [n, 3], energy float64 [1], forces [n, 3], virial [6],
        energies [n] on the module's GPU; cell and pbc on the host.  Raw device addresses (int) need `n`."""
        if n is None:
            n = _len_of(types, "types")
        n = int(n)
        cell = _as(cell, np.float64, (3, 3))
        pbc = _as(np.asarray(pbc).astype(bool), np.uint8, (3,))
        e = _dev_ptr(energy, "energy", np.float64, (1,))
        f = _dev_ptr(forces, "forces", np.float64, (n, 3), optional=True)
        v = _dev_ptr(virial, "virial", np.float64, (6,), optional=True)
        ea = _dev_ptr(energies, "energies", np.float64, (n,), optional=True)
        flags = (FLAG_ENERGIES if ea else 0) | (FLAG_ENERGY_ONLY if energy_only else 0)
        uq = [_dev_ptr(a, k, np.float64, (n,), optional=True)
              for a, k in ((gamma, "gamma"), (atomic_sigma, "atomic_sigma"), (gmm_cluster, "gmm_cluster"))]
        if any(uq):
            flags |= FLAG_UQ
            _check(_lib.grace_system_set_uq_outputs(self._h, *uq))
        try:
            _check(_lib.grace_system_compute_device(self._h, n, _dev_ptr(types, "types", np.int32, (n,)),
                                                    _dev_ptr(positions, "positions", np.float64, (n, 3)), _ptr(cell),
                                                    _ptr(pbc), flags, e, v, f, ea))
        finally:
            if any(uq):
                _lib.grace_system_set_uq_outputs(self._h, None, None, None)

    def neighbor_list(self):
        """Diagnostics: the device neighbour list of the last build (radius cutoff + skin) as (i, j, S [nb, 3]) in the
        caller's atom order; bond vector = x_j - x_i + S @ cell."""
        cnt = C.c_int64(0)
        _check(_lib.grace_system_neighbor_list(self._h, 0, None, None, None, C.addressof(cnt)))
        nb = cnt.value
        bi, bj, bs = np.zeros(nb, np.int32), np.zeros(nb, np.int32), np.zeros((nb, 3), np.int32)
        _check(_lib.grace_system_neighbor_list(self._h, nb, _ptr(bi), _ptr(bj), _ptr(bs), C.addressof(cnt)))
        return bi.astype(np.int64), bj.astype(np.int64), bs.astype(np.int64)


EXCHANGE_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p)    # (user, d_rows, width, stream)


class RunInput(C.Structure):
    """grace_run_input of include/grace_b200.h"""
    _fields_ = [("nlocal", C.c_int), ("nall", C.c_int), ("d_type", C.c_void_p), ("d_x", C.c_void_p),
                ("d_numneigh", C.c_void_p), ("d_neighbors", C.c_void_p), ("maxneigh", C.c_int), ("flags", C.c_int),
                ("forward", EXCHANGE_FN), ("reverse", EXCHANGE_FN), ("user", C.c_void_p)]


class Engine:
    """The engine interface for callers with their own neighbour list and ghost atoms (RunInput / RunOutput / Exchange of
    libgrace/include/grace/kk/grace_2l_kk.h:87-119): `run` adds forces to f [nall, 3] (ghost rows included) and per-atom
    energies to eatom [nlocal], and returns (energy, virial[6]) of the local atoms.  forward / reverse: callables
    (rows_address, width, stream_address) for the message rows of GRACE-2L."""

    def __init__(self, model, species, spline=1024, chunksize=-1):
        lib = load_library()
        h = C.c_void_p()
        self._model = model
        _check(lib.grace_engine_create(model._h, _names(species), len(species), int(spline), int(chunksize), C.addressof(h)))
        self._h = h

    def __del__(self):
        if getattr(self, "_h", None) and _lib is not None:
            _lib.grace_engine_free(self._h)
            self._h = None

    @property
    def cutoff(self):
        return _lib.grace_engine_cutoff(self._h)

    @property
    def comm_width(self):
        return _lib.grace_engine_comm_width(self._h)

    def run(self, nlocal, nall, types, x, numneigh, neighbors, maxneigh, f, eatom=None, forward=None, reverse=None,
            energy_only=False):
        errors = []

        def wrap(fn):
            def call(user, rows, width, stream):
                try:
                    fn(rows, width, stream)
                except Exception as e:      # an exception must not cross the C frames
                    errors.append(e)
            return EXCHANGE_FN(call) if fn else C.cast(None, EXCHANGE_FN)
        fw, rv = wrap(forward), wrap(reverse)
        inp = RunInput(int(nlocal), int(nall), _dev_ptr(types, "types", np.int32, (nall,)),
                       _dev_ptr(x, "x", np.float64, (nall, 3)), _dev_ptr(numneigh, "numneigh", np.int32, (nlocal,)),
                       _dev_ptr(neighbors, "neighbors", np.int32, (nlocal, maxneigh)), int(maxneigh),
                       FLAG_ENERGY_ONLY if energy_only else 0, fw, rv, None)
        e, v = np.zeros(1), np.zeros(6)
        _check(_lib.grace_engine_run(self._h, C.addressof(inp), _ptr(e), _ptr(v),
                                     _dev_ptr(f, "f", np.float64, (nall, 3), optional=energy_only),
                                     _dev_ptr(eatom, "eatom", np.float64, (nlocal,), optional=True)))
        if errors:
            raise errors[0]
        return float(e[0]), v


class Batch:
    """Many structures per engine pass (kk_api.h:92-156)."""

    def __init__(self, model, species, spline=1024, chunksize=-1):
        lib = load_library()
        h = C.c_void_p()
        self._model = model
        _check(lib.grace_batch_create(model._h, _names(species), len(species), int(spline), int(chunksize),
                                      C.addressof(h)))
        self._h = h

    def __del__(self):
        if getattr(self, "_h", None) and _lib is not None:
            _lib.grace_batch_free(self._h)
            self._h = None

    @property
    def cutoff(self):
        return _lib.grace_batch_cutoff(self._h)

    @property
    def passes(self):
        return _lib.grace_batch_passes(self._h)

    @property
    def last_host_seconds(self):
        return _lib.grace_batch_host_seconds(self._h)

    @property
    def keep_buffers(self):
        return getattr(self, "_keep", False)

    @keep_buffers.setter
    def keep_buffers(self, on):
        self._keep = bool(on)
        _check(_lib.grace_batch_set_keep_buffers(self._h, int(bool(on))))

    def release_buffers(self):
        _check(_lib.grace_batch_release_buffers(self._h))

    def compute(self, natoms, types, positions, cells, pbc, energies=False, uq=False, energy_only=False,
                max_nall=2097152, dispersion_parts=False):
        natoms = _as(natoms, np.int32)
        nsys = len(natoms)
        types = _as(types, np.int32)
        ntot = len(types)
        positions = _as(positions, np.float64, (ntot, 3))
        cells = _as(cells, np.float64, (nsys, 3, 3))
        pbc = _as(np.asarray(pbc).astype(bool), np.uint8, (nsys, 3))
        flags = (FLAG_ENERGIES if energies else 0) | (FLAG_ENERGY_ONLY if energy_only else 0) | (FLAG_UQ if uq else 0)
        e = np.zeros(nsys)
        v = np.zeros((nsys, 6))
        f = None if energy_only else np.zeros((ntot, 3))
        ea = np.zeros(ntot) if energies else None
        if uq:
            g, sg, cl = np.zeros(ntot), np.zeros(ntot), np.zeros(ntot)
            _check(_lib.grace_batch_set_uq_outputs(self._h, _ptr(g), _ptr(sg), _ptr(cl)))
        try:
            _check(_lib.grace_batch_compute(self._h, nsys, _ptr(natoms), ntot, _ptr(types), _ptr(positions),
                                            _ptr(cells), _ptr(pbc), flags, int(max_nall), _ptr(e),
                                            None if energy_only else _ptr(v), _ptr(f), _ptr(ea)))
        finally:
            if uq:
                _lib.grace_batch_set_uq_outputs(self._h, None, None, None)
        r = {"energy": e}
        if uq:      # keys of python/kk/kk_module.cpp:116-119
            r.update(gamma=g, atomic_sigma=sg, gmm_cluster=cl)
        if not energy_only:
            r["forces"] = f
            r["virial"] = v
        if energies:
            r["energies"] = ea
        return r

    def compute_device(self, natoms, types, positions, cells, pbc, energy, forces=None, virial=None, energies=None,
                       gamma=None, atomic_sigma=None, gmm_cluster=None, energy_only=False, max_nall=1 << 21,
                       dispersion_energy=None, dispersion_forces=None, dispersion_virial=None,
                       dispersion_energies=None):
        """Batch.compute_device of the reference (python/kk/kk_module.cpp:142-197,258-266): types int32 [N], positions
        float64 [N, 3] and the float64 outputs energy [S], forces [N, 3], virial [S, 6], energies [N] on the module's
        GPU, taken without conversion; natoms, cells, pbc on the host; gamma, atomic_sigma, gmm_cluster float64 [N]
        (all three or none) ask for the UQ outputs.  Dispersion outputs are not part of this backend: asking for one
        raises RuntimeError (unsupported)."""
        natoms = _as(natoms, np.int32)
        nsys = len(natoms)
        ntot = int(natoms.sum())
        if any(x is not None for x in (dispersion_energy, dispersion_forces, dispersion_virial, dispersion_energies)):
            raise RuntimeError("dispersion corrections are not part of this backend")
        cells = _as(cells, np.float64, (nsys, 3, 3))
        pbc = _as(np.asarray(pbc).astype(bool), np.uint8, (nsys, 3))
        t = _dev_ptr(types, "types", np.int32, (ntot,))
        x = _dev_ptr(positions, "positions", np.float64, (ntot, 3))
        e = _dev_ptr(energy, "energy", np.float64, (nsys,))
        f = _dev_ptr(forces, "forces", np.float64, (ntot, 3), optional=True)
        v = _dev_ptr(virial, "virial", np.float64, (nsys, 6), optional=True)
        ea = _dev_ptr(energies, "energies", np.float64, (ntot,), optional=True)
        flags = (FLAG_ENERGIES if ea else 0) | (FLAG_ENERGY_ONLY if energy_only else 0)
        uq = [_dev_ptr(a, k, np.float64, (ntot,), optional=True)
              for a, k in ((gamma, "gamma"), (atomic_sigma, "atomic_sigma"), (gmm_cluster, "gmm_cluster"))]
        if any(uq):
            flags |= FLAG_UQ
            _check(_lib.grace_batch_set_uq_outputs(self._h, *uq))
        try:
            _check(_lib.grace_batch_compute_device(self._h, nsys, _ptr(natoms), ntot, t, x, _ptr(cells), _ptr(pbc),
                                                   flags, int(max_nall), e, v, f, ea))
        finally:
            if any(uq):
                _lib.grace_batch_set_uq_outputs(self._h, None, None, None)
