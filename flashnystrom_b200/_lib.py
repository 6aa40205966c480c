"""ctypes binding of the C ABI declared in include/flashnystrom_b200.h.

The shared library is built in-tree (flashnystrom_b200/lib/).  Loading never falls back to
another implementation: if the library is missing and cannot be built, import of the
compute entry points raises."""
import ctypes as C
import os
import threading

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libflashnystrom_b200.so")

FNB_F32, FNB_F16, FNB_BF16 = 0, 1, 2
FNB_FLAG_FORCE_GENERIC = 1
FNB_FLAG_TEST_DROP_LOAD = 0x100
FNB_LAYOUT_BHND, FNB_LAYOUT_BNHD = 0, 1


class Shape(C.Structure):
    _fields_ = [("batch", C.c_int64), ("heads", C.c_int64), ("seq_len", C.c_int64),
                ("head_dim", C.c_int32), ("num_landmarks", C.c_int32),
                ("newton_iter", C.c_int32), ("dtype", C.c_int32),
                ("kappa_star", C.c_float), ("flags", C.c_uint32),
                ("layout", C.c_int32), ("reserved", C.c_int32)]


class FwdArgs(C.Structure):
    _fields_ = [("shape", Shape),
                ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
                ("lse1", C.c_void_p), ("q_landmarks", C.c_void_p), ("k_landmarks", C.c_void_p),
                ("k2", C.c_void_p), ("lse2", C.c_void_p), ("ns_iterates", C.c_void_p),
                ("k2_inv", C.c_void_p), ("bmat", C.c_void_p), ("lse3", C.c_void_p),
                ("step2", C.c_void_p),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
                ("device", C.c_int32), ("stream", C.c_void_p), ("device_status", C.c_void_p)]


class BwdArgs(C.Structure):
    _fields_ = [("shape", Shape),
                ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("d_out", C.c_void_p),
                ("lse1", C.c_void_p), ("q_landmarks", C.c_void_p), ("k_landmarks", C.c_void_p),
                ("k2", C.c_void_p), ("ns_iterates", C.c_void_p), ("k2_inv", C.c_void_p),
                ("bmat", C.c_void_p), ("lse3", C.c_void_p), ("step2", C.c_void_p),
                ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
                ("device", C.c_int32), ("stream", C.c_void_p), ("device_status", C.c_void_p)]


class SpInfo(C.Structure):
    _fields_ = [("rank", C.c_int32), ("world", C.c_int32), ("stage", C.c_int32),
                ("seq_len_global", C.c_int64), ("xfer", C.c_void_p), ("xfer_floats", C.c_size_t)]


class Caps(C.Structure):
    _fields_ = [("abi_version", C.c_int32), ("cc_major", C.c_int32), ("cc_minor", C.c_int32),
                ("sm_count", C.c_int32), ("max_smem_per_block", C.c_int32),
                ("l2_bytes", C.c_int64), ("total_mem_bytes", C.c_int64)]


class KernelTime(C.Structure):
    _fields_ = [("name", C.c_char * 48), ("ms", C.c_float)]


class KernelInfo(C.Structure):
    _fields_ = [("name", C.c_char * 48), ("registers", C.c_int32), ("static_smem_bytes", C.c_int32),
                ("dynamic_smem_bytes", C.c_int32), ("local_bytes_per_thread", C.c_int32),
                ("threads", C.c_int32), ("blocks_per_sm", C.c_int32)]


class ConvArgs(C.Structure):
    _fields_ = [("batch", C.c_int64), ("heads", C.c_int64), ("seq_len", C.c_int64),
                ("head_dim", C.c_int32), ("kernel_size", C.c_int32), ("dtype", C.c_int32), ("layout", C.c_int32),
                ("v", C.c_void_p), ("base", C.c_void_p), ("result", C.c_void_p), ("weight", C.c_void_p),
                ("transposed", C.c_int32), ("device", C.c_int32), ("stream", C.c_void_p)]


class ConvDwArgs(C.Structure):
    _fields_ = [("batch", C.c_int64), ("heads", C.c_int64), ("seq_len", C.c_int64),
                ("head_dim", C.c_int32), ("kernel_size", C.c_int32), ("dtype", C.c_int32), ("layout", C.c_int32),
                ("v", C.c_void_p), ("d_out", C.c_void_p), ("d_weight", C.c_void_p),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
                ("device", C.c_int32), ("stream", C.c_void_p)]


# every symbol include/flashnystrom_b200.h declares, with its ctypes signature
SIGNATURES = {
    "fnb_last_error": (C.c_char_p, []),
    "fnb_version": (C.c_int, []),
    "fnb_capabilities": (C.c_int, [C.c_int, C.POINTER(Caps)]),
    "fnb_fwd_workspace_bytes": (C.c_size_t, [C.POINTER(Shape)]),
    "fnb_bwd_workspace_bytes": (C.c_size_t, [C.POINTER(Shape)]),
    "fnb_check_shape": (C.c_int, [C.POINTER(Shape)]),
    "fnb_forward": (C.c_int, [C.POINTER(FwdArgs)]),
    "fnb_backward": (C.c_int, [C.POINTER(BwdArgs)]),
    "fnb_sp_xfer_floats": (C.c_size_t, [C.POINTER(Shape), C.c_int, C.c_int, C.c_int]),
    "fnb_sp_forward": (C.c_int, [C.POINTER(FwdArgs), C.POINTER(SpInfo)]),
    "fnb_sp_backward": (C.c_int, [C.POINTER(BwdArgs), C.POINTER(SpInfo)]),
    "fnb_debug_pinv_forward": (C.c_int, [C.c_int64, C.c_int32, C.c_int32, C.c_float, C.c_void_p,
                                         C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                                         C.c_int32, C.c_void_p]),
    "fnb_debug_pinv_backward": (C.c_int, [C.c_int64, C.c_int32, C.c_int32, C.c_float, C.c_void_p,
                                          C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                          C.c_size_t, C.c_int32, C.c_void_p]),
    "fnb_pinv_backward_noalloc": (C.c_int, [C.c_int64, C.c_int32, C.c_int32, C.c_float, C.c_void_p,
                                            C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "fnb_debug_pinv_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int32]),
    "fnb_debug_set_wait_limit_ms": (C.c_int, [C.c_int, C.c_int]),
    "fnb_debug_ns_bwd_step": (C.c_int, [C.c_int64, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_void_p, C.c_int32, C.c_void_p]),
    "fnb_debug_ns_bwd_final": (C.c_int, [C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_int32, C.c_void_p]),
    "fnb_kernel_report": (C.c_int, [C.c_int, C.POINTER(KernelInfo), C.c_int]),
    "fnb_conv_residual": (C.c_int, [C.POINTER(ConvArgs)]),
    "fnb_conv_dweight_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int64, C.c_int32]),
    "fnb_conv_residual_dweight": (C.c_int, [C.POINTER(ConvDwArgs)]),
    "fnb_set_profiling": (C.c_int, [C.c_int]),
    "fnb_last_profile": (C.c_int, [C.POINTER(KernelTime), C.c_int]),
}

_lock = threading.Lock()
_lib = None


def load(build_if_missing=True):
    """Return the loaded library, building it with nvcc first if it is absent."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            if not build_if_missing:
                raise ImportError(f"{LIB_PATH} not found; run python -m flashnystrom_b200.build")
            from . import build as _build
            _build.build()
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
        return lib


def last_error():
    return load().fnb_last_error().decode("utf-8", "replace")


def check(rc):
    if rc != 0:
        raise RuntimeError(f"flashnystrom_b200: {last_error()} (status {rc})")
