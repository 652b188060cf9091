"""ctypes binding of libfdp_b200.so (the C ABI declared in include/fdp_b200.h).

There is no fallback: if the library is missing or the device is not a B200, calls raise.
"""
import ctypes
import os

PKG = os.path.dirname(os.path.abspath(__file__))
# FDP_B200_LIB points at another build of the same ABI (used to compare builds on one GPU)
LIB_PATH = os.environ.get("FDP_B200_LIB") or os.path.join(PKG, "libfdp_b200.so")

ABI_VERSION = 3
FDP_OK = 0
FDP_ERR_ARG, FDP_ERR_DTYPE, FDP_ERR_SHAPE, FDP_ERR_ALIGN = -1, -2, -3, -4
FDP_ERR_WORKSPACE, FDP_ERR_ARCH, FDP_ERR_LAUNCH, FDP_ERR_TIMEOUT = -5, -6, -7, -8
FDP_ERR_STATIC_LIMIT = -9
FDP_STATIC_SCRATCH_BYTES = 8 << 20
FDP_F32, FDP_BF16, FDP_F16 = 0, 1, 2
FDP_OUT_IN, FDP_IN_OUT = 0, 1
FDP_NORM_AUTO, FDP_NORM_DIRECT, FDP_NORM_GRAM = 0, 1, 2
FDP_FP32_TENSOR = 16

c_void_p, c_int, c_size_t, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_float


class DPParams(ctypes.Structure):
    """struct fdp_dp_params"""
    _fields_ = [("C", c_float), ("clamp_value", c_float), ("noise_std", c_float),
                ("batch_divisor", ctypes.c_int32), ("seed", ctypes.c_uint64),
                ("param_id", ctypes.c_uint32), ("param_id2", ctypes.c_uint32),
                ("step", ctypes.c_uint32), ("noise_rank", ctypes.c_int32),
                ("noise_world", ctypes.c_int32), ("step_device", c_void_p)]


# name -> (restype, argtypes); every function include/fdp_b200.h declares
SIGNATURES = {
    "fdp_abi_version": (c_int, []),
    "fdp_status_string": (ctypes.c_char_p, [c_int]),
    "fdp_check_device": (c_int, [c_int]),
    "fdp_device_status": (c_int, [c_void_p, c_void_p]),
    "fdp_async_status": (c_int, [c_int]),
    "fdp_clear_async_status": (c_int, [c_int]),
    "fdp_selftest_wait_timeout": (c_int, [ctypes.c_longlong, c_void_p, c_size_t, c_void_p]),
    "fdp_set_sm_reserve": (c_int, [c_int]),
    "fdp_launch_count": (ctypes.c_ulonglong, []),
    "fdp_profile_enable": (c_int, [c_int]),
    "fdp_profile_read": (c_int, [ctypes.POINTER(c_float), c_int]),
    "fdp_linear_wgrad_workspace_bytes": (c_size_t, [c_int] * 6),
    "fdp_linear_wgrad": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 8 +
                         [ctypes.POINTER(DPParams), c_void_p, c_size_t, c_void_p]),
    "fdp_bias_grad_workspace_bytes": (c_size_t, [c_int] * 4),
    "fdp_bias_grad": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 5 +
                      [ctypes.POINTER(DPParams), c_void_p, c_size_t, c_void_p]),
    "fdp_bias_grad_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 5 +
                             [ctypes.POINTER(DPParams), c_void_p]),
    "fdp_linear_dgrad_workspace_bytes": (c_size_t, [c_int] * 4),
    "fdp_linear_dgrad": (c_int, [c_void_p, c_void_p, c_void_p] + [c_int] * 6 +
                         [c_void_p, c_size_t, c_void_p]),
    "fdp_linear_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 6 +
                       [c_void_p, c_size_t, c_void_p]),
    "fdp_layernorm_fwd": (c_int, [c_void_p] * 6 + [c_int, c_int, c_float, c_int, c_int, c_void_p]),
    "fdp_layernorm_bwd_workspace_bytes": (c_size_t, [c_int] * 3),
    "fdp_layernorm_saturate_workspace_bytes": (c_size_t, [c_int, c_int]),
    "fdp_layernorm_saturate_groups": (c_int, [c_int, c_int]),
    "fdp_layernorm_bwd_saturate": (c_int, [c_void_p] * 6 + [c_int] * 4 + [c_float, c_float, c_void_p, c_size_t, c_void_p]),
    "fdp_layernorm_bwd": (c_int, [c_void_p] * 10 + [c_int] * 5 +
                          [ctypes.POINTER(DPParams), c_void_p, c_size_t, c_void_p]),
}

_lib = None


def load():
    """Load the shared library (once) and attach the signatures."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m flashdp4review_b200.build` "
                "(needs nvcc; there is no CPU or PyTorch fallback for the DP kernels)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        if lib.fdp_abi_version() != ABI_VERSION:
            raise ImportError("libfdp_b200.so: ABI version mismatch, rebuild the library")
        _lib = lib
    return _lib


_EXC = {FDP_ERR_ARG: ValueError, FDP_ERR_DTYPE: KeyError, FDP_ERR_SHAPE: RuntimeError,
        FDP_ERR_ALIGN: RuntimeError, FDP_ERR_WORKSPACE: RuntimeError, FDP_ERR_ARCH: RuntimeError,
        FDP_ERR_LAUNCH: RuntimeError, FDP_ERR_TIMEOUT: RuntimeError}


def check(status, what):
    """Map a status code to the exception class the reference raises for that kind of error
    (KeyError for an unsupported dtype -- flashdp/core/bmtm_clip_loop.py:139-142; RuntimeError
    for shapes -- flashdp/layers/linear.py:97-102; ValueError for bad arguments)."""
    if status != FDP_OK:
        msg = load().fdp_status_string(status).decode()
        raise _EXC.get(status, RuntimeError)(f"{what}: {msg} (status {status})")
