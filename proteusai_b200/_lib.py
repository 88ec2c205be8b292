"""ctypes binding of libproteus_b200.so (the C ABI declared in include/proteus_b200.h).

There is no fallback: if the library is missing or an entry point reports an error, the call
raises.  Pointers are raw device addresses (``tensor.data_ptr()``), the stream is the raw
``cudaStream_t`` of PyTorch's current stream.
"""
import ctypes
import os
from ctypes import c_char_p, c_double, c_float, c_int, c_int64, c_size_t, c_uint32, c_void_p

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("PROTEUS_B200_LIB", os.path.join(_PKG, "libproteus_b200.so"))

_I64P = ctypes.POINTER(c_int64)  # host array of three element strides (z, h, n)

# name -> (restype, argtypes); mirrors include/proteus_b200.h
SIGNATURES = {
    "pai_abi_version": (c_int, []),
    "pai_status_str": (c_char_p, [c_int]),
    "pai_device_status": (c_int, [c_void_p]),
    "pai_we_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                           c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_uint32, c_uint32, c_void_p]),
    "pai_we_bwd_dk_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "pai_we_bwd_dk": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                              c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "pai_we_aniso_fwd": (c_int, [c_void_p] * 8 + [c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "pai_we_aniso_bwd_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "pai_we_aniso_bwd": (c_int, [c_void_p] * 6 + [c_size_t, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "pai_we_bwd_dk_static_max_k": (c_int, []),
    "pai_we_bwd_dk_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "pai_geoattn_plan_bytes": (c_size_t, [c_int, c_int]),
    "pai_geoattn_plan": (c_int, [c_void_p, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "pai_geoattn_schedule_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "pai_geoattn_schedule": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "pai_geoattn_fwd": (c_int, [c_void_p] * 9 + [c_int, c_void_p, c_void_p] + [c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_int,
                                c_int, c_int, c_int, c_int, c_void_p]),
    "pai_geoattn_fwd_strided": (c_int, [c_void_p, _I64P, c_void_p, _I64P, c_void_p, _I64P] + [c_void_p] * 6 + [c_int, c_void_p] + [_I64P, c_void_p] +
                                [c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "pai_geoattn_bwd_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "pai_geoattn_bwd": (c_int, [c_void_p] * 12 + [c_int] + [c_void_p] * 5 + [c_void_p, c_size_t, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_int,
                                c_int, c_int, c_int, c_int, c_void_p]),
    "pai_add_layernorm_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, ctypes.c_longlong, c_int, c_float, c_void_p]),
    "pai_gelu_bf16": (c_int, [c_void_p, c_void_p, ctypes.c_longlong, c_void_p]),
    "pai_knn_neighbors": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p]),
    "pai_edge_rbf": (c_int, [c_void_p, c_void_p, c_void_p, c_double, c_void_p, c_void_p, c_float, c_void_p,
                             c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "pai_measure_sfu_peak": (c_int, [ctypes.POINTER(c_double), ctypes.POINTER(c_double)]),
    "pai_tune_set": (c_int, [c_int, c_int]),
    "pai_selftest_wait_timeout": (c_int, [c_void_p]),
}

# enum pai_we_flags / enum pai_tune_key of the header
WE_REPRODUCIBLE = 1
TUNE = {"we_ks": 0, "we_tj": 1, "we_waves": 2, "we_range_reduce": 3, "we_poly_pairs": 4, "we_no_tma": 5,
        "ga_no_far_skip": 6, "ga_no_order": 7, "we_mixed": 8}
TUNE_DEFAULTS = {"we_poly_pairs": 2}

_lib = None


def lib():
    """The loaded library (loads on first use; raises if it has not been built)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: build it with `python -m proteusai_b200.build` "
                "(nvcc, sm_100a).  There is no CPU or PyTorch fallback.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status, what):
    """Raise RuntimeError for a non-zero status returned by an entry point."""
    if status != 0:
        msg = lib().pai_status_str(int(status)).decode()
        raise RuntimeError(f"{what} failed: {msg} (status {status})")


def ptr(t):
    """Device address of a tensor (None -> NULL)."""
    return None if t is None else c_void_p(t.data_ptr())


def current_stream():
    import torch
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def device_status():
    """Synchronise the current stream and raise if a kernel reported a bounded-wait timeout."""
    check(lib().pai_device_status(current_stream()), "device status")


def tune(**knobs):
    """Test-only: set tuning knobs of the kernels by name (see ``enum pai_tune_key``); ``tune_reset()`` restores them."""
    for name, value in knobs.items():
        check(lib().pai_tune_set(TUNE[name], int(value)), f"pai_tune_set({name})")


def tune_reset():
    tune(**{name: TUNE_DEFAULTS.get(name, 0) for name in TUNE})


def measure_sfu_peak():
    """(sin+cos pairs per second, elapsed ms) of the register-only SFU loop on the current device."""
    rate, ms = c_double(0.0), c_double(0.0)
    check(lib().pai_measure_sfu_peak(ctypes.byref(rate), ctypes.byref(ms)), "pai_measure_sfu_peak")
    return rate.value, ms.value
