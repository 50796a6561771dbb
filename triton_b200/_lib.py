"""ctypes binding of the C ABI declared in include/triton_b200.h.

The shared library is built in-tree by `python -m triton_b200.build`.  There is no
fallback: if the library is missing, loading raises; if no sm_100 device is current,
every compute call raises RuntimeError with the library's error text.
"""
import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libtriton_b200.so")

F16, BF16, E4M3, F32, E5M2 = 0, 1, 2, 3, 4
ERR_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_DEVICE, ERR_KERNEL = 1, 2, 3, 4, 5
ACT_NONE, ACT_LEAKY_RELU, ACT_SOFTMAX = 0, 1, 2
BIAS_NONE, BIAS_MATRIX, BIAS_ROWS, BIAS_COLS = 0, 1, 2, 3

_i, _i64, _p, _f = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.c_float
_s4 = ctypes.c_int64 * 4  # an element-stride quadruple {z, h, n, d}

# name -> argument types; every function returns int except where noted below
SIGNATURES = {
    "b200_version": [],
    "b200_last_error": [],
    "b200_status": [ctypes.POINTER(ctypes.c_uint), _i],
    "b200_selftest_wait_timeout": [_p, ctypes.c_uint],
    "b200_matmul": [_p, _p, _p, _p, _i, _i, _i, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _p, _p],
    "b200_matmul_plan": [_i, _i, _i, _i, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_size_t)],
    "b200_matmul_splitk": [_p, _p, _p, _p, _i, _i, _i, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _p, _p, _i, _p],
    "b200_matmul_bias": [_p, _p, _p, _p, _i, _i, _i, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _p, _p,
                         _p, _i, _i64, _i64, _i, _p],
    "b200_matmul_chain": [_p, _p, _p, _p, _p, _i, _i, _i, _i, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i],
    "b200_grouped_matmul_workspace": [_i],
    "b200_grouped_matmul": [_p, _i, _p, _p, _p, _p, _p, _i, _i, _p],
    "b200_grouped_matmul_prepare": [_p, _i, _p, _p, _p, _p, _p, _i, _i, _p, ctypes.POINTER(ctypes.c_int)],
    "b200_grouped_matmul_run": [_p, _p, _i, _i, _i],
    "b200_attention_fwd": [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _s4, _s4, _s4, _s4, _f, _i, _i],
    "b200_attention_fwd_stats": [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _s4, _s4, _s4, _s4, _f, _i, _i],
    "b200_attention_bwd": [_p] + [_p] * 10 + [_i, _i, _i, _i] + [_s4] * 8 + [_f, _i, _i],
    "b200_attention_bwd_onepass": [_p] + [_p] * 11 + [_i, _i, _i, _i] + [_s4] * 8 + [_f, _i, _i],
    "b200_attention_bwd_onepass_workspace": [_i, _i, _i, _i],
    "b200_attention_bwd_wide": [_p] + [_p] * 10 + [_i, _i, _i, _i] + [_s4] * 8 + [_f, _i, _i, _p],
    "b200_attention_bwd_wide_workspace": [_i],
    "b200_attention_bwd_noalloc": [_p] + [_p] * 9 + [_i, _i, _i, _i] + [_s4] * 8 + [_f, _i, _i],
    "b200_attention_bwd_noalloc_capacity": [],
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        # TRITON_B200_LIB (read at first use) selects another build of the same library: the
        # instrumented one of triton_b200/trace.py
        path = os.environ.get("TRITON_B200_LIB") or LIB_PATH
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: build it with `python -m triton_b200.build` (needs nvcc); "
                "there is no fallback implementation")
        L = ctypes.CDLL(path)
        for name, args in SIGNATURES.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = (ctypes.c_char_p if name == "b200_last_error" else
                          ctypes.c_longlong if name.endswith("_capacity") else
                          ctypes.c_size_t if name.endswith("_workspace") else ctypes.c_int)
        _lib = L
    return _lib


def last_error():
    return lib().b200_last_error().decode()


def check(code, what):
    if code != 0:
        raise RuntimeError(f"triton_b200 error [{what}] code {code}: {last_error()}")


def strides4(t):
    return _s4(*t.stride())


def status(clear=True):
    """Device status word (0 = all kernels completed normally). Synchronises the device."""
    v = ctypes.c_uint(0)
    check(lib().b200_status(ctypes.byref(v), 1 if clear else 0), "status")
    return v.value
