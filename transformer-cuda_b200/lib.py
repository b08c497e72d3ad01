"""ctypes binding of lib/libb200attn.so (the C ABI declared in include/b200attn.h).

There is no fallback: if the shared library is missing, `load()` raises and tells how to build it.
"""
import ctypes
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(HERE, "lib", "libb200attn.so")
HEADER_PATH = os.path.join(HERE, "..", "include", "b200attn.h")

OK = 0
ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED, ERR_CUDA, ERR_SCRATCH, ERR_DEVICE_FAULT = -1, -2, -3, -4, -5
MATH_FP32, MATH_BF16 = 0, 1
NOALLOC_SCRATCH_BYTES = 32 * 1024 * 1024


class B200AttnError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"b200attn error {code}: {message}")
        self.code = code


_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_LL, _ULL = ctypes.c_longlong, ctypes.c_ulonglong
_SIGNATURES = {
    "b200attn_version": ([], _I),
    "b200attn_last_error": ([], ctypes.c_char_p),
    "b200attn_set_math_mode": ([_I], _I),
    "b200attn_get_math_mode": ([], _I),
    "b200attn_set_fused_convert": ([_I], _I),
    "b200attn_get_fused_convert": ([], _I),
    "b200attn_fused_convert_hits": ([], _LL),
    "b200attn_reserve": ([_I, _I, _I], _I),
    "b200attn_release": ([], _I),
    "b200attn_check_device_fault": ([ctypes.POINTER(ctypes.c_uint)], _I),
    "b200attn_selftest_bounded_wait": ([_P, _P], _I),
    "b200attn_kernel_timing": ([_I], _I),
    "b200attn_kernel_times": ([ctypes.POINTER(ctypes.c_double), ctypes.POINTER(_I), ctypes.POINTER(ctypes.c_double),
                               ctypes.POINTER(_I)], _I),
    "b200attn_kernel_time_samples": ([_I, ctypes.POINTER(ctypes.c_float), _I, ctypes.POINTER(_I)], _I),
    "b200attn_qkv_split_f32": ([_P, _P, _P, _P, _I, _I, _I, _I, _P], _I),
    "b200attn_qkv_merge_grad_f32": ([_P, _P, _P, _P, _I, _I, _I, _I, _P], _I),
    "b200attn_causal_softmax_fwd_f32": ([_P, _P, _I, _I, _I, _F, _P], _I),
    "b200attn_causal_softmax_bwd_f32": ([_P, _P, _P, _I, _I, _I, _F, _P], _I),
    "b200attn_fwd_f32": ([_P, _P, _P, _P, _I, _I, _I, _I, _F, _P, _P, _P], _I),
    "b200attn_dot_do_o_f32": ([_P, _P, _P, _I, _I, _I, _I, _P], _I),
    "b200attn_bwd_f32": ([_P] * 11 + [_I, _I, _I, _I, _F, _P], _I),
    "b200attn_merge_heads_f32": ([_P, _P, _I, _I, _I, _I, _P], _I),
    "b200attn_split_heads_f32": ([_P, _P, _I, _I, _I, _I, _P], _I),
    "b200attn_fwd_bf16": ([_P, _P, _P, _P, _P, _I, _I, _I, _F, _P], _I),
    "b200attn_bwd_bf16": ([_P] * 9 + [_I, _I, _I, _F, _P], _I),
    "b200attn_bwd_bf16_noalloc": ([_P] * 9 + [_I, _I, _I, _F, _P], _I),
    "b200attn_fwd_bf16_packed": ([_P] * 3 + [_I, _I, _I, _I, _F, _P], _I),
    "b200attn_bwd_bf16_packed": ([_P] * 5 + [_I, _I, _I, _I, _F, _P], _I),
    "b200attn_qkv_split_bf16": ([_P, _P, _P, _P, _I, _I, _I, _I, _P], _I),
    "b200attn_qkv_merge_grad_bf16": ([_P, _P, _P, _P, _I, _I, _I, _I, _P], _I),
    "b200attn_merge_heads_bf16": ([_P, _P, _I, _I, _I, _I, _P], _I),
    "b200attn_split_heads_bf16": ([_P, _P, _I, _I, _I, _I, _P], _I),
    "b200attn_fill_normal_f32": ([_P, _LL, _ULL, _LL, _P], _I),
    "b200attn_fill_normal_bf16": ([_P, _LL, _ULL, _LL, _P], _I),
}

_lib = None


def declared_symbols():
    """Names of every function the public header declares (parsed from include/b200attn.h)."""
    with open(HEADER_PATH) as f:
        text = f.read()
    return sorted(set(re.findall(r"\b(b200attn_[a-z0-9_]+)\s*\(", text)))


def load():
    """Load the shared library once and attach argument types. Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(SO_PATH):
        raise B200AttnError(ERR_CUDA, f"{SO_PATH} is missing; build it with `python -c \"import __graft_entry__ as e; e.build()\"` "
                                      "(needs nvcc). There is no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(SO_PATH)
    for name, (argtypes, restype) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype
    _lib = lib
    return lib


def check(rc):
    if rc != OK:
        raise B200AttnError(rc, load().b200attn_last_error().decode("utf-8", "replace"))


def call(name, *args):
    """Call a C-ABI function by name and raise B200AttnError on a non-zero status."""
    check(getattr(load(), name)(*args))
