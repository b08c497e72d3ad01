"""ctypes binding of lib/libb200loss.so (include/b200loss.h) and the launcher of the reference's loss header over it.

`cross_entropy_forward_backward` keeps the name and argument meaning of include/kernels/loss.cuh:8-15 of
sarimahsan/transformer-cuda with torch CUDA tensors in place of raw pointers. There is no fallback: a missing
library raises."""
import ctypes
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(HERE, "lib", "libb200loss.so")
HEADER_PATH = os.path.join(HERE, "..", "include", "b200loss.h")

_P, _I = ctypes.c_void_p, ctypes.c_int
_SIGNATURES = {
    "b200loss_cross_entropy": ([_P, _P, _P, _P, _I, _I, _I, _P], _I),
    "b200loss_kernel_path": ([_P, _P, _I], _I),
    "b200loss_max_resident_vocab": ([], _I),
    "b200loss_check_device_fault": ([], _I),
    "b200loss_release": ([], None),
    "b200loss_last_error": ([], ctypes.c_char_p),
}
_lib = None


class B200LossError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"b200loss error {code}: {message}")
        self.code = code


def declared_symbols():
    with open(HEADER_PATH) as f:
        return sorted(set(re.findall(r"\b(b200loss_[a-z0-9_]+)\s*\(", f.read())))


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise RuntimeError(f"{SO_PATH} is missing: run `python -c 'import __graft_entry__ as e; e.build()'` (needs nvcc); "
                               "there is no CPU or PyTorch fallback")
        lib = ctypes.CDLL(SO_PATH)
        for name, (args, res) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, res
        _lib = lib
    return _lib


def _check(code):
    if code != 0:
        raise B200LossError(code, load().b200loss_last_error().decode())


def cross_entropy_forward_backward(logits, targets, dlogits=None, want_loss=True):
    """logits (B, T, V) float32, targets (B, T) int32 -> (dlogits, loss): dlogits = (softmax - onehot) / (B*T) and
    loss a 0-d CUDA tensor holding the mean (None when `want_loss` is false). Asynchronous on the current stream."""
    import torch
    if logits.dtype != torch.float32 or not logits.is_cuda or not logits.is_contiguous() or logits.dim() != 3:
        raise ValueError("logits must be a contiguous CUDA float32 tensor of shape (B, T, V)")
    B, T, V = logits.shape
    if targets.dtype != torch.int32 or not targets.is_cuda or not targets.is_contiguous() or targets.numel() != B * T:
        raise ValueError("targets must be a contiguous CUDA int32 tensor with B * T elements")
    if dlogits is None:
        dlogits = torch.empty_like(logits)
    elif dlogits.dtype != torch.float32 or not dlogits.is_cuda or not dlogits.is_contiguous() or dlogits.numel() != logits.numel():
        raise ValueError("dlogits must be a contiguous CUDA float32 tensor with the size of logits")
    loss = torch.zeros((), dtype=torch.float32, device=logits.device) if want_loss else None
    stream = torch.cuda.current_stream(logits.device).cuda_stream
    with torch.cuda.device(logits.device):
        _check(load().b200loss_cross_entropy(logits.data_ptr(), targets.data_ptr(), dlogits.data_ptr(),
                                             loss.data_ptr() if want_loss else None, B, T, V, stream))
    return dlogits, loss


def kernel_path(logits, dlogits):
    return load().b200loss_kernel_path(logits.data_ptr(), dlogits.data_ptr(), logits.shape[-1])


def check_device_fault():
    _check(load().b200loss_check_device_fault())
