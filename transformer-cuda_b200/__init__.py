"""b200attn: causal multi-head self-attention (forward + backward) for NVIDIA B200 (sm_100a).

Host-side Python mirror of the launch API of sarimahsan/transformer-cuda's attention path
(include/kernels/attention.cuh) over the engine's C ABI (include/b200attn.h). The directory name
carries a hyphen, so load the package through `__graft_entry__.load_package()` (it registers the
module as `transformer_cuda_b200`).

    ops     the nine launchers with their reference names + the BF16 tensor-core entry points
    mha     CausalSelfAttention module (interface of pytorch_src/model.py:7-58) running on the engine
    shard   (batch, head) partitioning across ranks
    lib     ctypes binding of libb200attn.so
"""
from . import lib, ops, shard  # noqa: F401

__all__ = ["lib", "ops", "shard", "mha"]


def __getattr__(name):
    if name == "mha":
        import importlib
        return importlib.import_module(__name__ + ".mha")
    raise AttributeError(name)
