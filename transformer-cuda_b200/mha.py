"""CausalSelfAttention with the interface of the reference's PyTorch module
(pytorch_src/model.py:7-58: `d_model`, `num_heads`, `max_seq_len`; `qkv_proj`, `out_proj`), whose
split-transpose, attention core and head merge run on the engine through the launch API in `ops`.

The two projections stay `torch.nn.Linear` (they are library GEMMs outside the attention path, as in
the reference's model.cu:289,342); autograd reaches the engine through `AttentionCoreFunction`, which
calls the same launcher sequence as the reference's model.cu:305-336 (forward) and :602-653 (backward).
"""
import math

import torch

from . import ops


class AttentionCoreFunction(torch.autograd.Function):
    """qkv (B,T,3C) FP32 -> merged heads (B,T,C) FP32; `math` is 'fp32' or 'bf16'."""

    @staticmethod
    def forward(ctx, qkv, num_heads, math_mode):
        B, T, C3 = qkv.shape
        C = C3 // 3
        H, d = num_heads, C // num_heads
        scale = 1.0 / math.sqrt(d)
        qkv = qkv.contiguous()
        dev = qkv.device
        merged = torch.empty(B, T, C, device=dev, dtype=torch.float32)
        if math_mode == "bf16":
            q, k, v = (torch.empty(B, H, T, d, device=dev, dtype=torch.bfloat16) for _ in range(3))
            ops.qkv_split_transpose_forward_bf16(qkv, q, k, v, B, T, H, d)
            out, lse = ops.attention_forward_bf16(q, k, v, scale)
            ops.head_merge_transpose_forward_bf16(out, merged, B, H, T, d)
            ctx.save_for_backward(q, k, v, out, lse)
        else:
            q, k, v, out = (torch.empty(B, H, T, d, device=dev, dtype=torch.float32) for _ in range(4))
            m, l = (torch.empty(B, H, T, device=dev, dtype=torch.float32) for _ in range(2))
            ops.qkv_split_transpose_forward(qkv, q, k, v, B, T, H, d)
            prev = ops.get_math_mode()
            ops.set_math_mode("fp32")
            try:
                ops.tiled_causal_attention_forward(q, k, v, out, B, H, T, d, scale, m, l)
            finally:
                ops.set_math_mode(prev)
            ops.head_merge_transpose_forward(out, merged, B, H, T, d)
            ctx.save_for_backward(q, k, v, out, m, l)
        ctx.dims = (B, H, T, d, scale, math_mode)
        return merged

    @staticmethod
    def backward(ctx, dmerged):
        B, H, T, d, scale, math_mode = ctx.dims
        dmerged = dmerged.contiguous()
        dev = dmerged.device
        dqkv = torch.empty(B, T, 3 * H * d, device=dev, dtype=torch.float32)
        if math_mode == "bf16":
            q, k, v, out, lse = ctx.saved_tensors
            dout = torch.empty(B, H, T, d, device=dev, dtype=torch.bfloat16)
            ops.head_merge_transpose_backward_bf16(dmerged, dout, B, H, T, d)
            dq, dk, dv = ops.attention_backward_bf16(q, k, v, out, dout, lse, scale)
            ops.qkv_split_transpose_backward_bf16(dq, dk, dv, dqkv, B, T, H, d)
        else:
            q, k, v, out, m, l = ctx.saved_tensors
            dout, dq, dk, dv = (torch.empty(B, H, T, d, device=dev, dtype=torch.float32) for _ in range(4))
            ws = torch.empty(B, H, T, device=dev, dtype=torch.float32)
            ops.head_merge_transpose_backward(dmerged, dout, B, H, T, d)
            prev = ops.get_math_mode()
            ops.set_math_mode("fp32")
            try:
                ops.tiled_causal_attention_backward(q, k, v, out, dout, m, l, dq, dk, dv, ws, B, H, T, d, scale)
            finally:
                ops.set_math_mode(prev)
            ops.qkv_split_transpose_backward(dq, dk, dv, dqkv, B, T, H, d)
        return dqkv, None, None


class CausalSelfAttention(torch.nn.Module):
    """Same constructor and parameters as pytorch_src/model.py:12-29; `math` selects the engine's
    FP32 parity path or the BF16 tensor-core path (d_head must then be 64 or 128)."""

    def __init__(self, d_model: int = 256, num_heads: int = 8, max_seq_len: int = 256, math: str = "fp32"):
        super().__init__()
        assert d_model % num_heads == 0, f"d_model {d_model} must be divisible by num_heads {num_heads}"
        self.d_model, self.num_heads, self.d_head = d_model, num_heads, d_model // num_heads
        self.max_seq_len = max_seq_len
        self.math = math
        self.qkv_proj = torch.nn.Linear(d_model, 3 * d_model, bias=True)
        self.out_proj = torch.nn.Linear(d_model, d_model, bias=True)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        qkv = self.qkv_proj(x)
        y = AttentionCoreFunction.apply(qkv, self.num_heads, self.math)
        return self.out_proj(y)
