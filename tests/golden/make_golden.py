"""Generate the golden vectors under tests/golden/ by running the reference's own PyTorch module.

Run once in a container that has the reference checkout (it cannot travel to the GPU box):

    python tests/golden/make_golden.py --reference /path/to/transformer-cuda

It imports `pytorch_src.model.CausalSelfAttention` from that checkout unmodified, feeds it seeded
inputs, and records, through forward hooks and retained gradients, every tensor that crosses one of
the launchers of the attention path:

    qkv (B,T,3C) -> q,k,v (B,H,T,d)      qkv_split_transpose_forward
    q,k,v -> out (B,H,T,d)               tiled_causal_attention_forward (m, l are derived, see below)
    out -> merged (B,T,C)                head_merge_transpose_forward
    d(merged) -> dout                    head_merge_transpose_backward
    dout -> dq,dk,dv                     tiled_causal_attention_backward
    dq,dk,dv -> dqkv                     qkv_split_transpose_backward
    x, weights, dY -> y, dx, dW, db      the whole block (with a gamma=1, beta=0 LayerNorm in front)

The module does not expose softmax statistics, so m and l are recomputed here from the module's
own q, k with torch ops that mirror pytorch_src/model.py:44-51 and stored beside the rest.
Outputs are float32 .npz files of a few hundred KB.
"""
import argparse
import math
import os
import sys

import numpy as np
import torch

CASES = {
    # name: (B, T, C, H, seed, keep)   keep = "block": every tensor of the block;
    #                                  keep = "core": only the attention core (q,k,v,dout -> out,m,l,dq,dk,dv)
    "config1_B4_T64_C128_H4": (4, 64, 128, 4, 1234, "block"),    # the CPU-runnable case of the benchmark spec
    "paritygate_B4_T16_C64_H4": (4, 16, 64, 4, 42, "block"),     # shape of scripts/compare_parity.py:37-44
    "ragged_B2_T37_C64_H2": (2, 37, 64, 2, 7, "core"),           # T not a multiple of any tile, d = 32
    "d64_B1_T130_C128_H2": (1, 130, 128, 2, 99, "core"),         # d = 64, T straddles a 128-row tile
    "d128_B1_T72_C256_H2": (1, 72, 256, 2, 5, "core"),           # d = 128
}
CORE_KEYS = ("shape", "seed", "q", "k", "v", "out", "m", "l", "dout", "dq", "dk", "dv")


def run_case(CausalSelfAttention, B, T, C, H, seed):
    torch.manual_seed(seed)
    d = C // H
    attn = CausalSelfAttention(d_model=C, num_heads=H, max_seq_len=max(T, 16))
    ln = torch.nn.LayerNorm(C, eps=1e-5)  # gamma = 1, beta = 0 by construction
    with torch.no_grad():
        attn.qkv_proj.weight.normal_(0.0, 0.02)
        attn.out_proj.weight.normal_(0.0, 0.02)
        attn.qkv_proj.bias.zero_()
        attn.out_proj.bias.zero_()
    x = torch.randn(B, T, C, requires_grad=True)
    dY = torch.randn(B, T, C)

    kept = {}

    def keep_qkv(_mod, _inp, out):
        out.retain_grad()
        kept["qkv"] = out

    def keep_merged(_mod, inp):
        inp[0].retain_grad()
        kept["merged"] = inp[0]

    h1 = attn.qkv_proj.register_forward_hook(keep_qkv)
    h2 = attn.out_proj.register_forward_pre_hook(keep_merged)
    y = attn(ln(x))
    y.backward(dY)
    h1.remove()
    h2.remove()

    qkv, merged = kept["qkv"], kept["merged"]
    dqkv, dmerged = qkv.grad, merged.grad

    def heads(t3):  # (B,T,C) -> (B,H,T,d)
        return t3.view(B, T, H, d).transpose(1, 2).contiguous()

    qc, kc, vc = qkv.detach().chunk(3, dim=-1)
    q, k, v = heads(qc), heads(kc), heads(vc)
    dqc, dkc, dvc = dqkv.chunk(3, dim=-1)
    dq, dk, dv = heads(dqc), heads(dkc), heads(dvc)
    out = heads(merged.detach())
    dout = heads(dmerged)

    scale = 1.0 / math.sqrt(d)
    att = (q @ k.transpose(-2, -1)) * scale
    att = att.masked_fill(torch.tril(torch.ones(T, T)) == 0, float("-inf"))
    m = att.max(dim=-1).values
    l = torch.exp(att - m[..., None]).sum(dim=-1)

    f = lambda t: t.detach().numpy().astype(np.float32)
    return dict(
        shape=np.array([B, T, C, H], dtype=np.int64), seed=np.array([seed], dtype=np.int64),
        x=f(x), dY=f(dY),
        # Linear weights are stored (out, in) by torch; the CUDA blob stores (in, out)
        # (pytorch_src/utils.py:7-42 transposes on export), so the fixtures hold (in, out).
        w_qkv=f(attn.qkv_proj.weight.t().contiguous()), b_qkv=f(attn.qkv_proj.bias),
        w_proj=f(attn.out_proj.weight.t().contiguous()), b_proj=f(attn.out_proj.bias),
        y=f(y), dx=f(x.grad),
        dw_qkv=f(attn.qkv_proj.weight.grad.t().contiguous()), db_qkv=f(attn.qkv_proj.bias.grad),
        dw_proj=f(attn.out_proj.weight.grad.t().contiguous()), db_proj=f(attn.out_proj.bias.grad),
        qkv=f(qkv), q=f(q), k=f(k), v=f(v), out=f(out), merged=f(merged), m=f(m), l=f(l),
        dmerged=f(dmerged), dout=f(dout), dq=f(dq), dk=f(dk), dv=f(dv), dqkv=f(dqkv),
    )


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of a transformer-cuda checkout")
    ap.add_argument("--out", default=os.path.dirname(os.path.abspath(__file__)))
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    from pytorch_src.model import CausalSelfAttention  # the reference's module, unmodified

    torch.set_num_threads(1)  # bit-reproducible reductions
    for name, (B, T, C, H, seed, keep) in CASES.items():
        data = run_case(CausalSelfAttention, B, T, C, H, seed)
        if keep == "core":
            data = {k: data[k] for k in CORE_KEYS}
        path = os.path.join(args.out, name + ".npz")
        np.savez_compressed(path, **data)
        print(f"wrote {path} ({os.path.getsize(path) / 1024:.0f} KB)")


if __name__ == "__main__":
    main()
