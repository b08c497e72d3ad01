"""CPU restatement of the reference's whole GPT training step (config 4) with the library the reference uses.

TEST / BASELINE INFRASTRUCTURE ONLY (see attention_oracle.py): the timed CPU baseline of `bench.py --workload c4`
and a cross-check in tests; never on the product path.

`gpt_forward` repeats PyTorchGPT.forward of the reference (pytorch_src/model.py:81-133: token + position embedding,
pre-LayerNorm blocks of causal self-attention (:31-58) and a tanh-GELU MLP (:60-78), final LayerNorm, un-embedding
head, mean cross-entropy) as a function of ONE flat FP32 parameter vector laid out the way the reference exports its
weights to the CUDA side (pytorch_src/utils.py:7-42: tok_emb (V,C), pos_emb (T,C), per layer ln_1 w,b | W_qkv (C,3C)
| b_qkv | W_proj (C,C) | b_proj | ln_2 w,b | W_ffn1 (C,4C) | b | W_ffn2 (4C,C) | b, then ln_f w,b and head (C,V);
every matrix stored (in, out)). Gradients of that flat vector come from autograd, as in the reference's training
loop; the optimizer is torch.optim.AdamW as in PyTorchGPT.configure_optimizers (:135-136).
tests/test_oracle_golden.py pins logits, loss and the flat gradient to the files the reference's own generator wrote
(tests/golden/parity_audit*/)."""
import time

import torch
import torch.nn.functional as F

from .torch_port import attention_core


def _take(flat, offset, *shape):
    n = 1
    for s in shape:
        n *= s
    return flat[offset:offset + n].view(*shape), offset + n


def gpt_forward(flat, idx, targets, V, T_max, C, L, H, eps=1e-5):
    """flat: (P,) FP32 parameters; idx, targets: (B, T) int64. Returns (logits (B,T,V), mean cross-entropy loss)."""
    B, T = idx.shape
    d = C // H
    o = 0
    tok, o = _take(flat, o, V, C)
    pos, o = _take(flat, o, T_max, C)
    x = tok[idx] + pos[:T]
    for _ in range(L):
        g1, o = _take(flat, o, C); b1, o = _take(flat, o, C)
        wqkv, o = _take(flat, o, C, 3 * C); bqkv, o = _take(flat, o, 3 * C)
        wproj, o = _take(flat, o, C, C); bproj, o = _take(flat, o, C)
        g2, o = _take(flat, o, C); b2, o = _take(flat, o, C)
        w1, o = _take(flat, o, C, 4 * C); bb1, o = _take(flat, o, 4 * C)
        w2, o = _take(flat, o, 4 * C, C); bb2, o = _take(flat, o, C)
        h = F.layer_norm(x, (C,), g1, b1, eps)
        q, k, v = (h @ wqkv + bqkv).chunk(3, dim=-1)
        q, k, v = (t.view(B, T, H, d).transpose(1, 2) for t in (q, k, v))
        att = attention_core(q, k, v, 1.0 / d ** 0.5).transpose(1, 2).contiguous().view(B, T, C)
        x = x + att @ wproj + bproj
        h = F.layer_norm(x, (C,), g2, b2, eps)
        x = x + F.gelu(h @ w1 + bb1, approximate="tanh") @ w2 + bb2
    gf, o = _take(flat, o, C); bf, o = _take(flat, o, C)
    head, o = _take(flat, o, C, V)
    assert o == flat.numel(), (o, flat.numel())
    logits = F.layer_norm(x, (C,), gf, bf, eps) @ head
    loss = F.cross_entropy(logits.view(-1, V), targets.view(-1)) if targets is not None else None
    return logits, loss


def num_parameters(V, T_max, C, L):
    return V * C + T_max * C + L * (2 * C + C * 3 * C + 3 * C + C * C + C + 2 * C + C * 4 * C + 4 * C + 4 * C * C + C) + 2 * C + C * V


def time_training_step(V, T, C, L, H, batch, steps=1, seed=0, lr=3e-4, betas=(0.9, 0.95), wd=0.1, clip=1.0):
    """`steps` full training steps (forward, autograd backward, global-norm clip, AdamW) of the config on the host
    CPU with every thread torch has, on `batch` rows of T seeded tokens; weights ~ N(0, 0.02). Returns
    dict(seconds_per_step, tokens_per_step, threads, loss)."""
    g = torch.Generator().manual_seed(seed)
    flat = (0.02 * torch.randn(num_parameters(V, T, C, L), generator=g)).requires_grad_(True)
    opt = torch.optim.AdamW([flat], lr=lr, betas=betas, weight_decay=wd)
    idx = torch.randint(0, V, (batch, T), generator=g)
    tgt = torch.randint(0, V, (batch, T), generator=g)
    t0 = time.perf_counter()
    loss = None
    for _ in range(steps):
        opt.zero_grad(set_to_none=True)
        _, loss = gpt_forward(flat, idx, tgt, V, T, C, L, H)
        loss.backward()
        torch.nn.utils.clip_grad_norm_([flat], clip)
        opt.step()
    el = time.perf_counter() - t0
    return dict(seconds_per_step=el / steps, tokens_per_step=batch * T, threads=torch.get_num_threads(), loss=float(loss.detach()))
