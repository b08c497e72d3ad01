"""The kernels of a BF16 forward + backward are launched with programmatic stream serialisation: each may be
scheduled while the one before it drains and waits on the device before it touches memory. These tests
drive many steps back to back on one stream, with the inputs of consecutive steps different and every step
sharing the library's scratch (FP32 dQ accumulator, D, lse2), and require every step's results to equal what
the same step gives when it runs alone with the stream drained on both sides. Any kernel that read or wrote
global memory before its predecessor had finished would show up as a difference in the deterministic
outputs (O, lse, dK, dV are bit-reproducible; dQ meets in floating-point reductions and gets a tolerance)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _sets(ops, n, BH, T, d, seed):
    sets = []
    for s in range(n):
        q, k, v, dO = (ops.fill_normal_(torch.empty(BH, T, d, device="cuda", dtype=BF16), seed=seed + 10 * s + i)
                       for i in range(4))
        sets.append(dict(q=q, k=k, v=v, dO=dO, o=torch.empty_like(q), lse=torch.empty(BH, T, device="cuda"),
                         dq=torch.empty_like(q), dk=torch.empty_like(q), dv=torch.empty_like(q)))
    return sets


def _step(ops, s, scale):
    ops.attention_forward_bf16(s["q"], s["k"], s["v"], scale, s["o"], s["lse"])
    ops.attention_backward_bf16(s["q"], s["k"], s["v"], s["o"], s["dO"], s["lse"], scale, s["dq"], s["dk"], s["dv"])


@pytest.mark.parametrize("BH,T,d", [(24, 640, 64), (6, 1536, 128), (96, 130, 64)])
def test_back_to_back_steps_equal_isolated_steps(pkg, BH, T, d):
    ops = pkg.ops
    scale = 1.0 / math.sqrt(d)
    n_sets, rounds = 3, 12
    sets = _sets(ops, n_sets, BH, T, d, seed=4000 + T)
    ops.reserve(BH, T, d)
    want = []
    for s in sets:  # each step alone, stream drained on both sides
        torch.cuda.synchronize()
        _step(ops, s, scale)
        torch.cuda.synchronize()
        want.append({key: s[key].clone() for key in ("o", "lse", "dq", "dk", "dv")})
    got = [[None] * n_sets for _ in range(rounds)]
    for r in range(rounds):  # no synchronisation anywhere in here
        for i, s in enumerate(sets):
            for key in ("o", "dq", "dk", "dv"):
                s[key].zero_()
            _step(ops, s, scale)
            got[r][i] = {key: s[key].clone() for key in ("o", "lse", "dq", "dk", "dv")}
    torch.cuda.synchronize()
    ops.check_device_fault()
    for r in range(rounds):
        for i in range(n_sets):
            for key in ("o", "lse", "dk", "dv"):
                assert torch.equal(got[r][i][key], want[i][key]), (r, i, key)
            diff = (got[r][i]["dq"].float() - want[i]["dq"].float()).abs().max().item()
            assert diff <= 2.0 ** -6 * max(1.0, want[i]["dq"].float().abs().max().item()), (r, i, diff)


def test_uninterrupted_chain(pkg):
    """Nothing but the library's own launches on the stream (no copies or fills in between, so every kernel's
    predecessor is another kernel of the chain, across step boundaries too); the state after the loop must be
    the isolated results."""
    ops = pkg.ops
    BH, T, d = 96, 1024, 64
    scale = 1.0 / math.sqrt(d)
    sets = _sets(ops, 3, BH, T, d, seed=5000)
    ops.reserve(BH, T, d)
    want = []
    for s in sets:
        torch.cuda.synchronize()
        _step(ops, s, scale)
        torch.cuda.synchronize()
        want.append({key: s[key].clone() for key in ("o", "lse", "dq", "dk", "dv")})
        for key in ("o", "dq", "dk", "dv"):
            s[key].zero_()
    torch.cuda.synchronize()
    for _ in range(40):
        for s in sets:
            _step(ops, s, scale)
    torch.cuda.synchronize()
    ops.check_device_fault()
    for s, w in zip(sets, want):
        for key in ("o", "lse", "dk", "dv"):
            assert torch.equal(s[key], w[key]), key
        assert (s["dq"].float() - w["dq"].float()).abs().max().item() <= 2.0 ** -6 * max(1.0, w["dq"].float().abs().max().item())


def test_packed_chain_back_to_back(pkg):
    """The same for the interleaved-layout entry points, which share the scratch with the slab entry points:
    alternate the two kinds of call without synchronisation."""
    ops = pkg.ops
    B, T, H, d = 2, 520, 4, 64
    C = H * d
    scale = 1.0 / math.sqrt(d)
    qkv = ops.fill_normal_(torch.empty(B, T, 3 * C, device="cuda", dtype=BF16), seed=77)
    dout = ops.fill_normal_(torch.empty(B, T, C, device="cuda", dtype=BF16), seed=78)
    slab = _sets(ops, 1, B * H, T, d, seed=79)[0]
    ops.reserve(B * H, T, d)
    torch.cuda.synchronize()
    out, lse = ops.attention_forward_bf16_packed(qkv, H, scale)
    dqkv = ops.attention_backward_bf16_packed(qkv, out, dout, lse, H, scale)
    torch.cuda.synchronize()
    _step(ops, slab, scale)
    torch.cuda.synchronize()
    want_out, want_g = out.clone(), dqkv.clone()
    want_slab = {key: slab[key].clone() for key in ("o", "dk", "dv")}
    for _ in range(10):
        out.zero_(), dqkv.zero_()
        ops.attention_forward_bf16_packed(qkv, H, scale, out=out, lse=lse)
        ops.attention_backward_bf16_packed(qkv, out, dout, lse, H, scale, dqkv=dqkv)
        keep_out, keep_g = out.clone(), dqkv.clone()
        _step(ops, slab, scale)
        torch.cuda.synchronize()
        assert torch.equal(keep_out, want_out)
        assert torch.equal(keep_g.view(B, T, 3, C)[:, :, 1:], want_g.view(B, T, 3, C)[:, :, 1:])  # dK, dV
        assert (keep_g.view(B, T, 3, C)[:, :, 0].float() - want_g.view(B, T, 3, C)[:, :, 0].float()).abs().max().item() <= 2e-2
        for key in ("o", "dk", "dv"):
            assert torch.equal(slab[key], want_slab[key])
    ops.check_device_fault()


@pytest.mark.parametrize("BH,T,d,iters", [(96, 1024, 64, 80), (8, 2048, 128, 20)])
def test_fresh_inputs_every_step(pkg, BH, T, d, iters):
    """New values in newly allocated memory before every step, kernels right behind the fills, no
    synchronisation; then the same step again with the stream drained around each call. A kernel that
    read a tile before its producer had finished - another kernel, or an earlier step of the same CTA
    (the dS^T tile in shared memory, for one, is rewritten every step while dK / dQ of the step before
    may still be reading it) - shows up as a difference."""
    ops = pkg.ops
    scale = 1.0 / math.sqrt(d)
    for it in range(iters):
        q, k, v, dO = (ops.fill_normal_(torch.empty(BH, T, d, device="cuda", dtype=BF16), seed=1000 * it + i)
                       for i in range(4))
        o, lse = ops.attention_forward_bf16(q, k, v, scale)
        dq, dk, dv = ops.attention_backward_bf16(q, k, v, o, dO, lse, scale)
        got = [t.clone() for t in (o, lse, dk, dv, dq)]
        torch.cuda.synchronize()
        o2, lse2 = ops.attention_forward_bf16(q, k, v, scale)
        torch.cuda.synchronize()
        dq2, dk2, dv2 = ops.attention_backward_bf16(q, k, v, o2, dO, lse2, scale)
        torch.cuda.synchronize()
        for name, g, r in zip(("o", "lse", "dk", "dv"), got, (o2, lse2, dk2, dv2)):
            assert torch.equal(g, r), (it, name)
        assert (got[4].float() - dq2.float()).abs().max().item() <= 2.0 ** -6 * max(1.0, dq2.float().abs().max().item()), it
    ops.check_device_fault()
