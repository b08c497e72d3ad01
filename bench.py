#!/usr/bin/env python
"""Benchmark of the causal attention path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c2|c3|...]

One "step" is one forward + backward pass of the attention core over one batch of seeded synthetic
BF16 Q, K, V, dO ~ N(0,1). The default workload is the GPT-2-small shape of the benchmark spec
(B=8, H=12, T=1024, d=64). With N > 1 (one process per GPU, launched by torchrun) every rank owns a
contiguous range of (batch, head) slabs of a batch N times larger - the per-GPU work is fixed, no
collective is on the data path, and the reported value is all ranks' FLOPs over the slowest rank's time.

Rank 0 prints ONE JSON line. `value` is device-timed with inputs resident in HBM; `e2e` is the same
metric through the public API with pinned HOST buffers, host<->device copies inside the timed region;
`roofline` is the dominant kernel (the tcgen05 backward) against the measured dense-BF16 peak;
`cpu_baseline` times the reference's own math (PyTorch, FP32, autograd) on the host cores.

`--impl reference` runs only that CPU implementation, with all host threads, on the same workload
definition (each step a bounded sample of it) and prints the same line with "impl": "reference".
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, H, T, d) per GPU
    "c2": (8, 12, 1024, 64),      # GPT-2-small-shaped causal attention (the headline configuration)
    "c3": (2, 16, 8192, 128),     # long context
    "c5_512": (64, 32, 512, 128), "c5_1024": (32, 32, 1024, 128), "c5_2048": (16, 32, 2048, 128),
    "c5_4096": (8, 32, 4096, 128), "c5_8192": (4, 32, 8192, 128), "c5_16384": (2, 32, 16384, 128),
}
METRIC = "causal_attention_fwd_bwd_tflops"
UNIT = "TFLOP/s"
L2_BYTES = 126 * 1024 * 1024


def flops(B, H, T, d):
    """Algorithmic count, causal pairs as half the square: fwd 2*BH*T^2*d, bwd 5*BH*T^2*d."""
    return 7.0 * B * H * T * T * d


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return dict(bf16=float(p["bf16_tflops"]), bf16_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                    hbm=float(p["hbm_gbs"]), source="measured")
    except Exception:
        return dict(bf16=1590.0, bf16_sustained=1400.0, hbm=6650.0, source="fallback")


def ncu_traffic_per_launch(workload):
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary, if one covers this workload."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            return json.load(f).get(workload, {}).get("attn_bwd_tc_kernel_bytes_per_launch")
    except Exception:
        return None


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.proc, self.path = None, f"/tmp/b200attn_clocks_{os.getpid()}.csv"
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=self.out,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def wait_first_sample(self, timeout_s=3.0):
        t0 = time.perf_counter()
        while self.proc is not None and time.perf_counter() - t0 < timeout_s:
            try:
                if os.path.getsize(self.path) > 0:
                    break
            except OSError:
                pass
            time.sleep(0.02)
        self.t_region = time.perf_counter()

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 6 or not parts[0].isdigit():
                    continue
                sm.append(int(parts[0]))
                mx.append(int(parts[1]))
                for n, v in zip(names, parts[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.remove(self.path)
        except Exception:
            pass
        if not sm:
            return None
        busy = [x for x in sm if x > 0.5 * max(sm)] or sm
        return dict(sm_mhz=statistics.median(busy), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))


def cpu_baseline(B, H, T, d, budget_s):
    """The reference's math on the host cores: PyTorch FP32 forward + autograd backward
    (oracle/torch_port.py), all threads, on a bounded sample of the workload's slabs."""
    import torch
    from oracle import torch_port
    torch.set_num_threads(os.cpu_count() or 1)
    r = torch_port.time_forward_backward(B * H, T, d, budget_s=budget_s)
    tf = flops(1, 1, T, d) / r["seconds_per_slab"] / 1e12
    return dict(value=tf, unit=UNIT, cores=r["threads"], kind="port",
                sample=f"{r['slabs_timed']} (batch,head) slab passes of the workload's {B * H} slabs, {r['slabs_per_call']} per "
                       f"call, {r['calls']} calls after 1 warm-up, PyTorch FP32 forward + autograd backward")


def run_reference(args, B, H, T, d):
    """--impl reference: K timed steps of the CPU implementation, each a bounded sample (a few slabs)."""
    import torch
    from oracle import torch_port
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    per_step = max(1, min(8, B * H, (1 << 28) // (T * T)))
    g = torch.Generator().manual_seed(0)
    q, k, v, dO = (torch.randn(per_step, T, d, generator=g) for _ in range(4))
    scale = 1.0 / math.sqrt(d)
    for _ in range(args.warmup):
        torch_port.forward_backward(q, k, v, dO, scale)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        torch_port.forward_backward(q, k, v, dO, scale)
    el = time.perf_counter() - t0
    tf = flops(1, per_step, T, d) * args.steps / el / 1e12
    sample = f"{per_step} of {B * H} (batch,head) slabs per step, PyTorch FP32 autograd on host CPU"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": tf, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": el / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args, B, H, T, d), "sample": sample},
        "cpu_baseline": {"value": tf, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def run_gpt_step(args):
    """Config 4: full synthetic GPT training step (L=12, C=768, H=12, d_ff=3072, V=50257, T=1024, per-GPU B=16,
    AdamW), data-parallel with one NCCL all-reduce of the gradient buffer per step. The step is the reference's
    own model code linked against this engine (transformer-cuda_b200/harness/gpt_step_dp.cu; binary prebuilt into
    build/ by transformer-cuda_b200/harness/Makefile where the reference checkout exists). Launched by torchrun, every bench.py rank starts the
    binary as its rank's process (RANK / WORLD_SIZE / LOCAL_RANK / MASTER_PORT are inherited); rank 0 relays the
    JSON line. `--impl reference` runs the same harness linked against the reference's own attention kernels."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    # --gemm reference: the reference's FP32 cuBLAS wrappers; fp32 / bf16: the GEMM drop-in
    # (transformer-cuda_b200/gemm/matmul_dropin.cu) in that arithmetic
    if args.impl == "reference":
        name = "gpt_step_dp_ref"
    else:
        name = "gpt_step_dp_b200" if args.gemm == "reference" else \
            ("gpt_step_dp_b200_all" if args.loss_adamw == "dropin" else "gpt_step_dp_b200_gemm")
    exe = os.path.join(ROOT, "build", name)
    if not os.path.exists(exe):
        if rank == 0:
            print(json.dumps({"impl": args.impl, "metric": "gpt_step_tokens_per_s",
                              "unavailable": f"build/{name} is built by transformer-cuda_b200/harness/Makefile where a reference checkout exists; not present here"}))
        return
    steps = max(1, min(args.steps, 20))
    env = dict(os.environ)
    env.setdefault("B200ATTN_MATH", "bf16")  # attention through the tcgen05 kernels (the reference arm ignores it)
    env.setdefault("B200ATTN_FUSED_CONVERT", "1")  # BF16 copies of q, k, v, dO come out of the layout launchers
    if args.gemm != "reference":
        env["B200GEMM_MATH"] = args.gemm
        # the reference model never rewrites a gradient between the dW and dX products that read it (src/model.cu:451-700)
        env.setdefault("B200GEMM_REUSE_STAGED", "1")
        # ... and its LayerNorm outputs, LayerNorm / attention gradients are written by the drop-ins only: BF16 twins
        env.setdefault("B200GEMM_TWINS", "1")
    res = subprocess.run([exe, "--steps", str(steps), "--warmup", str(min(args.warmup, 3))], env=env, capture_output=True, text=True)
    if res.returncode != 0:
        raise SystemExit(f"{name} failed on rank {rank}: {res.stderr[-2000:]}")
    if rank != 0:
        return
    child = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    line = {"metric": "gpt_step_tokens_per_s", "value": child["value"], "unit": "tokens/s", "n_gpus": world, "steps": steps,
            "warmup": min(args.warmup, 3), "ms_per_step": child["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None,
            "dtype": "f32" if args.impl == "reference" else
                     ("f32 buffers, bf16 attention and bf16 GEMM operands" if args.gemm == "bf16" else "f32 model, bf16 attention"),
            "data": "synthetic", "impl": args.impl,
            "config": {"workload": "c4: GPT training step L=12 C=768 H=12 d_ff=3072 V=50257 T=1024, per-GPU B=16, AdamW, "
                                   "data-parallel NCCL all-reduce of gradients", **child["config"], "attention": child["attention"],
                       "gemm": "reference FP32 cuBLAS wrappers" if (args.impl == "reference" or args.gemm == "reference")
                               else f"GEMM drop-in, B200GEMM_MATH={args.gemm}",
                       "loss_adamw": "loss and AdamW drop-ins (libb200loss, optim/adamw_dropin.cu)" if name.endswith("_all")
                                     else "reference loss.cu and optimizer.cu"},
            "loss_after_last_step": child["loss"], "gemm_dropin": child.get("gemm_dropin"),
            "allreduce_ms_per_step": child.get("allreduce_ms_per_step"),
            "allreduce_overlapped": child.get("allreduce_overlapped"),
            "allreduce": ("in-place ncclAllReduce(avg) of the 163 M-float gradient buffer in 14 parts on a second stream, each issued when "
                          "the backward pass has finished that part; allreduce_ms_per_step = what the compute stream still waits for (rank 0)")
                         if child.get("allreduce_overlapped") else
                         "one in-place ncclAllReduce(avg) of the 163 M-float gradient buffer per step, timed with CUDA events on rank 0"}
    if world == 1 and args.impl != "reference" and not args.no_cpu_baseline:
        # the reference's PyTorch twin of the whole step on the host cores (a port: the checkout is not on this machine)
        import torch
        from oracle import torch_gpt_port
        torch.set_num_threads(os.cpu_count() or 1)
        c = child["config"]
        r = torch_gpt_port.time_training_step(c["V"], c["T"], c["C"], c["L"], c["H"], batch=1, steps=1)
        line["cpu_baseline"] = {"value": r["tokens_per_step"] / r["seconds_per_step"], "unit": "tokens/s", "cores": r["threads"],
                                "kind": "port",
                                "sample": f"one un-warmed training step (forward, autograd backward, clip, AdamW) on 1 of the "
                                          f"{c['per_gpu_batch']} rows of the per-GPU batch ({r['tokens_per_step']} tokens), "
                                          f"{r['seconds_per_step']:.1f} s, PyTorch FP32"}
    print(json.dumps(line), flush=True)


def time_loss_kernel(pkg, dev, peaks, rows, iters=10):
    """The loss launcher at the head of the model's backward (cross_entropy_forward_backward, loss.cu:97) on `rows` rows
    of the GPT step's vocabulary (16384 rows: 3.3 GB in, 3.3 GB out, far beyond L2): algorithmic bytes = 8 per logit."""
    import importlib
    import torch
    loss_ops = importlib.import_module(pkg.__name__ + ".loss_ops")
    V = 50257
    logits = torch.randn(1, rows, V, device=dev)
    targets = torch.randint(0, V, (rows,), device=dev, dtype=torch.int32)
    dlogits = torch.empty_like(logits)
    for _ in range(3):
        loss_ops.cross_entropy_forward_backward(logits, targets, dlogits=dlogits)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        loss_ops.cross_entropy_forward_backward(logits, targets, dlogits=dlogits)
    e1.record()
    torch.cuda.synchronize()
    loss_ops.check_device_fault()
    ms, nbytes = e0.elapsed_time(e1) / iters, 8 * rows * V
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"launcher": f"cross_entropy_forward_backward (rows={rows}, V={V})", "replaces": "loss.cu:97", "ms": round(ms, 4),
            "algorithmic_bytes": nbytes, "achieved_gbs": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peaks["hbm"], 3)}


def run_loss_kernel(args):
    import torch
    import __graft_entry__ as entry
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = measured_peaks()
    row = time_loss_kernel(entry.load_package(), dev, peaks, args.loss_rows, iters=max(1, min(args.steps, 10)))
    print(json.dumps({"suite": "loss", "unit": "GB/s", "hbm_peak_gbs": peaks["hbm"], "peak_source": peaks["source"], "kernels": [row]}),
          flush=True)


def run_path_kernels(args, B, H, T, d):
    """The HBM-bound launchers of the path (and the FP32 parity kernels) on the workload's shape, one GPU:
    achieved GB/s = algorithmic bytes / CUDA-event time, against the measured HBM copy bandwidth."""
    import torch
    import __graft_entry__ as entry
    pkg = entry.load_package()
    ops = pkg.ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = measured_peaks()
    n, rows = B * H * T * d, B * H * T
    f32, bf16 = torch.float32, torch.bfloat16
    iters = max(5, min(args.steps, 50))

    def timed(fn, copies=1):
        for _ in range(3):
            fn(0)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            fn(i % copies)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    # enough rotating copies of every buffer set to exceed L2
    copies = max(2, math.ceil(2.0 * L2_BYTES / (24 * n)))
    qkv = [ops.fill_normal_(torch.empty(B, T, 3 * H * d, device=dev), seed=50 + c) for c in range(copies)]
    q32, k32, v32 = ([torch.empty(B, H, T, d, device=dev) for _ in range(copies)] for _ in range(3))
    qb, kb, vb = ([torch.empty(B, H, T, d, device=dev, dtype=bf16) for _ in range(copies)] for _ in range(3))
    merged = [torch.empty(B, T, H * d, device=dev) for _ in range(copies)]
    out = []

    def row(name, ref, ms, nbytes):
        gbs = nbytes / (ms * 1e-3) / 1e9
        out.append({"launcher": name, "replaces": ref, "ms": round(ms, 4), "algorithmic_bytes": nbytes,
                    "achieved_gbs": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peaks["hbm"], 3)})

    row("qkv_split_transpose_forward (FP32)", "attention.cu:381",
        timed(lambda c: ops.qkv_split_transpose_forward(qkv[c], q32[c], k32[c], v32[c], B, T, H, d), copies), 24 * n)
    row("qkv_split_transpose_backward (FP32)", "attention.cu:408",
        timed(lambda c: ops.qkv_split_transpose_backward(q32[c], k32[c], v32[c], qkv[c], B, T, H, d), copies), 24 * n)
    row("qkv split + BF16 conversion", "attention.cu:381",
        timed(lambda c: ops.qkv_split_transpose_forward_bf16(qkv[c], qb[c], kb[c], vb[c], B, T, H, d), copies), 18 * n)
    row("dqkv merge from BF16", "attention.cu:408",
        timed(lambda c: ops.qkv_split_transpose_backward_bf16(qb[c], kb[c], vb[c], qkv[c], B, T, H, d), copies), 18 * n)
    row("head_merge_transpose_forward (FP32)", "attention.cu:466",
        timed(lambda c: ops.head_merge_transpose_forward(q32[c], merged[c], B, H, T, d), copies), 8 * n)
    row("head_merge_transpose_backward (FP32)", "attention.cu:491",
        timed(lambda c: ops.head_merge_transpose_backward(merged[c], q32[c], B, H, T, d), copies), 8 * n)
    row("head merge from BF16", "attention.cu:466",
        timed(lambda c: ops.head_merge_transpose_forward_bf16(qb[c], merged[c], B, H, T, d), copies), 6 * n)
    D = torch.empty(B, H, T, device=dev)
    row("attention_precompute_dot_do_o (FP32)", "attention.cu:679",
        timed(lambda c: ops.attention_precompute_dot_do_o(q32[c], k32[c], D, B, H, T, d), copies), 8 * n + 4 * rows)
    # materialised softmax of the non-tiled branch: one slab batch small enough to hold (rows x T floats)
    Bs = max(1, min(B, (1 << 28) // (H * T * T)))
    srows = Bs * H * T
    scores = [ops.fill_normal_(torch.empty(srows, T, device=dev), seed=70 + c) for c in range(2)]
    probs = [torch.empty(srows, T, device=dev) for _ in range(2)]
    ms = timed(lambda c: ops.causal_softmax_forward(scores[c], probs[c], Bs, H, T, 0.125), 2)
    row(f"causal_softmax_forward (B={Bs})", "attention.cu:435", ms, srows * T * 4 // 2 + srows * T * 4)  # reads j<=i, writes all
    ms = timed(lambda c: ops.causal_softmax_backward(scores[c], probs[c], scores[1 - c], Bs, H, T, 0.125), 2)
    row(f"causal_softmax_backward (B={Bs})", "attention.cu:450", ms, srows * T * 4 + srows * T * 4)  # reads 2 halves, writes all
    # FP32 parity kernels: compute-bound SIMT, reported in TFLOP/s
    o32, m32, l32 = torch.empty_like(q32[0]), torch.empty(B, H, T, device=dev), torch.empty(B, H, T, device=dev)
    dq, dk, dv, ws = torch.empty_like(o32), torch.empty_like(o32), torch.empty_like(o32), torch.empty(B, H, T, device=dev)
    ops.set_math_mode("fp32")
    scale = 1.0 / math.sqrt(d)
    iters = 3
    ms_f = timed(lambda c: ops.tiled_causal_attention_forward(q32[0], k32[0], v32[0], o32, B, H, T, d, scale, m32, l32))
    ms_b = timed(lambda c: ops.tiled_causal_attention_backward(q32[0], k32[0], v32[0], o32, merged[0].view(B, H, T, d), m32,
                                                               l32, dq, dk, dv, ws, B, H, T, d, scale))
    fl = flops(B, H, T, d)
    # interleaved-layout entry points against the chain they replace, BF16 end to end:
    #   chain: (B,T,3C) -> split -> attention fwd -> merge;  merge^T -> attention bwd -> split^T -> (B,T,3C)
    iters = max(5, min(args.steps, 50))
    pq = [ops.fill_normal_(torch.empty(B, T, 3 * H * d, device=dev, dtype=bf16), seed=90 + c) for c in range(copies)]
    pdo = [ops.fill_normal_(torch.empty(B, T, H * d, device=dev, dtype=bf16), seed=95 + c) for c in range(copies)]
    pout = [torch.empty(B, T, H * d, device=dev, dtype=bf16) for _ in range(copies)]
    pdqkv = [torch.empty_like(pq[c]) for c in range(copies)]
    plse = torch.empty(B, H, T, device=dev)
    ops.reserve(B * H, T, d)

    def packed_step(c):
        ops.attention_forward_bf16_packed(pq[c], H, scale, out=pout[c], lse=plse)
        ops.attention_backward_bf16_packed(pq[c], pout[c], pdo[c], plse, H, scale, dqkv=pdqkv[c])

    def chain_step(c):
        x = pq[c].view(B, T, 3, H, d).permute(2, 0, 3, 1, 4).contiguous()          # split (one torch copy kernel)
        o, lse = ops.attention_forward_bf16(x[0], x[1], x[2], scale)
        pout[c].copy_(o.view(B, H, T, d).permute(0, 2, 1, 3).reshape(B, T, H * d))  # merge
        do = pdo[c].view(B, T, H, d).permute(0, 2, 1, 3).contiguous()               # merge^T
        dq_, dk_, dv_ = ops.attention_backward_bf16(x[0], x[1], x[2], o, do, lse, scale)
        g = pdqkv[c].view(B, T, 3, H, d)                                            # split^T
        g[:, :, 0].copy_(dq_.view(B, H, T, d).permute(0, 2, 1, 3))
        g[:, :, 1].copy_(dk_.view(B, H, T, d).permute(0, 2, 1, 3))
        g[:, :, 2].copy_(dv_.view(B, H, T, d).permute(0, 2, 1, 3))

    ms_packed = timed(packed_step, copies)
    ms_chain = timed(chain_step, copies)
    del pq, pdo, pout, pdqkv, qkv, q32, k32, v32, qb, kb, vb, merged, scores, probs
    torch.cuda.empty_cache()
    out.append(time_loss_kernel(pkg, dev, peaks, args.loss_rows))
    print(json.dumps({
        "suite": "path-kernels", "unit": "GB/s", "hbm_peak_gbs": peaks["hbm"], "peak_source": peaks["source"],
        "config": {"workload": workload_name(args, B, H, T, d), "l2": f"{copies} rotating buffer sets"},
        "kernels": out,
        "fp32_parity_mode": {"forward_ms": round(ms_f, 3), "backward_ms": round(ms_b, 3),
                             "tflops": round(fl / ((ms_f + ms_b) * 1e-3) / 1e12, 3),
                             "note": "SIMT FP32, exact expf: the <=1e-5 parity path, not the fast path"},
        "interleaved_layout": {"packed_fwd_bwd_ms": round(ms_packed, 4), "split_attention_merge_chain_ms": round(ms_chain, 4),
                               "packed_tflops": round(fl / (ms_packed * 1e-3) / 1e12, 1),
                               "chain_tflops": round(fl / (ms_chain * 1e-3) / 1e12, 1),
                               "note": "BF16 (B,T,3C) in, (B,T,C) out and back; the chain uses torch copy kernels for the "
                                       "four layout passes that b200attn_*_bf16_packed folds into TMA strides"},
    }), flush=True)


class DeviceWorkload:
    """Seeded BF16 Q, K, V, dO of one workload resident on one GPU (this rank's (batch, head) slabs of a batch
    `world` times the per-GPU batch), rotating over enough buffer sets to exceed L2, and the forward + backward step."""

    def __init__(self, pkg, dev, rank, world, B, H, T, d, strong=False):
        import torch
        self.pkg, self.ops, self.dev, self.torch = pkg, pkg.ops, dev, torch
        ops = self.ops
        # weak: every rank holds one full per-GPU workload; strong: the ranks share the B * H slabs of ONE workload
        mine = pkg.shard.slab_range(B * H * (1 if strong else world), rank, world)
        self.BH, self.T, self.d = mine.count, T, d
        self.n = self.BH * T * d
        self.scale = 1.0 / math.sqrt(d)
        bf16 = torch.bfloat16
        self.set_bytes = 9 * self.n * 2  # q,k,v,o,dO,dq,dk,dv in BF16 + about one tensor of scratch traffic
        self.n_sets = max(2, math.ceil(2.0 * L2_BYTES / self.set_bytes))  # a step's inputs were evicted from L2
        self.sets = []
        for s in range(self.n_sets):
            ts = []
            for i in range(4):  # q, k, v, dO: counter-based streams indexed by global element, distinct per set
                t = torch.empty(self.BH, T, d, device=dev, dtype=bf16)
                ops.fill_normal_(t, seed=1000 + 10 * s + i, offset=pkg.shard.element_offset(mine, T, d))
                ts.append(t)
            q, k, v, dO = ts
            self.sets.append(dict(q=q, k=k, v=v, dO=dO, o=torch.empty_like(q), lse=torch.empty(self.BH, T, device=dev),
                                  dq=torch.empty_like(q), dk=torch.empty_like(q), dv=torch.empty_like(q)))
        ops.reserve(self.BH, T, d)

    def step(self, s):
        ops, scale = self.ops, self.scale
        ops.attention_forward_bf16(s["q"], s["k"], s["v"], scale, s["o"], s["lse"])
        ops.attention_backward_bf16(s["q"], s["k"], s["v"], s["o"], s["dO"], s["lse"], scale, s["dq"], s["dk"], s["dv"])

    def timed_steps(self, steps, warmup, stride, sampler=None, after=0):
        """`warmup` untimed steps, then exactly `steps` steps between barrier + synchronize on both sides, CUDA events on
        the launching stream, maximum over ranks; every `stride`-th launch of each kernel inside the region and every
        launch of `after` further steps behind it is bracketed with events of its own.
        Returns (total ms, per-kernel event times)."""
        torch, ops = self.torch, self.ops
        from transformer_cuda_b200 import dist as pdist
        for i in range(warmup):
            self.step(self.sets[i % self.n_sets])
        torch.cuda.synchronize()
        ops.check_device_fault()
        if sampler:
            sampler.wait_first_sample()
        ops.kernel_timing(True, every=stride)
        pdist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            self.step(self.sets[i % self.n_sets])
        e1.record()
        torch.cuda.synchronize()
        pdist.barrier()
        ms_total = pdist.max_over_ranks(e0.elapsed_time(e1), device=self.dev)
        kt = ops.kernel_times()
        kt["fwd_samples"], kt["bwd_samples"] = ops.kernel_time_samples(False), ops.kernel_time_samples(True)
        # further steps right after the timed region, same buffers and stream, every launch bracketed: the events that
        # cost the timed region its back-to-back launches cost nothing here, so short runs still get enough samples
        kt["region_bwd_launches"], kt["region_fwd_launches"] = kt["bwd_launches"], kt["fwd_launches"]
        if after > 0:
            ops.kernel_timing(True, every=1)
            for i in range(after):
                self.step(self.sets[(steps + i) % self.n_sets])
            torch.cuda.synchronize()
            more = ops.kernel_times()
            for k in ("fwd_ms", "fwd_launches", "bwd_ms", "bwd_launches"):
                kt[k] += more[k]
            kt["fwd_samples"] += ops.kernel_time_samples(False)
            kt["bwd_samples"] += ops.kernel_time_samples(True)
        ops.kernel_timing(False)
        return ms_total, kt

    def timed_graph_steps(self, steps, warmup):
        """The same `steps` steps replayed from CUDA graphs captured once per buffer set (the reference's benchmark has such
        a mode, src/benchmark.cu:158-175), barrier + synchronize on both sides, maximum over ranks. Returns total ms."""
        torch, ops = self.torch, self.ops
        from transformer_cuda_b200 import dist as pdist
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graphs = []
            for s_ in self.sets:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    self.step(s_)
                graphs.append(g)
            for i in range(max(3, warmup)):
                graphs[i % self.n_sets].replay()
            side.synchronize()
            pdist.barrier()
            torch.cuda.synchronize()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record(side)
            for i in range(steps):
                graphs[i % self.n_sets].replay()
            g1.record(side)
            torch.cuda.synchronize()
            pdist.barrier()
        torch.cuda.current_stream().wait_stream(side)
        ms_total = pdist.max_over_ranks(g0.elapsed_time(g1), device=self.dev)
        ops.check_device_fault()
        del graphs
        return ms_total


GRAPH_BELOW_MS = 1.0     # steps shorter than this are launch-bound from Python: timed from CUDA graph replay as well
SAMPLED_STEPS_AFTER = 8  # steps behind the timed region whose every kernel launch is bracketed with events


def default_event_stride(steps):
    """Which launches of the timed region carry events of their own. An event between two kernels undoes their
    programmatic back-to-back launch for that step (about a quarter of a c2 step), so the sampled share of the region
    is kept small: about eight launches of a long run, four of a run of a few dozen steps."""
    return max(1, steps // 8) if steps >= 160 else max(1, -(-steps // 4))


def fwd_kernel_name(T, d):
    """The forward variant launch_attn_fwd_tc dispatches to (csrc/attn_tc_fwd.cu): the two-CTAs-per-SM kernel for
    d = 64 and for d = 128 up to T = 4096, the one-CTA-per-SM kernel beyond."""
    return "attn_fwd_tc_short_kernel" if (d == 64 or T <= 4096) else "attn_fwd_tc_kernel"


def median(xs):
    xs = sorted(xs)
    return 0.0 if not xs else (xs[len(xs) // 2] if len(xs) & 1 else 0.5 * (xs[len(xs) // 2 - 1] + xs[len(xs) // 2]))


def kernel_rooflines(kt, BH, T, d, peaks):
    """Per-launch duration (the median of the sampled launches) and the rate it means, backward and forward kernel."""
    bwd_ms = median(kt["bwd_samples"])
    fwd_ms = median(kt["fwd_samples"])
    bwd_tf = 5.0 * BH * T * T * d / (bwd_ms * 1e-3) / 1e12 if bwd_ms > 0 else 0.0
    fwd_tf = 2.0 * BH * T * T * d / (fwd_ms * 1e-3) / 1e12 if fwd_ms > 0 else 0.0
    return bwd_ms, fwd_ms, bwd_tf, fwd_tf


def extra_workloads(pkg, dev, rank, world, local, peaks, names):
    """Device-timed forward + backward of the other benchmark shapes (long context, the scaling sweep), a short
    run each (about half a second of steps after 3 warm-up steps), each with its own clock record."""
    import torch
    from transformer_cuda_b200 import dist as pdist
    out = {}
    # with more than one GPU, the fixed-size problems sharded by (batch, head) as well: strong scaling of c2 and c3
    runs = [(n, False) for n in names] + ([(n, True) for n in ("c2", "c3") if world > 1 and n in WORKLOADS])
    for name, strong in runs:
        B, H, T, d = WORKLOADS[name]
        if strong and B * H < world:
            continue
        W = DeviceWorkload(pkg, dev, rank, world, B, H, T, d, strong=strong)
        # calibrate the step count on three untimed steps
        for i in range(3):
            W.step(W.sets[i % W.n_sets])
        torch.cuda.synchronize()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for i in range(3):
            W.step(W.sets[i % W.n_sets])
        c1.record()
        torch.cuda.synchronize()
        est = pdist.max_over_ranks(c0.elapsed_time(c1), device=dev) / 3
        steps = int(max(8, min(400, math.ceil(500.0 / max(est, 1e-3)))))
        sampler = ClockSampler(local) if rank == 0 else None
        ms_total, kt = W.timed_steps(steps, 3, default_event_stride(steps), sampler, after=SAMPLED_STEPS_AFTER)
        stream_ms = ms_total / steps
        graph_ms = W.timed_graph_steps(steps, 3) / steps if stream_ms < GRAPH_BELOW_MS else None
        clocks = sampler.stop() if sampler else None
        ms = graph_ms if graph_ms is not None else stream_ms
        fl = pdist.sum_over_ranks(flops(1, W.BH, T, d), device=dev)
        value = fl / (ms * 1e-3) / 1e12
        bwd_ms, fwd_ms, bwd_tf, fwd_tf = kernel_rooflines(kt, W.BH, T, d, peaks)
        out[name + "_strong" if strong else name] = {
                     "workload": f"B={B} H={H} T={T} d={d} " + (f"in total, {W.BH} of its {B * H} (batch, head) slabs on each of {world} GPUs"
                                                            if strong else "per GPU"),
                     "scaling": "strong" if strong else "weak", "steps": steps, "warmup": 6, "ms_per_step": ms,
                     "value": value, "unit": UNIT, "frac_of_bf16_peak": value / world / peaks["bf16"],
                     "frac_of_bf16_sustained_peak": value / world / peaks["bf16_sustained"],
                     "bwd_kernel": {"launch_ms": bwd_ms, "achieved": bwd_tf, "frac": bwd_tf / peaks["bf16"],
                                    "timed_launches": kt["bwd_launches"]},
                     "fwd_kernel": {"kernel": fwd_kernel_name(T, d), "launch_ms": fwd_ms, "achieved": fwd_tf,
                                    "frac": fwd_tf / peaks["bf16"], "timed_launches": kt["fwd_launches"]},
                     "launch": "cuda graph replay" if graph_ms is not None else "stream",
                     "stream_launched_value": fl / (stream_ms * 1e-3) / 1e12,
                     "l2": f"{W.n_sets} rotating buffer sets", "clocks": clocks}
        del W
        torch.cuda.empty_cache()
        pkg.ops.release()
    return out


def workload_name(args, B, H, T, d):
    return f"{args.workload}: causal attention fwd+bwd, B={B} H={H} T={T} d={d} per GPU, BF16, scale=1/sqrt(d)"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + ["c4"],
                    help="c2 (default), c3, c5_*: the attention path; c4: the data-parallel GPT training step around it")
    ap.add_argument("--cpu-budget-s", type=float, default=12.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gemm", default="bf16", choices=["reference", "fp32", "bf16"],
                    help="c4 only: the model's GEMM wrappers - the reference's own FP32 ones, or the drop-in in FP32 / BF16 arithmetic")
    ap.add_argument("--loss-adamw", default="dropin", choices=["reference", "dropin"],
                    help="c4 only, with a GEMM drop-in: the model's loss launcher and optimizer - the reference's, or the drop-ins")
    ap.add_argument("--kernel-event-stride", type=int, default=0,
                    help="bracket every N-th launch of each tensor-core kernel with CUDA events inside the timed region "
                         "(roofline durations); events between kernels undo their back-to-back launch, so N=1 slows the "
                         "step. Default 0 = steps // 8 for 160 steps or more, a quarter of the steps rounded up below; "
                         "every launch of eight further steps behind the timed region is sampled as well")
    ap.add_argument("--extra", default="c3,c5_512,c5_1024,c5_2048,c5_4096,c5_8192,c5_16384",
                    help="comma-separated other workloads measured briefly (device-timed) after the main one and reported "
                         "under `extra`; empty string: none")
    ap.add_argument("--loss-rows", type=int, default=16384, help="rows of 50257 logits for the loss-kernel timing")
    ap.add_argument("--suite", default="attention", choices=["attention", "path-kernels", "loss"],
                    help="'path-kernels': time every other launcher of the path (layout, softmax, pre-pass, FP32 parity "
                         "kernels) against the HBM roofline and print one JSON line with a table")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.workload == "c4":
        run_gpt_step(args)
        return
    B, H, T, d = WORKLOADS[args.workload]

    if args.impl == "reference":
        run_reference(args, B, H, T, d)
        return
    if args.suite == "path-kernels":
        run_path_kernels(args, B, H, T, d)
        return
    if args.suite == "loss":
        run_loss_kernel(args)
        return

    import torch
    import __graft_entry__ as entry
    pkg = entry.load_package()
    ops = pkg.ops
    from transformer_cuda_b200 import dist as pdist

    rank, world, local = pdist.init()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU fallback (use --impl reference for the CPU arm)")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)

    # ---- weak scaling: the global batch is `world` times the per-GPU batch, split by (batch, head) slabs
    stride = args.kernel_event_stride if args.kernel_event_stride > 0 else default_event_stride(args.steps)
    sampler = ClockSampler(local) if rank == 0 else None  # started early: nvidia-smi needs a moment to come up
    W = DeviceWorkload(pkg, dev, rank, world, B, H, T, d)
    BH, n, scale, sets, n_sets, set_bytes, step = W.BH, W.n, W.scale, W.sets, W.n_sets, W.set_bytes, W.step
    ms_total, kt = W.timed_steps(args.steps, args.warmup, stride, sampler, after=SAMPLED_STEPS_AFTER)

    # ---- the same K steps replayed from CUDA graphs, one captured per buffer set (the reference's benchmark has such a
    # mode, src/benchmark.cu:158-175), for steps short enough for launch overhead to matter. Where it runs it is the
    # headline: a step of four kernels of 7-60 us is launch-bound from Python until the host has run far enough ahead for
    # the kernels' programmatic overlap to engage, which a run of a few dozen steps never reaches; the stream-launched
    # region above is reported beside it and carries the per-kernel events.
    graph_ms = None
    if ms_total / args.steps < GRAPH_BELOW_MS:
        graph_ms = W.timed_graph_steps(args.steps, args.warmup) / args.steps
    clocks = sampler.stop() if sampler else None
    ops.check_device_fault()
    stream_ms_per_step = ms_total / args.steps
    ms_per_step = graph_ms if graph_ms is not None else stream_ms_per_step
    step_flops = flops(1, BH, T, d)
    all_flops = pdist.sum_over_ranks(step_flops, device=dev)
    value = all_flops / (ms_per_step * 1e-3) / 1e12

    # ---- end to end: pinned host buffers -> device -> forward + backward -> host, every step.
    # Every step copies its own inputs in and its own results out; the three legs run on three streams
    # over two device buffer sets, so step i+1's upload and step i-1's download overlap step i's kernels.
    bf16 = torch.bfloat16
    host_in = [torch.empty(BH, T, d, dtype=bf16).pin_memory() for _ in range(4)]
    for hbuf, key in zip(host_in, ("q", "k", "v", "dO")):
        hbuf.copy_(sets[0][key])
    host_out = [[torch.empty(BH, T, d, dtype=bf16).pin_memory() for _ in range(4)] for _ in range(2)]
    e2e_sets = [sets[-1], sets[-2]]
    e2e_steps = max(4, min(args.steps, 40))
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    s_cmp = torch.cuda.current_stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_cmp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_step(i):
        b = i & 1
        st = e2e_sets[b]
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(ev_cmp[b])  # the kernels of step i-2 have consumed this set's inputs
            for hbuf, key in zip(host_in, ("q", "k", "v", "dO")):
                st[key].copy_(hbuf, non_blocking=True)
            ev_in[b].record(s_in)
        s_cmp.wait_event(ev_in[b])
        if i >= 2:
            s_cmp.wait_event(ev_out[b])  # the results of step i-2 have left this set's output buffers
        step(st)
        ev_cmp[b].record(s_cmp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_cmp[b])
            for hbuf, key in zip(host_out[b], ("o", "dq", "dk", "dv")):
                hbuf.copy_(st[key], non_blocking=True)
            ev_out[b].record(s_out)

    for i in range(4):
        e2e_step(i)
    torch.cuda.synchronize()
    pdist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    torch.cuda.synchronize()  # all three streams: the last result is on the host
    wall_ms = (time.perf_counter() - t0) * 1e3
    pdist.barrier()
    e2e_ms = pdist.max_over_ranks(wall_ms, device=dev) / e2e_steps
    e2e_value = all_flops / (e2e_ms * 1e-3) / 1e12
    # the last step's results, read on the host: a checksum proves the data made the round trip
    e2e_checksum = float(host_out[(e2e_steps - 1) & 1][0].float().abs().mean())

    # ---- the ceiling of that loop: the same pinned buffers, streams and event chain with no kernel in between.
    # With N ranks copying at once the host's memory system and the PCIe root complexes are shared, so this is
    # measured at every N; e2e is then reported as a fraction of it.
    def copy_only_step(i):
        b = i & 1
        st = e2e_sets[b]
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(ev_out[b])
            for hbuf, key in zip(host_in, ("q", "k", "v", "dO")):
                st[key].copy_(hbuf, non_blocking=True)
            ev_in[b].record(s_in)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_in[b])
            for hbuf, key in zip(host_out[b], ("o", "dq", "dk", "dv")):
                hbuf.copy_(st[key], non_blocking=True)
            ev_out[b].record(s_out)

    for i in range(4):
        copy_only_step(i)
    torch.cuda.synchronize()
    pdist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        copy_only_step(i)
    torch.cuda.synchronize()
    copy_wall_ms = (time.perf_counter() - t0) * 1e3
    pdist.barrier()
    copy_ms = pdist.max_over_ranks(copy_wall_ms, device=dev) / e2e_steps

    # ---- the other benchmark shapes, briefly (every rank takes part: weak scaling like the main workload)
    peaks = measured_peaks()
    extra_names = [x for x in args.extra.split(",") if x and x != args.workload]
    del W, sets, e2e_sets, step
    host_in = host_out = None
    torch.cuda.empty_cache()
    ops.release()
    extra = extra_workloads(pkg, dev, rank, world, local, peaks, extra_names) if extra_names else {}

    if rank != 0:
        if world > 1:
            torch.distributed.destroy_process_group()
        return

    bwd_ms, fwd_ms, bwd_tf, fwd_tf = kernel_rooflines(kt, BH, T, d, peaks)
    # algorithmic HBM bytes of one step: BF16 q,k,v read + o written + lse (forward); q,k,v,o,dO read + dq,dk,dv
    # written + lse (backward) = 24 bytes per element of one tensor, 8 per row
    step_bytes = 24 * n + 8 * BH * T
    hbm_gbs = step_bytes / (ms_per_step * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": workload_name(args, B, H, T, d), "global_batch": B * world,
                   "sharding": f"(batch,head) slabs, {B * H} per GPU, no collective",
                   "l2": f"inputs rotate over {n_sets} buffer sets ({n_sets * set_bytes >> 20} MiB > L2) so a step reads from HBM",
                   "launch": ("each step (forward, backward pre-pass, backward, dQ convert) replayed from a CUDA graph "
                              "captured once per buffer set; the same K steps launched on the stream: `stream_launched`")
                             if graph_ms is not None else "each step's kernels launched on the stream",
                   "flops_per_step_per_gpu": step_flops},
        "frac_of_bf16_peak": value / world / peaks["bf16"],
        "tokens_per_s": B * world * T / (ms_per_step * 1e-3),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 4 * n * 2, "d2h_bytes_per_step": 4 * n * 2,
                "ms_per_step": e2e_ms, "steps": e2e_steps, "timing": "host wall clock around the steps, synchronised both sides",
                "copy_only": {"ms_per_step": copy_ms, "gbs_per_gpu_each_way": 4 * n * 2 / (copy_ms * 1e-3) / 1e9,
                              "e2e_frac_of_copy_only": copy_ms / e2e_ms,
                              "note": "the same pinned buffers, streams and events with no kernel in between: the ceiling "
                                      "the host<->device copy leg sets at this number of GPUs"},
                "host_result_checksum": e2e_checksum,
                "path": "pinned host BF16 q,k,v,dO -> device -> b200attn_fwd_bf16 + b200attn_bwd_bf16 -> host o,dq,dk,dv; "
                        "upload, kernels and download of consecutive steps overlap on three streams"},
        "gpu_launches": 4 * args.steps,  # per step: forward kernel, backward pre-pass, backward kernel, dQ convert
        "roofline": {"bound": "tensor", "kernel": "attn_bwd_tc64_kernel" if d == 64 else "attn_bwd_tc_kernel", "achieved": bwd_tf, "peak": peaks["bf16"],
                     "unit": UNIT, "frac": bwd_tf / peaks["bf16"], "peak_source": f"{peaks['source']} (burst cuBLAS BF16)",
                     "traffic": ncu_traffic_per_launch(args.workload), "launch_ms": bwd_ms,
                     "launch_ms_mean": kt["bwd_ms"] / max(1, kt["bwd_launches"]),
                     "timed_launches": kt["bwd_launches"], "of_which_inside_timed_region": kt["region_bwd_launches"],
                     "timing": f"CUDA events around every {stride}-th launch inside the stream-launched timed region and around every launch "
                               f"of {SAMPLED_STEPS_AFTER} further steps right behind it (median over all of them)",
                     "flops_per_launch": 5.0 * BH * T * T * d,
                     "forward_kernel": {"kernel": fwd_kernel_name(T, d), "achieved": fwd_tf, "launch_ms": fwd_ms,
                                        "frac": fwd_tf / peaks["bf16"], "timed_launches": kt["fwd_launches"]},
                     "hbm": {"bound": "hbm", "achieved": hbm_gbs, "peak": peaks["hbm"], "unit": "GB/s",
                             "frac": hbm_gbs / peaks["hbm"], "bytes_per_step": step_bytes,
                             "note": "algorithmic bytes of a whole step over ms_per_step: the step is not HBM-bound"}},
        "clocks": clocks,
    }
    if extra:
        line["extra"] = extra
    if graph_ms is not None:
        line["stream_launched"] = {"ms_per_step": stream_ms_per_step, "value": all_flops / (stream_ms_per_step * 1e-3) / 1e12,
                                   "unit": UNIT, "steps": args.steps,
                                   "note": "the same K steps launched kernel by kernel from Python, barrier + synchronize on "
                                           "both sides; the launches that carry the roofline's events are inside this region"}
    if world == 1 and not args.no_cpu_baseline:  # the CPU arm runs beside the 1-GPU measurement only
        line["cpu_baseline"] = cpu_baseline(B, H, T, d, args.cpu_budget_s)
    print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
