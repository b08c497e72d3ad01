"""Builds the engine in-tree with nvcc for sm_100a: lib/libb200attn.so (C ABI + the C++ launch API)
and lib/libb200attn.a (the same objects, for static linking in place of the reference's
src/kernels/attention.cu); beside them the drop-ins for the callers of the path: lib/libb200gemm.a
(src/kernels/matmul.cu), lib/libb200loss.so / .a (src/kernels/loss.cu) and lib/libb200norm.a
(src/kernels/layernorm.cu), lib/libb200ffn.a (src/kernels/ffn.cu). Rebuilds only when a source is newer than the library."""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(LIBDIR, "obj")
SOURCES = ["api.cu", "launch_api.cu", "layout_kernels.cu", "softmax_kernels.cu", "attn_f32.cu", "attn_f32_tiled.cu", "attn_tc_fwd.cu", "attn_tc_fwd_short.cu",
           "attn_tc_bwd.cu", "attn_tc_bwd64.cu", "static_scratch.cu", "wait_selftest.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall"]
SO = os.path.join(LIBDIR, "libb200attn.so")
AR = os.path.join(LIBDIR, "libb200attn.a")
GEMM_AR = os.path.join(LIBDIR, "libb200gemm.a")
NORM_AR = os.path.join(LIBDIR, "libb200norm.a")
FFN_AR = os.path.join(LIBDIR, "libb200ffn.a")
LOSS_SO = os.path.join(LIBDIR, "libb200loss.so")
LOSS_AR = os.path.join(LIBDIR, "libb200loss.a")


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the engine has no prebuilt or CPU fallback")


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose=False, force=False, ptxas_info=False):
    os.makedirs(OBJDIR, exist_ok=True)
    nvcc = _nvcc()
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers += [os.path.join(HERE, "..", "include", "b200attn.h"),
                os.path.join(HERE, "..", "include", "kernels", "attention.cuh")]
    objs, procs = [], []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJDIR, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + headers):
            cmd = [nvcc] + ARCH + FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", s, "-o", o]
            if verbose:
                print(" ".join(cmd), flush=True)
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"--- nvcc failed for {src} ---\n{out}\n")
        elif verbose or ptxas_info:
            print(out)
    if failed:
        raise RuntimeError("nvcc compilation failed")
    if force or _stale(SO, objs):
        subprocess.check_call([nvcc] + ARCH + ["-shared", "-o", SO] + objs + ["-lcudart"])
    if force or _stale(AR, objs):
        if os.path.exists(AR):
            os.remove(AR)
        subprocess.check_call(["ar", "rcs", AR] + objs)
    # the GEMM drop-in for the reference model (links against cuBLAS, so it stays out of libb200attn): the wrappers and
    # the hand-written tcgen05 GEMM they can route staged products to
    gemm_objs = []
    gemm_hdrs = [os.path.join(HERE, "..", "include", "kernels", "matmul.cuh"), os.path.join(HERE, "gemm", "gemm_tc.h"),
                 os.path.join(CSRC, "tc_common.cuh")]
    for name in ("matmul_dropin", "gemm_tc"):
        src = os.path.join(HERE, "gemm", name + ".cu")
        obj = os.path.join(OBJDIR, name + ".o")
        gemm_objs.append(obj)
        if force or _stale(obj, [src] + gemm_hdrs):
            subprocess.check_call([nvcc] + ARCH + FLAGS + ["-I", os.path.join(HERE, "..", "include"), "-I", CSRC, "-c", src, "-o", obj])
    if force or _stale(GEMM_AR, gemm_objs):
        if os.path.exists(GEMM_AR):
            os.remove(GEMM_AR)
        subprocess.check_call(["ar", "rcs", GEMM_AR] + gemm_objs)
    # the loss drop-in (fused softmax cross-entropy): its own shared + static library, no dependency on the attention engine
    loss_src = os.path.join(HERE, "loss", "cross_entropy.cu")
    loss_obj = os.path.join(OBJDIR, "cross_entropy.o")
    loss_deps = [loss_src, os.path.join(CSRC, "tc_common.cuh"), os.path.join(HERE, "..", "include", "kernels", "loss.cuh"),
                 os.path.join(HERE, "..", "include", "b200loss.h")]
    if force or _stale(loss_obj, loss_deps):
        subprocess.check_call([nvcc] + ARCH + FLAGS + ["-I", os.path.join(HERE, "..", "include"), "-I", CSRC, "-c", loss_src, "-o", loss_obj])
    if force or _stale(LOSS_SO, [loss_obj]):
        subprocess.check_call([nvcc] + ARCH + ["-shared", "-o", LOSS_SO, loss_obj, "-lcudart"])
    if force or _stale(LOSS_AR, [loss_obj]):
        if os.path.exists(LOSS_AR):
            os.remove(LOSS_AR)
        subprocess.check_call(["ar", "rcs", LOSS_AR, loss_obj])
    # the LayerNorm drop-in (static library only: its interface is the C++ header of the reference)
    norm_src = os.path.join(HERE, "norm", "layernorm_dropin.cu")
    norm_obj = os.path.join(OBJDIR, "layernorm_dropin.o")
    if force or _stale(norm_obj, [norm_src, os.path.join(HERE, "..", "include", "kernels", "layernorm.cuh")]):
        subprocess.check_call([nvcc] + ARCH + FLAGS + ["--use_fast_math", "-I", os.path.join(HERE, "..", "include"), "-c", norm_src, "-o", norm_obj])
    if force or _stale(NORM_AR, [norm_obj]):
        if os.path.exists(NORM_AR):
            os.remove(NORM_AR)
        subprocess.check_call(["ar", "rcs", NORM_AR, norm_obj])
    # the GELU drop-in
    ffn_src = os.path.join(HERE, "ffn", "gelu_dropin.cu")
    ffn_obj = os.path.join(OBJDIR, "gelu_dropin.o")
    if force or _stale(ffn_obj, [ffn_src, os.path.join(HERE, "..", "include", "kernels", "ffn.cuh")]):
        subprocess.check_call([nvcc] + ARCH + FLAGS + ["--use_fast_math", "-I", os.path.join(HERE, "..", "include"), "-c", ffn_src, "-o", ffn_obj])
    if force or _stale(FFN_AR, [ffn_obj]):
        if os.path.exists(FFN_AR):
            os.remove(FFN_AR)
        subprocess.check_call(["ar", "rcs", FFN_AR, ffn_obj])
    return SO


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv, ptxas_info="--ptxas" in sys.argv))
