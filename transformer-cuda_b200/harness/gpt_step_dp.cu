// Data-parallel GPT training step around the reference model (config 4 of the benchmark spec).
//
// One process per GPU. Each rank owns a full replica of sarimahsan/transformer-cuda's
// TransformerModel (its own src/model.cu, compiled unmodified from the reference checkout) with
// use_tiled_attention = true, so every attention launcher of the step - qkv_split_transpose_*,
// tiled_causal_attention_forward/backward, head_merge_transpose_* - resolves to whichever attention
// object the binary is linked against: libb200attn (this engine) or the reference's own
// src/kernels/attention.cu (the "reference kernels on the same GPU" arm). Per step:
//
//     forward -> backward -> ncclAllReduce(avg) of the contiguous gradient buffer over NVLink
//             -> AdamW::fused_step (global-norm clip + AdamW + zero-grad)
//
// The mean over ranks is taken inside the collective (ncclAvg), so no separate pass scales the 163 M-float buffer.
//
// The all-reduce runs once per step on the finished buffer, before fused_step, because the
// reference accumulates bias / LayerNorm / embedding gradients with atomics into a buffer that
// fused_step clears (src/optimizer.cu:225-249). Attention itself issues no collective.
// Ranks find each other through RANK / WORLD_SIZE / LOCAL_RANK (torchrun's variables); the NCCL
// unique id travels through a file named after MASTER_PORT in /tmp. Rank 0 prints one JSON line.
//
//   gpt_step_dp [--steps K] [--warmup W] [--B 16] [--T 1024] [--C 768] [--L 12] [--H 12] [--V 50257]
#include <nccl.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

#include "common.h"
#include "config.h"
#include "model.h"
#include "optimizer.h"
#ifdef B200ATTN_DROPIN
#include "b200attn.h"
#endif

#define NCCL_CHECK(x)                                                                       \
    do {                                                                                    \
        ncclResult_t r_ = (x);                                                              \
        if (r_ != ncclSuccess) {                                                            \
            fprintf(stderr, "NCCL error %s at %s:%d\n", ncclGetErrorString(r_), __FILE__, __LINE__); \
            exit(2);                                                                        \
        }                                                                                   \
    } while (0)

static int env_int(const char* name, int dflt) {
    const char* s = getenv(name);
    return s ? atoi(s) : dflt;
}

// Counters of the GEMM drop-in, present when libb200gemm is linked in (weak: the other builds have none).
extern "C" long long b200gemm_tc_launches(void) __attribute__((weak));
extern "C" long long b200gemm_staged_reuses(void) __attribute__((weak));
extern "C" long long b200gemm_twin_hits(void) __attribute__((weak));

// Hook of the LayerNorm drop-in (weak: builds that link the reference's own layernorm.cu have none).
extern "C" void b200norm_set_backward_hook(void (*fn)(int, cudaStream_t, void*), void* user) __attribute__((weak));
extern "C" void b200norm_reset_backward_count(void) __attribute__((weak));

// Bucketed all-reduce overlapped with the backward pass. The gradient buffer is laid out [embeddings | layer 0 ... layer
// L-1 | final LayerNorm | head] (src/model.cu:45-58) and the backward pass finishes those parts from the back: head and
// final LayerNorm first (done once the final LayerNorm's backward has been launched: the 1st layernorm_backward call), then
// layer L-1 (its LN1 backward is the 3rd call), ... layer 0 (call 1 + 2 L), the embeddings last. After each of those calls
// the part that has just become final is all-reduced in place on a second stream, ordered behind the compute stream by an
// event; the optimizer waits for the second stream. Every rank issues the same collectives in the same order.
struct OverlapState {
    ncclComm_t comm = nullptr;
    cudaStream_t comm_stream = nullptr;
    float* base = nullptr;
    std::vector<std::pair<size_t, size_t>> part_after_call;  // [call index] -> (offset, count); count 0: nothing
    std::vector<cudaEvent_t> events;
};
static void reduce_part(OverlapState* o, size_t offset, size_t count, cudaEvent_t ev, cudaStream_t compute) {
    CUDA_CHECK(cudaEventRecord(ev, compute));
    CUDA_CHECK(cudaStreamWaitEvent(o->comm_stream, ev, 0));
    NCCL_CHECK(ncclAllReduce(o->base + offset, o->base + offset, count, ncclFloat, ncclAvg, o->comm, o->comm_stream));
}
static void on_layernorm_backward(int call, cudaStream_t stream, void* user) {
    OverlapState* o = static_cast<OverlapState*>(user);
    if (call >= (int)o->part_after_call.size() || o->part_after_call[call].second == 0) return;
    reduce_part(o, o->part_after_call[call].first, o->part_after_call[call].second, o->events[call], stream);
}

int main(int argc, char** argv) {
    int steps = 5, warmup = 2;
    TransformerConfig cfg;
    cfg.batch_size = 16;
    cfg.max_seq_len = 1024;
    cfg.d_model = 768;
    cfg.num_layers = 12;
    cfg.num_heads = 12;
    cfg.vocab_size = 50257;
    cfg.learning_rate = 3e-4f;
    cfg.beta1 = 0.9f;
    cfg.beta2 = 0.95f;
    cfg.weight_decay = 0.1f;
    cfg.grad_clip = 1.0f;
    for (int i = 1; i + 1 < argc; i += 2) {
        std::string a = argv[i];
        long v = atol(argv[i + 1]);
        if (a == "--steps") steps = (int)v;
        else if (a == "--warmup") warmup = (int)v;
        else if (a == "--B") cfg.batch_size = v;
        else if (a == "--T") cfg.max_seq_len = v;
        else if (a == "--C") cfg.d_model = v;
        else if (a == "--L") cfg.num_layers = v;
        else if (a == "--H") cfg.num_heads = v;
        else if (a == "--V") cfg.vocab_size = v;
        else { fprintf(stderr, "unknown option %s\n", a.c_str()); return 1; }
    }
    cfg.d_head = cfg.d_model / cfg.num_heads;
    cfg.d_ff = 4 * cfg.d_model;
    cfg.use_tiled_attention = true;

    const int rank = env_int("RANK", 0), world = env_int("WORLD_SIZE", 1), local = env_int("LOCAL_RANK", rank);
    CUDA_CHECK(cudaSetDevice(local));

    ncclComm_t comm = nullptr;
    if (world > 1) {
        ncclUniqueId id;
        const std::string path = std::string("/tmp/b200attn_nccl_") + (getenv("MASTER_PORT") ? getenv("MASTER_PORT") : "0") + ".id";
        if (rank == 0) {
            NCCL_CHECK(ncclGetUniqueId(&id));
            const std::string tmp = path + ".tmp";
            std::ofstream f(tmp, std::ios::binary);
            f.write(reinterpret_cast<const char*>(&id), sizeof(id));
            f.close();
            rename(tmp.c_str(), path.c_str());
        } else {
            bool ok = false;
            for (int tries = 0; tries < 6000 && !ok; ++tries) {  // up to a minute
                std::ifstream f(path, std::ios::binary);
                if (f.good() && f.read(reinterpret_cast<char*>(&id), sizeof(id))) ok = true;
                else usleep(10000);
            }
            if (!ok) { fprintf(stderr, "rank %d: no NCCL id at %s\n", rank, path.c_str()); return 2; }
        }
        NCCL_CHECK(ncclCommInitRank(&comm, world, id, rank));
        if (rank == 0) { usleep(200000); unlink(path.c_str()); }
    }

    TransformerModel model(cfg);  // identical initial weights on every rank (seed 42 inside the reference)
    AdamW optimizer(model.get_params_memory(), model.get_grads_memory(), model.get_num_parameters(), cfg);
    const int B = (int)cfg.batch_size, T = (int)cfg.max_seq_len;
    const size_t n_tok = (size_t)B * T, n_params = model.get_num_parameters();
#ifdef B200ATTN_DROPIN
    b200attn_reserve(B * (int)cfg.num_heads, T, (int)cfg.d_head);
#endif

    std::vector<int> h_tok(n_tok), h_tgt(n_tok);
    unsigned long long s = 0x9E3779B97F4A7C15ull * (unsigned long long)(rank + 1);  // distinct data per rank
    auto next = [&]() { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return s; };
    for (size_t i = 0; i < n_tok; ++i) {
        h_tok[i] = (int)(next() % cfg.vocab_size);
        h_tgt[i] = (int)(next() % cfg.vocab_size);
    }
    int *d_tok, *d_tgt;
    CUDA_CHECK(cudaMalloc(&d_tok, n_tok * sizeof(int)));
    CUDA_CHECK(cudaMalloc(&d_tgt, n_tok * sizeof(int)));
    CUDA_CHECK(cudaMemcpy(d_tok, h_tok.data(), n_tok * sizeof(int), cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(d_tgt, h_tgt.data(), n_tok * sizeof(int), cudaMemcpyHostToDevice));

    cudaStream_t stream;
    CUDA_CHECK(cudaStreamCreate(&stream));
    float* d_time;
    CUDA_CHECK(cudaMalloc(&d_time, sizeof(float)));
    float host_loss = 0.f;

    // overlapped, bucketed all-reduce: needs the LayerNorm drop-in's hook; B200_DP_OVERLAP=0 keeps the single all-reduce
    OverlapState overlap;
    const bool use_overlap = world > 1 && b200norm_set_backward_hook != nullptr && env_int("B200_DP_OVERLAP", 1) != 0;
    cudaEvent_t tail_event = nullptr, comm_done = nullptr;
    size_t embeddings_count = 0;
    if (use_overlap) {
        const TransformerParameters& gp = model.get_gradients().params;
        const int L = (int)cfg.num_layers;
        overlap.comm = comm, overlap.base = model.get_grads_memory();
        CUDA_CHECK(cudaStreamCreateWithFlags(&overlap.comm_stream, cudaStreamNonBlocking));
        overlap.part_after_call.assign(2 * L + 2, std::make_pair(size_t(0), size_t(0)));
        overlap.events.resize(2 * L + 2);
        for (auto& e : overlap.events) CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        const size_t off_lnf = gp.ln_f_gamma - overlap.base;
        overlap.part_after_call[1] = {off_lnf, n_params - off_lnf};  // final LayerNorm + head
        for (int l = L - 1; l >= 0; --l) {
            const size_t begin = gp.layers[l].ln1_gamma - overlap.base;
            const size_t end = (l + 1 < L ? gp.layers[l + 1].ln1_gamma : gp.ln_f_gamma) - overlap.base;
            overlap.part_after_call[1 + 2 * (L - l)] = {begin, end - begin};
        }
        embeddings_count = (L > 0 ? gp.layers[0].ln1_gamma : gp.ln_f_gamma) - overlap.base;
        CUDA_CHECK(cudaEventCreateWithFlags(&tail_event, cudaEventDisableTiming));
        CUDA_CHECK(cudaEventCreateWithFlags(&comm_done, cudaEventDisableTiming));
        b200norm_set_backward_hook(on_layernorm_backward, &overlap);
    }

    // events around every all-reduce of the timed steps: the collective's share of a step is reported (with the overlap:
    // the part of it the compute stream waits for after the backward pass)
    std::vector<cudaEvent_t> ar_events;
    bool time_allreduce = false;
    auto step = [&](float* loss) {
        model.forward(d_tok, stream);
        if (use_overlap) b200norm_reset_backward_count();
        model.backward(d_tok, d_tgt, loss, stream);
        if (use_overlap) {
            cudaEvent_t a0 = nullptr, a1 = nullptr;
            if (time_allreduce) {
                CUDA_CHECK(cudaEventCreate(&a0));
                CUDA_CHECK(cudaEventCreate(&a1));
                CUDA_CHECK(cudaEventRecord(a0, stream));
            }
            reduce_part(&overlap, 0, embeddings_count, tail_event, stream);  // the embeddings: final only now
            CUDA_CHECK(cudaEventRecord(comm_done, overlap.comm_stream));
            CUDA_CHECK(cudaStreamWaitEvent(stream, comm_done, 0));
            if (time_allreduce) {
                CUDA_CHECK(cudaEventRecord(a1, stream));
                ar_events.push_back(a0);
                ar_events.push_back(a1);
            }
        } else if (world > 1) {
            cudaEvent_t a0 = nullptr, a1 = nullptr;
            if (time_allreduce) {
                CUDA_CHECK(cudaEventCreate(&a0));
                CUDA_CHECK(cudaEventCreate(&a1));
                CUDA_CHECK(cudaEventRecord(a0, stream));
            }
            NCCL_CHECK(ncclAllReduce(model.get_grads_memory(), model.get_grads_memory(), n_params, ncclFloat, ncclAvg, comm, stream));
            if (time_allreduce) {
                CUDA_CHECK(cudaEventRecord(a1, stream));
                ar_events.push_back(a0);
                ar_events.push_back(a1);
            }
        }
        optimizer.fused_step(cfg.learning_rate, cfg.grad_clip, stream);
    };

    for (int i = 0; i < warmup; ++i) step(nullptr);
    CUDA_CHECK(cudaStreamSynchronize(stream));
    if (world > 1) {  // barrier: a tiny all-reduce
        NCCL_CHECK(ncclAllReduce(d_time, d_time, 1, ncclFloat, ncclMax, comm, stream));
        CUDA_CHECK(cudaStreamSynchronize(stream));
    }
    cudaEvent_t e0, e1;
    CUDA_CHECK(cudaEventCreate(&e0));
    CUDA_CHECK(cudaEventCreate(&e1));
    time_allreduce = true;
    CUDA_CHECK(cudaEventRecord(e0, stream));
    for (int i = 0; i < steps; ++i) step(i == steps - 1 ? &host_loss : nullptr);
    CUDA_CHECK(cudaEventRecord(e1, stream));
    CUDA_CHECK(cudaEventSynchronize(e1));
    float ms = 0.f;
    CUDA_CHECK(cudaEventElapsedTime(&ms, e0, e1));
    if (world > 1) {  // the slowest rank's time
        CUDA_CHECK(cudaMemcpy(d_time, &ms, sizeof(float), cudaMemcpyHostToDevice));
        NCCL_CHECK(ncclAllReduce(d_time, d_time, 1, ncclFloat, ncclMax, comm, stream));
        CUDA_CHECK(cudaStreamSynchronize(stream));
        CUDA_CHECK(cudaMemcpy(&ms, d_time, sizeof(float), cudaMemcpyDeviceToHost));
    }
    double ar_ms = 0.0;
    for (size_t i = 0; i + 1 < ar_events.size(); i += 2) {
        float t = 0.f;
        CUDA_CHECK(cudaEventElapsedTime(&t, ar_events[i], ar_events[i + 1]));
        ar_ms += t;
    }
    if (rank == 0) {
        const double ms_step = ms / steps;
#ifdef B200ATTN_DROPIN
        const char* attn = b200attn_get_math_mode() == B200ATTN_MATH_BF16 ? "b200attn (BF16 tensor cores)" : "b200attn (FP32 parity mode)";
#else
        const char* attn = "reference src/kernels/attention.cu";
#endif
        printf("{\"metric\": \"gpt_step_tokens_per_s\", \"value\": %.1f, \"unit\": \"tokens/s\", \"n_gpus\": %d, \"steps\": %d, "
               "\"warmup\": %d, \"ms_per_step\": %.3f, \"allreduce_ms_per_step\": %.3f, \"loss\": %.5f, \"attention\": \"%s\", \"params\": %zu, "
               "\"config\": {\"L\": %zu, \"C\": %zu, \"H\": %zu, \"d_ff\": %zu, \"V\": %zu, \"T\": %d, \"per_gpu_batch\": %d, "
               "\"optimizer\": \"AdamW lr=3e-4 betas=(0.9,0.95) wd=0.1 clip=1.0\", \"parallelism\": \"dp%d, one ncclAllReduce(avg) of the gradient buffer per step\"}, "
               "\"allreduce_overlapped\": %s, \"gemm_dropin\": {\"linked\": %s, \"tcgen05_launches\": %lld, \"staged_reuses\": %lld, \"twin_hits\": %lld}}\n",
               (double)world * B * T / (ms_step * 1e-3), world, steps, warmup, ms_step, ar_ms / steps, host_loss, attn, n_params,
               cfg.num_layers, cfg.d_model, cfg.num_heads, cfg.d_ff, cfg.vocab_size, T, B, world,
               use_overlap ? "true" : "false", b200gemm_tc_launches ? "true" : "false", b200gemm_tc_launches ? b200gemm_tc_launches() : 0LL,
               b200gemm_staged_reuses ? b200gemm_staged_reuses() : 0LL, b200gemm_twin_hits ? b200gemm_twin_hits() : 0LL);
    }
    if (comm) ncclCommDestroy(comm);
    return 0;
}
