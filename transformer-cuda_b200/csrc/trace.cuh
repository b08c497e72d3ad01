// clock64 stamps for debug builds (-DB200ATTN_TRACE); in every other build the macros expand to nothing and no
// symbol is emitted. A kernel file names one buffer with B200ATTN_TRACE_DEFINE(name, slots), which also exports
// b200attn_debug_read_<name>(host_ptr, count) to copy it back, and stamps with B200ATTN_TRACE_POINT.
#pragma once

#ifdef B200ATTN_TRACE
#define B200ATTN_TRACE_DEFINE(name, slots)                                                              \
    __device__ long long g_trace_##name[slots];                                                         \
    extern "C" int b200attn_debug_read_##name(long long* host, int count) {                             \
        return (int)cudaMemcpyFromSymbol(host, g_trace_##name, sizeof(long long) * (size_t)count);      \
    }
#define B200ATTN_TRACE_POINT(name, cond, slot)             \
    do {                                                   \
        if (cond) g_trace_##name[slot] = clock64();        \
    } while (0)
#else
#define B200ATTN_TRACE_DEFINE(name, slots)
#define B200ATTN_TRACE_POINT(name, cond, slot) \
    do {                                       \
    } while (0)
#endif
