// Device-side launch trace, compiled in only with -DW8A8_TRACE (a diagnostic build; the product library has none
// of it). Thread 0 of the first and of the last CTA of a traced kernel records the GPU's nanosecond timer at kernel
// entry, after the dependency wait (griddepcontrol.wait) and at the end of the CTA, into a buffer that is private to
// the translation unit; W8A8_TRACE_READER(name) exports `w8a8_trace_read_<name>` to copy it out and clear it. No
// profiler is involved, so launches overlap exactly as they do in a normal run.
#pragma once

#ifdef W8A8_TRACE
#include <cuda_runtime.h>

namespace w8a8 {
namespace trace {

constexpr int kCap = 16384;
struct Rec {
    unsigned long long t_entry, t_waited, t_end;
    unsigned id, cta, ctas, aux;
};
static __device__ Rec g_recs[kCap];
static __device__ unsigned g_n;

__device__ __forceinline__ unsigned long long now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

struct Scope {
    unsigned long long t0, t1;
    unsigned cta, ctas;
    bool on;
    __device__ __forceinline__ Scope() {
        ctas = gridDim.x * gridDim.y * gridDim.z;
        cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
        on = threadIdx.x == 0 && (cta == 0 || cta == ctas - 1);
        t0 = t1 = on ? now() : 0ull;
    }
    __device__ __forceinline__ void waited() {
        if (on) t1 = now();
    }
    __device__ __forceinline__ void end(unsigned id, unsigned aux = 0) {
        if (!on) return;
        const unsigned i = atomicAdd(&g_n, 1u);
        if (i < kCap) g_recs[i] = Rec{t0, t1, now(), id, cta, ctas, aux};
    }
};

inline int read_and_clear(void* out, int cap_records) {
    unsigned n = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&n, g_n, sizeof n) != cudaSuccess) return -1;
    if (n > static_cast<unsigned>(kCap)) n = kCap;
    if (static_cast<int>(n) > cap_records) n = cap_records;
    if (n && cudaMemcpyFromSymbol(out, g_recs, n * sizeof(Rec)) != cudaSuccess) return -1;
    const unsigned zero = 0;
    cudaMemcpyToSymbol(g_n, &zero, sizeof zero);
    return static_cast<int>(n);
}

}  // namespace trace
}  // namespace w8a8

#define W8A8_TRACE_SCOPE() w8a8::trace::Scope w8a8_trace_scope
#define W8A8_TRACE_WAITED() w8a8_trace_scope.waited()
#define W8A8_TRACE_END(...) w8a8_trace_scope.end(__VA_ARGS__)
#define W8A8_TRACE_READER(name)                                                                          \
    extern "C" __attribute__((visibility("default"))) int w8a8_trace_read_##name(void* out, int cap) { \
        return w8a8::trace::read_and_clear(out, cap);                                                    \
    }
#else
#define W8A8_TRACE_SCOPE() do {} while (0)
#define W8A8_TRACE_WAITED() do {} while (0)
#define W8A8_TRACE_END(...) do {} while (0)
#define W8A8_TRACE_READER(name)
#endif
