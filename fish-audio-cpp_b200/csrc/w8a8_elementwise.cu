// Elementwise neighbours of the linear layer and the loader-side gate/up pre-pack.
//
// silu / mul / residual_add keep the reference's arithmetic (fp32 math, one fp16
// rounding per call: ffn_activations.cu:12-17, :35-45) but move 8 halves per thread
// with 128-bit accesses. They exist so that a caller that has not switched to the
// fused epilogues still finds every operator it used next to the linear layer.
#include "w8a8_internal.h"

namespace w8a8 {
namespace {

enum { OP_SILU = 0, OP_MUL = 1, OP_ADD = 2 };

template <int OP>
__device__ __forceinline__ __half apply(__half a, __half b) {
    float av = __half2float(a);
    if (OP == OP_SILU) return __float2half(av / (1.0f + expf(-av)));
    if (OP == OP_MUL) return __float2half(av * __half2float(b));
    return __float2half(av + __half2float(b));
}

template <int OP>
__global__ void __launch_bounds__(256) eltwise_kernel(__half* __restrict__ a, const __half* __restrict__ b,
                                                      long n, int vec_ok) {
    const long stride = static_cast<long>(gridDim.x) * blockDim.x;
    long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (vec_ok) {
        const long nv = n / 8;
        for (long v = i; v < nv; v += stride) {
            uint4 ua = reinterpret_cast<uint4*>(a)[v];
            uint4 ub = OP == OP_SILU ? ua : reinterpret_cast<const uint4*>(b)[v];
            __half* ha = reinterpret_cast<__half*>(&ua);
            const __half* hb = reinterpret_cast<const __half*>(&ub);
#pragma unroll
            for (int e = 0; e < 8; ++e) ha[e] = apply<OP>(ha[e], hb[e]);
            reinterpret_cast<uint4*>(a)[v] = ua;
        }
        for (long t = nv * 8 + i; t < n; t += stride) a[t] = apply<OP>(a[t], OP == OP_SILU ? a[t] : b[t]);
    } else {
        for (long t = i; t < n; t += stride) a[t] = apply<OP>(a[t], OP == OP_SILU ? a[t] : b[t]);
    }
}

template <int OP>
int launch(__half* a, const __half* b, long n, cudaStream_t s) {
    if (n <= 0) return W8A8_OK;
    int vec_ok = (reinterpret_cast<uintptr_t>(a) & 15u) == 0 &&
                 (OP == OP_SILU || (reinterpret_cast<uintptr_t>(b) & 15u) == 0);
    long work = vec_ok ? (n + 7) / 8 : n;
    long blocks = (work + 255) / 256;
    if (blocks > 148L * 16) blocks = 148L * 16;  // grid-stride beyond 16 CTAs per SM
    eltwise_kernel<OP><<<static_cast<unsigned>(blocks), 256, 0, s>>>(a, b, n, vec_ok);
    return check_launch("eltwise_kernel");
}

// Block-16 interleave: packed row 16*t + i      <- gate row 8*t + i
//                      packed row 16*t + 8 + i  <- up   row 8*t + i        (i < 8)
__global__ void __launch_bounds__(256) pack_gate_up_kernel(const int8_t* __restrict__ wg,
                                                           const __half* __restrict__ sg,
                                                           const int8_t* __restrict__ wu,
                                                           const __half* __restrict__ su, int inter, int K,
                                                           int G, int8_t* __restrict__ Wo,
                                                           __half* __restrict__ So) {
    const int pr = blockIdx.x;  // packed row
    const int t = pr / 16, i = pr % 16;
    const bool up = i >= 8;
    const int src = t * 8 + (i & 7);
    const int8_t* w = (up ? wu : wg) + static_cast<size_t>(src) * K;
    const __half* sc = (up ? su : sg) + static_cast<size_t>(src) * G;
    int8_t* wo = Wo + static_cast<size_t>(pr) * K;
    if ((K & 15) == 0 && ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(wo)) & 15u) == 0) {
        for (int v = threadIdx.x; v < K / 16; v += blockDim.x)
            reinterpret_cast<uint4*>(wo)[v] = reinterpret_cast<const uint4*>(w)[v];
    } else {
        for (int k = threadIdx.x; k < K; k += blockDim.x) wo[k] = w[k];
    }
    for (int j = threadIdx.x; j < G; j += blockDim.x) So[static_cast<size_t>(pr) * G + j] = sc[j];
}

}  // namespace

int launch_silu(__half* a, long n, cudaStream_t s) { return launch<OP_SILU>(a, nullptr, n, s); }
int launch_mul(__half* a, const __half* b, long n, cudaStream_t s) { return launch<OP_MUL>(a, b, n, s); }
int launch_residual_add(__half* a, const __half* b, long n, cudaStream_t s) { return launch<OP_ADD>(a, b, n, s); }

int launch_pack_gate_up(const int8_t* wg, const __half* sg, const int8_t* wu, const __half* su,
                        int inter, int K, int G, int8_t* Wo, __half* So, cudaStream_t s) {
    if (inter <= 0) return W8A8_OK;
    pack_gate_up_kernel<<<2 * inter, 256, 0, s>>>(wg, sg, wu, su, inter, K, G, Wo, So);
    return check_launch("pack_gate_up_kernel");
}

}  // namespace w8a8
