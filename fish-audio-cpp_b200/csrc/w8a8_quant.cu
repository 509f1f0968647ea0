// Row kernels: residual add -> RMSNorm -> activation quantiser, any subset, one launch.
//
// One CTA owns one token row and keeps it in shared memory from the first load
// to the last store, so the chain
//     residual_add (ffn_activations.cu:41-45) -> rms_norm (rms_norm.cu:10-58)
//     -> quantize_activation_groups_kernel (int8_gemm.cu:147-211)
// costs one read of the row instead of three round trips through HBM. Every
// value that the reference would have rounded to fp16 on its way through global
// memory is rounded to fp16 here too, so the int8 codes and the fp32 scales are
// bit-identical to those of the unfused reference chain.
#include <cstdlib>

#include "w8a8_internal.h"
#include "w8a8_trace.cuh"

namespace w8a8 {
namespace {

constexpr int kWarp = 32;

struct RowQuantParams {
    const __half* x_in;
    __half* x_out;            // where x_in + residual goes (null: not stored)
    const __half* residual;   // null: no add
    const __half* norm_weight;  // null: no norm
    float eps;
    const __half* smooth_inv;
    const __half* act_scale;  // static scales [G] or null
    __half* normed_out;       // null: not stored
    int8_t* Xq;               // null: no quantisation (plain rms_norm)
    float* Xs;
    int K, g, G;
    int per_token;
    int vec_ok;               // K % 8 == 0 and all fp16 pointers 16-byte aligned
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = kWarp / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__global__ void __launch_bounds__(1024) rowquant_kernel(const RowQuantParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* row = reinterpret_cast<__half*>(smem_raw);
    float* gscale = reinterpret_cast<float*>(smem_raw + ((static_cast<size_t>(p.K) * 2 + 15) & ~size_t(15)));
    __shared__ float s_red[kWarp];

    const int tid = threadIdx.x;
    const int T = blockDim.x;
    const int K = p.K;
    const size_t base = static_cast<size_t>(blockIdx.x) * K;
    // Let the next kernel in the stream start its own prologue; wait for the one before this.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- stage the row (+ residual add, rounded to fp16 like residual_add_kernel) ----
    if (p.vec_ok) {
        const uint4* src = reinterpret_cast<const uint4*>(p.x_in + base);
        const uint4* res = p.residual ? reinterpret_cast<const uint4*>(p.residual + base) : nullptr;
        uint4* dst = p.x_out ? reinterpret_cast<uint4*>(p.x_out + base) : nullptr;
        for (int v = tid; v < K / 8; v += T) {
            uint4 u = src[v];
            if (res) {
                uint4 r = res[v];
                __half2* uh = reinterpret_cast<__half2*>(&u);
                const __half2* rh = reinterpret_cast<const __half2*>(&r);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float2 a = __half22float2(uh[i]), b = __half22float2(rh[i]);
                    uh[i] = __halves2half2(__float2half(a.x + b.x), __float2half(a.y + b.y));
                }
                if (dst) dst[v] = u;
            }
            reinterpret_cast<uint4*>(row)[v] = u;
        }
    } else {
        for (int i = tid; i < K; i += T) {
            __half h = p.x_in[base + i];
            if (p.residual) {
                h = __float2half(__half2float(h) + __half2float(p.residual[base + i]));
                if (p.x_out) p.x_out[base + i] = h;
            }
            row[i] = h;
        }
    }
    __syncthreads();

    // ---- RMSNorm, with the reference's summation order (rms_norm.cu:23-49): thread t sums
    // elements t, t+T, ...; shuffle-down tree inside each warp; shuffle-down tree over warps. ----
    if (p.norm_weight) {
        float local_sum = 0.0f;
        for (int i = tid; i < K; i += T) {
            float val = __half2float(row[i]);
            local_sum += val * val;
        }
        for (int offset = kWarp / 2; offset > 0; offset /= 2)
            local_sum += __shfl_down_sync(0xffffffffu, local_sum, offset);
        if ((tid & (kWarp - 1)) == 0) s_red[tid / kWarp] = local_sum;
        __syncthreads();
        float total_sum = 0.0f;
        int num_warps = (T + kWarp - 1) / kWarp;
        if (tid < num_warps) total_sum = s_red[tid];
        for (int offset = kWarp / 2; offset > 0; offset /= 2)
            total_sum += __shfl_down_sync(0xffffffffu, total_sum, offset);
        __syncthreads();
        if (tid == 0) s_red[0] = rsqrtf(total_sum / K + p.eps);
        __syncthreads();
        const float rms = s_red[0];
        for (int i = tid; i < K; i += T) {
            float val = __half2float(row[i]) * rms;
            __half o = __float2half(val * __half2float(p.norm_weight[i]));
            row[i] = o;
            if (p.normed_out) p.normed_out[base + i] = o;
        }
        __syncthreads();
    }
    if (!p.Xq) return;

    // ---- scales: one warp per group; absmax is order-free (int8_gemm.cu:177-199) ----
    const int lane = tid & (kWarp - 1), warp = tid / kWarp, nwarps = T / kWarp;
    const int g = p.g, G = p.G;
    if (p.act_scale) {
        for (int j = tid; j < G; j += T) {
            float s = __half2float(p.act_scale[j]);
            gscale[j] = s < 1e-8f ? 1e-8f : s;
        }
    } else {
        for (int j = warp; j < G; j += nwarps) {
            int start = j * g, end = min(start + g, K);
            float m = 0.0f;
            for (int k = start + lane; k < end; k += kWarp) {
                float v = __half2float(row[k]);
                if (p.smooth_inv) v *= __half2float(p.smooth_inv[k]);
                m = fmaxf(m, fabsf(v));
            }
            m = warp_max(m);
            if (lane == 0) gscale[j] = m;  // absmax for now
        }
        __syncthreads();
        if (p.per_token) {
            float m = 0.0f;
            for (int j = tid; j < G; j += T) m = fmaxf(m, gscale[j]);
            m = warp_max(m);
            if (lane == 0) s_red[warp] = m;
            __syncthreads();
            m = 0.0f;
            for (int w = 0; w < nwarps; ++w) m = fmaxf(m, s_red[w]);
            __syncthreads();
            for (int j = tid; j < G; j += T) gscale[j] = m;
            __syncthreads();
        }
        for (int j = tid; j < G; j += T) {
            float s = gscale[j] / 127.0f;
            gscale[j] = s < 1e-8f ? 1e-8f : s;
        }
    }
    __syncthreads();
    for (int j = tid; j < G; j += T) p.Xs[static_cast<size_t>(blockIdx.x) * G + j] = gscale[j];

    // ---- codes (int8_gemm.cu:201-210) ----
    int8_t* q_row = p.Xq + base;
    if ((K & 3) == 0 && (g & 3) == 0) {
        for (int w4 = tid; w4 < K / 4; w4 += T) {
            const int k0 = w4 * 4;
            const float inv_scale = 1.0f / gscale[k0 / g];
            uint32_t packed = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float v = __half2float(row[k0 + i]);
                if (p.smooth_inv) v *= __half2float(p.smooth_inv[k0 + i]);
                int q = __float2int_rn(v * inv_scale);
                q = max(-127, min(127, q));
                packed |= (static_cast<uint32_t>(q) & 0xffu) << (8 * i);
            }
            reinterpret_cast<uint32_t*>(q_row)[w4] = packed;
        }
    } else {
        for (int k = tid; k < K; k += T) {
            const float inv_scale = 1.0f / gscale[k / g];
            float v = __half2float(row[k]);
            if (p.smooth_inv) v *= __half2float(p.smooth_inv[k]);
            int q = __float2int_rn(v * inv_scale);
            q = max(-127, min(127, q));
            q_row[k] = static_cast<int8_t>(q);
        }
    }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Register-resident form of the fused row kernel for rows of at most 4 x blockDim elements (the decode
// case: K = 2560 with 1024 threads). Same arithmetic and the same summation order as rowquant_kernel —
// thread t owns elements t, t+T, t+2T, ... exactly like the reference's rms_norm launch — but nothing is
// staged in shared memory and only three block barriers separate the first load from the last store;
// at 8 rows per launch the kernel's length is a latency chain, not a bandwidth figure. Needs g % 32 == 0
// so that the 32 lanes of a warp always sit in one quantisation group.
constexpr int kFastElems = 4;
__global__ void __launch_bounds__(1024) rowquant_fast_kernel(const RowQuantParams p) {
    __shared__ float s_red[kWarp];
    __shared__ unsigned s_gmax[160];  // absmax per group as float bits (non-negative floats order like uints)
    const int tid = threadIdx.x, T = blockDim.x, K = p.K, g = p.g, G = p.G;
    const int lane = tid & (kWarp - 1), warp = tid / kWarp;
    const size_t base = static_cast<size_t>(blockIdx.x) * K;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // the norm weight and the smoothing vector are parameters, not results of the kernel before this one
    __half nw[kFastElems], sm[kFastElems];
#pragma unroll
    for (int i = 0; i < kFastElems; ++i) {
        const int e = tid + i * T;
        if (e < K) {
            if (p.norm_weight) nw[i] = p.norm_weight[e];
            if (p.smooth_inv) sm[i] = p.smooth_inv[e];
        }
    }
    for (int j = tid; j < G; j += T) s_gmax[j] = 0u;
    asm volatile("griddepcontrol.wait;" ::: "memory");

    __half h[kFastElems], res[kFastElems];
    float local_sum = 0.0f;
    // every load is requested before the first store: x_out may be x_in, so a load placed after a store
    // would have to wait for it, one memory round trip per element
#pragma unroll
    for (int i = 0; i < kFastElems; ++i) {
        const int e = tid + i * T;
        if (e < K) {
            h[i] = p.x_in[base + e];
            if (p.residual) res[i] = p.residual[base + e];
        }
    }
#pragma unroll
    for (int i = 0; i < kFastElems; ++i) {
        const int e = tid + i * T;
        if (e < K) {
            __half v = h[i];
            if (p.residual) {
                v = __float2half(__half2float(v) + __half2float(res[i]));
                if (p.x_out) p.x_out[base + e] = v;
            }
            h[i] = v;
            float val = __half2float(v);
            local_sum += val * val;
        }
    }
    if (p.norm_weight) {
        for (int offset = kWarp / 2; offset > 0; offset /= 2)
            local_sum += __shfl_down_sync(0xffffffffu, local_sum, offset);
        if (lane == 0) s_red[warp] = local_sum;
        __syncthreads();
        float total_sum = 0.0f;
        const int num_warps = (T + kWarp - 1) / kWarp;
        if (tid < num_warps) total_sum = s_red[tid];
        if (warp == 0) {
            for (int offset = kWarp / 2; offset > 0; offset /= 2)
                total_sum += __shfl_down_sync(0xffffffffu, total_sum, offset);
        }
        __syncthreads();
        if (tid == 0) s_red[0] = rsqrtf(total_sum / K + p.eps);
        __syncthreads();
        const float rms = s_red[0];
#pragma unroll
        for (int i = 0; i < kFastElems; ++i) {
            const int e = tid + i * T;
            if (e < K) {
                float val = __half2float(h[i]) * rms;
                h[i] = __float2half(val * __half2float(nw[i]));
                if (p.normed_out) p.normed_out[base + e] = h[i];
            }
        }
    }
    if (!p.Xq) return;
    float v[kFastElems];
#pragma unroll
    for (int i = 0; i < kFastElems; ++i) {
        const int e = tid + i * T;
        v[i] = 0.0f;
        if (e < K) {
            v[i] = __half2float(h[i]);
            if (p.smooth_inv) v[i] *= __half2float(sm[i]);
        }
    }
    if (!p.act_scale) {
#pragma unroll
        for (int i = 0; i < kFastElems; ++i) {
            const int e0 = warp * kWarp + i * T;  // first element of this warp's run
            if (e0 < K) {
                float m = warp_max(fabsf(v[i]));
                if (lane == 0) atomicMax(&s_gmax[p.per_token ? 0 : e0 / g], __float_as_uint(m));
            }
        }
    }
    __syncthreads();
    for (int j = tid; j < G; j += T) {
        float sc = p.act_scale ? __half2float(p.act_scale[j]) : __uint_as_float(s_gmax[p.per_token ? 0 : j]) / 127.0f;
        if (sc < 1e-8f) sc = 1e-8f;
        p.Xs[static_cast<size_t>(blockIdx.x) * G + j] = sc;
    }
#pragma unroll
    for (int i = 0; i < kFastElems; ++i) {
        const int e = tid + i * T;
        if (e < K) {
            const int j = e / g;
            float sc = p.act_scale ? __half2float(p.act_scale[j]) : __uint_as_float(s_gmax[p.per_token ? 0 : j]) / 127.0f;
            if (sc < 1e-8f) sc = 1e-8f;
            const float inv_scale = 1.0f / sc;
            int q = __float2int_rn(v[i] * inv_scale);
            q = max(-127, min(127, q));
            p.Xq[base + e] = static_cast<int8_t>(q);
        }
    }
}

// residual add + RMSNorm + group quantiser for the decode step, in little code: 256 threads per row, the row
// staged in shared memory, g in {64, 128, 256}, K a multiple of 256 up to 4096. The sum of squares follows the
// reference's T-thread launch (rms_norm.cu:23-49, :69-70): real warp w plays virtual warps w*VW .. w*VW+VW-1
// (VW = T / 256), so the normed values are the reference's; normalising and quantising then go 8 elements (one
// 128-bit piece) per thread, the g/8 threads of a group finding its absmax with shuffles. Plain loops on purpose:
// a launch runs this code once, and what it costs is the instruction fetch as much as the arithmetic.
template <int GM>
__global__ void __launch_bounds__(256) rowquant_compact_kernel(const RowQuantParams p, int T) {
    constexpr int LANES = GM / 8, kThreads = 256;
    __shared__ float s_red[32];
    __shared__ __align__(16) __half row_s[4096];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = p.K, VW = T / kThreads, G = p.G, row = blockIdx.x;
    const size_t base = static_cast<size_t>(row) * K;
    const int pieces = K / 8;
    W8A8_TRACE_SCOPE();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint4 xv[2], dv[2], wv[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int c8 = tid + i * kThreads;
        wv[i] = __ldg(reinterpret_cast<const uint4*>(p.norm_weight) + (c8 < pieces ? c8 : 0));
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    W8A8_TRACE_WAITED();
#pragma unroll
    for (int i = 0; i < 2; ++i) {  // every load first (at most two pieces per thread)
        const int c8 = tid + i * kThreads;
        const int cc = c8 < pieces ? c8 : 0;
        xv[i] = *reinterpret_cast<const uint4*>(p.x_in + base + cc * 8);
        dv[i] = *reinterpret_cast<const uint4*>((p.residual ? p.residual : p.x_in) + base + cc * 8);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int c8 = tid + i * kThreads;
        if (c8 < pieces) {
            if (p.residual) {
                __half* hx = reinterpret_cast<__half*>(&xv[i]);
                const __half* hd = reinterpret_cast<const __half*>(&dv[i]);
#pragma unroll
                for (int e = 0; e < 8; ++e) hx[e] = __float2half(__half2float(hx[e]) + __half2float(hd[e]));
                if (p.x_out) *reinterpret_cast<uint4*>(p.x_out + base + c8 * 8) = xv[i];
            }
            reinterpret_cast<uint4*>(row_s)[c8] = xv[i];
        }
    }
    __syncthreads();
#pragma unroll 1
    for (int k = 0; k < VW; ++k) {
        float local_sum = 0.0f;
#pragma unroll 1
        for (int e = (warp * VW + k) * 32 + lane; e < K; e += T) {
            float val = __half2float(row_s[e]);
            local_sum += val * val;
        }
        for (int offset = 16; offset > 0; offset /= 2) local_sum += __shfl_down_sync(0xffffffffu, local_sum, offset);
        if (lane == 0) s_red[warp * VW + k] = local_sum;
    }
    __syncthreads();
    float total_sum = 0.0f;
    if (warp == 0) {
        if (lane < T / 32) total_sum = s_red[lane];
        for (int offset = 16; offset > 0; offset /= 2) total_sum += __shfl_down_sync(0xffffffffu, total_sum, offset);
    }
    __syncthreads();
    if (tid == 0) s_red[0] = rsqrtf(total_sum / K + p.eps);
    __syncthreads();
    const float rms = s_red[0];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int c8 = tid + i * kThreads;
        const bool live = c8 < pieces;  // whole warps are live or not (pieces is a multiple of 32)
        __half* hx = reinterpret_cast<__half*>(&xv[i]);
        const __half* hw = reinterpret_cast<const __half*>(&wv[i]);
        float v[8], amax = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float val = __half2float(hx[e]) * rms;
            hx[e] = __float2half(val * __half2float(hw[e]));
            v[e] = __half2float(hx[e]);
            amax = fmaxf(amax, fabsf(v[e]));
        }
        if (live && p.normed_out) *reinterpret_cast<uint4*>(p.normed_out + base + c8 * 8) = xv[i];
        if (!p.Xq) continue;
#pragma unroll
        for (int o = LANES / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (!live) continue;
        float scale = amax / 127.0f;
        if (scale < 1e-8f) scale = 1e-8f;
        if ((lane & (LANES - 1)) == 0) p.Xs[static_cast<size_t>(row) * G + (c8 * 8) / GM] = scale;
        const float inv_scale = 1.0f / scale;
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            int q = __float2int_rn(v[e] * inv_scale);
            q = max(-127, min(127, q));
            if (e < 4) lo |= (static_cast<uint32_t>(q) & 0xffu) << (8 * e);
            else hi |= (static_cast<uint32_t>(q) & 0xffu) << (8 * (e - 4));
        }
        *reinterpret_cast<uint2*>(p.Xq + base + c8 * 8) = make_uint2(lo, hi);
    }
    W8A8_TRACE_END(2u);
}

// The quantiser alone (int8_gemm.cu:147-211) for g in {64, 128, 256}: no shared memory, no block
// barrier. A thread owns 8 consecutive activations (one 128-bit load), the g/8 threads of a group
// find the absmax with shuffles, and each thread stores its 8 codes as one 64-bit word. At decode
// sizes the whole activation matrix is a few KB, so what counts is the length of the dependency
// chain (one load, log2(g/8) shuffles, one divide, one store), not bandwidth.
template <int LANES>  // threads per group = g / 8
__global__ void __launch_bounds__(128) groupquant_kernel(const __half* __restrict__ X,
                                                         const __half* __restrict__ smooth_inv,
                                                         const __half* __restrict__ act_scale,
                                                         int8_t* __restrict__ Xq, float* __restrict__ Xs, int K,
                                                         int G) {
    W8A8_TRACE_SCOPE();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    W8A8_TRACE_WAITED();
    const int m = blockIdx.y;
    const int e = (blockIdx.x * 128 + threadIdx.x) * 8;
    const bool live = e < K;
    float v[8];
    float amax = 0.0f;
    if (live) {
        const uint4 u = *reinterpret_cast<const uint4*>(X + static_cast<size_t>(m) * K + e);
        const __half* h = reinterpret_cast<const __half*>(&u);
        uint4 su = make_uint4(0, 0, 0, 0);
        if (smooth_inv) su = *reinterpret_cast<const uint4*>(smooth_inv + e);
        const __half* sh = reinterpret_cast<const __half*>(&su);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = __half2float(h[i]);
            if (smooth_inv) v[i] *= __half2float(sh[i]);
            amax = fmaxf(amax, fabsf(v[i]));
        }
    }
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (!live) return;
    const int j = e / (LANES * 8);
    float scale = act_scale ? __half2float(act_scale[j]) : amax / 127.0f;
    if (scale < 1e-8f) scale = 1e-8f;
    if ((threadIdx.x & (LANES - 1)) == 0) Xs[static_cast<size_t>(m) * G + j] = scale;
    const float inv_scale = 1.0f / scale;
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int q = __float2int_rn(v[i] * inv_scale);
        q = max(-127, min(127, q));
        if (i < 4) lo |= (static_cast<uint32_t>(q) & 0xffu) << (8 * i);
        else hi |= (static_cast<uint32_t>(q) & 0xffu) << (8 * (i - 4));
    }
    *reinterpret_cast<uint2*>(Xq + static_cast<size_t>(m) * K + e) = make_uint2(lo, hi);
    W8A8_TRACE_END(3u);
}

template <int LANES>
int launch_groupquant(const __half* X, const __half* smooth_inv, const __half* act_scale, int8_t* Xq, float* Xs,
                      int M, int K, int G, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((K + 1023) / 1024, M, 1);
    cfg.blockDim = dim3(128, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled(kPdlRow) ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, groupquant_kernel<LANES>, X, smooth_inv, act_scale, Xq, Xs, K, G);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "groupquant launch: %s", cudaGetErrorString(e));
    return W8A8_OK;
}

}  // namespace

int launch_rowquant(const __half* x_in, __half* x_out, const __half* residual,
                    const __half* norm_weight, float eps, const __half* smooth_inv,
                    const __half* act_scale, int M, int K, int g, int act_mode, __half* normed_out,
                    int8_t* Xq, float* Xs, cudaStream_t stream) {
    if (M == 0) return W8A8_OK;
    {   // the quantiser alone, common group sizes: the barrier-free kernel
        const int gn = norm_group(K, g);
        if (!residual && !norm_weight && !normed_out && Xq && act_mode == W8A8_ACT_PER_TOKEN_GROUP &&
            (gn == 64 || gn == 128 || gn == 256) && K % gn == 0 && M <= 65535 && aligned16(x_in) &&
            (reinterpret_cast<uintptr_t>(Xq) & 7u) == 0 && (!smooth_inv || aligned16(smooth_inv))) {
            const int G = K / gn;
            if (gn == 64) return launch_groupquant<8>(x_in, smooth_inv, act_scale, Xq, Xs, M, K, G, stream);
            if (gn == 128) return launch_groupquant<16>(x_in, smooth_inv, act_scale, Xq, Xs, M, K, G, stream);
            return launch_groupquant<32>(x_in, smooth_inv, act_scale, Xq, Xs, M, K, G, stream);
        }
    }
    RowQuantParams p;
    p.x_in = x_in;
    p.x_out = x_out;
    p.residual = residual;
    p.norm_weight = norm_weight;
    p.eps = eps;
    p.smooth_inv = smooth_inv;
    p.act_scale = act_scale;
    p.normed_out = normed_out;
    p.Xq = Xq;
    p.Xs = Xs;
    p.K = K;
    p.g = norm_group(K, g);
    p.G = num_groups(K, g);
    p.per_token = act_mode == W8A8_ACT_PER_TOKEN;
    p.vec_ok = (K % 8 == 0) && aligned16(x_in) && (!residual || aligned16(residual)) &&
               (!x_out || aligned16(x_out));
    // The norm must run with the reference's block size to reproduce its summation order:
    // min(1024, next_pow2(dim)), rms_norm.cu:69-70.
    int threads = 256;
    if (norm_weight) {
        threads = 1;
        while (threads < K && threads < 1024) threads <<= 1;
        if (threads < 32) threads = 32;  // shuffles need whole warps; lanes past K add 0.0f
    } else if (K >= 4096) {
        threads = 512;
    }
    static const bool compact_ok = [] {
        const char* v = std::getenv("W8A8_ROW_COMPACT");
        return v ? (*v && *v != '0') : true;
    }();
    if (compact_ok && norm_weight && threads >= 256 && K % 256 == 0 && K <= 4096 && !smooth_inv && !act_scale && !p.per_token &&
        (p.g == 64 || p.g == 128 || p.g == 256) && p.vec_ok && aligned16(norm_weight) &&
        (!normed_out || aligned16(normed_out)) && (!Xq || (reinterpret_cast<uintptr_t>(Xq) & 7u) == 0)) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(M, 1, 1);
        cfg.blockDim = dim3(256, 1, 1);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl_enabled(kPdlRow) ? 1 : 0;
        cudaError_t e = p.g == 64    ? cudaLaunchKernelEx(&cfg, rowquant_compact_kernel<64>, p, threads)
                        : p.g == 128 ? cudaLaunchKernelEx(&cfg, rowquant_compact_kernel<128>, p, threads)
                                     : cudaLaunchKernelEx(&cfg, rowquant_compact_kernel<256>, p, threads);
        if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "rowquant_compact launch: %s", cudaGetErrorString(e));
        return W8A8_OK;
    }
    if (norm_weight && threads >= 32 && K <= kFastElems * threads && p.g % 32 == 0 && p.G <= 160) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(M, 1, 1);
        cfg.blockDim = dim3(threads, 1, 1);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl_enabled(kPdlRow) ? 1 : 0;
        cudaError_t e = cudaLaunchKernelEx(&cfg, rowquant_fast_kernel, p);
        if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "rowquant_fast launch: %s", cudaGetErrorString(e));
        return W8A8_OK;
    }
    size_t smem = ((static_cast<size_t>(K) * 2 + 15) & ~size_t(15)) + static_cast<size_t>(p.G) * 4;
    if (smem > 200 * 1024) return fail(W8A8_ERR_UNSUPPORTED, "row of K=%d does not fit shared memory", K);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(rowquant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(smem));
        if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(M, 1, 1);
    cfg.blockDim = dim3(threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled(kPdlRow) ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, rowquant_kernel, p);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "rowquant launch: %s", cudaGetErrorString(e));
    return W8A8_OK;
}

}  // namespace w8a8

W8A8_TRACE_READER(quant)
