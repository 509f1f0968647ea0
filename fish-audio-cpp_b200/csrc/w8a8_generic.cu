// Shape-agnostic W8A8 linear kernel: one warp per (output row, token).
//
// This is the path for shapes the fast kernels decline (K or group size not a
// multiple of their vector width, ragged last group, unaligned pointers). It
// carries the reference's arithmetic in the plainest order there is: exact
// int32 sum per K-group (int8_gemm.cu:470-490), then groups ascending
//     acc = fma(float(P) * ws, xs, acc)                     (int8_gemm.cu:213-234)
// from 0.0f, then one rounding to fp16 (int8_gemm.cu:236-243). Not tuned.
#include "w8a8_internal.h"

namespace w8a8 {
namespace {

struct GenericParams {
    LinearArgs a;
    int words_ok;  // K % 4 == 0, g % 4 == 0, W and Xq 4-byte aligned
};

__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ float row_dot(const GenericParams& p, int n, int m, int lane) {
    const LinearArgs& a = p.a;
    const int8_t* w_row = a.W + static_cast<size_t>(n) * a.K;
    const int8_t* x_row = a.Xq + static_cast<size_t>(m) * a.K;
    float acc = 0.0f;
    for (int j = 0; j < a.G; ++j) {
        const int start = j * a.g, end = min(start + a.g, a.K);
        int dot = 0;
        if (p.words_ok) {
            const int* w4 = reinterpret_cast<const int*>(w_row + start);
            const int* x4 = reinterpret_cast<const int*>(x_row + start);
            for (int i = lane; i < (end - start) / 4; i += 32) dot = __dp4a(w4[i], x4[i], dot);
        } else {
            for (int k = start + lane; k < end; k += 32)
                dot += static_cast<int>(w_row[k]) * static_cast<int>(x_row[k]);
        }
        dot = warp_sum(dot);
        if (a.dump && lane == 0) a.dump[(static_cast<size_t>(m) * a.N + n) * a.G + j] = dot;
        const float ws = __half2float(a.w_scale[static_cast<size_t>(n) * a.G + j]);
        const float xs = a.Xs[static_cast<size_t>(m) * a.G + j];
        acc = __fmaf_rn(__fmul_rn(static_cast<float>(dot), ws), xs, acc);
    }
    return acc;
}

__global__ void __launch_bounds__(256) linear_generic_kernel(const GenericParams p) {
    const LinearArgs& a = p.a;
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);
    const int m = blockIdx.y;
    if (a.epilogue == W8A8_EPI_SWIGLU) {
        const int H = a.N / 2;
        if (unit >= H) return;
        const int gate_row = 16 * (unit / 8) + (unit % 8);
        const float gt = row_dot(p, gate_row, m, lane);
        const float up = row_dot(p, gate_row + 8, m, lane);
        if (lane == 0) {
            const float g16 = __half2float(__float2half(gt));
            const __half s16 = __float2half(g16 / (1.0f + expf(-g16)));
            const float u16 = __half2float(__float2half(up));
            a.Y[static_cast<size_t>(m) * H + unit] = __float2half(__half2float(s16) * u16);
        }
        return;
    }
    if (unit >= a.N) return;
    const float acc = row_dot(p, unit, m, lane);
    if (lane == 0) {
        const size_t o = static_cast<size_t>(m) * a.N + unit;
        __half y = __float2half(acc);
        if (a.epilogue == W8A8_EPI_RESIDUAL) y = __float2half(__half2float(y) + __half2float(a.residual[o]));
        a.Y[o] = y;
    }
}

}  // namespace

int launch_linear_generic(const LinearArgs& a, cudaStream_t s) {
    if (a.M == 0) return W8A8_OK;
    if (!a.Xq || !a.Xs) return fail(W8A8_ERR_INVALID_ARG, "generic kernel needs codes and scales");
    GenericParams p;
    p.a = a;
    p.words_ok = (a.K % 4 == 0) && (a.g % 4 == 0) &&
                 ((reinterpret_cast<uintptr_t>(a.W) | reinterpret_cast<uintptr_t>(a.Xq)) & 3u) == 0;
    const int units = a.epilogue == W8A8_EPI_SWIGLU ? a.N / 2 : a.N;
    for (int m0 = 0; m0 < a.M; m0 += 65535) {  // gridDim.y limit
        GenericParams q = p;
        const int mc = a.M - m0 < 65535 ? a.M - m0 : 65535;
        const int outN = a.epilogue == W8A8_EPI_SWIGLU ? a.N / 2 : a.N;
        q.a.Xq = a.Xq + static_cast<size_t>(m0) * a.K;
        q.a.Xs = a.Xs + static_cast<size_t>(m0) * a.G;
        q.a.Y = a.Y + static_cast<size_t>(m0) * outN;
        if (a.residual) q.a.residual = a.residual + static_cast<size_t>(m0) * a.N;
        if (a.dump) q.a.dump = a.dump + static_cast<size_t>(m0) * a.N * a.G;
        dim3 grid((units + 7) / 8, mc);
        linear_generic_kernel<<<grid, 256, 0, s>>>(q);
        int rc = check_launch("linear_generic_kernel");
        if (rc) return rc;
    }
    return W8A8_OK;
}

}  // namespace w8a8
