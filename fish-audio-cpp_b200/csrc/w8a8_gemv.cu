// Small-M (decode) W8A8 linear: a weight-streaming kernel bound by HBM bandwidth.
//
// Replaces int8_matvec_dequant_kernel / int8_smallbatch_dequant_kernel and, for
// 4 < tokens <= 32, the per-group cuBLAS loop of int8_gemm.cu:245-505.
//
// Work split: grid = (row tiles of 64 weight rows) x (S slices of K); the S CTAs
// that share a row tile form one thread-block cluster and add their fp32 partial
// tiles through distributed shared memory in a fixed order, so split-K needs no
// global scratch and the result does not depend on scheduling.
//
// Per warp: 16 weight rows. Each lane streams two 16-byte pieces per 64-byte
// K-chunk (rows r and r+8) straight from the row-major [N,K] matrix; the bytes
// feed mma.sync.m16n8k32.s8 as the A operand with the tokens as the 8-wide B
// operand. Integer dot products do not care in which order K is visited, so the
// kernel lets "MMA k index" be a permutation of the real k that makes every
// load 128-bit and contiguous; activations are read with the same permutation.
// The int32 sums of one K-group are exact and complete inside one warp; they are
// promoted with acc = fma(float(P) * ws, xs, acc) in ascending group order.
//
// The activation slice comes either as int8 codes + fp32 scales, or as fp16
// that the CTA quantises for itself in its prologue (per (token, K-group) scales
// only — every group lies wholly inside one slice, so no exchange is needed).
#include <cooperative_groups.h>

#include "w8a8_internal.h"

namespace cg = cooperative_groups;

namespace w8a8 {
namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kTileRows = kWarps * 16;
constexpr int kPartPitch = kTileRows + 4;  // floats; keeps fragment stores bank-conflict-free
constexpr int kNumSMs = 148;

struct GemvParams {
    LinearArgs a;
    int S;           // K-slices per row tile = cluster size along y
    int bpg;         // 256-byte blocks per group when g >= 256
    int xq_pitch;    // bytes per token row of the staged codes
    int xs_pitch;    // floats per token row of the staged scales
    int max_slice_groups;
};

__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream(const void* p) {
    return __ldcs(reinterpret_cast<const uint4*>(p));
}

struct WBlock {  // one lane's share of 4 K-chunks of its two rows, plus the scales they need
    uint4 a[4], b[4];
    __half sa[4], sb[4];
};

// CPG: 64-byte chunks per group when that is 1, 2 or 4 (g = 64, 128, 256); 0 means
// g is a multiple of 256 larger than 256 and p.bpg counts 256-byte blocks per group.
template <int MT, int CPG, bool FUSED>
__global__ void __launch_bounds__(kThreads) gemv_kernel(const GemvParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const LinearArgs& a = p.a;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, c = lane & 3;
    constexpr int TOK = MT * 8;

    // ---- this CTA's share: rows [n0, n0+64), groups [j0, j0+nj) ----
    const int S = p.S, s = blockIdx.y;
    const int base = a.G / S, rem = a.G % S;
    const int j0 = s * base + min(s, rem);
    const int nj = base + (s < rem ? 1 : 0);
    const int g = a.g;
    const int k0 = j0 * g;
    const int slice_bytes = nj * g;
    const int total_chunks = slice_bytes / 64;
    const int n0 = blockIdx.x * kTileRows;
    constexpr int GPB = CPG == 0 ? 1 : 4 / CPG;  // group boundaries that can fall inside one block

    unsigned char* xq_s = smem;
    float* xs_s = reinterpret_cast<float*>(smem + static_cast<size_t>(TOK) * p.xq_pitch);
    float* part_s = xs_s + TOK * p.xs_pitch;

    const int rowA_raw = n0 + warp * 16 + gq;
    const int rowA = min(rowA_raw, a.N - 1), rowB = min(rowA_raw + 8, a.N - 1);
    const int8_t* pa = a.W + static_cast<size_t>(rowA) * a.K + k0 + c * 16;
    const int8_t* pb = a.W + static_cast<size_t>(rowB) * a.K + k0 + c * 16;
    const __half* wsa = a.w_scale + static_cast<size_t>(rowA) * a.G + j0;
    const __half* wsb = a.w_scale + static_cast<size_t>(rowB) * a.G + j0;

    auto load_block = [&](int blk, WBlock& w) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int t = blk * 4 + i;
            if (t < total_chunks) {
                w.a[i] = ld_stream(pa + t * 64);
                w.b[i] = ld_stream(pb + t * 64);
            }
        }
#pragma unroll
        for (int q = 0; q < GPB; ++q) {
            const int jl = CPG == 0 ? blk / p.bpg : blk * GPB + q;
            if (jl < nj) {
                w.sa[q] = __ldg(wsa + jl);
                w.sb[q] = __ldg(wsb + jl);
            }
        }
    };

    // Weights do not depend on the kernel before this one: start streaming them at once.
    WBlock w0, w1;
    load_block(0, w0);
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- stage the activation slice ----
    if (FUSED) {
        // Quantise X[:, k0:k0+slice) here: int8_gemm.cu:147-211 per (token, group).
        const int vpg = g / 8;  // 16-byte vectors per group
        int lpp = 32;           // lanes per (token, group) pair: largest power of two <= min(32, vpg)
        while (lpp > vpg) lpp >>= 1;
        const int ppw = 32 / lpp, sub = lane % lpp, which = lane / lpp;
        const int pairs = a.M * nj;
        for (int pr0 = warp * ppw; pr0 < pairs; pr0 += kWarps * ppw) {
            const int pr = pr0 + which;
            const bool live = pr < pairs;
            const int m = live ? pr / nj : 0, jl = live ? pr % nj : 0;
            const __half* xg = a.X + static_cast<size_t>(m) * a.K + k0 + jl * g;
            const __half* sm = a.smooth_inv ? a.smooth_inv + k0 + jl * g : nullptr;
            float amax = 0.0f;
            if (live && !a.act_scale) {
                for (int v = sub; v < vpg; v += lpp) {
                    uint4 u = *reinterpret_cast<const uint4*>(xg + v * 8);
                    const __half* h = reinterpret_cast<const __half*>(&u);
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        float f = __half2float(h[e]);
                        if (sm) f *= __half2float(sm[v * 8 + e]);
                        amax = fmaxf(amax, fabsf(f));
                    }
                }
            }
            for (int o = lpp / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            float scale = a.act_scale ? __half2float(a.act_scale[j0 + jl]) : amax / 127.0f;
            if (scale < 1e-8f) scale = 1e-8f;
            const float inv_scale = 1.0f / scale;
            if (live) {
                if (sub == 0) xs_s[m * p.xs_pitch + jl] = scale;
                for (int v = sub; v < vpg; v += lpp) {
                    uint4 u = *reinterpret_cast<const uint4*>(xg + v * 8);
                    const __half* h = reinterpret_cast<const __half*>(&u);
                    uint32_t lo = 0, hi = 0;
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        float f = __half2float(h[e]);
                        if (sm) f *= __half2float(sm[v * 8 + e]);
                        int q = __float2int_rn(f * inv_scale);
                        q = max(-127, min(127, q));
                        if (e < 4) lo |= (static_cast<uint32_t>(q) & 0xffu) << (8 * e);
                        else hi |= (static_cast<uint32_t>(q) & 0xffu) << (8 * (e - 4));
                    }
                    *reinterpret_cast<uint2*>(xq_s + static_cast<size_t>(m) * p.xq_pitch + jl * g + v * 8) =
                        make_uint2(lo, hi);
                }
            }
        }
    } else {
        const int vec_per_row = slice_bytes / 16;
        for (int i = tid; i < a.M * vec_per_row; i += kThreads) {
            const int m = i / vec_per_row, v = i % vec_per_row;
            *reinterpret_cast<uint4*>(xq_s + static_cast<size_t>(m) * p.xq_pitch + v * 16) =
                *reinterpret_cast<const uint4*>(a.Xq + static_cast<size_t>(m) * a.K + k0 + v * 16);
        }
        for (int i = tid; i < a.M * nj; i += kThreads) {
            const int m = i / nj, jl = i % nj;
            xs_s[m * p.xs_pitch + jl] = a.Xs[static_cast<size_t>(m) * a.G + j0 + jl];
        }
    }
    // Token rows past M take part in the MMA as zeros.
    {
        const int vec_per_row = slice_bytes / 16;
        for (int i = tid; i < (TOK - a.M) * vec_per_row; i += kThreads) {
            const int m = a.M + i / vec_per_row, v = i % vec_per_row;
            *reinterpret_cast<uint4*>(xq_s + static_cast<size_t>(m) * p.xq_pitch + v * 16) = make_uint4(0, 0, 0, 0);
        }
        for (int i = tid; i < (TOK - a.M) * nj; i += kThreads)
            xs_s[(a.M + i / nj) * p.xs_pitch + i % nj] = 0.0f;
    }
    __syncthreads();

    // ---- main loop ----
    int P[MT][4];
    float acc[MT][4];
#pragma unroll
    for (int nt = 0; nt < MT; ++nt)
#pragma unroll
        for (int r = 0; r < 4; ++r) { P[nt][r] = 0; acc[nt][r] = 0.0f; }

    auto promote = [&](int jl, __half hsa, __half hsb) {
        const float fa = __half2float(hsa), fb = __half2float(hsb);
#pragma unroll
        for (int nt = 0; nt < MT; ++nt) {
            const int t0 = nt * 8 + 2 * c;
            const float x0 = xs_s[t0 * p.xs_pitch + jl], x1 = xs_s[(t0 + 1) * p.xs_pitch + jl];
            if (a.dump) {
                const int j = j0 + jl;
                const size_t NG = static_cast<size_t>(a.N) * a.G;
                if (rowA_raw < a.N) {
                    if (t0 < a.M) a.dump[t0 * NG + static_cast<size_t>(rowA_raw) * a.G + j] = P[nt][0];
                    if (t0 + 1 < a.M) a.dump[(t0 + 1) * NG + static_cast<size_t>(rowA_raw) * a.G + j] = P[nt][1];
                }
                if (rowA_raw + 8 < a.N) {
                    if (t0 < a.M) a.dump[t0 * NG + static_cast<size_t>(rowA_raw + 8) * a.G + j] = P[nt][2];
                    if (t0 + 1 < a.M) a.dump[(t0 + 1) * NG + static_cast<size_t>(rowA_raw + 8) * a.G + j] = P[nt][3];
                }
            }
            acc[nt][0] = __fmaf_rn(__fmul_rn(static_cast<float>(P[nt][0]), fa), x0, acc[nt][0]);
            acc[nt][1] = __fmaf_rn(__fmul_rn(static_cast<float>(P[nt][1]), fa), x1, acc[nt][1]);
            acc[nt][2] = __fmaf_rn(__fmul_rn(static_cast<float>(P[nt][2]), fb), x0, acc[nt][2]);
            acc[nt][3] = __fmaf_rn(__fmul_rn(static_cast<float>(P[nt][3]), fb), x1, acc[nt][3]);
            P[nt][0] = P[nt][1] = P[nt][2] = P[nt][3] = 0;
        }
    };

    auto process = [&](int blk, const WBlock& w) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int t = blk * 4 + i;
            if (t < total_chunks) {
#pragma unroll
                for (int nt = 0; nt < MT; ++nt) {
                    const uint4 xv = *reinterpret_cast<const uint4*>(
                        xq_s + static_cast<size_t>(nt * 8 + gq) * p.xq_pitch + t * 64 + c * 16);
                    mma_s8(P[nt], w.a[i].x, w.b[i].x, w.a[i].y, w.b[i].y, xv.x, xv.y);
                    mma_s8(P[nt], w.a[i].z, w.b[i].z, w.a[i].w, w.b[i].w, xv.z, xv.w);
                }
                if (CPG != 0) {
                    if ((i + 1) % (CPG == 0 ? 1 : CPG) == 0) {
                        const int q = i / (CPG == 0 ? 1 : CPG);
                        promote(blk * GPB + q, w.sa[q], w.sb[q]);
                    }
                } else if (i == 3 && (blk + 1) % p.bpg == 0) {
                    promote(blk / p.bpg, w.sa[0], w.sb[0]);
                }
            }
        }
    };

    const int nblk = (total_chunks + 3) / 4;
    for (int blk = 0; blk < nblk; blk += 2) {
        load_block(blk + 1, w1);
        process(blk, w0);
        load_block(blk + 2, w0);
        process(blk + 1, w1);
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // ---- fp32 partial tile -> shared memory, [token][row] ----
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) {
        const int t0 = nt * 8 + 2 * c, r = warp * 16 + gq;
        part_s[t0 * kPartPitch + r] = acc[nt][0];
        part_s[(t0 + 1) * kPartPitch + r] = acc[nt][1];
        part_s[t0 * kPartPitch + r + 8] = acc[nt][2];
        part_s[(t0 + 1) * kPartPitch + r + 8] = acc[nt][3];
    }

    cg::cluster_group cluster = cg::this_cluster();
    if (S > 1) cluster.sync(); else __syncthreads();

    // ---- reduce over the S slices in slice order, apply the epilogue, store ----
    // CTA s of the cluster finishes a contiguous 1/S of the tile's rows (of its channels when SwiGLU).
    auto peer_tile = [&](int q) -> const float* {
        return S > 1 ? cluster.map_shared_rank(part_s, q) : part_s;
    };
    if (a.epilogue == W8A8_EPI_SWIGLU) {
        const int H = a.N / 2;
        // 32 channels per tile; channel u lives in rows 16*(u/8) + u%8 (gate) and that + 8 (up).
        const int u_begin = s * 32 / S, u_cnt = (s + 1) * 32 / S - u_begin;
        for (int i = tid; i < u_cnt * a.M; i += kThreads) {
            const int u = u_begin + i % u_cnt, m = i / u_cnt;
            const int rg = 16 * (u / 8) + (u % 8);
            if (n0 + rg + 8 >= a.N) continue;
            float gt = 0.0f, up = 0.0f;
            for (int q = 0; q < S; ++q) {
                const float* t = peer_tile(q);
                gt += t[m * kPartPitch + rg];
                up += t[m * kPartPitch + rg + 8];
            }
            const float g16 = __half2float(__float2half(gt));
            const __half s16 = __float2half(g16 / (1.0f + expf(-g16)));
            const float u16 = __half2float(__float2half(up));
            a.Y[static_cast<size_t>(m) * H + n0 / 2 + u] = __float2half(__half2float(s16) * u16);
        }
    } else {
        const int r_begin = s * kTileRows / S, r_cnt = (s + 1) * kTileRows / S - r_begin;
        for (int i = tid; i < r_cnt * a.M; i += kThreads) {
            const int r = r_begin + i % r_cnt, m = i / r_cnt;
            if (n0 + r >= a.N) continue;
            float v = 0.0f;
            for (int q = 0; q < S; ++q) v += peer_tile(q)[m * kPartPitch + r];
            const size_t o = static_cast<size_t>(m) * a.N + n0 + r;
            __half y = __float2half(v);
            if (a.epilogue == W8A8_EPI_RESIDUAL) y = __float2half(__half2float(y) + __half2float(a.residual[o]));
            a.Y[o] = y;
        }
    }
    if (S > 1) cluster.sync();  // nobody leaves while a peer may still read its tile
}

struct Plan {
    int MT, CPG, S, bpg, xq_pitch, xs_pitch, max_slice_groups;
    size_t smem;
};

bool make_plan(const LinearArgs& a, Plan& pl) {
    if (a.M < 1 || a.M > 32) return false;
    if (a.K % 64 != 0 || a.g % 64 != 0 || a.K % a.g != 0) return false;
    if (a.g > 256 && a.g % 256 != 0) return false;
    if (a.g == 192) return false;
    const bool fused = a.Xq == nullptr;
    uintptr_t al = reinterpret_cast<uintptr_t>(a.W);
    if (fused) al |= reinterpret_cast<uintptr_t>(a.X);
    else al |= reinterpret_cast<uintptr_t>(a.Xq);
    if (al & 15u) return false;
    if (a.epilogue == W8A8_EPI_SWIGLU && a.N % 16 != 0) return false;
    pl.MT = a.M <= 8 ? 1 : (a.M <= 16 ? 2 : 4);
    pl.CPG = a.g == 64 ? 1 : a.g == 128 ? 2 : a.g == 256 ? 4 : 0;
    pl.bpg = a.g >= 256 ? a.g / 256 : 1;
    const int tiles = (a.N + kTileRows - 1) / kTileRows;
    int S = a.split_k;
    if (S <= 0) {
        // Pick the slice count that minimises (CTAs per SM, rounded up) x (bytes per CTA + a fixed
        // per-CTA cost): enough CTAs to cover the SMs, slices of equal group counts preferred.
        double best = 1e30;
        S = 1;
        for (int cand = 1; cand <= 8 && cand <= a.G; ++cand) {
            const int slice_groups = (a.G + cand - 1) / cand;
            const int waves = (tiles * cand + kNumSMs - 1) / kNumSMs;
            const double cost = static_cast<double>(waves) * (static_cast<double>(slice_groups) * a.g + 768.0);
            if (cost < best * 0.999) { best = cost; S = cand; }
        }
    }
    if (S > 8 || S > a.G || S < 1) return false;
    pl.S = S;
    pl.max_slice_groups = (a.G + S - 1) / S;
    const int slice_bytes = pl.max_slice_groups * a.g;
    pl.xq_pitch = (slice_bytes % 128 == 0) ? slice_bytes + 64 : slice_bytes;  // == 64 mod 128
    pl.xs_pitch = pl.max_slice_groups | 1;
    const int TOK = pl.MT * 8;
    pl.smem = static_cast<size_t>(TOK) * pl.xq_pitch + sizeof(float) * TOK * pl.xs_pitch +
              sizeof(float) * TOK * kPartPitch;
    pl.smem = (pl.smem + 15) & ~size_t(15);
    return pl.smem <= 200 * 1024;
}

template <int MT, int CPG, bool FUSED>
int launch_variant(const GemvParams& p, const Plan& pl, cudaStream_t stream) {
    auto kern = gemv_kernel<MT, CPG, FUSED>;
    if (pl.smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(pl.smem));
        if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.a.N + kTileRows - 1) / kTileRows, pl.S, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = pl.S;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "gemv launch: %s", cudaGetErrorString(e));
    return W8A8_OK;
}

template <int MT, bool FUSED>
int launch_cpg(const GemvParams& p, const Plan& pl, cudaStream_t s) {
    switch (pl.CPG) {
        case 1: return launch_variant<MT, 1, FUSED>(p, pl, s);
        case 2: return launch_variant<MT, 2, FUSED>(p, pl, s);
        case 4: return launch_variant<MT, 4, FUSED>(p, pl, s);
        default: return launch_variant<MT, 0, FUSED>(p, pl, s);
    }
}

template <bool FUSED>
int launch_mt(const GemvParams& p, const Plan& pl, cudaStream_t s) {
    switch (pl.MT) {
        case 1: return launch_cpg<1, FUSED>(p, pl, s);
        case 2: return launch_cpg<2, FUSED>(p, pl, s);
        default: return launch_cpg<4, FUSED>(p, pl, s);
    }
}

}  // namespace

bool gemv_supports(const LinearArgs& a) {
    Plan pl;
    return make_plan(a, pl);
}

int launch_linear_gemv(const LinearArgs& a, cudaStream_t s) {
    Plan pl;
    if (!make_plan(a, pl)) return fail(W8A8_ERR_UNSUPPORTED, "gemv kernel does not take this shape");
    GemvParams p;
    p.a = a;
    p.S = pl.S;
    p.bpg = pl.bpg;
    p.xq_pitch = pl.xq_pitch;
    p.xs_pitch = pl.xs_pitch;
    p.max_slice_groups = pl.max_slice_groups;
    return a.Xq ? launch_mt<false>(p, pl, s) : launch_mt<true>(p, pl, s);
}

}  // namespace w8a8
