// Small-M (decode) W8A8 linear: a weight-streaming kernel bound by HBM bandwidth.
//
// Replaces int8_matvec_dequant_kernel / int8_smallbatch_dequant_kernel and, for
// 4 < tokens <= 32, the per-group cuBLAS loop of int8_gemm.cu:245-505. Input is the
// activation codes and scales (int8_gemm.cu:147-211 is the row kernel in w8a8_quant.cu).
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
// load 128-bit and contiguous; activation codes are read with the same
// permutation, straight from global memory: they are a few KB shared by every
// CTA, so after first touch they are L1 hits. The int32 sums of one K-group are
// exact and complete inside one warp; they are promoted with
// acc = fma(float(P) * ws, xs, acc) in ascending group order.
//
// Launched with programmatic dependent launch: the first weight block is
// requested before griddepcontrol.wait, i.e. while the kernel that produces the
// activations is still running. Weights must not be written by that kernel.
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
    int S;    // K-slices per row tile = cluster size along y
    int bpg;  // 256-byte blocks per group when g >= 256
};

__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Weights are read once: stream them past L1.
__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

struct WBlock {  // one lane's share of 4 K-chunks of its two rows, plus the scales they need
    uint4 a[4], b[4];
    __half sa[4], sb[4];
};

// CPG: 64-byte chunks per group when that is 1, 2 or 4 (g = 64, 128, 256); 0 means
// g is a multiple of 256 larger than 256 and p.bpg counts 256-byte blocks per group.
template <int MT, int CPG>
__global__ void __launch_bounds__(kThreads) gemv_kernel(const GemvParams p) {
    __shared__ float part_s[MT * 8 * kPartPitch];
    const LinearArgs& a = p.a;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, c = lane & 3;

    // ---- this CTA's share: rows [n0, n0+64), groups [j0, j0+nj) ----
    const int S = p.S, s = blockIdx.y;
    const int base = a.G / S, rem = a.G % S;
    const int j0 = s * base + min(s, rem);
    const int nj = base + (s < rem ? 1 : 0);
    const int g = a.g;
    const int k0 = j0 * g;
    const int total_chunks = nj * (g / 64);
    const int n0 = blockIdx.x * kTileRows;
    constexpr int GPB = CPG == 0 ? 1 : 4 / CPG;  // group boundaries that can fall inside one block

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
    load_block(1, w1);
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // Token rows past M read the last real row; their results are never stored.
    const int8_t* xq[MT];
    const float* xsp[MT][2];
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) {
        xq[nt] = a.Xq + static_cast<size_t>(min(nt * 8 + gq, a.M - 1)) * a.K + k0 + c * 16;
        xsp[nt][0] = a.Xs + static_cast<size_t>(min(nt * 8 + 2 * c, a.M - 1)) * a.G + j0;
        xsp[nt][1] = a.Xs + static_cast<size_t>(min(nt * 8 + 2 * c + 1, a.M - 1)) * a.G + j0;
    }

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
            const float x0 = __ldg(xsp[nt][0] + jl), x1 = __ldg(xsp[nt][1] + jl);
            if (a.dump) {
                const int t0 = nt * 8 + 2 * c, j = j0 + jl;
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
        // Activation codes come from L1; request a whole block's worth up front (two chunks at a
        // time when 32 tokens make that too many registers).
        constexpr int XB = MT <= 2 ? 4 : 2;
        uint4 xv[XB][MT];
#pragma unroll
        for (int i0 = 0; i0 < 4; i0 += XB) {
#pragma unroll
            for (int i = 0; i < XB; ++i)
#pragma unroll
                for (int nt = 0; nt < MT; ++nt)
                    if (blk * 4 + i0 + i < total_chunks)
                        xv[i][nt] = __ldg(reinterpret_cast<const uint4*>(xq[nt] + (blk * 4 + i0 + i) * 64));
#pragma unroll
            for (int ii = 0; ii < XB; ++ii) {
                const int i = i0 + ii;
                const int t = blk * 4 + i;
                if (t < total_chunks) {
#pragma unroll
                    for (int nt = 0; nt < MT; ++nt) {
                        mma_s8(P[nt], w.a[i].x, w.b[i].x, w.a[i].y, w.b[i].y, xv[ii][nt].x, xv[ii][nt].y);
                        mma_s8(P[nt], w.a[i].z, w.b[i].z, w.a[i].w, w.b[i].w, xv[ii][nt].z, xv[ii][nt].w);
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
        }
    };

    const int nblk = (total_chunks + 3) / 4;
    for (int blk = 0; blk < nblk; blk += 2) {
        process(blk, w0);
        load_block(blk + 2, w0);
        process(blk + 1, w1);
        load_block(blk + 3, w1);
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
    int MT, CPG, S, bpg;
};

bool make_plan(const LinearArgs& a, Plan& pl) {
    if (a.M < 1 || a.M > 32 || !a.Xq || !a.Xs) return false;
    if (a.K % 64 != 0 || a.g % 64 != 0 || a.K % a.g != 0) return false;
    if (a.g > 256 && a.g % 256 != 0) return false;
    if (a.g == 192) return false;
    if ((reinterpret_cast<uintptr_t>(a.W) | reinterpret_cast<uintptr_t>(a.Xq)) & 15u) return false;
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
    return true;
}

template <int MT, int CPG>
int launch_variant(const GemvParams& p, const Plan& pl, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.a.N + kTileRows - 1) / kTileRows, pl.S, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = pl.S;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled(kPdlLinear) ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_kernel<MT, CPG>, p);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "gemv launch: %s", cudaGetErrorString(e));
    return W8A8_OK;
}

template <int MT>
int launch_cpg(const GemvParams& p, const Plan& pl, cudaStream_t s) {
    switch (pl.CPG) {
        case 1: return launch_variant<MT, 1>(p, pl, s);
        case 2: return launch_variant<MT, 2>(p, pl, s);
        case 4: return launch_variant<MT, 4>(p, pl, s);
        default: return launch_variant<MT, 0>(p, pl, s);
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
    switch (pl.MT) {
        case 1: return launch_cpg<1>(p, pl, s);
        case 2: return launch_cpg<2>(p, pl, s);
        default: return launch_cpg<4>(p, pl, s);
    }
}

}  // namespace w8a8
