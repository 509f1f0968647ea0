// Decode-step neighbours of the linear layer inside one transformer layer:
//   (1) split the fused qkv row, per-head RMSNorm of q and k, interleaved-pair RoPE, and the write
//       of k / v into the paged cache — one launch instead of the reference's three device copies,
//       two rms_norm launches, rope_qk and 2 x n_kv cudaMemcpyAsync per layer
//       (src/engine/dual_ar_engine.cc:585-628, src/kernels/rope.cu:9-65);
//   (2) single-query paged attention over 16-token blocks with GQA
//       (src/kernels/paged_attention.cu:13-110), one CTA cluster per (sequence, kv head) so that the
//       four query heads of a group share every K/V byte, the context split over the cluster and over
//       warps, partial softmax states merged through (distributed) shared memory; the epilogue can
//       emit the o-projection's int8 codes and scales directly.
// Both follow the reference's fp16 rounding points; (1) also follows its summation order, so q, k and
// the cache contents are bit-identical to the reference chain. (2) sums in a different order than
// the reference's one-warp-per-head loop and is compared at a tolerance.
#include <cooperative_groups.h>

#include "sm100_ptx.cuh"
#include "w8a8_internal.h"
#include "w8a8_trace.cuh"

namespace cg = cooperative_groups;

namespace w8a8 {
namespace {

constexpr int kHeadDim = 128;
constexpr int kBlockTokens = 16;

struct RopeParams {
    const __half* qkv;        // [B, (n_q + 2 n_kv) * 128]
    const __half* q_norm_w;   // [128] or null (no qk-norm: the fast AR)
    const __half* k_norm_w;
    float eps;
    const float* freqs;       // [64]
    const int* positions;     // [B] position of the new token
    const int* block_table;   // [B, max_blocks]
    int max_blocks;
    __half* k_cache;
    __half* v_cache;          // [blocks, n_layers, n_kv, 16, 128]
    int layer, n_layers, n_q, n_kv;
    __half* q_out;            // [B, n_q, 128]
};

// One warp per (sequence, head). Lane i holds elements i, 32+i, 64+i, 96+i: the four 32-element
// runs are the four "warps" of the reference's 128-thread rms_norm launch, so four shuffle-down
// trees followed by (p0+p2)+(p1+p3) reproduce its sum bit for bit (rms_norm.cu:23-49).
__global__ void __launch_bounds__(128) qknorm_rope_kvwrite_kernel(const RopeParams p) {
    ptx::pdl_launch_dependents();
    const int b = blockIdx.x;
    const int head = blockIdx.y * 4 + (threadIdx.x >> 5);  // 0..n_q-1 q, then k heads, then v heads
    const int lane = threadIdx.x & 31;
    const int total_heads = p.n_q + 2 * p.n_kv;
    if (head >= total_heads) return;
    const __half* src = p.qkv + (static_cast<size_t>(b) * total_heads + head) * kHeadDim;
    const bool is_q = head < p.n_q, is_k = !is_q && head < p.n_q + p.n_kv;
    // parameters (norm weights, rotation frequencies) are requested before the wait for the qkv projection
    const __half* w = is_q ? p.q_norm_w : (is_k ? p.k_norm_w : nullptr);
    __half wv[4];
    float fr[4];
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        wv[v] = w ? w[v * 32 + lane] : __float2half(1.0f);
        fr[v] = p.freqs[(v * 32 + lane) >> 1];
    }
    ptx::pdl_wait();
    const int pos = p.positions[b];
    __half h[4];
#pragma unroll
    for (int v = 0; v < 4; ++v) h[v] = src[v * 32 + lane];
    // the cache slot of the new token: a second dependent load, started now rather than after the arithmetic
    int phys = 0;
    if (!is_q) phys = p.block_table[static_cast<size_t>(b) * p.max_blocks + pos / kBlockTokens];

    if (is_q || is_k) {
        if (w) {
            float part[4];
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                float val = __half2float(h[v]);
                float local_sum = 0.0f;
                local_sum += val * val;
                for (int offset = 16; offset > 0; offset /= 2)
                    local_sum += __shfl_down_sync(0xffffffffu, local_sum, offset);
                part[v] = __shfl_sync(0xffffffffu, local_sum, 0);
            }
            // the reference's second tree over its four warp partials (lanes 4..31 hold 0.0f)
            float total_sum = (part[0] + part[2]) + (part[1] + part[3]);
            const float rms = rsqrtf(total_sum / kHeadDim + p.eps);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                float val = __half2float(h[v]) * rms;
                h[v] = __float2half(val * __half2float(wv[v]));
            }
        }
        // RoPE on interleaved pairs (2i, 2i+1): neighbours in the same run (rope.cu:36-45)
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            const float freq = fr[v];
            float angle = freq * static_cast<float>(pos);
            float cos_a = cosf(angle), sin_a = sinf(angle);
            const float mine = __half2float(h[v]);
            const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
            float q0 = (lane & 1) ? other : mine, q1 = (lane & 1) ? mine : other;
            h[v] = (lane & 1) ? __float2half(q0 * sin_a + q1 * cos_a) : __float2half(q0 * cos_a - q1 * sin_a);
        }
    }
    if (is_q) {
        __half* dst = p.q_out + (static_cast<size_t>(b) * p.n_q + head) * kHeadDim;
#pragma unroll
        for (int v = 0; v < 4; ++v) dst[v * 32 + lane] = h[v];
    } else {
        const int kvh = is_k ? head - p.n_q : head - p.n_q - p.n_kv;
        if (phys < 0) return;
        __half* cache = is_k ? p.k_cache : p.v_cache;
        __half* dst = cache + ((((static_cast<size_t>(phys) * p.n_layers + p.layer) * p.n_kv + kvh) * kBlockTokens) +
                               pos % kBlockTokens) * kHeadDim;
#pragma unroll
        for (int v = 0; v < 4; ++v) dst[v * 32 + lane] = h[v];
    }
}

// ---------------------------------------------------------------------------------------------
struct AttnParams {
    const __half* q;          // [B, n_q, 128]
    const __half* k_cache;
    const __half* v_cache;
    const int* block_table;
    const int* seq_lens;
    int max_blocks;
    int n_q, n_kv, layer, n_layers;
    float sm_scale;
    __half* out;              // [B, n_q, 128] or null
    int8_t* Xq;               // [B, n_q*128] or null: codes of `out` for the following linear
    float* Xs;                // [B, n_q*128/g]
    int g;
    int S;                    // context slices = cluster size
    // fused prologue (ROPE form): q, k, v of the new token come from the qkv projection's output
    const __half* qkv;        // [B, (n_q + 2 n_kv) * 128]
    const __half* q_norm_w;   // [128] or null
    const __half* k_norm_w;
    float eps;
    const float* freqs;       // [64]
    const int* positions;     // [B]
    __half* k_cache_w;        // the caches again, writable
    __half* v_cache_w;
};

constexpr int kAttnWarps = 8;
constexpr int kQPerKv = 4;  // query heads per kv head handled by one CTA

// K and V of one 16-token block as one lane sees them (64 registers):
//   k[j][i]: token j*8 + (lane>>2), 16-byte piece i*4 + (lane&3) of its 128 dims;
//   v[q][h]: token {2t, 2t+1, 2t+8, 2t+9}[q] with t = lane&3, 16-byte piece (lane>>2) + 8h.
struct KvFrag {
    uint4 k[2][4];
    uint4 v[4][2];
};

__device__ __forceinline__ uint4 ld_stream16(const __half* ptr) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(ptr));
    return r;
}

__device__ __forceinline__ uint4 ld_cg16(const __half* ptr) {
    uint4 r;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(ptr));
    return r;
}

// One warp, one head of the new token: per-head RMSNorm in the reference's order (rms_norm.cu:23-49 with a
// 128-thread block) and interleaved-pair RoPE (rope.cu:36-45) — the arithmetic of qknorm_rope_kvwrite_kernel.
// h: elements lane, 32+lane, 64+lane, 96+lane; w, fr: norm weights and frequencies of the same elements.
__device__ __forceinline__ void head_norm_rope(__half (&h)[4], bool with_norm, const __half (&w)[4], float eps,
                                               const float (&fr)[4], int pos, int lane) {
    if (with_norm) {
        float part[4];
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            float val = __half2float(h[v]);
            float local_sum = 0.0f;
            local_sum += val * val;
            for (int offset = 16; offset > 0; offset /= 2) local_sum += __shfl_down_sync(0xffffffffu, local_sum, offset);
            part[v] = __shfl_sync(0xffffffffu, local_sum, 0);
        }
        float total_sum = (part[0] + part[2]) + (part[1] + part[3]);
        const float rms = rsqrtf(total_sum / kHeadDim + eps);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            float val = __half2float(h[v]) * rms;
            h[v] = __float2half(val * __half2float(w[v]));
        }
    }
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        float angle = fr[v] * static_cast<float>(pos);
        float cos_a = cosf(angle), sin_a = sinf(angle);
        const float mine = __half2float(h[v]);
        const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
        float q0 = (lane & 1) ? other : mine, q1 = (lane & 1) ? mine : other;
        h[v] = (lane & 1) ? __float2half(q0 * sin_a + q1 * cos_a) : __float2half(q0 * cos_a - q1 * sin_a);
    }
}

// D(16x8, fp32) += A(16x16 fp16, rows 8..15 zero) x B(16x8 fp16). Only rows 0..7 of D are kept.
__device__ __forceinline__ void mma_top_rows(float& d0, float& d1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    float j2, j3;
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=f"(d0), "=f"(d1), "=f"(j2), "=f"(j3)
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(d0), "f"(d1), "f"(0.0f), "f"(0.0f));
}

__device__ __forceinline__ uint32_t reg_of(const uint4& v, int i) {
    return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

// grid (S, n_kv, B), cluster (S,1,1), 8 warps. The four query heads of a kv group are rows 0..3 of a
// 16-row tensor-core tile (mma.sync.m16n8k16, fp32 accumulate): scores = Q K^T with tokens as the
// n index, then out += P V with P rounded to fp16 (the softmax denominator is summed from the same
// rounded values, so the weights stay normalised). The sums over head dims (QK) and over tokens (PV)
// do not depend on order, so each lane takes whole 16-byte pieces straight from the cache and the
// "k index" of an MMA is a permutation of the real one, applied to q alike; V's token pairs are put
// side by side with one byte-permute per register. Nothing is staged in shared memory. Each warp
// keeps the next block's 8 KB in flight while it works on the current one.
//
// ROPE form: the launch also does what qknorm_rope_kvwrite_kernel does. Warps 0..3 norm and rotate the four
// query heads into shared memory; in the CTA that attends over the block the new token joins, warps 4 and 5
// write the new k and v rows into the cache first. The first two KV blocks of every warp are requested
// before that work, so its latency hides under theirs.
template <bool ROPE>
__global__ void __launch_bounds__(kAttnWarps * 32, 1) paged_attention_decode_kernel(const AttnParams p) {
    W8A8_TRACE_SCOPE();
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    W8A8_TRACE_WAITED();
    __shared__ __align__(16) __half q_s[ROPE ? kQPerKv : 1][kHeadDim];
    __shared__ float red_m[kAttnWarps][kQPerKv], red_l[kAttnWarps][kQPerKv];
    __shared__ float red_acc[kAttnWarps][kQPerKv][kHeadDim];
    __shared__ float cta_m[kQPerKv], cta_l[kQPerKv];
    __shared__ __align__(16) float cta_acc[kQPerKv][kHeadDim];
    __shared__ __align__(16) __half out_s[kQPerKv * kHeadDim];

    const int s = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, S = p.S;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int seq_len = p.seq_lens[b];
    // 16-token blocks are dealt round-robin: first over the cluster's CTAs, then over the warps. The physical
    // numbers of this warp's next 32 blocks, one per lane, are requested before seq_len is used anywhere (the
    // read is bounded by the table's width), so that the two reads are one round trip, not two.
    const int stride = S * kAttnWarps, first = s + warp * S;
    auto fetch_phys = [&](int it0) -> int {
        const int bi = first + (it0 + lane) * stride;
        return bi < p.max_blocks ? p.block_table[static_cast<size_t>(b) * p.max_blocks + bi] : 0;
    };
    int phys_mine = fetch_phys(0);
    const int heads_here = p.n_q / p.n_kv;  // == kQPerKv (checked on the host)

    // ROPE: everything the prologue reads is requested here, before the first value is used
    int pos = 0;
    bool owner = false;
    const bool role_q = warp < kQPerKv, is_k = warp == kQPerKv, is_v = warp == kQPerKv + 1;
    __half hq[4], wq[4];
    float fr[4];
    const __half* norm_w = nullptr;
    if constexpr (ROPE) {
        pos = p.positions[b];
        norm_w = role_q ? p.q_norm_w : p.k_norm_w;
        const int total_heads = p.n_q + 2 * p.n_kv;
        const __half* src = p.qkv + (static_cast<size_t>(b) * total_heads +
                                     (role_q ? kvh * heads_here + warp : p.n_q + (is_k ? 0 : p.n_kv) + kvh)) * kHeadDim;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            hq[v] = (role_q || is_k || is_v) ? src[v * 32 + lane] : __float2half(0.0f);
            wq[v] = norm_w ? norm_w[v * 32 + lane] : __float2half(1.0f);
            fr[v] = p.freqs[(v * 32 + lane) >> 1];
        }
        owner = ((pos / kBlockTokens) % S) == s;  // this CTA attends over the block the new token joins
    }

    const int n_blocks = (seq_len + kBlockTokens - 1) / kBlockTokens;
    const int n_mine = first < n_blocks ? (n_blocks - first + stride - 1) / stride : 0;

    auto load = [&](KvFrag& f, int it) {
        if ((it & 31) == 0 && it > 0) phys_mine = fetch_phys(it);
        const int phys = __shfl_sync(0xffffffffu, phys_mine, it & 31);
        const int bi = first + it * stride;
        const int tokens = min(kBlockTokens, seq_len - bi * kBlockTokens);
        const size_t base = (((static_cast<size_t>(phys) * p.n_layers + p.layer) * p.n_kv + kvh) * kBlockTokens) * kHeadDim;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int tok = j * 8 + g;
            const __half* row = p.k_cache + base + static_cast<size_t>(tok < tokens ? tok : 0) * kHeadDim;
#pragma unroll
            for (int i = 0; i < 4; ++i) f.k[j][i] = ROPE ? ld_cg16(row + (i * 4 + t) * 8) : ld_stream16(row + (i * 4 + t) * 8);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int tok = 2 * t + (q & 1) + 8 * (q >> 1);
            const __half* row = p.v_cache + base + static_cast<size_t>(tok < tokens ? tok : 0) * kHeadDim;
#pragma unroll
            for (int h = 0; h < 2; ++h) f.v[q][h] = ROPE ? ld_cg16(row + (g + 8 * h) * 8) : ld_stream16(row + (g + 8 * h) * 8);
        }
    };

    KvFrag fa, fb;
    const int new_bi = pos / kBlockTokens;
    const bool pre0 = n_mine > 0 && !(ROPE && owner && first == new_bi);
    const bool pre1 = n_mine > 1 && !(ROPE && owner && first + stride == new_bi);
    if (pre0) load(fa, 0);
    if (pre1) load(fb, 1);
    if constexpr (ROPE) {
        if (role_q || ((is_k || is_v) && owner)) {
            if (!is_v) head_norm_rope(hq, norm_w != nullptr, wq, p.eps, fr, pos, lane);
            if (role_q) {
#pragma unroll
                for (int v = 0; v < 4; ++v) q_s[warp][v * 32 + lane] = hq[v];
            } else {
                const int phys = p.block_table[static_cast<size_t>(b) * p.max_blocks + new_bi];
                if (phys >= 0) {
                    __half* dst = (is_k ? p.k_cache_w : p.v_cache_w) +
                                  ((((static_cast<size_t>(phys) * p.n_layers + p.layer) * p.n_kv + kvh) * kBlockTokens) +
                                   pos % kBlockTokens) * kHeadDim;
#pragma unroll
                    for (int v = 0; v < 4; ++v) dst[v * 32 + lane] = hq[v];
                }
            }
        }
        __syncthreads();  // q in shared memory; the new k and v rows written (read back past L1)
        if (n_mine > 0 && !pre0) load(fa, 0);
        if (n_mine > 1 && !pre1) load(fb, 1);
    }
    // q of head g (rows 4..15 of the tile are zero), in the same piece order as K
    uint32_t qa[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (g < kQPerKv) {
            if constexpr (ROPE) v = *reinterpret_cast<const uint4*>(&q_s[g][(i * 4 + t) * 8]);
            else v = *reinterpret_cast<const uint4*>(p.q + (static_cast<size_t>(b) * p.n_q + kvh * heads_here + g) * kHeadDim +
                                                     (i * 4 + t) * 8);
        }
        qa[i][0] = v.x; qa[i][1] = v.y; qa[i][2] = v.z; qa[i][3] = v.w;
    }

    float m_run = -1e30f, l_run = 0.0f;
    float o[16][2];  // head g; tile n = 8h + e holds dims (2t + 8h)*8 + e and (2t + 1 + 8h)*8 + e
#pragma unroll
    for (int n = 0; n < 16; ++n) { o[n][0] = 0.0f; o[n][1] = 0.0f; }

    auto compute = [&](const KvFrag& f, int it) {
        const int bi = first + it * stride;
        const int tokens = min(kBlockTokens, seq_len - bi * kBlockTokens);
        float sc[2][2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            sc[j][0] = 0.0f; sc[j][1] = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    mma_top_rows(sc[j][0], sc[j][1], qa[i][2 * h], qa[i][2 * h + 1], reg_of(f.k[j][i], 2 * h),
                                 reg_of(f.k[j][i], 2 * h + 1));
            }
        }
        float mx = -1e30f;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int tok = j * 8 + 2 * t + e;
                sc[j][e] = tok < tokens ? sc[j][e] * p.sm_scale : -1e30f;
                mx = fmaxf(mx, sc[j][e]);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float new_m = fmaxf(m_run, mx);
        const float corr = __expf(m_run - new_m);
        m_run = new_m;
        const __half2 p0 = __floats2half2_rn(__expf(sc[0][0] - new_m), __expf(sc[0][1] - new_m));
        const __half2 p1 = __floats2half2_rn(__expf(sc[1][0] - new_m), __expf(sc[1][1] - new_m));
        const float2 f0 = __half22float2(p0), f1 = __half22float2(p1);
        l_run = l_run * corr + ((f0.x + f0.y) + (f1.x + f1.y));
        const uint32_t pa0 = *reinterpret_cast<const uint32_t*>(&p0), pa2 = *reinterpret_cast<const uint32_t*>(&p1);
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int n = h * 8 + e;
                const uint32_t sel = (e & 1) ? 0x7632u : 0x5410u;
                const uint32_t b0 = __byte_perm(reg_of(f.v[0][h], e >> 1), reg_of(f.v[1][h], e >> 1), sel);
                const uint32_t b1 = __byte_perm(reg_of(f.v[2][h], e >> 1), reg_of(f.v[3][h], e >> 1), sel);
                o[n][0] *= corr;
                o[n][1] *= corr;
                mma_top_rows(o[n][0], o[n][1], pa0, pa2, b0, b1);
            }
    };

    for (int it = 0; it < n_mine;) {  // fa holds block `it`, fb block `it + 1`
        compute(fa, it);
        if (it + 2 < n_mine) load(fa, it + 2);
        if (++it >= n_mine) break;
        compute(fb, it);
        if (it + 2 < n_mine) load(fb, it + 2);
        ++it;
    }
    // the four lanes of a quad hold the same head: their partial denominators add up
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (g < kQPerKv) {
        if (t == 0) { red_m[warp][g] = m_run; red_l[warp][g] = l_run; }
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                red_acc[warp][g][(2 * t + 8 * h) * 8 + e] = o[h * 8 + e][0];
                red_acc[warp][g][(2 * t + 1 + 8 * h) * 8 + e] = o[h * 8 + e][1];
            }
    }
    __syncthreads();
    // ---- merge the warps: thread -> (head, 4 dims) ----
    if (threadIdx.x < kQPerKv * 32) {
        const int hh = threadIdx.x >> 5, d0 = (threadIdx.x & 31) * 4;
        float m = -1e30f;
        for (int w = 0; w < kAttnWarps; ++w) m = fmaxf(m, red_m[w][hh]);
        float l = 0.0f, a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int w = 0; w < kAttnWarps; ++w) {
            const float scw = __expf(red_m[w][hh] - m);
            l += red_l[w][hh] * scw;
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] += red_acc[w][hh][d0 + i] * scw;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) cta_acc[hh][d0 + i] = a[i];
        if ((threadIdx.x & 31) == 0) { cta_m[hh] = m; cta_l[hh] = l; }
    }
    cg::cluster_group cluster = cg::this_cluster();
    if (S > 1) cluster.sync(); else __syncthreads();
    // ---- CTA 0 of the cluster merges the S context slices and writes the 4 heads ----
    if (s == 0 && threadIdx.x < kQPerKv * 32) {
        const int hh = threadIdx.x >> 5, d0 = (threadIdx.x & 31) * 4;
        float m = -1e30f;
        for (int r = 0; r < S; ++r) m = fmaxf(m, (S > 1 ? cluster.map_shared_rank(cta_m, r) : cta_m)[hh]);
        float l = 0.0f, a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int r = 0; r < S; ++r) {
            const float* pm = S > 1 ? cluster.map_shared_rank(cta_m, r) : cta_m;
            const float* pl = S > 1 ? cluster.map_shared_rank(cta_l, r) : cta_l;
            const float* pa = S > 1 ? cluster.map_shared_rank(&cta_acc[0][0], r) : &cta_acc[0][0];
            const float scr = __expf(pm[hh] - m);
            l += pl[hh] * scr;
            const float4 v4 = *reinterpret_cast<const float4*>(pa + hh * kHeadDim + d0);
            a[0] += v4.x * scr; a[1] += v4.y * scr; a[2] += v4.z * scr; a[3] += v4.w * scr;
        }
        const float inv = seq_len > 0 ? 1.0f / l : 0.0f;  // empty sequence -> zeros (paged_attention.cu:44-50)
        __align__(8) __half o4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) o4[i] = __float2half(seq_len > 0 ? a[i] * inv : 0.0f);
#pragma unroll
        for (int i = 0; i < 4; ++i) out_s[hh * kHeadDim + d0 + i] = o4[i];
        const size_t oo = (static_cast<size_t>(b) * p.n_q + kvh * heads_here + hh) * kHeadDim + d0;
        if (p.out) *reinterpret_cast<uint2*>(p.out + oo) = *reinterpret_cast<const uint2*>(o4);
    }
    if (S > 1) cluster.sync(); else __syncthreads();
    // ---- optional: quantise these 512 channels for the o-projection (int8_gemm.cu:147-211) ----
    if (s == 0 && p.Xq) {
        const int gsz = p.g, K = p.n_q * kHeadDim, G = K / gsz;
        const int ch0 = kvh * heads_here * kHeadDim;          // first channel of this CTA
        const int groups_here = (kQPerKv * kHeadDim) / gsz;   // 2 at g=256, 8 at g=64
        for (int j = warp; j < groups_here; j += kAttnWarps) {
            float amax = 0.0f;
            for (int e = lane; e < gsz; e += 32) amax = fmaxf(amax, fabsf(__half2float(out_s[j * gsz + e])));
            for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
            float scale = amax / 127.0f;
            if (scale < 1e-8f) scale = 1e-8f;
            if (lane == 0) p.Xs[static_cast<size_t>(b) * G + ch0 / gsz + j] = scale;
            const float inv_scale = 1.0f / scale;
            for (int e = lane; e < gsz; e += 32) {
                int qv = __float2int_rn(__half2float(out_s[j * gsz + e]) * inv_scale);
                qv = max(-127, min(127, qv));
                p.Xq[static_cast<size_t>(b) * K + ch0 + j * gsz + e] = static_cast<int8_t>(qv);
            }
        }
    }
    W8A8_TRACE_END(4u);
}

}  // namespace

int launch_qknorm_rope_kvwrite(const __half* qkv, const __half* q_norm_w, const __half* k_norm_w, float eps,
                               const float* freqs, const int* positions, const int* block_table, int max_blocks,
                               __half* k_cache, __half* v_cache, int layer, int n_layers, int B, int n_q, int n_kv,
                               __half* q_out, cudaStream_t stream) {
    if (B == 0) return W8A8_OK;
    RopeParams p = {qkv, q_norm_w, k_norm_w, eps, freqs, positions, block_table, max_blocks, k_cache, v_cache,
                    layer, n_layers, n_q, n_kv, q_out};
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(B, (n_q + 2 * n_kv + 3) / 4, 1);
    cfg.blockDim = dim3(128, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled(kPdlAttn) ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, qknorm_rope_kvwrite_kernel, p);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "qknorm_rope_kvwrite launch: %s", cudaGetErrorString(e));
    return W8A8_OK;
}

namespace {
int launch_attention(const AttnParams& base, int B, int splits, cudaStream_t stream);
}

int launch_paged_attention_decode(const __half* q, const __half* k_cache, const __half* v_cache,
                                  const int* block_table, const int* seq_lens, int B, int n_q, int n_kv,
                                  int max_blocks, float sm_scale, int layer, int n_layers, __half* out, int g,
                                  int8_t* Xq, float* Xs, int splits, cudaStream_t stream) {
    AttnParams p = {};
    p.q = q; p.k_cache = k_cache; p.v_cache = v_cache; p.block_table = block_table; p.seq_lens = seq_lens;
    p.max_blocks = max_blocks; p.n_q = n_q; p.n_kv = n_kv; p.layer = layer; p.n_layers = n_layers; p.sm_scale = sm_scale;
    p.out = out; p.Xq = Xq; p.Xs = Xs; p.g = g;
    return launch_attention(p, B, splits, stream);
}

int launch_qkv_attention_decode(const __half* qkv, const __half* q_norm_w, const __half* k_norm_w, float eps,
                                const float* freqs, const int* positions, __half* k_cache, __half* v_cache,
                                const int* block_table, const int* seq_lens, int B, int n_q, int n_kv, int max_blocks,
                                float sm_scale, int layer, int n_layers, __half* out, int g, int8_t* Xq, float* Xs,
                                int splits, cudaStream_t stream) {
    AttnParams p = {};
    p.k_cache = k_cache; p.v_cache = v_cache; p.block_table = block_table; p.seq_lens = seq_lens;
    p.max_blocks = max_blocks; p.n_q = n_q; p.n_kv = n_kv; p.layer = layer; p.n_layers = n_layers; p.sm_scale = sm_scale;
    p.out = out; p.Xq = Xq; p.Xs = Xs; p.g = g;
    p.qkv = qkv; p.q_norm_w = q_norm_w; p.k_norm_w = k_norm_w; p.eps = eps; p.freqs = freqs; p.positions = positions;
    p.k_cache_w = k_cache; p.v_cache_w = v_cache;
    return launch_attention(p, B, splits, stream);
}

namespace {
int launch_attention(const AttnParams& base, int B, int splits, cudaStream_t stream) {
    const int n_q = base.n_q, n_kv = base.n_kv, g = base.g;
    const int8_t* Xq = base.Xq;
    if (B == 0) return W8A8_OK;
    if (n_kv <= 0 || n_q != n_kv * kQPerKv)
        return fail(W8A8_ERR_UNSUPPORTED, "paged attention here handles 4 query heads per kv head (got %d / %d)", n_q, n_kv);
    if (Xq && (g <= 0 || (kQPerKv * kHeadDim) % g != 0))
        return fail(W8A8_ERR_UNSUPPORTED, "fused output quantisation needs a group size dividing 512 (got %d)", g);
    if (splits <= 0) {  // one CTA per SM: as many context slices as the (sequence, kv head) pairs leave room for
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
        const int want = sms / (B * n_kv);
        splits = want >= 8 ? 8 : want >= 4 ? 4 : want >= 2 ? 2 : 1;
    }
    if (splits > 8) splits = 8;
    AttnParams p = base;
    p.S = splits;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, n_kv, B);
    cfg.blockDim = dim3(kAttnWarps * 32, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled(kPdlAttn) ? 2 : 1;
    cudaError_t e = p.qkv ? cudaLaunchKernelEx(&cfg, paged_attention_decode_kernel<true>, p)
                          : cudaLaunchKernelEx(&cfg, paged_attention_decode_kernel<false>, p);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "paged_attention_decode launch: %s", cudaGetErrorString(e));
    return W8A8_OK;
}
}  // namespace

}  // namespace w8a8

W8A8_TRACE_READER(attn)
