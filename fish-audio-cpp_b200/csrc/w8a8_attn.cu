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
    int* status;              // error word for bounded waits that ran out
};

#ifndef W8A8_ATTN_WARPS
#define W8A8_ATTN_WARPS 8
#endif
#ifndef W8A8_ATTN_RING
#define W8A8_ATTN_RING 16
#endif
constexpr int kAttnWarps = W8A8_ATTN_WARPS;      // consumer warps
constexpr int kAttnThreads = (kAttnWarps + 1) * 32;  // + one producer warp
constexpr int kQPerKv = 4;                       // query heads per kv head handled by one CTA
constexpr int kBoxBytes = kBlockTokens * 128;    // a TMA box: 16 token rows x 128 bytes (64 dims), 128-byte swizzle
constexpr int kBlkBytes = 2 * kBoxBytes;         // one 16-token block of K (or of V): dims 0..63, then dims 64..127
constexpr int kStageBytes = 2 * kBlkBytes;       // K block, then V block
constexpr int kRing = W8A8_ATTN_RING;            // stages of the CTA's ring, 8 KB each: two per consumer warp, so that a
                                                 // warp's next block is on its way while it works on the current one

// Byte offset, inside a K or V block in shared memory, of the 16-byte chunk that holds dims [8 c16, 8 c16 + 8) of
// token row r: the box of its 64-dim half, the row's 128 bytes, the chunk XOR-ed with the row (what the tensor
// map's 128-byte swizzle does, and what makes eight rows of one chunk column fall into eight different bank groups).
__device__ __forceinline__ uint32_t kv_chunk(int r, int c16) {
    return (c16 >> 3) * kBoxBytes + r * 128 + (((c16 & 7) ^ (r & 7)) << 4);
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

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void consumer_barrier() {  // the eight consumer warps only
    asm volatile("bar.sync 1, %0;" ::"n"(kAttnWarps * 32) : "memory");
}

// grid (S, n_kv, B), cluster (S,1,1); eight consumer warps and one producer warp per CTA.
//
// The K and V of one (sequence, kv head) are 4 KB blocks scattered over the paged cache. The producer warp brings them
// into a ring of shared-memory stages with TMA (cp.async.bulk.tensor.2d over the cache seen as rows of 256 bytes,
// two 16 x 128-byte boxes per block, 128-byte swizzle, completion counted on the stage's mbarrier; single 256-byte
// row copies were tried first and are bound by the copy engine's request rate) — no registers are tied up by bytes in flight, so the kernel fits beside a CTA of
// the linear before it, and everything the producer needs (sequence length, block table, every block but the
// sequence's last) does not depend on that linear: with programmatic dependent launch the ring is already full when
// the query arrives. 16-token blocks are dealt round-robin, first over the cluster's CTAs, then over the consumer
// warps; a consumer waits for its block, computes on it from shared memory (ldmatrix into mma.sync.m16n8k16 with
// fp32 accumulation: scores = Q K^T with the four query heads of the group as rows 0..3 of the tile, then
// out += P V with P rounded to fp16 and the softmax denominator summed from the same rounded values) and hands the
// stage back. Partial softmax states are merged over the warps in shared memory and over the cluster through
// distributed shared memory; the epilogue can emit the o-projection's int8 codes and scales directly.
//
// ROPE form: the launch also does what qknorm_rope_kvwrite_kernel does. Consumer warps 0..3 norm and rotate the four
// query heads into shared memory; warps 4 and 5 do the same for the new k and v rows, which go to shared memory and,
// in the CTA that owns the block the new token joins, to the cache. That block is read from the cache like any other
// (possibly before the new rows are there) and the new rows are put over it in shared memory.
// Without ROPE the new rows were written by the launch before this one, so the sequence's last block is requested
// only after the dependency wait.
#ifdef W8A8_TRACE
// Diagnostic build only: nanosecond stamps of the phases of CTA (0, 0, 0), written by consumer thread 0, kept from
// the last launch; read out by w8a8_trace_read_attn_phases.
__device__ unsigned long long g_attn_phase[8];
#define ATTN_PHASE(i)                                                                     \
    do {                                                                                  \
        if (threadIdx.x == 0 && (blockIdx.x | blockIdx.y | blockIdx.z) == 0) g_attn_phase[i] = w8a8::trace::now(); \
    } while (0)
#else
#define ATTN_PHASE(i) do {} while (0)
#endif

template <bool ROPE>
__global__ void __maxnreg__(120) paged_attention_decode_kernel(const __grid_constant__ CUtensorMap map_k,
                                                               const __grid_constant__ CUtensorMap map_v,
                                                               const AttnParams p) {
    extern __shared__ unsigned char attn_smem[];
    __shared__ __align__(8) uint64_t full_bar[kRing], empty_bar[kRing];
    __shared__ __align__(16) __half q_s[kQPerKv][kHeadDim];
    __shared__ __align__(16) __half kv_new_s[2][kHeadDim];
    __shared__ float red_m[kAttnWarps][kQPerKv], red_l[kAttnWarps][kQPerKv];
    __shared__ float red_acc[kAttnWarps][kQPerKv][kHeadDim];
    __shared__ float cta_m[kQPerKv], cta_l[kQPerKv];
    __shared__ __align__(16) float cta_acc[kQPerKv][kHeadDim];
    __shared__ __align__(16) __half out_s[kQPerKv * kHeadDim];
    __shared__ int s_fail;
    W8A8_TRACE_SCOPE();
    ATTN_PHASE(0);
    ptx::pdl_launch_dependents();

    const int s = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, S = p.S;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t ring = (ptx::smem_u32(attn_smem) + 1023u) & ~1023u;  // the swizzle pattern repeats every 1024 bytes
    if (threadIdx.x == 0) {
        ptx::prefetch_tensormap(&map_k);
        ptx::prefetch_tensormap(&map_v);
        for (int i = 0; i < kRing; ++i) {
            ptx::mbar_init(&full_bar[i], 1);
            ptx::mbar_init(&empty_bar[i], 1);
        }
        s_fail = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
    }
    __syncthreads();  // the only whole-CTA barrier: from here on the producer warp runs by itself

    // Read before the dependency wait: these are not results of the launch before this one. The producer asks for the
    // first 32 block numbers without waiting for the sequence length (the read is bounded by the table's width), so
    // that the two reads are one round trip, not two.
    int phys_first = 0;
    if (warp == kAttnWarps) {
        const int bi = s + lane * S;
        phys_first = bi < p.max_blocks ? p.block_table[static_cast<size_t>(b) * p.max_blocks + bi] : 0;
    }
    const int seq_len = p.seq_lens[b];
    const int n_blocks = (seq_len + kBlockTokens - 1) / kBlockTokens;
    const int n_local = s < n_blocks ? (n_blocks - s + S - 1) / S : 0;  // blocks s, s + S, s + 2 S, ...
    const int heads_here = p.n_q / p.n_kv;                                // == kQPerKv (checked on the host)

    if (warp == kAttnWarps) {
        // ------------------------------ producer ------------------------------
        // Eight blocks per round, four lanes per block (one TMA box each): a single lane issuing every copy of the
        // CTA one after the other costs more than the copies take.
        bool waited = false;
        int phys_mine = phys_first;
        bool failed = false;
        for (int li0 = 0; li0 < n_local && !failed; li0 += 8) {
            if ((li0 & 31) == 0 && li0 > 0) {  // the physical numbers of the next 32 local blocks, one per lane
                const int bi = s + (li0 + lane) * S;
                phys_mine = (bi < n_blocks && bi < p.max_blocks) ? p.block_table[static_cast<size_t>(b) * p.max_blocks + bi] : 0;
            }
            const int li = li0 + (lane >> 2), box = lane & 3;
            const int phys = __shfl_sync(0xffffffffu, phys_mine, li & 31);
            const int bi = s + li * S, st = li % kRing;
            const bool live = li < n_local;
            // Without ROPE the newest rows come from the launch before this one: wait for it before the round that
            // holds the sequence's last block.
            if (!ROPE && !waited && s + (li0 + 7) * S >= n_blocks - 1) {
                ptx::pdl_wait();
                waited = true;
            }
            if (live && li >= kRing && !ptx::mbar_wait_bounded(&empty_bar[st], ((li / kRing) - 1) & 1)) {
                if (box == 0) { atomicExch(p.status, 800 + st); s_fail = 1; }
                failed = true;
            }
            failed = __any_sync(0xffffffffu, failed);
            if (failed) break;
            if (live && box == 0) ptx::mbar_arrive_expect_tx(&full_bar[st], kStageBytes);
            __syncwarp();
            if (live) {  // box 0: K dims 0..63, 1: K dims 64..127, 2: V dims 0..63, 3: V dims 64..127
                const int y = ((phys < 0 ? 0 : phys) * p.n_layers + p.layer) * p.n_kv * kBlockTokens + kvh * kBlockTokens;
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                    ::"r"(ring + st * kStageBytes + box * kBoxBytes), "l"(box < 2 ? &map_k : &map_v),
                      "r"(ptx::smem_u32(&full_bar[st])), "r"((box & 1) * 128), "r"(y)
                    : "memory");
            }
        }
        if (!waited) ptx::pdl_wait();
    } else {
        // ------------------------------ consumers ------------------------------
        int pos = 0;
        bool owner = false;
        float fr[4];
        if constexpr (ROPE) {  // parameters first: they do not depend on the launch before this one
            pos = p.positions[b];
#pragma unroll
            for (int v = 0; v < 4; ++v) fr[v] = p.freqs[(v * 32 + lane) >> 1];
            owner = ((pos / kBlockTokens) % S) == s;  // this CTA attends over the block the new token joins
        }
        ptx::pdl_wait();
        W8A8_TRACE_WAITED();
        ATTN_PHASE(1);
        const int new_bi = pos / kBlockTokens;
        if constexpr (ROPE) {
            // six head rows of the new token: the group's four query heads, then its k and its v; a warp per row
            const int total_heads = p.n_q + 2 * p.n_kv;
            for (int h = warp; h < kQPerKv + 2; h += kAttnWarps) {
                const bool role_q = h < kQPerKv, is_k = h == kQPerKv, is_v = h == kQPerKv + 1;
                const __half* norm_w = role_q ? p.q_norm_w : p.k_norm_w;
                const __half* src = p.qkv + (static_cast<size_t>(b) * total_heads +
                                             (role_q ? kvh * heads_here + h : p.n_q + (is_k ? 0 : p.n_kv) + kvh)) * kHeadDim;
                __half hq[4], wq[4];
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    hq[v] = src[v * 32 + lane];
                    wq[v] = (norm_w && !is_v) ? norm_w[v * 32 + lane] : __float2half(1.0f);
                }
                if (!is_v) head_norm_rope(hq, norm_w != nullptr, wq, p.eps, fr, pos, lane);
                if (role_q) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) q_s[h][v * 32 + lane] = hq[v];
                } else {
#pragma unroll
                    for (int v = 0; v < 4; ++v) kv_new_s[is_v ? 1 : 0][v * 32 + lane] = hq[v];
                    if (owner) {
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
            }
            consumer_barrier();  // q and the new k / v rows are in shared memory
        }
        // q of head g (rows 4..15 of the tile are zero): A fragments of the eight 16-dim steps
        uint32_t qa[8][2];
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
            qa[kk][0] = 0u;
            qa[kk][1] = 0u;
            if (g < kQPerKv) {
                if constexpr (ROPE) {
                    qa[kk][0] = *reinterpret_cast<const uint32_t*>(&q_s[g][16 * kk + 2 * t]);
                    qa[kk][1] = *reinterpret_cast<const uint32_t*>(&q_s[g][16 * kk + 8 + 2 * t]);
                } else {
                    const __half* qrow = p.q + (static_cast<size_t>(b) * p.n_q + kvh * heads_here + g) * kHeadDim;
                    qa[kk][0] = *reinterpret_cast<const uint32_t*>(qrow + 16 * kk + 2 * t);
                    qa[kk][1] = *reinterpret_cast<const uint32_t*>(qrow + 16 * kk + 8 + 2 * t);
                }
            }
        }

        ATTN_PHASE(2);  // q (and the new k / v rows) are ready
        float m_run = -1e30f, l_run = 0.0f;
        float o[16][2];  // head g, dims 8 n + 2 t, 8 n + 2 t + 1
#pragma unroll
        for (int n = 0; n < 16; ++n) { o[n][0] = 0.0f; o[n][1] = 0.0f; }

        for (int li = warp; li < n_local; li += kAttnWarps) {
            const int st = li % kRing, bi = s + li * S;
            if (!ptx::mbar_wait_bounded(&full_bar[st], (li / kRing) & 1)) {
                if (lane == 0) { atomicExch(p.status, 810 + st); s_fail = 1; }
                break;
            }
            if (li == warp) ATTN_PHASE(3);  // the warp's first block is in shared memory
            const uint32_t ks = ring + st * kStageBytes, vs = ks + kBlkBytes;
            const int tokens = min(kBlockTokens, seq_len - bi * kBlockTokens);
            if (ROPE && bi == new_bi) {  // the new token's rows over whatever the cache held there (lane: 4 dims)
                const int r = pos % kBlockTokens;
                const uint2 kn = reinterpret_cast<const uint2*>(kv_new_s[0])[lane], vn = reinterpret_cast<const uint2*>(kv_new_s[1])[lane];
                const uint32_t off = kv_chunk(r, lane >> 1) + (lane & 1) * 8;
                asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(ks + off), "r"(kn.x), "r"(kn.y) : "memory");
                asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(vs + off), "r"(vn.x), "r"(vn.y) : "memory");
            }
            // V rows past the sequence's end: their weights are exactly zero, but whatever lies there (it may not be
            // a number) must not meet the multiply. (K rows past the end only feed scores that are replaced below.)
            for (int r = tokens; r < kBlockTokens; ++r)
                asm volatile("st.shared.v2.u32 [%0], {%1,%1};" ::"r"(vs + (lane >> 4) * kBoxBytes + r * 128 + (lane & 15) * 8), "r"(0u)
                             : "memory");
            __syncwarp();
            // scores: two tiles of 8 tokens x eight steps of 16 dims
            float sc[2][2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                sc[j][0] = 0.0f; sc[j][1] = 0.0f;
#pragma unroll
                for (int k2 = 0; k2 < 4; ++k2) {  // matrices: dims 32 k2 + 8 (lane >> 3) of tokens 8 j + (lane & 7)
                    uint32_t r4[4];
                    ldmatrix_x4(r4, ks + kv_chunk(8 * j + (lane & 7), 4 * k2 + (lane >> 3)));
                    mma_top_rows(sc[j][0], sc[j][1], qa[2 * k2][0], qa[2 * k2][1], r4[0], r4[1]);
                    mma_top_rows(sc[j][0], sc[j][1], qa[2 * k2 + 1][0], qa[2 * k2 + 1][1], r4[2], r4[3]);
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
            for (int n2 = 0; n2 < 8; ++n2) {  // matrices (transposed): tokens 8 (m & 1) + (lane & 7), dims 16 n2 + 8 (m >> 1)
                uint32_t r4[4];
                const int m = lane >> 3;
                ldmatrix_x4_trans(r4, vs + kv_chunk(8 * (m & 1) + (lane & 7), 2 * n2 + (m >> 1)));
                o[2 * n2][0] *= corr; o[2 * n2][1] *= corr;
                o[2 * n2 + 1][0] *= corr; o[2 * n2 + 1][1] *= corr;
                mma_top_rows(o[2 * n2][0], o[2 * n2][1], pa0, pa2, r4[0], r4[1]);
                mma_top_rows(o[2 * n2 + 1][0], o[2 * n2 + 1][1], pa0, pa2, r4[2], r4[3]);
            }
            // the stage goes back to the producer; the writes above (the new rows) are ordered before its next copy
            ptx::fence_proxy_async();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&empty_bar[st]);
        }
        ATTN_PHASE(4);  // the warp's blocks are done
        // the four lanes of a quad hold the same head: their partial denominators add up
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
        if (g < kQPerKv) {
            if (t == 0) { red_m[warp][g] = m_run; red_l[warp][g] = l_run; }
#pragma unroll
            for (int n = 0; n < 16; ++n) {
                red_acc[warp][g][8 * n + 2 * t] = o[n][0];
                red_acc[warp][g][8 * n + 2 * t + 1] = o[n][1];
            }
        }
        consumer_barrier();
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
    }
    // ---- every thread of the cluster (the producer warps included) ----
    ATTN_PHASE(5);  // warps merged
    cg::cluster_group cluster = cg::this_cluster();
    if (S > 1) cluster.sync(); else __syncthreads();
    ATTN_PHASE(6);  // every CTA of the cluster has its partial state ready
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
    if (s == 0 && p.Xq && warp < kAttnWarps) {
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
    if (s_fail) {  // a bounded wait ran out: give copies that may still be in flight time to land before the CTA goes
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    ATTN_PHASE(7);
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
                                  int8_t* Xq, float* Xs, int splits, int* status, cudaStream_t stream) {
    AttnParams p = {};
    p.status = status;
    p.q = q; p.k_cache = k_cache; p.v_cache = v_cache; p.block_table = block_table; p.seq_lens = seq_lens;
    p.max_blocks = max_blocks; p.n_q = n_q; p.n_kv = n_kv; p.layer = layer; p.n_layers = n_layers; p.sm_scale = sm_scale;
    p.out = out; p.Xq = Xq; p.Xs = Xs; p.g = g;
    return launch_attention(p, B, splits, stream);
}

int launch_qkv_attention_decode(const __half* qkv, const __half* q_norm_w, const __half* k_norm_w, float eps,
                                const float* freqs, const int* positions, __half* k_cache, __half* v_cache,
                                const int* block_table, const int* seq_lens, int B, int n_q, int n_kv, int max_blocks,
                                float sm_scale, int layer, int n_layers, __half* out, int g, int8_t* Xq, float* Xs,
                                int splits, int* status, cudaStream_t stream) {
    AttnParams p = {};
    p.status = status;
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
    // The caches as rows of 256 bytes (one token of one head); a box is 16 rows x 128 bytes. The row count only bounds
    // the coordinates the kernel may ask for: the physical block numbers come from the caller's block table.
    CUtensorMap map_k, map_v;
    int rc = make_tensor_map_2d_u8(&map_k, p.k_cache, kHeadDim * 2, uint64_t(1) << 30, kHeadDim * 2, 128, kBlockTokens, 1);
    if (rc) return rc;
    rc = make_tensor_map_2d_u8(&map_v, p.v_cache, kHeadDim * 2, uint64_t(1) << 30, kHeadDim * 2, 128, kBlockTokens, 1);
    if (rc) return rc;
    const size_t smem = static_cast<size_t>(kRing) * kStageBytes + 1024;
    {  // per device, so on every launch (a host-side table write)
        cudaError_t e = cudaFuncSetAttribute(paged_attention_decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(smem));
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(paged_attention_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem));
        if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, n_kv, B);
    cfg.blockDim = dim3(kAttnThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
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
    cudaError_t e = p.qkv ? cudaLaunchKernelEx(&cfg, paged_attention_decode_kernel<true>, map_k, map_v, p)
                          : cudaLaunchKernelEx(&cfg, paged_attention_decode_kernel<false>, map_k, map_v, p);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "paged_attention_decode launch: %s", cudaGetErrorString(e));
    return W8A8_OK;
}
}  // namespace

}  // namespace w8a8

W8A8_TRACE_READER(attn)
#ifdef W8A8_TRACE
extern "C" __attribute__((visibility("default"))) int w8a8_trace_read_attn_phases(unsigned long long* out8) {
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    return cudaMemcpyFromSymbol(out8, w8a8::g_attn_phase, 8 * sizeof(unsigned long long)) == cudaSuccess ? 8 : -1;
}
#endif
