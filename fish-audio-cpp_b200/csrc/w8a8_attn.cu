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
    ptx::pdl_wait();
    const int b = blockIdx.x;
    const int head = blockIdx.y * 4 + (threadIdx.x >> 5);  // 0..n_q-1 q, then k heads, then v heads
    const int lane = threadIdx.x & 31;
    const int total_heads = p.n_q + 2 * p.n_kv;
    if (head >= total_heads) return;
    const __half* src = p.qkv + (static_cast<size_t>(b) * total_heads + head) * kHeadDim;
    const bool is_q = head < p.n_q, is_k = !is_q && head < p.n_q + p.n_kv;
    const int pos = p.positions[b];

    __half h[4];
#pragma unroll
    for (int v = 0; v < 4; ++v) h[v] = src[v * 32 + lane];

    if (is_q || is_k) {
        const __half* w = is_q ? p.q_norm_w : p.k_norm_w;
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
                h[v] = __float2half(val * __half2float(w[v * 32 + lane]));
            }
        }
        // RoPE on interleaved pairs (2i, 2i+1): neighbours in the same run (rope.cu:36-45)
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            const int e = v * 32 + lane;
            const float freq = p.freqs[e >> 1];
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
        const int phys = p.block_table[static_cast<size_t>(b) * p.max_blocks + pos / kBlockTokens];
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
};

constexpr int kAttnWarps = 4;
constexpr int kQPerKv = 4;  // query heads per kv head handled by one CTA

struct SoftState {  // per (head) running softmax state of one lane group: 16 of the 128 dims
    float m, l;
    float acc[16];
};

// grid (S, n_kv, B), cluster (S,1,1). Lane layout: 8 lanes per token (16 dims each), 4 tokens per pass.
__global__ void __launch_bounds__(kAttnWarps * 32) paged_attention_decode_kernel(const AttnParams p) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    __shared__ float red_m[kAttnWarps][kQPerKv], red_l[kAttnWarps][kQPerKv];
    __shared__ float red_acc[kAttnWarps][kQPerKv][kHeadDim];
    __shared__ float cta_m[kQPerKv], cta_l[kQPerKv];
    __shared__ __align__(16) float cta_acc[kQPerKv][kHeadDim];
    __shared__ __align__(16) __half out_s[kQPerKv * kHeadDim];

    const int s = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, S = p.S;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grp = lane >> 3, sub = lane & 7;  // token within a pass, 16-dim slice
    const int seq_len = p.seq_lens[b];
    const int n_blocks = (seq_len + kBlockTokens - 1) / kBlockTokens;
    const int heads_here = p.n_q / p.n_kv;  // == kQPerKv (checked on the host)

    // q of the 4 heads as fp32 in shared memory (read back as broadcast 128-bit loads)
    __shared__ __align__(16) float q_s[kQPerKv][kHeadDim];
    for (int i = threadIdx.x; i < kQPerKv * kHeadDim; i += blockDim.x)
        q_s[i / kHeadDim][i % kHeadDim] =
            __half2float(p.q[(static_cast<size_t>(b) * p.n_q + kvh * heads_here + i / kHeadDim) * kHeadDim + i % kHeadDim]);
    __syncthreads();
    SoftState st[kQPerKv];
#pragma unroll
    for (int hh = 0; hh < kQPerKv; ++hh) {
        st[hh].m = -1e30f; st[hh].l = 0.0f;
#pragma unroll
        for (int d = 0; d < 16; ++d) st[hh].acc[d] = 0.0f;
    }

    // 16-token blocks are dealt round-robin: first over the cluster's CTAs, then over the warps. All 16
    // loads of a block (4 passes x K and V halves) are requested before any arithmetic, so that a warp
    // keeps 8 KB in flight instead of paying one memory round trip per pass.
    for (int bi = s + warp * S; bi < n_blocks; bi += S * kAttnWarps) {
        const int phys = p.block_table[static_cast<size_t>(b) * p.max_blocks + bi];
        const size_t base = (((static_cast<size_t>(phys) * p.n_layers + p.layer) * p.n_kv + kvh) * kBlockTokens) * kHeadDim;
        const int tokens = min(kBlockTokens, seq_len - bi * kBlockTokens);
        uint4 kraw[4][2], vraw[4][2];
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
            const int t = pass * 4 + grp;
            const size_t off = base + static_cast<size_t>(t < tokens ? t : 0) * kHeadDim + sub * 16;
            kraw[pass][0] = *reinterpret_cast<const uint4*>(p.k_cache + off);
            kraw[pass][1] = *reinterpret_cast<const uint4*>(p.k_cache + off + 8);
            vraw[pass][0] = *reinterpret_cast<const uint4*>(p.v_cache + off);
            vraw[pass][1] = *reinterpret_cast<const uint4*>(p.v_cache + off + 8);
        }
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
            const int t = pass * 4 + grp;
            const bool live = t < tokens;
            float kf[16], vf[16];
            {
                const __half* a0 = reinterpret_cast<const __half*>(&kraw[pass][0]);
                const __half* a1 = reinterpret_cast<const __half*>(&kraw[pass][1]);
                const __half* b0 = reinterpret_cast<const __half*>(&vraw[pass][0]);
                const __half* b1 = reinterpret_cast<const __half*>(&vraw[pass][1]);
#pragma unroll
                for (int d = 0; d < 8; ++d) {
                    kf[d] = __half2float(a0[d]); kf[8 + d] = __half2float(a1[d]);
                    vf[d] = __half2float(b0[d]); vf[8 + d] = __half2float(b1[d]);
                }
            }
#pragma unroll
            for (int hh = 0; hh < kQPerKv; ++hh) {
                float dot = 0.0f;
#pragma unroll
                for (int d4 = 0; d4 < 4; ++d4) {
                    const float4 q4 = *reinterpret_cast<const float4*>(&q_s[hh][sub * 16 + d4 * 4]);
                    dot = fmaf(q4.x, kf[d4 * 4 + 0], dot);
                    dot = fmaf(q4.y, kf[d4 * 4 + 1], dot);
                    dot = fmaf(q4.z, kf[d4 * 4 + 2], dot);
                    dot = fmaf(q4.w, kf[d4 * 4 + 3], dot);
                }
                dot += __shfl_xor_sync(0xffffffffu, dot, 1);
                dot += __shfl_xor_sync(0xffffffffu, dot, 2);
                dot += __shfl_xor_sync(0xffffffffu, dot, 4);
                if (live) {
                    const float score = dot * p.sm_scale;
                    const float new_max = fmaxf(st[hh].m, score);
                    const float scale = expf(st[hh].m - new_max);
                    const float e = expf(score - new_max);
                    st[hh].l = st[hh].l * scale + e;
#pragma unroll
                    for (int d = 0; d < 16; ++d) st[hh].acc[d] = st[hh].acc[d] * scale + e * vf[d];
                    st[hh].m = new_max;
                }
            }
        }
    }
    // ---- merge the 4 lane groups of the warp (xor 8, 16), same 16-dim slice in each ----
#pragma unroll
    for (int hh = 0; hh < kQPerKv; ++hh) {
#pragma unroll
        for (int o = 8; o <= 16; o <<= 1) {
            const float om = __shfl_xor_sync(0xffffffffu, st[hh].m, o);
            const float ol = __shfl_xor_sync(0xffffffffu, st[hh].l, o);
            const float nm = fmaxf(st[hh].m, om);
            const float sa = expf(st[hh].m - nm), sb = expf(om - nm);
            st[hh].l = st[hh].l * sa + ol * sb;
#pragma unroll
            for (int d = 0; d < 16; ++d) {
                const float oa = __shfl_xor_sync(0xffffffffu, st[hh].acc[d], o);
                st[hh].acc[d] = st[hh].acc[d] * sa + oa * sb;
            }
            st[hh].m = nm;
        }
        if (grp == 0) {
            if (sub == 0) { red_m[warp][hh] = st[hh].m; red_l[warp][hh] = st[hh].l; }
#pragma unroll
            for (int d = 0; d < 16; ++d) red_acc[warp][hh][sub * 16 + d] = st[hh].acc[d];
        }
    }
    __syncthreads();
    // ---- merge the warps: thread -> (head, 4 dims) ----
    {
        const int hh = threadIdx.x >> 5, d0 = (threadIdx.x & 31) * 4;
        float m = -1e30f;
        for (int w = 0; w < kAttnWarps; ++w) m = fmaxf(m, red_m[w][hh]);
        float l = 0.0f, a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int w = 0; w < kAttnWarps; ++w) {
            const float sc = expf(red_m[w][hh] - m);
            l += red_l[w][hh] * sc;
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] += red_acc[w][hh][d0 + i] * sc;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) cta_acc[hh][d0 + i] = a[i];
        if ((threadIdx.x & 31) == 0) { cta_m[hh] = m; cta_l[hh] = l; }
    }
    cg::cluster_group cluster = cg::this_cluster();
    if (S > 1) cluster.sync(); else __syncthreads();
    // ---- CTA 0 of the cluster merges the S context slices and writes the 4 heads ----
    if (s == 0) {
        const int hh = threadIdx.x >> 5, d0 = (threadIdx.x & 31) * 4;
        float m = -1e30f;
        for (int r = 0; r < S; ++r) m = fmaxf(m, (S > 1 ? cluster.map_shared_rank(cta_m, r) : cta_m)[hh]);
        float l = 0.0f, a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int r = 0; r < S; ++r) {
            const float* pm = S > 1 ? cluster.map_shared_rank(cta_m, r) : cta_m;
            const float* pl = S > 1 ? cluster.map_shared_rank(cta_l, r) : cta_l;
            const float* pa = S > 1 ? cluster.map_shared_rank(&cta_acc[0][0], r) : &cta_acc[0][0];
            const float sc = expf(pm[hh] - m);
            l += pl[hh] * sc;
            const float4 v4 = *reinterpret_cast<const float4*>(pa + hh * kHeadDim + d0);
            a[0] += v4.x * sc; a[1] += v4.y * sc; a[2] += v4.z * sc; a[3] += v4.w * sc;
        }
        const float inv = seq_len > 0 ? 1.0f / l : 0.0f;  // empty sequence -> zeros (paged_attention.cu:44-50)
        __align__(8) __half o4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) o4[i] = __float2half(seq_len > 0 ? a[i] * inv : 0.0f);
#pragma unroll
        for (int i = 0; i < 4; ++i) out_s[hh * kHeadDim + d0 + i] = o4[i];
        const size_t o = (static_cast<size_t>(b) * p.n_q + kvh * heads_here + hh) * kHeadDim + d0;
        if (p.out) *reinterpret_cast<uint2*>(p.out + o) = *reinterpret_cast<const uint2*>(o4);
    }
    if (S > 1) cluster.sync(); else __syncthreads();
    // ---- optional: quantise these 512 channels for the o-projection (int8_gemm.cu:147-211) ----
    if (s == 0 && p.Xq) {
        const int g = p.g, K = p.n_q * kHeadDim, G = K / g;
        const int ch0 = kvh * heads_here * kHeadDim;        // first channel of this CTA
        const int groups_here = (kQPerKv * kHeadDim) / g;   // 2 at g=256, 8 at g=64
        // warp per group (8 warps)
        for (int j = warp; j < groups_here; j += kAttnWarps) {
            float amax = 0.0f;
            for (int e = lane; e < g; e += 32) amax = fmaxf(amax, fabsf(__half2float(out_s[j * g + e])));
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            float scale = amax / 127.0f;
            if (scale < 1e-8f) scale = 1e-8f;
            if (lane == 0) p.Xs[static_cast<size_t>(b) * G + ch0 / g + j] = scale;
            const float inv_scale = 1.0f / scale;
            for (int e = lane; e < g; e += 32) {
                int qv = __float2int_rn(__half2float(out_s[j * g + e]) * inv_scale);
                qv = max(-127, min(127, qv));
                p.Xq[static_cast<size_t>(b) * K + ch0 + j * g + e] = static_cast<int8_t>(qv);
            }
        }
    }
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
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, qknorm_rope_kvwrite_kernel, p);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "qknorm_rope_kvwrite launch: %s", cudaGetErrorString(e));
    return W8A8_OK;
}

int launch_paged_attention_decode(const __half* q, const __half* k_cache, const __half* v_cache,
                                  const int* block_table, const int* seq_lens, int B, int n_q, int n_kv,
                                  int max_blocks, float sm_scale, int layer, int n_layers, __half* out, int g,
                                  int8_t* Xq, float* Xs, int splits, cudaStream_t stream) {
    if (B == 0) return W8A8_OK;
    if (n_kv <= 0 || n_q != n_kv * kQPerKv)
        return fail(W8A8_ERR_UNSUPPORTED, "paged attention here handles 4 query heads per kv head (got %d / %d)", n_q, n_kv);
    if (Xq && (g <= 0 || (kQPerKv * kHeadDim) % g != 0))
        return fail(W8A8_ERR_UNSUPPORTED, "fused output quantisation needs a group size dividing 512 (got %d)", g);
    if (splits <= 0) splits = 4;
    if (splits > 8) splits = 8;
    AttnParams p = {q, k_cache, v_cache, block_table, seq_lens, max_blocks, n_q, n_kv, layer, n_layers, sm_scale,
                    out, Xq, Xs, g, splits};
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
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, paged_attention_decode_kernel, p);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "paged_attention_decode launch: %s", cudaGetErrorString(e));
    return W8A8_OK;
}

}  // namespace w8a8
