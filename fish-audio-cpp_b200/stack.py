"""Slow-AR decoder stack harness: the layer loop of DualAREngine::decode_step
(src/engine/dual_ar_engine.cc:554-658) on top of the C ABI, with random-init weights.

It exists to measure decode tokens/s of the whole stack (36 layers, hidden 2560, 32 q / 8 kv heads of
128, SwiGLU 9728, W8A8 at g256, fp16 paged KV with 16-token blocks) at tensor-parallel degree 1/2/4/8.
Per layer it issues eight launches where the reference issues ~23 plus 19 device copies:

    rmsnorm_quantize (+ residual add of the previous projection)      rms_norm + residual_add + quantiser
    linear_q  wqkv                                                     int8_dequant_gemm_fp16
    qknorm_rope_kvwrite                                                3 copies, 2 rms_norm, rope_qk, 16 copies
    paged_attention_decode (+ quantiser for wo)                        paged_attention_decode + quantiser
    linear_q  wo            -> partial        [all-reduce when TP > 1]
    rmsnorm_quantize (+ residual add)                                  residual_add + rms_norm + quantiser
    linear_q  w1|w3 packed, SwiGLU epilogue                            2 GEMMs + silu + mul
    quantize ; linear_q  w2 -> partial        [all-reduce when TP > 1]

Tensor parallelism (the reference has none): wqkv and w1|w3 are column-parallel (whole heads, whole
SwiGLU channels per rank), wo and w2 row-parallel with K cut at quantisation-group boundaries, so every
per-group int32 sum and every activation scale stays on one rank; the only exchange is one fp16 sum
all-reduce of [batch, 2560] after wo and after w2.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass

import numpy as np

from . import capi


@dataclass
class SlowARConfig:
    n_layer: int = 36
    dim: int = 2560
    n_head: int = 32
    n_kv: int = 8
    head_dim: int = 128
    inter: int = 9728
    rope_base: float = 1e6
    eps: float = 1e-6
    group: int = 256
    block_tokens: int = 16
    qk_norm: bool = True   # per-head RMSNorm of q and k before RoPE (slow AR: yes, fast AR: no; dual_ar_config.h:19,28)


def shard_bounds(total_groups: int, world: int):
    """Row-parallel cut of K at group boundaries: rank r owns groups [b[r], b[r+1]). Sizes differ by at
    most one group (38 groups over 4 ranks -> 10, 10, 9, 9)."""
    base, rem = divmod(total_groups, world)
    b = [0]
    for r in range(world):
        b.append(b[-1] + base + (1 if r < rem else 0))
    return b


def shard_plan(cfg: SlowARConfig, tp_size: int, tp_rank: int):
    """Shapes of one rank's shard: (q heads, kv heads, rows of wqkv, K of wo, first and last intermediate channel).
    Column-parallel wqkv / w1|w3 by heads and intermediate channels, row-parallel wo / w2 with K cut at quantisation
    group boundaries (so every per-group int32 sum stays on one rank)."""
    c, g = cfg, cfg.group
    assert c.n_kv % tp_size == 0 and c.n_head == 4 * c.n_kv and c.head_dim == 128
    nq_l, nkv_l = c.n_head // tp_size, c.n_kv // tp_size
    qkv_n, attn_k = (nq_l + 2 * nkv_l) * c.head_dim, nq_l * c.head_dim
    assert attn_k % g == 0, "attention shard must hold whole quantisation groups"
    assert c.inter % g == 0
    # cut in units of 256 channels when the group size divides 256: the decode kernel's packed weight format
    # wants K in multiples of 256, and a multiple of 256 is a multiple of the group size too
    unit = 256 if (256 % g == 0 and c.inter % 256 == 0) else g
    gb = shard_bounds(c.inter // unit, tp_size)
    lo, hi = gb[tp_rank] * unit, gb[tp_rank + 1] * unit
    assert hi > lo and (hi - lo) % 8 == 0
    return nq_l, nkv_l, qkv_n, attn_k, lo, hi


def _seeded(torch, dev, seed, tag):
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed * 1000003 + tag)
    return gen


def random_weight(torch, n, k, g, seed, tag, dev="cuda"):
    """int8 uniform [-127, 127] weights [n, k] and fp16 scales in [1e-3, 5e-3] per (row, group), seeded."""
    gen = _seeded(torch, dev, seed, tag)
    w = torch.randint(-127, 128, (n, k), dtype=torch.int8, device=dev, generator=gen)
    s = torch.empty((n, k // g), dtype=torch.float32, device=dev).uniform_(1e-3, 5e-3, generator=gen).half()
    return w, s


def random_vector(torch, n, seed, tag, dev="cuda"):
    gen = _seeded(torch, dev, seed, tag)
    return torch.empty((n,), dtype=torch.float32, device=dev).uniform_(0.8, 1.2, generator=gen).half()


def layer_tensors(torch, cfg: SlowARConfig, l: int, seed: int, dev="cuda"):
    """The UNSHARDED random-init tensors of layer l, as a checkpoint would hold them (w1 and w3 apart, like the
    reference's loader sees them): every rank of a tensor-parallel run, the single-GPU stack and the
    reference-kernel chain all cut or use the same values. torch only; no call into the library."""
    c, g, D, t = cfg, cfg.group, cfg.head_dim, l * 16
    wqkv, sqkv = random_weight(torch, (c.n_head + 2 * c.n_kv) * D, c.dim, g, seed, t + 1, dev)
    wo, so = random_weight(torch, c.dim, c.n_head * D, g, seed, t + 2, dev)
    w1, s1 = random_weight(torch, c.inter, c.dim, g, seed, t + 3, dev)
    w3, s3 = random_weight(torch, c.inter, c.dim, g, seed, t + 4, dev)
    w2, s2 = random_weight(torch, c.dim, c.inter, g, seed, t + 5, dev)
    return dict(wqkv=wqkv, sqkv=sqkv, wo=wo, so=so, w1=w1, s1=s1, w3=w3, s3=s3, w2=w2, s2=s2,
                attn_norm=random_vector(torch, c.dim, seed, t + 6, dev), ffn_norm=random_vector(torch, c.dim, seed, t + 7, dev),
                q_norm=random_vector(torch, D, seed, t + 8, dev) if c.qk_norm else None,
                k_norm=random_vector(torch, D, seed, t + 9, dev) if c.qk_norm else None)


def final_norm_weight(torch, cfg: SlowARConfig, seed: int, dev="cuda"):
    return random_vector(torch, cfg.dim, seed, 999983, dev)


def rope_frequencies(torch, cfg: SlowARConfig, dev="cuda"):
    """freq_i = base^(-2i/D) in fp32 on the host, as DualAREngine::init computes them (dual_ar_engine.cc:161-167)."""
    D = cfg.head_dim
    freqs = (1.0 / np.power(np.float32(cfg.rope_base), (np.float32(2.0) * np.arange(D // 2, dtype=np.float32) /
                                                          np.float32(D)))).astype(np.float32)
    return torch.from_numpy(freqs).to(dev)


def synthetic_kv(torch, cfg: SlowARConfig, batch: int, context: int, max_new: int, seed: int, dev="cuda",
                 kv_heads=None):
    """Paged fp16 KV cache [blocks, layers, kv heads, 16, head_dim] already holding `context` tokens per sequence
    (a synthetic prefill) with a shuffled block table. kv_heads = (first, count) keeps only those heads (one
    tensor-parallel rank's share of the same cache). Returns (k_cache, v_cache, block_table, max_blocks)."""
    c, bt = cfg, cfg.block_tokens
    max_blocks = (context + max_new + bt - 1) // bt
    nblocks = batch * max_blocks
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed + 4242)
    lo, n = kv_heads if kv_heads is not None else (0, c.n_kv)
    caches = []
    for _ in range(2):  # k, then v; generated layer by layer over all heads so that every rank sees the same values
        full = torch.empty((nblocks, c.n_layer, n, bt, c.head_dim), dtype=torch.float16, device=dev)
        for l in range(c.n_layer):
            part = torch.randn((nblocks, c.n_kv, bt, c.head_dim), dtype=torch.float32, device=dev, generator=gen) * 0.5
            full[:, l] = part[:, lo:lo + n].half()
        caches.append(full)
    perm = torch.randperm(nblocks, device=dev, generator=gen).to(torch.int32)
    return caches[0], caches[1], perm.view(batch, max_blocks).contiguous(), max_blocks


class SlowARStack:
    def __init__(self, torch, ctx: capi.Context, cfg: SlowARConfig, batch: int, context: int, max_new: int = 256,
                 tp_rank: int = 0, tp_size: int = 1, seed: int = 0, all_reduce=None, pack: bool = True,
                 attn_splits: int = 0, tp_mode: str = "fused", gather_handles=None, fuse_norm: bool = True):
        self.torch, self.ctx, self.cfg = torch, ctx, cfg
        self.B, self.tp_rank, self.tp_size = batch, tp_rank, tp_size
        self.all_reduce = all_reduce
        self.attn_splits = int(os.environ.get("W8A8_STACK_ATTN_SPLITS", attn_splits))
        # "fused": the exchange happens inside the residual+norm+quant kernel over peer memory;
        # "nccl": a library all-reduce between the projection and that kernel (the baseline).
        self.tp_fused = tp_size > 1 and tp_mode == "fused"
        if self.tp_fused:
            handle = ctx.tp_create(tp_rank, tp_size, batch, cfg.dim)
            ctx.tp_connect(b"".join(gather_handles(handle)))
            self.all_reduce = None
        # On one GPU the residual add + RMSNorm + quantiser before wqkv and w13 run inside the linear's own
        # launch (w8a8_rmsnorm_linear); with TP the exchange sits in that place instead.
        self.fuse_norm = fuse_norm and tp_size == 1 and pack and os.environ.get("W8A8_STACK_FUSE_NORM", "0") == "1"
        # W8A8_STACK_TAILS=1 (one GPU, batch <= 8): the small kernels between the linears run as TAILS of the linear
        # before them (w8a8_linear_q_tail): residual add + RMSNorm + quantiser after wo and w2, the quantiser after
        # w1|w3; five launches per layer. Measured slower than the eight-launch form inside a replayed graph (a tail
        # costs what the launch it replaces costs, and the next linear's prefetch overlaps less), so it is off by default.
        self.tails = (tp_size == 1 and pack and batch <= 8 and cfg.group in (64, 128, 256) and not self.fuse_norm and
                      os.environ.get("W8A8_STACK_TAILS", "0") == "1")
        # qk-norm + RoPE + KV write inside the attention launch (W8A8_STACK_FUSE_ROPE=0: as two launches)
        self.fuse_rope = os.environ.get("W8A8_STACK_FUSE_ROPE", "1") == "1"
        c = cfg
        g = c.group
        self.nq_l, self.nkv_l, self.qkv_n, self.attn_k, self.inter_lo, self.inter_hi = shard_plan(cfg, tp_size, tp_rank)
        self.inter_l = self.inter_hi - self.inter_lo
        dev = "cuda"

        D = c.head_dim
        q_lo, q_hi = tp_rank * self.nq_l * D, (tp_rank + 1) * self.nq_l * D
        kv_lo, kv_hi = tp_rank * self.nkv_l * D, (tp_rank + 1) * self.nkv_l * D
        self.layers = []
        self._keep = []
        self._registered = []
        for l in range(c.n_layer):
            f = layer_tensors(torch, cfg, l, seed, dev)
            kq, kk = c.n_head * D, c.n_kv * D
            rows = torch.cat([torch.arange(q_lo, q_hi), kq + torch.arange(kv_lo, kv_hi),
                              kq + kk + torch.arange(kv_lo, kv_hi)]).to(dev)
            wqkv, sqkv = f["wqkv"][rows].contiguous(), f["sqkv"][rows].contiguous()
            wo = f["wo"][:, q_lo:q_hi].contiguous()
            so = f["so"][:, q_lo // g:q_hi // g].contiguous()
            w1, s1 = f["w1"][self.inter_lo:self.inter_hi].contiguous(), f["s1"][self.inter_lo:self.inter_hi].contiguous()
            w3, s3 = f["w3"][self.inter_lo:self.inter_hi].contiguous(), f["s3"][self.inter_lo:self.inter_hi].contiguous()
            G = c.dim // g
            w13 = torch.empty((2 * self.inter_l, c.dim), dtype=torch.int8, device=dev)
            s13 = torch.empty((2 * self.inter_l, G), dtype=torch.float16, device=dev)
            ctx.pack_gate_up(w1, s1, w3, s3, self.inter_l, c.dim, G, w13, s13)
            w2 = f["w2"][:, self.inter_lo:self.inter_hi].contiguous()
            s2 = f["s2"][:, self.inter_lo // g:self.inter_hi // g].contiguous()
            torch.cuda.synchronize()
            lw = dict(attn_norm=f["attn_norm"], ffn_norm=f["ffn_norm"], q_norm=f["q_norm"], k_norm=f["k_norm"],
                      wqkv=wqkv, sqkv=sqkv, wo=wo, so=so, w13=w13, s13=s13, w2=w2, s2=s2)
            del f, w1, w3, s1, s3
            if pack:  # what the loader does once per weight: pack for the decode kernel and register the pair
                for name, sname, n, k in (("wqkv", "sqkv", self.qkv_n, c.dim), ("wo", "so", c.dim, self.attn_k),
                                          ("w13", "s13", 2 * self.inter_l, c.dim), ("w2", "s2", c.dim, self.inter_l)):
                    nbytes = ctx.packed_weight_bytes(n, k, g)
                    if nbytes:
                        P = torch.empty((nbytes,), dtype=torch.uint8, device=dev)
                        ctx.pack_weight(lw[name], lw[sname], n, k, g, P)
                        ctx.register_packed_weight(lw[name], P, n, k, g)
                        self._registered.append(lw[name])
                        self._keep.append(P)
                        lw[name + "_packed"] = P
            self.layers.append(lw)
        self.final_norm = final_norm_weight(torch, cfg, seed, dev)
        self.freqs = rope_frequencies(torch, cfg, dev)
        # paged KV, already holding `context` tokens per sequence (synthetic prefill); a rank keeps its kv heads
        self.k_cache, self.v_cache, self.block_table, self.max_blocks = synthetic_kv(
            torch, cfg, batch, context, max_new, seed, dev, kv_heads=(tp_rank * self.nkv_l, self.nkv_l))
        self.positions = torch.full((batch,), context, dtype=torch.int32, device=dev)   # the new token's position
        self.seq_lens = torch.full((batch,), context + 1, dtype=torch.int32, device=dev)
        self.context0 = context

        B = batch
        h16 = dict(dtype=torch.float16, device=dev)
        self.x = torch.zeros((B, c.dim), **h16)          # residual stream
        self.x_alt = torch.zeros((B, c.dim), **h16)      # its other copy when the fused form ping-pongs
        self.delta = torch.zeros((B, c.dim), **h16)      # output of wo / w2 (summed over ranks when TP > 1)
        self.have_delta = False
        self.xq = torch.empty((B, c.dim), dtype=torch.int8, device=dev)
        self.xs = torch.empty((B, c.dim // g), dtype=torch.float32, device=dev)
        self.qkv = torch.empty((B, self.qkv_n), **h16)
        self.q = torch.empty((B, self.nq_l, D), **h16)
        self.aq = torch.empty((B, self.attn_k), dtype=torch.int8, device=dev)
        self.as_ = torch.empty((B, self.attn_k // g), dtype=torch.float32, device=dev)
        self.act = torch.empty((B, self.inter_l), **h16)
        self.actq = torch.empty((B, self.inter_l), dtype=torch.int8, device=dev)
        self.acts = torch.empty((B, self.inter_l // g), dtype=torch.float32, device=dev)
        self.out = torch.empty((B, c.dim), **h16)
        self.launches_per_step = c.n_layer * ((7 if self.fuse_norm else 9) - (1 if self.fuse_rope else 0)) + 2
        if self.tails:
            self.launches_per_step = c.n_layer * (5 if self.fuse_rope else 6) + 1
        # bytes the step must move at least once (per rank): weights + scales + the KV it reads
        wbytes = sum(lw[n].numel() + lw[s].numel() * 2 for lw in self.layers
                     for n, s in (("wqkv", "sqkv"), ("wo", "so"), ("w13", "s13"), ("w2", "s2")))
        self.weight_bytes = wbytes
        self.kv_bytes_per_step = lambda ctx_len: 2 * B * ctx_len * c.n_layer * self.nkv_l * D * 2

    # ------------------------------------------------------------------------------------------
    def decode_step(self, x_in=None):
        """One token for every sequence. x_in fp16 [B, dim] (the embedding of the new token); returns
        the final-normed hidden state in self.out. All launches go to the current stream."""
        c, ctx, B, g = self.cfg, self.ctx, self.B, self.cfg.group
        D = c.head_dim
        if x_in is not None:
            self.x.copy_(x_in, non_blocking=True)
        sm_scale = 1.0 / math.sqrt(D)
        if self.tails:
            return self._decode_step_tails(sm_scale)
        pending = False  # a projection output waiting to be added to the residual stream
        x, x_alt = self.x, self.x_alt
        for l, lw in enumerate(self.layers):
            if self.fuse_norm:
                ctx.rmsnorm_linear(lw["wqkv"], lw["sqkv"], g, x, lw["attn_norm"], c.eps, self.qkv, B, self.qkv_n,
                                   c.dim, residual=self.delta if pending else None, x_out=x_alt if pending else None)
                if pending:
                    x, x_alt = x_alt, x
            elif pending and self.tp_fused:
                ctx.tp_allreduce_rmsnorm_quantize(self.x, None, lw["attn_norm"], c.eps, B, c.dim, g,
                                                  Xq=self.xq, Xs=self.xs)
            else:
                ctx.rmsnorm_quantize(self.x, lw["attn_norm"], c.eps, B, c.dim, g, self.xq, self.xs,
                                     residual=self.delta if pending else None)
            if not self.fuse_norm:
                ctx.linear_q(lw["wqkv"], lw["sqkv"], g, self.xq, self.xs, self.qkv, B, self.qkv_n, c.dim)
            if self.fuse_rope:
                ctx.qkv_attention_decode(self.qkv, lw["q_norm"], lw["k_norm"], c.eps, self.freqs, self.positions,
                                         self.k_cache, self.v_cache, self.block_table, self.seq_lens, None, B, self.nq_l,
                                         D, self.max_blocks, sm_scale, l, c.n_layer, self.nkv_l, quant_group_size=g,
                                         Xq=self.aq, Xs=self.as_, context_splits=self.attn_splits)
            else:
                ctx.qknorm_rope_kvwrite(self.qkv, lw["q_norm"], lw["k_norm"], c.eps, self.freqs, self.positions,
                                        self.block_table, self.max_blocks, self.k_cache, self.v_cache, l, c.n_layer, B,
                                        self.nq_l, self.nkv_l, D, self.q)
                ctx.paged_attention_decode(self.q, self.k_cache, self.v_cache, self.block_table, self.seq_lens, None, B,
                                           self.nq_l, D, self.max_blocks, sm_scale, l, c.n_layer, self.nkv_l,
                                           quant_group_size=g, Xq=self.aq, Xs=self.as_,
                                           context_splits=self.attn_splits)
            if self.tp_fused:  # the partial goes from the kernel's epilogue into every rank's exchange buffer
                ctx.tp_linear_q(lw["wo"], lw["so"], g, self.aq, self.as_, B, c.dim, self.attn_k)
            else:
                ctx.linear_q(lw["wo"], lw["so"], g, self.aq, self.as_, self.delta, B, c.dim, self.attn_k)
            if self.all_reduce is not None:
                self.all_reduce(self.delta)
            if self.fuse_norm:
                ctx.rmsnorm_linear(lw["w13"], lw["s13"], g, x, lw["ffn_norm"], c.eps, self.act, B, 2 * self.inter_l,
                                   c.dim, residual=self.delta, x_out=x_alt, epilogue=capi.EPI_SWIGLU)
                x, x_alt = x_alt, x
            else:
                if self.tp_fused:
                    ctx.tp_allreduce_rmsnorm_quantize(self.x, None, lw["ffn_norm"], c.eps, B, c.dim, g,
                                                      Xq=self.xq, Xs=self.xs)
                else:
                    ctx.rmsnorm_quantize(self.x, lw["ffn_norm"], c.eps, B, c.dim, g, self.xq, self.xs,
                                         residual=self.delta)
                ctx.linear_q(lw["w13"], lw["s13"], g, self.xq, self.xs, self.act, B, 2 * self.inter_l, c.dim,
                             epilogue=capi.EPI_SWIGLU)
            ctx.quantize(self.act, B, self.inter_l, g, self.actq, self.acts)
            if self.tp_fused:
                ctx.tp_linear_q(lw["w2"], lw["s2"], g, self.actq, self.acts, B, c.dim, self.inter_l)
            else:
                ctx.linear_q(lw["w2"], lw["s2"], g, self.actq, self.acts, self.delta, B, c.dim, self.inter_l)
            if self.all_reduce is not None:
                self.all_reduce(self.delta)
            pending = True
        if self.tp_fused:
            ctx.tp_allreduce_rmsnorm_quantize(self.x, None, self.final_norm, c.eps, B, c.dim, g, normed_out=self.out)
        else:
            ctx.residual_add(x, self.delta, B * c.dim)
            ctx.rms_norm(x, self.final_norm, self.out, B, c.dim, c.eps)
        self.positions.add_(1)
        self.seq_lens.add_(1)
        return self.out

    def _attention(self, l, lw, sm_scale):
        c, ctx, B, g, D = self.cfg, self.ctx, self.B, self.cfg.group, self.cfg.head_dim
        if self.fuse_rope:
            ctx.qkv_attention_decode(self.qkv, lw["q_norm"], lw["k_norm"], c.eps, self.freqs, self.positions,
                                     self.k_cache, self.v_cache, self.block_table, self.seq_lens, None, B, self.nq_l,
                                     D, self.max_blocks, sm_scale, l, c.n_layer, self.nkv_l, quant_group_size=g,
                                     Xq=self.aq, Xs=self.as_, context_splits=self.attn_splits)
        else:
            ctx.qknorm_rope_kvwrite(self.qkv, lw["q_norm"], lw["k_norm"], c.eps, self.freqs, self.positions,
                                    self.block_table, self.max_blocks, self.k_cache, self.v_cache, l, c.n_layer, B,
                                    self.nq_l, self.nkv_l, D, self.q)
            ctx.paged_attention_decode(self.q, self.k_cache, self.v_cache, self.block_table, self.seq_lens, None, B,
                                       self.nq_l, D, self.max_blocks, sm_scale, l, c.n_layer, self.nkv_l,
                                       quant_group_size=g, Xq=self.aq, Xs=self.as_, context_splits=self.attn_splits)

    def _decode_step_tails(self, sm_scale):
        """The step with the small kernels as tails of the linears (one GPU): per layer wqkv, attention,
        wo [+ residual add, RMSNorm, quantiser], w1|w3 + SwiGLU [+ quantiser], w2 [+ residual add, the next layer's
        RMSNorm, quantiser]; one row kernel in front of the first layer."""
        c, ctx, B, g = self.cfg, self.ctx, self.B, self.cfg.group
        ctx.rmsnorm_quantize(self.x, self.layers[0]["attn_norm"], c.eps, B, c.dim, g, self.xq, self.xs)
        for l, lw in enumerate(self.layers):
            ctx.linear_q(lw["wqkv"], lw["sqkv"], g, self.xq, self.xs, self.qkv, B, self.qkv_n, c.dim)
            self._attention(l, lw, sm_scale)
            ctx.linear_q_tail(lw["wo"], lw["so"], g, self.aq, self.as_, self.delta, B, c.dim, self.attn_k,
                              capi.TAIL_ROWNORM, g, tail_Xq=self.xq, tail_Xs=self.xs, x=self.x,
                              norm_weight=lw["ffn_norm"], eps=c.eps)
            ctx.linear_q_tail(lw["w13"], lw["s13"], g, self.xq, self.xs, self.act, B, 2 * self.inter_l, c.dim,
                              capi.TAIL_GROUPQUANT, g, tail_Xq=self.actq, tail_Xs=self.acts, epilogue=capi.EPI_SWIGLU)
            last = l + 1 == len(self.layers)
            ctx.linear_q_tail(lw["w2"], lw["s2"], g, self.actq, self.acts, self.delta, B, c.dim, self.inter_l,
                              capi.TAIL_ROWNORM, g, tail_Xq=None if last else self.xq, tail_Xs=None if last else self.xs,
                              x=self.x, norm_weight=self.final_norm if last else self.layers[l + 1]["attn_norm"],
                              eps=c.eps, normed_out=self.out if last else None)
        self.positions.add_(1)
        self.seq_lens.add_(1)
        return self.out

    def one_launch_descriptor(self):
        """The w8a8_decode_stack descriptor of this stack (single GPU, packed weights), built once."""
        if getattr(self, "_desc", None) is not None:
            return self._desc
        assert self.tp_size == 1, "the one-launch step is the single-GPU form"
        torch, c = self.torch, self.cfg
        rows = []
        for lw in self.layers:
            rows.append([lw["attn_norm"].data_ptr(), lw["ffn_norm"].data_ptr(),
                         lw["q_norm"].data_ptr() if c.qk_norm else 0, lw["k_norm"].data_ptr() if c.qk_norm else 0] + [lw[n + "_packed"].data_ptr() for n in ("wqkv", "wo", "w13", "w2")])
        table = np.asarray(rows, dtype=np.int64)
        assert table.shape[1] == capi.DECODE_LAYER_POINTERS
        self._layer_table = torch.from_numpy(table).to(self.x.device)
        d = capi.DecodeStack()
        d.n_layers, d.batch, d.dim, d.n_q_heads, d.n_kv_heads = c.n_layer, self.B, c.dim, self.nq_l, self.nkv_l
        d.head_dim, d.inter, d.group_size = c.head_dim, self.inter_l, c.group
        d.eps, d.sm_scale = c.eps, 1.0 / math.sqrt(c.head_dim)
        d.layers, d.final_norm, d.rope_freqs = self._layer_table.data_ptr(), self.final_norm.data_ptr(), self.freqs.data_ptr()
        d.positions, d.seq_lens, d.block_table = self.positions.data_ptr(), self.seq_lens.data_ptr(), self.block_table.data_ptr()
        d.max_blocks_per_seq = self.max_blocks
        d.k_cache, d.v_cache, d.x, d.out = self.k_cache.data_ptr(), self.v_cache.data_ptr(), self.x.data_ptr(), self.out.data_ptr()
        self._desc = d
        return d

    def decode_step_one_launch(self, x_in=None):
        """The same step as decode_step through w8a8_decode_stack_step: one persistent kernel."""
        if x_in is not None:
            self.x.copy_(x_in, non_blocking=True)
        self.ctx.decode_stack_step(self.one_launch_descriptor())
        self.positions.add_(1)
        self.seq_lens.add_(1)
        return self.out

    def linears_only(self):
        """Only the four W8A8 linears of every layer, on whatever the activation buffers hold: the
        benchmark times these alone to put the dominant kernel on the roofline."""
        c, ctx, B, g = self.cfg, self.ctx, self.B, self.cfg.group
        for lw in self.layers:
            ctx.linear_q(lw["wqkv"], lw["sqkv"], g, self.xq, self.xs, self.qkv, B, self.qkv_n, c.dim)
            ctx.linear_q(lw["wo"], lw["so"], g, self.aq, self.as_, self.delta, B, c.dim, self.attn_k)
            ctx.linear_q(lw["w13"], lw["s13"], g, self.xq, self.xs, self.act, B, 2 * self.inter_l, c.dim,
                         epilogue=capi.EPI_SWIGLU)
            ctx.linear_q(lw["w2"], lw["s2"], g, self.actq, self.acts, self.delta, B, c.dim, self.inter_l)

    def close(self):
        """Removes this stack's weights from the context's packed-weight registry (before the tensors are freed)."""
        for W in self._registered:
            self.ctx.register_packed_weight(W, None)
        self._registered = []

    def reset_positions(self):
        self.positions.fill_(self.context0)
        self.seq_lens.fill_(self.context0 + 1)
