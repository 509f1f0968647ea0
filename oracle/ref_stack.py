"""The slow-AR decode step built from the REFERENCE's own CUDA kernels (_ref/libfishref.so). TEST INFRASTRUCTURE:
used by the GPU parity tests and by the benchmark's `--impl reference` arm, never by the product.

The kernels are called through their stock entry points in the order of DualAREngine::decode_step
(src/engine/dual_ar_engine.cc:576-657) at batch B: rms_norm, int8_dequant_gemm_fp16 x5 (gate and up apart), silu, mul,
residual_add x2, qk rms_norm x2, rope_qk, paged_attention_decode. The engine itself cannot be built here (its build
fetches dependencies from the network and it wants a checkpoint); its per-head cudaMemcpyAsync KV writes, which are
batch-1 host code, are stood in for by one vectorised scatter per layer. Launches are eager: the reference linear
allocates inside the call. Single GPU (the reference has no multi-GPU path).

Weights, norms, KV cache and block table are the same seeded tensors the repository's own stack cuts its shards from
(fish-audio-cpp_b200/stack.py: layer_tensors, synthetic_kv), built with torch alone: nothing here loads the product
library.
"""
from __future__ import annotations

from . import fishref


class ReferenceStack:
    def __init__(self, torch, cfg, batch: int, context: int, max_new: int = 128, seed: int = 0):
        from fish_audio_cpp_b200 import stack as S

        self.f, self.torch, self.cfg, self.B = fishref, torch, cfg, batch
        c, D, B = cfg, cfg.head_dim, batch
        self.layers = [S.layer_tensors(torch, cfg, l, seed) for l in range(c.n_layer)]
        self.final_norm = S.final_norm_weight(torch, cfg, seed)
        self.freqs = S.rope_frequencies(torch, cfg)
        self.k_cache, self.v_cache, self.block_table, self.max_blocks = S.synthetic_kv(torch, cfg, batch, context,
                                                                                       max_new, seed)
        self.context0 = context
        self.pos = context
        self.seq_lens = torch.full((B,), context + 1, dtype=torch.int32, device="cuda")
        h16 = dict(dtype=torch.float16, device="cuda")
        self.qkv_n = (c.n_head + 2 * c.n_kv) * D
        self.x = torch.zeros((B, c.dim), **h16)
        self.out = torch.empty((B, c.dim), **h16)
        self.ws1 = torch.empty((B, max(c.dim, c.inter)), **h16)
        self.ws2 = torch.empty((B, max(self.qkv_n, c.inter, c.dim)), **h16)
        self.up = torch.empty((B, c.inter), **h16)
        self.qb = torch.empty((B, c.n_head, D), **h16)
        self.kb = torch.empty((B, c.n_kv, D), **h16)
        self.vb = torch.empty((B, c.n_kv, D), **h16)
        self.att = torch.empty((B, c.n_head * D), **h16)

    def reset_positions(self):
        self.pos = self.context0
        self.seq_lens.fill_(self.context0 + 1)

    def gemm(self, W, S, X, Y, n_out, tokens, K):
        self.f.int8_dequant_gemm_fp16(W.data_ptr(), S.data_ptr(), self.cfg.group, None, None, X.data_ptr(),
                                      Y.data_ptr(), n_out, tokens, K)

    def decode_step(self, x_in, advance: bool = True):
        f, c, B, D = self.f, self.cfg, self.B, self.cfg.head_dim
        x = self.x
        x.copy_(x_in)
        p = lambda tt: tt.data_ptr()  # noqa: E731
        pos = int(self.pos)
        for l, lw in enumerate(self.layers):
            f.rms_norm(p(x), p(lw["attn_norm"]), p(self.ws1), B, c.dim, c.eps)
            self.gemm(lw["wqkv"], lw["sqkv"], self.ws1, self.ws2, self.qkv_n, B, c.dim)
            qkv = self.ws2.view(-1)[:B * self.qkv_n].view(B, self.qkv_n)
            self.qb.copy_(qkv[:, :c.n_head * D].reshape(B, c.n_head, D))
            self.kb.copy_(qkv[:, c.n_head * D:(c.n_head + c.n_kv) * D].reshape(B, c.n_kv, D))
            self.vb.copy_(qkv[:, (c.n_head + c.n_kv) * D:].reshape(B, c.n_kv, D))
            if c.qk_norm:
                f.rms_norm(p(self.qb), p(lw["q_norm"]), p(self.qb), B * c.n_head, D, c.eps)
                f.rms_norm(p(self.kb), p(lw["k_norm"]), p(self.kb), B * c.n_kv, D, c.eps)
            f.rope_qk(p(self.qb), p(self.kb), p(self.freqs), B, c.n_head, c.n_kv, 1, D, pos)
            phys = self.block_table[:, pos // c.block_tokens].long()
            self.k_cache[phys, l, :, pos % c.block_tokens] = self.kb
            self.v_cache[phys, l, :, pos % c.block_tokens] = self.vb
            f.paged_attention_decode(p(self.qb), p(self.k_cache), p(self.v_cache), p(self.block_table), p(self.seq_lens),
                                     p(self.att), B, c.n_head, D, self.max_blocks, 1.0 / D ** 0.5, l, c.n_layer, c.n_kv)
            self.gemm(lw["wo"], lw["so"], self.att, self.ws1, c.dim, B, c.n_head * D)
            f.residual_add(p(x), p(self.ws1), B * c.dim)
            f.rms_norm(p(x), p(lw["ffn_norm"]), p(self.ws2), B, c.dim, c.eps)
            self.gemm(lw["w1"], lw["s1"], self.ws2, self.ws1, c.inter, B, c.dim)
            f.silu(p(self.ws1), B * c.inter)
            self.gemm(lw["w3"], lw["s3"], self.ws2, self.up, c.inter, B, c.dim)
            f.mul(p(self.ws1), p(self.up), B * c.inter)
            self.gemm(lw["w2"], lw["s2"], self.ws1, self.ws2, c.dim, B, c.inter)
            f.residual_add(p(x), p(self.ws2), B * c.dim)
        f.rms_norm(p(x), p(self.final_norm), p(self.out), B, c.dim, c.eps)
        if advance:
            self.pos += 1
            self.seq_lens.add_(1)
        return self.out
