"""The decoder-stack harness (layer loop of DualAREngine::decode_step) against the oracle chain, small config."""
import numpy as np
import pytest
import torch

from fish_audio_cpp_b200 import stack as S

pytestmark = pytest.mark.gpu


def oracle_step(oracle, st, x_in, k_cache, v_cache, bt, positions, jitter=None):
    """One decode step on the CPU. With `jitter` (a numpy Generator) the attention output is moved by one
    fp16 ulp up or down at random: what a different but equally valid summation order does to it."""
    c = st.cfg
    g, D, B = c.group, c.head_dim, x_in.shape[0]
    cpu = lambda t: t.cpu().numpy()
    freqs = cpu(st.freqs)
    x = x_in.copy()
    pending = None
    for l, lw in enumerate(st.layers):
        if pending is not None:
            x = oracle.residual_add(x, pending)
        h = oracle.rms_norm(x, cpu(lw["attn_norm"]), c.eps)
        qkv = oracle.linear(cpu(lw["wqkv"]), cpu(lw["sqkv"]), g, h).reshape(B, st.nq_l + 2 * st.nkv_l, D)
        q = np.empty((B, st.nq_l, D), np.float16)
        for b in range(B):
            pos = int(positions[b])
            qn = cpu(lw["q_norm"]) if c.qk_norm else None
            kn = cpu(lw["k_norm"]) if c.qk_norm else None
            q[b] = oracle.qknorm_rope(qkv[b, :st.nq_l], qn, c.eps, freqs, pos)
            kk = oracle.qknorm_rope(qkv[b, st.nq_l:st.nq_l + st.nkv_l], kn, c.eps, freqs, pos)
            phys = bt[b, pos // 16]
            k_cache[phys, l, :, pos % 16] = kk
            v_cache[phys, l, :, pos % 16] = qkv[b, st.nq_l + st.nkv_l:]
        att = oracle.paged_attention_decode(q, k_cache, v_cache, bt, positions + 1, l, 1.0 / np.sqrt(D))
        att16 = att.astype(np.float16).reshape(B, st.attn_k)
        if jitter is not None:
            bits = att16.view(np.uint16).astype(np.int32) + jitter.integers(-1, 2, att16.shape)
            att16 = np.clip(bits, 0, 0xFFFF).astype(np.uint16).view(np.float16)
        delta = oracle.linear(cpu(lw["wo"]), cpu(lw["so"]), g, att16)
        x = oracle.residual_add(x, delta)
        h2 = oracle.rms_norm(x, cpu(lw["ffn_norm"]), c.eps)
        act = oracle.linear(cpu(lw["w13"]), cpu(lw["s13"]), g, h2, epilogue=oracle.EPI_SWIGLU)
        pending = oracle.linear(cpu(lw["w2"]), cpu(lw["s2"]), g, act)
    x = oracle.residual_add(x, pending)
    return oracle.rms_norm(x, cpu(st.final_norm), c.eps)


@pytest.mark.parametrize("group,dim,qk_norm,context", [(64, 512, True, 37), (256, 512, True, 37), (256, 1024, True, 37),
                                                        (64, 1024, False, 3)])  # the last: the fast AR's form
def test_stack_matches_oracle_chain(ctx, oracle, group, dim, qk_norm, context):
    cfg = S.SlowARConfig(n_layer=2, dim=dim, n_head=4, n_kv=1, inter=512, group=group, qk_norm=qk_norm)
    B = 3
    st = S.SlowARStack(torch, ctx, cfg, B, context, max_new=8, seed=5)
    rng = np.random.default_rng(group)
    x_in = rng.standard_normal((B, cfg.dim)).astype(np.float16)
    kc, vc = st.k_cache.cpu().numpy().copy(), st.v_cache.cpu().numpy().copy()
    bt, pos = st.block_table.cpu().numpy(), st.positions.cpu().numpy().copy()
    out = st.decode_step(torch.from_numpy(x_in).cuda())
    torch.cuda.synchronize()
    ctx.check_device_status()
    want = oracle_step(oracle, st, x_in, kc.copy(), vc.copy(), bt, pos).astype(np.float32)
    got = out.cpu().numpy().astype(np.float32)
    rel = np.linalg.norm(got - want) / np.linalg.norm(want)
    # The attention kernel sums in another order than the oracle (tolerance parity), and the quantisers
    # after it turn a last-bit difference into a flipped code now and then. The yardstick is therefore the
    # oracle's own sensitivity: how far its result moves when its attention output is jittered by one ulp.
    noise = max(np.linalg.norm(oracle_step(oracle, st, x_in, kc.copy(), vc.copy(), bt, pos,
                                           jitter=np.random.default_rng(s)).astype(np.float32) - want)
                for s in range(3)) / np.linalg.norm(want)
    assert rel < max(2e-2, 3.0 * noise), (rel, noise)
    assert int(st.positions[0]) == context + 1 and int(st.seq_lens[0]) == context + 2
    # graph replay gives the same bits as the eager step from the same state
    st.reset_positions()
    st.k_cache.copy_(torch.from_numpy(kc).cuda()); st.v_cache.copy_(torch.from_numpy(vc).cuda())
    xin = torch.from_numpy(x_in).cuda()
    st.decode_step(xin); torch.cuda.synchronize()   # warm (attributes set), state advanced
    st.reset_positions()
    st.k_cache.copy_(torch.from_numpy(kc).cuda()); st.v_cache.copy_(torch.from_numpy(vc).cuda())
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        st.decode_step(xin)
    st.reset_positions()
    st.k_cache.copy_(torch.from_numpy(kc).cuda()); st.v_cache.copy_(torch.from_numpy(vc).cuda())
    gr.replay(); torch.cuda.synchronize()
    assert np.array_equal(st.out.cpu().numpy().view(np.uint16), out.cpu().numpy().view(np.uint16)) or \
        np.linalg.norm(st.out.cpu().numpy().astype(np.float32) - got) / np.linalg.norm(got) < 1e-3
    st.close()


def test_stack_at_benchmark_width_matches_oracle_and_reference_chain(pkg, oracle):
    """The benchmarked configuration's own shapes (hidden 2560, 32 q / 8 kv heads of 128, SwiGLU 9728, g256, batch 8,
    context 1024), two layers deep: one decode step against (a) the CPU oracle chain and (b) the reference's own CUDA
    kernels chained like DualAREngine::decode_step (oracle/ref_stack.py) on the same seeded weights, cache and input.

    What may differ: the attention kernels sum in different orders (tolerance parity), the decode linears add their
    K-groups per warp range instead of strictly ascending, and a quantiser behind either turns a last-bit difference
    into a flipped int8 code now and then. The yardstick is the oracle's own sensitivity to a one-ulp jitter of its
    attention output ("noise"); the bar is max(5e-3, 3 x noise) in relative L2 norm of the final hidden state.
    The K and V rows layer 0 writes depend on the norm, wqkv, qk-norm and RoPE only: at most 2 fp16 ulp from the
    oracle for 99.9 % of the elements."""
    from oracle import fishref, ref_stack

    ctx = pkg.Context(0, 1 << 22)
    cfg = S.SlowARConfig(n_layer=2)
    B, context = 8, 1024
    st = S.SlowARStack(torch, ctx, cfg, B, context, max_new=8, seed=21)
    try:
        rng = np.random.default_rng(17)
        x_in = (rng.standard_normal((B, cfg.dim)) * 0.5).astype(np.float16)
        kc, vc = st.k_cache.cpu().numpy().copy(), st.v_cache.cpu().numpy().copy()
        bt, pos = st.block_table.cpu().numpy(), st.positions.cpu().numpy().copy()
        out = st.decode_step(torch.from_numpy(x_in).cuda())
        torch.cuda.synchronize()
        ctx.check_device_status()
        got = out.cpu().numpy().astype(np.float32)
        kw, vw = kc.copy(), vc.copy()
        want = oracle_step(oracle, st, x_in, kw, vw, bt, pos).astype(np.float32)
        noise = max(np.linalg.norm(oracle_step(oracle, st, x_in, kc.copy(), vc.copy(), bt, pos,
                                               jitter=np.random.default_rng(s)).astype(np.float32) - want)
                    for s in range(2)) / np.linalg.norm(want)
        rel = np.linalg.norm(got - want) / np.linalg.norm(want)
        bar = max(5e-3, 3.0 * noise)
        print(f"[stack@2560] ours vs oracle chain: rel L2 {rel:.3e}, one-ulp-jitter noise {noise:.3e}")
        assert rel < bar, (rel, noise)
        # rows written by layer 0
        phys = bt[np.arange(B), pos // 16]
        for cache_got, cache_want in ((st.k_cache, kw), (st.v_cache, vw)):
            g0 = cache_got[torch.from_numpy(phys).long().cuda(), 0][:, :, int(pos[0]) % 16].cpu().numpy()
            w0 = cache_want[phys, 0][:, :, int(pos[0]) % 16]
            ulp = oracle.ulp_distance_fp16(g0, w0)
            assert (ulp <= 2).mean() >= 0.999 and ulp.max() <= 16, (ulp.max(), (ulp <= 2).mean())
        if fishref.available():
            ref = ref_stack.ReferenceStack(torch, cfg, B, context, max_new=8, seed=21)
            assert torch.equal(ref.k_cache, torch.from_numpy(kc).cuda()) and torch.equal(ref.block_table, st.block_table)
            rout = ref.decode_step(torch.from_numpy(x_in).cuda()).cpu().numpy().astype(np.float32)
            torch.cuda.synchronize()
            rel_ref = np.linalg.norm(got - rout) / np.linalg.norm(rout)
            rel_ro = np.linalg.norm(rout - want) / np.linalg.norm(want)
            print(f"[stack@2560] ours vs reference-kernel chain: rel L2 {rel_ref:.3e}; reference chain vs oracle {rel_ro:.3e}")
            assert rel_ref < bar, (rel_ref, noise)
            assert rel_ro < bar, (rel_ro, noise)
    finally:
        st.close()
        ctx.close()


def test_fast_ar_frame_matches_oracle_chain(pkg, oracle):
    """One frame of the fast-AR codebook decoder at its real width: ten codebook steps of a 4-layer stack (hidden 2560,
    32 q / 8 kv heads, SwiGLU 9728, no qk-norm, g64) at batch 8 over a cache that starts empty, each followed by the
    final norm and the codebook head 2560 -> 4096 (the order of DualAREngine::fast_codebook_decode_device,
    src/engine/dual_ar_engine.cc:769-844), against the CPU oracle chain fed with the same inputs step by step (each
    side keeps its own cache). Bar per step: relative L2 distance of the logits within max(5e-3, 3 x the distance by
    which a one-ulp jitter of the oracle's own attention output moves its logits)."""
    from fish_audio_cpp_b200 import synth

    ctx = pkg.Context(0, 1 << 22)
    cfg = S.SlowARConfig(n_layer=4, group=64, qk_norm=False)
    B, steps, vocab = 8, 10, 4096
    st = S.SlowARStack(torch, ctx, cfg, B, 0, max_new=16, seed=41)
    rng = np.random.default_rng(9)
    hw, hs = synth.weights(rng, vocab, cfg.dim), synth.weight_scales(rng, vocab, cfg.dim // 64)
    dhw, dhs = torch.from_numpy(hw).cuda(), torch.from_numpy(hs).cuda()
    img = torch.empty((ctx.packed_weight_bytes(vocab, cfg.dim, 64),), dtype=torch.uint8, device="cuda")
    ctx.pack_weight(dhw, dhs, vocab, cfg.dim, 64, img)
    ctx.register_packed_weight(dhw, img, vocab, cfg.dim, 64)
    try:
        kc, vc = st.k_cache.cpu().numpy().copy(), st.v_cache.cpu().numpy().copy()
        kj, vj = kc.copy(), vc.copy()
        bt = st.block_table.cpu().numpy()
        logits = torch.empty((B, vocab), dtype=torch.float16, device="cuda")
        worst = 0.0
        for step in range(steps):
            x_in = (rng.standard_normal((B, cfg.dim)) * 0.5).astype(np.float16)
            pos = np.full((B,), step, np.int32)
            out = st.decode_step(torch.from_numpy(x_in).cuda())
            ctx.linear(dhw, dhs, 64, out, logits, B, vocab, cfg.dim)
            torch.cuda.synchronize()
            ctx.check_device_status()
            got = logits.cpu().numpy().astype(np.float32)
            want_h = oracle_step(oracle, st, x_in, kc, vc, bt, pos)
            want = oracle.linear(hw, hs, 64, want_h).astype(np.float32)
            jit_h = oracle_step(oracle, st, x_in, kj, vj, bt, pos, jitter=np.random.default_rng(step))
            noise = np.linalg.norm(oracle.linear(hw, hs, 64, jit_h).astype(np.float32) - want) / np.linalg.norm(want)
            rel = np.linalg.norm(got - want) / np.linalg.norm(want)
            worst = max(worst, rel / max(5e-3, 3.0 * noise))
            assert rel < max(5e-3, 3.0 * noise), (step, rel, noise)
        print(f"[fast-AR frame] worst step at {worst:.2f} of its bar")
        assert int(st.positions[0]) == steps
    finally:
        ctx.register_packed_weight(dhw, None)
        st.close()
        ctx.close()


@pytest.mark.parametrize("group,dim,n_kv,inter,layers,B,context", [
    (256, 512, 1, 512, 2, 3, 37), (64, 1024, 2, 768, 3, 8, 100), (128, 2560, 8, 1024, 2, 8, 530), (256, 2560, 8, 9728, 2, 5, 1024),
    (256, 2560, 8, 9728, 1, 8, 1024)])
def test_one_launch_step_matches_the_chain_of_launches(ctx, group, dim, n_kv, inter, layers, B, context):
    """w8a8_decode_stack_step (one persistent cooperative kernel) against decode_step (eight launches per
    layer) from the same state, two steps. Both run the same arithmetic; the one difference is how many CTAs
    share a linear's row tiles (148 there, up to 296 in the separate launches), hence where its K range is cut
    between warps, i.e. the grouping of its fp32 partial sums, so outputs of a
    linear may differ in the last fp16 bit and, now and then, a quantiser after it flips a code. The bars:
    hidden state within 2e-2 in relative L2 norm after several layers; the KV rows written by layer 0 within
    3 fp16 ulp for at least 99 % of the elements and never beyond 1e-2 of the largest value; all KV rows
    within 2e-2 in relative L2 norm."""
    cfg = S.SlowARConfig(n_layer=layers, dim=dim, n_head=4 * n_kv, n_kv=n_kv, inter=inter, group=group)
    st = S.SlowARStack(torch, ctx, cfg, B, context, max_new=8, seed=11)
    need = ctx.decode_stack_workspace_bytes(st.one_launch_descriptor())
    assert 0 < need <= ctx.workspace_bytes
    rng = np.random.default_rng(dim + group)
    k0, v0 = st.k_cache.clone(), st.v_cache.clone()
    xs = [torch.from_numpy(rng.standard_normal((B, cfg.dim)).astype(np.float16)).cuda() for _ in range(2)]
    want = []
    for x_in in xs:
        st.decode_step(x_in)
        torch.cuda.synchronize()
        want.append(st.out.float().clone())
    kw, vw = st.k_cache.clone(), st.v_cache.clone()
    ctx.check_device_status()
    st.reset_positions()
    st.k_cache.copy_(k0); st.v_cache.copy_(v0)
    outs = []
    for x_in, out_w in zip(xs, want):
        st.decode_step_one_launch(x_in)
        torch.cuda.synchronize()
        ctx.check_device_status()
        got = st.out.float()
        rel = ((got - out_w).norm() / out_w.norm()).item()
        assert rel < 2e-2, rel
        outs.append(st.out.clone())
    for got_c, want_c, before in ((st.k_cache, kw, k0), (st.v_cache, vw, v0)):
        assert (want_c != before).any()
        # layer 0 sees the same hidden state in both forms: its new rows differ by last-bit effects only
        g0, w0 = got_c[:, 0].float(), want_c[:, 0].float()
        assert (g0 - w0).abs().max().item() <= 1e-2 * w0.abs().max().item()
        ulp = (got_c[:, 0].contiguous().view(torch.int16).int() - want_c[:, 0].contiguous().view(torch.int16).int()).abs()
        assert (ulp <= 3).float().mean().item() >= 0.99
        # deeper layers inherit the hidden state's difference
        assert ((got_c.float() - want_c.float()).norm() / want_c.float().norm()).item() < 2e-2
    # the step is deterministic: the same inputs from the same state give the same bits
    st.reset_positions()
    st.k_cache.copy_(k0); st.v_cache.copy_(v0)
    for x_in, first in zip(xs, outs):
        st.decode_step_one_launch(x_in)
        torch.cuda.synchronize()
        assert torch.equal(st.out.view(torch.int16), first.view(torch.int16))
    st.close()


@pytest.mark.parametrize("tp,rank", [(2, 1), (4, 0), (4, 3), (8, 0), (8, 7)])
@pytest.mark.parametrize("group", [256, 64])
def test_every_tensor_parallel_shard_shape_runs(ctx, tp, rank, group):
    """One rank's shard of the benchmark stack at TP 2 / 4 / 8 (uneven w2 shards included), run alone on one GPU
    with no exchange: the decode kernels must take every shard shape (packed weights, attention with 16 / 8 / 4
    query heads) and give finite numbers. The exchange itself is tested in test_gpu_tp.py."""
    cfg = S.SlowARConfig(n_layer=1, group=group)
    st = S.SlowARStack(torch, ctx, cfg, 8, 100, max_new=4, tp_rank=rank, tp_size=tp, seed=3, all_reduce=None,
                       tp_mode="nccl")
    x = torch.from_numpy(np.random.default_rng(tp + rank).standard_normal((8, cfg.dim)).astype(np.float16)).cuda()
    out = st.decode_step(x)
    torch.cuda.synchronize()
    ctx.check_device_status()
    assert torch.isfinite(out.float()).all()
    for name in ("wqkv", "wo", "w13", "w2"):
        assert name + "_packed" in st.layers[0], f"{name} shard of TP{tp} rank {rank} was not packable"
    st.close()
