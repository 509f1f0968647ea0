"""GPU parity of the decode-step neighbours: fused split + qk-norm + RoPE + KV write, and paged attention."""
import numpy as np
import pytest
import torch

from oracle import fishref

pytestmark = pytest.mark.gpu

N_Q, N_KV, D, LAYERS, BS = 32, 8, 128, 3, 16


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def make_cache(rng, B, ctx_len, max_blocks):
    nblk = B * max_blocks + 3
    kc = (rng.standard_normal((nblk, LAYERS, N_KV, BS, D)) * 0.5).astype(np.float16)
    vc = (rng.standard_normal((nblk, LAYERS, N_KV, BS, D)) * 0.5).astype(np.float16)
    perm = rng.permutation(nblk)[:B * max_blocks].reshape(B, max_blocks).astype(np.int32)  # scattered physical blocks
    return kc, vc, perm


@pytest.mark.parametrize("B,with_norm", [(1, True), (8, True), (3, False)])
def test_qknorm_rope_kvwrite(ctx, oracle, B, with_norm):
    rng = np.random.default_rng(B)
    layer, max_blocks = 1, 8
    qkv = rng.standard_normal((B, (N_Q + 2 * N_KV) * D)).astype(np.float16)
    qw = rng.uniform(0.5, 1.5, D).astype(np.float16)
    kw = rng.uniform(0.5, 1.5, D).astype(np.float16)
    freqs = oracle.rope_freqs(D, 1e6)
    positions = rng.integers(0, max_blocks * BS, B).astype(np.int32)
    kc, vc, bt = make_cache(rng, B, 0, max_blocks)
    dk, dv = dev(kc), dev(vc)
    dq = torch.empty((B, N_Q, D), dtype=torch.float16, device="cuda")
    dqkv, dqw, dkw, dfr, dpos, dbt = dev(qkv), dev(qw), dev(kw), dev(freqs), dev(positions), dev(bt)
    ctx.qknorm_rope_kvwrite(dqkv, dqw if with_norm else None, dkw if with_norm else None, 1e-6, dfr, dpos, dbt,
                            max_blocks, dk, dv, layer, LAYERS, B, N_Q, N_KV, D, dq)
    torch.cuda.synchronize()
    q3 = qkv.reshape(B, N_Q + 2 * N_KV, D)
    want_k, want_v = kc.copy(), vc.copy()
    for b in range(B):
        pos = int(positions[b])
        wq = oracle.qknorm_rope(q3[b, :N_Q], qw if with_norm else None, 1e-6, freqs, pos)
        wk = oracle.qknorm_rope(q3[b, N_Q:N_Q + N_KV], kw if with_norm else None, 1e-6, freqs, pos)
        assert oracle.ulp_distance_fp16(dq[b].cpu().numpy(), wq).max() <= 2
        phys = bt[b, pos // BS]
        got_k = dk[phys, layer, :, pos % BS].cpu().numpy()
        assert oracle.ulp_distance_fp16(got_k, wk).max() <= 2
        want_k[phys, layer, :, pos % BS] = got_k
        want_v[phys, layer, :, pos % BS] = q3[b, N_Q + N_KV:]
    # nothing but the B new rows changed, and v is a verbatim copy
    assert np.array_equal(dk.cpu().numpy(), want_k) and np.array_equal(dv.cpu().numpy(), want_v)
    if fishref.available():
        # the reference chain: rms_norm on q and k, rope_qk in place (one sequence at a time: it is batch-1 code)
        for b in range(B):
            rq, rk = dev(q3[b, :N_Q].copy()), dev(q3[b, N_Q:N_Q + N_KV].copy())
            if with_norm:
                fishref.rms_norm(rq.data_ptr(), dqw.data_ptr(), rq.data_ptr(), N_Q, D, 1e-6)
                fishref.rms_norm(rk.data_ptr(), dkw.data_ptr(), rk.data_ptr(), N_KV, D, 1e-6)
            fishref.rope_qk(rq.data_ptr(), rk.data_ptr(), dfr.data_ptr(), 1, N_Q, N_KV, 1, D, int(positions[b]))
            torch.cuda.synchronize()
            assert torch.equal(rq, dq[b]), "q must match the reference chain bit for bit"
            pos = int(positions[b])
            assert torch.equal(rk, dk[int(bt[b, pos // BS]), layer, :, pos % BS])


@pytest.mark.parametrize("B,lens", [(1, [1]), (2, [16, 17]), (8, [1024] * 8), (4, [5, 300, 0, 1000])])
@pytest.mark.parametrize("splits", [0, 1, 3])
def test_paged_attention_decode(ctx, oracle, B, lens, splits):
    rng = np.random.default_rng(B + len(lens))
    layer, max_blocks = 2, 128
    kc, vc, bt = make_cache(rng, B, max(lens), max_blocks)
    q = rng.standard_normal((B, N_Q, D)).astype(np.float16)
    seq = np.array(lens, np.int32)
    dq, dk, dv, dbt, dseq = dev(q), dev(kc), dev(vc), dev(bt), dev(seq)
    dout = torch.full((B, N_Q, D), 9.0, dtype=torch.float16, device="cuda")
    sm = 1.0 / np.sqrt(D)
    for g in (256, 64):
        dxq = torch.empty((B, N_Q * D), dtype=torch.int8, device="cuda")
        dxs = torch.empty((B, N_Q * D // g), dtype=torch.float32, device="cuda")
        ctx.paged_attention_decode(dq, dk, dv, dbt, dseq, dout, B, N_Q, D, max_blocks, sm, layer, LAYERS, N_KV,
                                   quant_group_size=g, Xq=dxq, Xs=dxs, context_splits=splits)
        torch.cuda.synchronize()
        got = dout.cpu().numpy()
        want = oracle.paged_attention_decode(q, kc, vc, bt, seq, layer, sm)
        assert np.abs(got.astype(np.float64) - want).max() <= 2e-3 * max(1.0, np.abs(want).max())
        # the fused quantiser == the stand-alone quantiser on the fp16 output
        wq, ws = oracle.quantize(got.reshape(B, N_Q * D), g)
        assert np.array_equal(dxq.cpu().numpy(), wq) and np.array_equal(dxs.cpu().numpy(), ws)
    if fishref.available():
        rout = torch.empty_like(dout)
        fishref.paged_attention_decode(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dbt.data_ptr(), dseq.data_ptr(),
                                       rout.data_ptr(), B, N_Q, D, max_blocks, sm, layer, LAYERS, N_KV)
        torch.cuda.synchronize()
        assert (rout.float() - dout.float()).abs().max().item() <= 2e-3 * max(1.0, rout.float().abs().max().item())


@pytest.mark.parametrize("B,positions", [(1, [0]), (3, [15, 16, 40]), (8, [1024] * 8), (4, [4, 299, 31, 999])])
@pytest.mark.parametrize("splits", [0, 1, 2, 3])
def test_qkv_attention_decode_equals_the_two_calls(ctx, B, positions, splits):
    """qk-norm + RoPE + KV write + attention (+ quantiser) as one launch against the two launches: attention
    output, codes, scales and both caches bit for bit."""
    rng = np.random.default_rng(B + sum(positions))
    layer, max_blocks, g = 1, 128, 256
    kc, vc, bt = make_cache(rng, B, max(positions) + 1, max_blocks)
    qkv = rng.standard_normal((B, (N_Q + 2 * N_KV) * D)).astype(np.float16)
    qw = rng.uniform(0.5, 1.5, D).astype(np.float16)
    kw = rng.uniform(0.5, 1.5, D).astype(np.float16)
    freqs = (1.0 / np.power(np.float32(1e6), np.float32(2.0) * np.arange(D // 2, dtype=np.float32) / np.float32(D))
             ).astype(np.float32)
    pos = np.array(positions, np.int32)
    dqkv, dqw, dkw, dfr, dpos, dbt = dev(qkv), dev(qw), dev(kw), dev(freqs), dev(pos), dev(bt)
    dseq = dev(pos + 1)
    sm = 1.0 / np.sqrt(D)

    def run(fused):
        dk, dv = dev(kc), dev(vc)
        out = torch.full((B, N_Q, D), 7.0, dtype=torch.float16, device="cuda")
        xq = torch.full((B, N_Q * D), 99, dtype=torch.int8, device="cuda")
        xs = torch.full((B, N_Q * D // g), -1.0, dtype=torch.float32, device="cuda")
        if fused:
            ctx.qkv_attention_decode(dqkv, dqw, dkw, 1e-6, dfr, dpos, dk, dv, dbt, dseq, out, B, N_Q, D, max_blocks, sm,
                                     layer, LAYERS, N_KV, quant_group_size=g, Xq=xq, Xs=xs, context_splits=splits)
        else:
            dq = torch.empty((B, N_Q, D), dtype=torch.float16, device="cuda")
            ctx.qknorm_rope_kvwrite(dqkv, dqw, dkw, 1e-6, dfr, dpos, dbt, max_blocks, dk, dv, layer, LAYERS, B, N_Q, N_KV,
                                    D, dq)
            ctx.paged_attention_decode(dq, dk, dv, dbt, dseq, out, B, N_Q, D, max_blocks, sm, layer, LAYERS, N_KV,
                                       quant_group_size=g, Xq=xq, Xs=xs, context_splits=splits)
        torch.cuda.synchronize()
        return out, xq, xs, dk, dv

    want, got = run(False), run(True)
    for w, gt, what in zip(want, got, ("attention output", "codes", "scales", "k cache", "v cache")):
        assert torch.equal(w.view(torch.uint8) if w.dtype != torch.int8 else w, gt.view(torch.uint8) if gt.dtype != torch.int8 else gt), what
    assert not torch.equal(got[3], dev(kc)), "the new k rows were written"
