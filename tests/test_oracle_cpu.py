"""The C oracle against an independent numpy restatement and the reference's own known answers.

The reference has no test of the W8A8 path; the known answers it does hold are for RMSNorm
(tests/test_kernels.cu:121-247) and silu / mul / residual_add (tests/test_kernels.cu:354-481).
Those are restated here with the reference's tolerances.
"""
import numpy as np
import pytest

from fish_audio_cpp_b200 import synth  # noqa: F401  (registered by the pkg fixture)


@pytest.fixture(autouse=True)
def _pkg(pkg):
    return pkg


def np_quantize(X, g, smooth=None, static=None, per_token=False):
    M, K = X.shape
    g = K if g <= 0 or g > K else g
    G = (K + g - 1) // g
    v = X.astype(np.float32)
    if smooth is not None:
        v = v * smooth.astype(np.float32)[None, :]
    Xq = np.zeros((M, K), np.int8)
    Xs = np.zeros((M, G), np.float32)
    for j in range(G):
        sl = slice(j * g, min((j + 1) * g, K))
        if static is not None:
            s = np.full(M, np.float32(static[j]), np.float32)
        elif per_token:
            s = np.abs(v).max(axis=1) / np.float32(127.0)
        else:
            s = np.abs(v[:, sl]).max(axis=1) / np.float32(127.0)
        s = np.maximum(s.astype(np.float32), np.float32(1e-8))
        Xs[:, j] = s
        inv = (np.float32(1.0) / s).astype(np.float32)
        r = (v[:, sl] * inv[:, None]).astype(np.float32)
        Xq[:, sl] = np.clip(np.rint(r), -127, 127).astype(np.int8)
    return Xq, Xs


def np_group_sums(W, Xq, g):
    N, K = W.shape
    g = K if g <= 0 or g > K else g
    G = (K + g - 1) // g
    P = np.zeros((Xq.shape[0], N, G), np.int32)
    for j in range(G):
        sl = slice(j * g, min((j + 1) * g, K))
        P[:, :, j] = Xq[:, sl].astype(np.int32) @ W[:, sl].astype(np.int32).T
    return P


CASES = [(1, 8, 64, 64), (3, 24, 256, 64), (5, 16, 320, 128), (2, 7, 100, 32), (4, 9, 72, 0), (16, 32, 512, 256),
         (2, 5, 52, 20)]


@pytest.mark.parametrize("M,N,K,g", CASES)
def test_quantize_matches_numpy(oracle, M, N, K, g):
    X, W, ws = synth.linear_case(11, M, N, K, g)
    Xq, Xs = oracle.quantize(X, g)
    nq, ns = np_quantize(X, g)
    assert np.array_equal(Xq, nq) and np.array_equal(Xs, ns)
    assert Xq.min() >= -127
    Xq2, Xs2 = oracle.quantize(X, g, act_mode=oracle.ACT_PER_TOKEN)
    nq2, ns2 = np_quantize(X, g, per_token=True)
    assert np.array_equal(Xq2, nq2) and np.array_equal(Xs2, ns2)


def test_quantize_smooth_static_and_zero_group(oracle):
    rng = np.random.default_rng(3)
    M, K, g = 3, 192, 64
    X = synth.activations(rng, M, K)
    X[1, 64:128] = 0  # an all-zero group: scale floors at 1e-8, codes are 0
    smooth = rng.uniform(0.25, 4.0, K).astype(np.float16)
    static = np.array([0.05, 1e-9, 0.5], np.float16)  # the middle one is below the floor
    Xq, Xs = oracle.quantize(X, g, smooth_inv=smooth)
    nq, ns = np_quantize(X, g, smooth=smooth)
    assert np.array_equal(Xq, nq) and np.array_equal(Xs, ns)
    assert Xs[1, 1] == np.float32(1e-8) and not Xq[1, 64:128].any()
    Xq, Xs = oracle.quantize(X, g, act_scale=static)
    nq, ns = np_quantize(X, g, static=static.astype(np.float32))
    assert np.array_equal(Xq, nq) and np.array_equal(Xs, ns)
    assert np.abs(Xq).max() == 127  # huge ratios clamp, never wrap


@pytest.mark.parametrize("M,N,K,g", CASES)
def test_group_sums_and_linear(oracle, M, N, K, g):
    X, W, ws = synth.linear_case(5, M, N, K, g)
    Xq, Xs = oracle.quantize(X, g)
    P = oracle.group_sums(W, Xq, g)
    assert np.array_equal(P, np_group_sums(W, Xq, g))
    Y, Yf, Yd = oracle.linear_q(W, ws, Xq, Xs, g, want_f32=True, want_f64=True)
    G = P.shape[2]
    s2 = ws.reshape(N, G).astype(np.float32)
    # fp32, ascending groups, fma: replay with exact arithmetic in float64 per step
    acc = np.zeros((M, N), np.float32)
    for j in range(G):
        t = (P[:, :, j].astype(np.float32) * s2[None, :, j]).astype(np.float32)
        acc = (t.astype(np.float64) * Xs[:, j].astype(np.float64)[:, None] + acc.astype(np.float64)).astype(np.float32)
    assert np.array_equal(acc, Yf)
    assert np.array_equal(Y, acc.astype(np.float16))
    ref64 = (P.astype(np.float64) * s2[None].astype(np.float64) * Xs[:, None, :].astype(np.float64)).sum(-1)
    assert np.allclose(Yd, ref64, rtol=1e-12, atol=1e-12)
    # the two promote orders agree to a couple of fp32 ulp, hence to <= 1 fp16 ulp
    Y2 = oracle.linear_q(W, ws, Xq, Xs, g, promote=oracle.PROMOTE_MUL_ADD)
    assert oracle.ulp_distance_fp16(Y, Y2).max() <= 1
    assert np.array_equal(oracle.linear(W, ws, g, X), Y)


def test_fused_epilogues_equal_the_unfused_chain(oracle):
    M, inter, K, g = 3, 16, 128, 64
    rng = np.random.default_rng(9)
    X = synth.activations(rng, M, K)
    wg, wu = synth.weights(rng, inter, K), synth.weights(rng, inter, K)
    sg, su = synth.weight_scales(rng, inter, 2), synth.weight_scales(rng, inter, 2)
    Wp, Sp = oracle.pack_gate_up(wg, sg, wu, su)
    fused = oracle.linear(Wp, Sp, g, X, epilogue=oracle.EPI_SWIGLU)
    chain = oracle.mul(oracle.silu(oracle.linear(wg, sg, g, X)), oracle.linear(wu, su, g, X))
    assert np.array_equal(fused, chain)
    R = rng.standard_normal((M, inter)).astype(np.float16)
    fused = oracle.linear(wg, sg, g, X, epilogue=oracle.EPI_RESIDUAL, residual=R)
    assert np.array_equal(fused, oracle.residual_add(R, oracle.linear(wg, sg, g, X)))


# ---- known answers held by the reference's own tests ----

def test_rmsnorm_known_answers(oracle):
    # RmsNormBasic: x = 1, w = 1 -> 1 (tol 1e-3)
    out = oracle.rms_norm(np.ones((4, 8), np.float16), np.ones(8, np.float16), 1e-6)
    assert np.abs(out.astype(np.float32) - 1.0).max() < 1e-3
    # RmsNormZeroInput: finite
    out = oracle.rms_norm(np.zeros((2, 4), np.float16), np.ones(4, np.float16), 1e-5)
    assert np.isfinite(out.astype(np.float32)).all()
    # RmsNormScale: x = [1,3,1,3], w = 2 -> x / sqrt(5 + eps) * 2 (tol 1e-2)
    x = np.array([[1, 3, 1, 3]], np.float16)
    out = oracle.rms_norm(x, np.full(4, 2, np.float16), 1e-6).astype(np.float32)
    assert np.abs(out - x.astype(np.float32) / np.sqrt(5 + 1e-6) * 2).max() < 1e-2
    # RmsNormMultiToken: N(0,1) rows, w = 1 -> rms of each output row is 1 (tol 1e-3)
    x = np.random.default_rng(42).standard_normal((3, 16)).astype(np.float16)
    out = oracle.rms_norm(x, np.ones(16, np.float16), 1e-6).astype(np.float32)
    assert np.abs(np.sqrt((out ** 2).mean(axis=1)) - 1.0).max() < 1e-3


def test_elementwise_known_answers(oracle):
    x = np.arange(-8, 8).astype(np.float16)  # SiluBasic, tol 1e-2
    xf = x.astype(np.float32)
    assert np.abs(oracle.silu(x).astype(np.float32) - xf / (1 + np.exp(-xf))).max() < 1e-2
    a = np.array([1, 2, 3, 4, 5, 6, 7, 8], np.float16)  # MulForward
    b = np.array([2, 3, 4, 5, 1, 1, 1, 1], np.float16)
    assert np.array_equal(oracle.mul(a, b).astype(np.float32), a.astype(np.float32) * b.astype(np.float32))
    b = np.array([10, 20, 30, 40, 0, -1, -2, -3], np.float16)  # ResidualAdd
    assert np.array_equal(oracle.residual_add(a, b).astype(np.float32), a.astype(np.float32) + b.astype(np.float32))


def test_empty_inputs(oracle):
    X, W, ws = synth.linear_case(1, 0, 8, 64, 64)
    assert oracle.linear(W, ws, 64, X).shape == (0, 8)
    assert oracle.quantize(X, 64)[0].shape == (0, 64)


# ---------------------------------------------------------------- the oracle's own helpers, pinned by scalar loops
def test_pack_gate_up_is_the_block_16_interleave(oracle):
    """Rows 16 b .. 16 b + 7 of the packed matrix are gate channels 8 b .. 8 b + 7, rows 16 b + 8 .. 16 b + 15 the up
    rows of the same channels; scales travel with their rows (src/engine/dual_ar_engine.cc:640-644 keeps w1 and w3
    apart; the interleave is this library's load-time pack)."""
    rng = np.random.default_rng(3)
    inter, K, G = 24, 64, 2
    wg, wu = rng.integers(-127, 128, (inter, K), dtype=np.int8), rng.integers(-127, 128, (inter, K), dtype=np.int8)
    sg = rng.uniform(1e-3, 5e-3, (inter, G)).astype(np.float16)
    su = rng.uniform(1e-3, 5e-3, (inter, G)).astype(np.float16)
    W, S = oracle.pack_gate_up(wg, sg, wu, su)
    assert W.shape == (2 * inter, K) and S.shape == (2 * inter, G)
    for ch in range(inter):
        b, r = divmod(ch, 8)
        assert np.array_equal(W[16 * b + r], wg[ch]) and np.array_equal(W[16 * b + 8 + r], wu[ch])
        assert np.array_equal(S[16 * b + r].view(np.uint16), sg[ch].view(np.uint16))
        assert np.array_equal(S[16 * b + 8 + r].view(np.uint16), su[ch].view(np.uint16))


@pytest.mark.parametrize("N,K,g", [(32, 512, 256), (24, 256, 64), (16, 768, 128), (40, 512, 0), (16, 1024, 512)])
def test_pack_weight_layout_byte_by_byte(oracle, N, K, g):
    """The decode stream, restated as the plainest possible loop: block (row tile rt, K-block kb) is 4096 code bytes
    [chunk c of 64 K-bytes][row half][lane][16 bytes], where lane = 4 * (row mod 8) + piece and the 16 bytes are K
    offsets 256 kb + 64 c + 16 piece .. + 15 of row 16 rt + (row mod 8) + 8 half, followed by the block's
    [16 rows][groups per block] fp16 scales. Rows past N are zeros."""
    rng = np.random.default_rng(N + K)
    ge = K if g <= 0 or g > K else g
    G = K // ge
    W = rng.integers(-127, 128, (N, K), dtype=np.int8)
    S = rng.uniform(1e-3, 5e-3, (N, G)).astype(np.float16)
    img = oracle.pack_weight(W, S, g)
    gpb = 1 if ge >= 256 else 256 // ge
    tiles, kblocks = (N + 15) // 16, K // 256
    block = 4096 + 32 * gpb
    assert img.dtype == np.uint8 and img.size == tiles * kblocks * block
    Wz = np.zeros((tiles * 16, K), np.int8)
    Wz[:N] = W
    Sz = np.zeros((tiles * 16, G), np.float16)
    Sz[:N] = S
    for rt in range(tiles):
        for kb in range(kblocks):
            b = img[(rt * kblocks + kb) * block:(rt * kblocks + kb + 1) * block]
            for c in range(4):
                for half in range(2):
                    for lane in range(32):
                        row, piece = 16 * rt + lane // 4 + 8 * half, lane % 4
                        k0 = 256 * kb + 64 * c + 16 * piece
                        got = b[((c * 2 + half) * 32 + lane) * 16:((c * 2 + half) * 32 + lane + 1) * 16].view(np.int8)
                        assert np.array_equal(got, Wz[row, k0:k0 + 16]), (rt, kb, c, half, lane)
            sc = b[4096:].view(np.float16).reshape(16, gpb)
            for r in range(16):
                for q in range(gpb):
                    j = (256 * kb) // ge + q if ge < 256 else (256 * kb) // ge
                    assert sc[r, q] == Sz[16 * rt + r, j], (rt, kb, r, q)


def test_rope_is_the_interleaved_pair_rotation(oracle):
    """rope.cu:36-45: pair (2 i, 2 i + 1) of a head is rotated by pos * base^(-2 i / D); position 0 is the identity,
    the rotation keeps every pair's length (to fp16 rounding), and without norm weights nothing else happens."""
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, 128)).astype(np.float16)
    fr = oracle.rope_freqs(128, 1e6)
    assert fr.shape == (64,) and fr[0] == 1.0 and abs(fr[63] - 1e6 ** (-126 / 128)) < 1e-9
    assert np.array_equal(oracle.qknorm_rope(x, None, 1e-6, fr, 0).view(np.uint16), x.view(np.uint16))
    y = oracle.qknorm_rope(x, None, 1e-6, fr, 1025).astype(np.float64)
    for h in range(3):
        for i in range(64):
            a = 1025.0 * float(fr[i])
            x0, x1 = float(x[h, 2 * i]), float(x[h, 2 * i + 1])
            assert abs(y[h, 2 * i] - (x0 * np.cos(a) - x1 * np.sin(a))) <= 2e-3 * max(1.0, abs(x0) + abs(x1))
            assert abs(y[h, 2 * i + 1] - (x0 * np.sin(a) + x1 * np.cos(a))) <= 2e-3 * max(1.0, abs(x0) + abs(x1))


def test_paged_attention_oracle_against_a_scalar_softmax(oracle):
    """paged_attention.cu:13-110 restated twice: the oracle's vectorised form against a scalar loop over the tokens
    of each sequence, on a cache whose blocks are scattered (block table not the identity), two layers, grouped
    query heads, one empty sequence (-> zeros, paged_attention.cu:44-50) and one that ends inside a block."""
    rng = np.random.default_rng(9)
    B, H, KvH, D, layers, nblocks = 3, 4, 2, 8, 2, 7
    q = rng.standard_normal((B, H, D)).astype(np.float16)
    kc = rng.standard_normal((nblocks, layers, KvH, 16, D)).astype(np.float16)
    vc = rng.standard_normal((nblocks, layers, KvH, 16, D)).astype(np.float16)
    table = np.array([[5, 2, 6], [0, 0, 0], [3, 1, 4]], dtype=np.int32)
    lens = np.array([37, 0, 16], dtype=np.int32)
    scale = 1.0 / np.sqrt(D)
    got = oracle.paged_attention_decode(q, kc, vc, table, lens, 1, scale)
    assert got.shape == (B, H, D) and not got[1].any()
    for b in (0, 2):
        for h in range(H):
            kv = h // (H // KvH)
            scores, vals = [], []
            for t in range(int(lens[b])):
                blk, off = table[b, t // 16], t % 16
                scores.append(float(np.dot(kc[blk, 1, kv, off].astype(np.float64), q[b, h].astype(np.float64))) * scale)
                vals.append(vc[blk, 1, kv, off].astype(np.float64))
            m = max(scores)
            w = [np.exp(s - m) for s in scores]
            want = sum(wi * vi for wi, vi in zip(w, vals)) / sum(w)
            assert np.allclose(got[b, h], want, rtol=1e-12, atol=1e-12)


# ---------------------------------------------------------------- size-independent properties (hypothesis)
from hypothesis import given, settings, strategies as st  # noqa: E402


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 5), st.sampled_from([32, 64, 96, 128, 256]), st.integers(1, 4), st.integers(0, 2 ** 31 - 1),
       st.sampled_from([0.0, 1e-9, 1e-3, 1.0, 300.0]))
def test_quantiser_properties(M, g, groups, seed, magnitude):
    """int8_gemm.cu:147-211 for any row: codes stay in [-127, 127] (never -128), the scale is amax / 127 floored at
    1e-8, the reconstruction error of every element is at most half a step (plus fp32 rounding of the product), and a
    ragged last group is scaled by its own elements only."""
    from oracle import oracle
    oracle.build()
    rng = np.random.default_rng(seed)
    K = g * groups - (g // 4 if groups > 1 and seed % 2 else 0)  # sometimes a ragged last group
    X = (rng.standard_normal((M, K)) * magnitude).astype(np.float16)
    Xq, Xs = oracle.quantize(X, g)
    G = oracle.num_groups(K, g)
    assert Xq.shape == (M, K) and Xs.shape == (M, G) and Xq.min(initial=0) >= -127 and Xq.max(initial=0) <= 127
    for j in range(G):
        seg = X[:, j * g:min(K, (j + 1) * g)].astype(np.float32)
        amax = np.abs(seg).max(axis=1)
        want = np.maximum(amax / np.float32(127.0), np.float32(1e-8)).astype(np.float32)
        assert np.array_equal(Xs[:, j], want)
        rec = Xq[:, j * g:min(K, (j + 1) * g)].astype(np.float32) * Xs[:, j:j + 1]
        assert (np.abs(rec - seg) <= 0.5 * Xs[:, j:j + 1] * (1 + 1e-5) + 1e-30).all()


@settings(max_examples=25, deadline=None)
@given(st.integers(1, 4), st.integers(1, 12), st.sampled_from([64, 128, 256]), st.integers(1, 3), st.integers(0, 2 ** 31 - 1),
       st.sampled_from([-3, -1, 1, 4]))
def test_linear_properties(M, N, g, groups, seed, shift):
    """(a) The integer sums of a K range are the sums of its parts: group sums of the two halves of K, side by side,
    are the group sums of the whole. (b) Multiplying every weight scale by a power of two multiplies the fp32 result
    by exactly that power (int8_gemm.cu:213-234 is one multiply and one fma per group; powers of two commute with
    both roundings while nothing overflows or goes subnormal). (c) Rows and tokens are independent: any sub-block of
    the output is the output of the sub-problem."""
    from oracle import oracle
    oracle.build()
    rng = np.random.default_rng(seed)
    K = 2 * g * groups
    W = rng.integers(-127, 128, (N, K), dtype=np.int8)
    ws = rng.uniform(1e-3, 5e-3, (N, K // g)).astype(np.float16)
    X = rng.standard_normal((M, K)).astype(np.float16)
    Xq, Xs = oracle.quantize(X, g)
    P = oracle.group_sums(W, Xq, g)
    h = K // 2
    Pl = oracle.group_sums(np.ascontiguousarray(W[:, :h]), np.ascontiguousarray(Xq[:, :h]), g)
    Pr = oracle.group_sums(np.ascontiguousarray(W[:, h:]), np.ascontiguousarray(Xq[:, h:]), g)
    assert np.array_equal(P, np.concatenate([Pl, Pr], axis=2))
    _, y32 = oracle.linear_q(W, ws, Xq, Xs, g, want_f32=True)
    ws2 = (ws.astype(np.float32) * np.float32(2.0 ** shift)).astype(np.float16)
    assert np.array_equal(ws2.astype(np.float32), ws.astype(np.float32) * np.float32(2.0 ** shift))  # still exact in fp16
    _, z32 = oracle.linear_q(W, ws2, Xq, Xs, g, want_f32=True)
    assert np.array_equal(z32, y32 * np.float32(2.0 ** shift))
    r0, t0 = N // 2, M // 2
    sub = oracle.linear_q(np.ascontiguousarray(W[r0:]), np.ascontiguousarray(ws[r0:]), np.ascontiguousarray(Xq[t0:]),
                          np.ascontiguousarray(Xs[t0:]), g)
    full = oracle.linear_q(W, ws, Xq, Xs, g)
    assert np.array_equal(sub.view(np.uint16), full[t0:, r0:].view(np.uint16))
