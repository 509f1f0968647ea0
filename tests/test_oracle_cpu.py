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
