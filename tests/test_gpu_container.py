"""Pre-packed sidecar of a ``.bin`` container: images made through the C ABI on the GPU, written in the
container format, read back, and streamed by the decode kernel — against the numpy restatements of the pack and
the oracle's linear."""
import numpy as np
import pytest
import torch

from fish_audio_cpp_b200 import container as ct
from fish_audio_cpp_b200 import synth
from test_gpu_parity import abs_term_sum, assert_close_fp16

pytestmark = pytest.mark.gpu
P0 = "text_model.model.layers.0."


def dev(a):
    return torch.from_numpy(np.array(a, order="C")).cuda()  # a copy: container views are read-only


def make_checkpoint(path, smooth_differs=False):
    rng = np.random.default_rng(11)
    t = {}

    def lin(name, N, K, g, smooth=None):
        t[name] = synth.weights(rng, N, K)
        t[name + "_scale"] = synth.weight_scales(rng, N, K // g)
        if smooth is not None:
            t[name + "_smooth_inv"] = smooth

    smooth = rng.uniform(0.5, 2.0, 512).astype(np.float16)
    other = smooth.copy()
    other[3] = np.float16(4.0)
    t[P0 + "attention_norm.weight"] = np.ones(512, np.float16)
    lin(P0 + "attention.wqkv.weight", 96, 512, 256)
    lin(P0 + "attention.wo.weight", 64, 256, 64)
    lin(P0 + "feed_forward.w1.weight", 40, 512, 256, smooth)
    lin(P0 + "feed_forward.w3.weight", 40, 512, 256, other if smooth_differs else smooth)
    lin(P0 + "feed_forward.w2.weight", 48, 768, 128)
    lin("odd.weight", 16, 320, 64)  # K % 256 != 0: cannot be streamed, stays row-major
    ct.write_container(path, t)
    return t


def test_sidecar_images_equal_the_numpy_pack_and_stream_through_the_decode_kernel(ctx, oracle, pkg, tmp_path):
    src = make_checkpoint(tmp_path / "model.bin")
    c = ct.Container(tmp_path / "model.bin")
    done = ct.write_packed_sidecar(ctx, c, tmp_path / "model.packed.bin")
    assert done == {P0 + "attention.wqkv.weight": (96, 512, 256), P0 + "attention.wo.weight": (64, 256, 64),
                    P0 + "feed_forward.w13.weight": (80, 512, 256), P0 + "feed_forward.w2.weight": (48, 768, 128)}
    side = ct.Container(tmp_path / "model.packed.bin")
    assert not side.has("odd.weight" + ct.PACKED_SUFFIX)

    # every image is the numpy restatement of the pack over the container's tensors
    for name, (rows, K, g) in done.items():
        if name.endswith("w13.weight"):
            W, S = oracle.pack_gate_up(src[P0 + "feed_forward.w1.weight"], src[P0 + "feed_forward.w1.weight_scale"],
                                       src[P0 + "feed_forward.w3.weight"], src[P0 + "feed_forward.w3.weight_scale"])
        else:
            W, S = src[name], src[name + "_scale"]
        image = side.get(name + ct.PACKED_SUFFIX)
        assert image.dtype == np.int8 and image.size == ctx.packed_weight_bytes(rows, K, g)
        assert np.array_equal(image.view(np.uint8), oracle.pack_weight(W, S, g)), name
        assert side.get(name + ct.META_SUFFIX).tolist() == [rows, K, g]

    # a loader maps the image, uploads it and registers it under the row-major pointer: M <= 32 calls stream it
    name, M = P0 + "feed_forward.w2.weight", 5
    lin = c.linear(name)
    X = synth.activations(np.random.default_rng(3), M, lin.K)
    dW, dS, dX = dev(lin.W), dev(lin.scale), dev(X)
    dImg = dev(side.get(name + ct.PACKED_SUFFIX).view(np.uint8))
    ctx.register_packed_weight(dW, dImg, lin.N, lin.K, lin.group_size)
    try:
        dY = torch.empty((M, lin.N), dtype=torch.float16, device="cuda")
        dD = torch.full((M, lin.N, lin.G), -1, dtype=torch.int32, device="cuda")
        ctx.linear(dW, dS, lin.group_size, dX, dY, M, lin.N, lin.K, dump=dD, kernel=pkg.KERNEL_GEMV_PACKED)
        torch.cuda.synchronize()
        ctx.check_device_status()
    finally:
        ctx.register_packed_weight(dW, None)
    Xq, Xs = oracle.quantize(X, lin.group_size)
    P = oracle.group_sums(lin.W, Xq, lin.group_size)
    assert np.array_equal(dD.cpu().numpy(), P)
    # the bar of the path (2 fp16 ulp or 2e-3 relative, with the summation-order slack of the packed kernel)
    assert_close_fp16(oracle, dY.cpu().numpy(), oracle.linear_q(lin.W, lin.scale, Xq, Xs, lin.group_size), "sidecar image",
                      abs_terms=abs_term_sum(P, np.asarray(lin.scale), Xs))


def test_gate_and_up_with_two_smooth_vectors_stay_apart(ctx, tmp_path):
    make_checkpoint(tmp_path / "model.bin", smooth_differs=True)
    done = ct.write_packed_sidecar(ctx, ct.Container(tmp_path / "model.bin"), tmp_path / "model.packed.bin")
    assert P0 + "feed_forward.w13.weight" not in done
    assert done[P0 + "feed_forward.w1.weight"] == (40, 512, 256) and done[P0 + "feed_forward.w3.weight"] == (40, 512, 256)


def test_sampled_rows_lm_head_equals_the_rows_of_the_full_head(ctx, oracle, pkg):
    """The compact LM head (semantic range + end of sequence, gathered and packed at load) against the oracle on
    those rows, and against the same rows of the full head's output."""
    from fish_audio_cpp_b200 import lm_head as lmh

    vocab, K, g, M = 2048, 512, 256, 8
    rng = np.random.default_rng(5)
    W, S = synth.weights(rng, vocab, K), synth.weight_scales(rng, vocab, K // g)
    X = synth.activations(rng, M, K)
    rows = lmh.sampled_rows(1500, 1999, 77)
    dW, dS, dX = dev(W), dev(S), dev(X)
    dWc, dSc = lmh.compact_head(dW, dS, rows)
    n = len(rows)
    img = torch.empty(ctx.packed_weight_bytes(n, K, g), dtype=torch.uint8, device="cuda")
    ctx.pack_weight(dWc, dSc, n, K, g, img)
    ctx.register_packed_weight(dWc, img, n, K, g)
    try:
        dYc = torch.empty((M, n), dtype=torch.float16, device="cuda")
        ctx.linear(dWc, dSc, g, dX, dYc, M, n, K, kernel=pkg.KERNEL_GEMV_PACKED)
        dY = torch.empty((M, vocab), dtype=torch.float16, device="cuda")
        ctx.linear(dW, dS, g, dX, dY, M, vocab, K)
        torch.cuda.synchronize()
        ctx.check_device_status()
    finally:
        ctx.register_packed_weight(dWc, None)
    Xq, Xs = oracle.quantize(X, g)
    Wc, Sc = lmh.compact_head(W, S, rows)
    P = oracle.group_sums(Wc, Xq, g)
    terms = abs_term_sum(P, Sc, Xs)
    assert_close_fp16(oracle, dYc.cpu().numpy(), oracle.linear_q(Wc, Sc, Xq, Xs, g), "compact head", abs_terms=terms)
    assert_close_fp16(oracle, dYc.cpu().numpy(), dY.cpu().numpy()[:, rows], "compact vs full head", abs_terms=terms)
