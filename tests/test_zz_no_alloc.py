"""w8a8_linear_static_scratch: the context-free entry point for callers that may not allocate
device memory (a plugin inside a host that owns the memory budget, a real-time audio thread).

Its scratch is one 8 MiB array built into the library and shared by every call on a GPU, so the
checks here are: same results as w8a8_linear through the C ABI, on two calls in a row whose shapes
and data differ (the second must not see anything the first left behind), and a clean refusal of a
call that would not fit. This file sorts last on purpose: a run that stops at the first failure has
then already run every other test.
"""
import numpy as np
import pytest
import torch

from fish_audio_cpp_b200 import synth

pytestmark = pytest.mark.gpu

ULP_BAR, REL_BAR = 2, 2e-3  # the bars of tests/test_gpu_parity.py


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def close(oracle, got, want):
    ulp = oracle.ulp_distance_fp16(got, want)
    g32, w32 = got.astype(np.float32), want.astype(np.float32)
    rel = np.abs(g32 - w32) / np.maximum(np.abs(w32), 1e-30)
    return not ((ulp > ULP_BAR) & (rel > REL_BAR)).any()


def test_static_scratch_matches_context_entry_point_twice_in_a_row(ctx, pkg, oracle):
    assert pkg.static_scratch_bytes() == 8 << 20
    # first a call that fills a good part of the array, then a smaller one with other data and
    # another group size, then the first shape again with new data
    for seed, (M, N, K, g) in enumerate([(160, 96, 2560, 64), (8, 256, 512, 256), (160, 96, 2560, 64),
                                         (40, 33, 200, 64)]):
        X, W, ws = synth.linear_case(50 + seed, M, N, K, g)
        dX, dW, dS = dev(X), dev(W), dev(ws)
        want = torch.empty((M, N), dtype=torch.float16, device="cuda")
        ctx.linear(dW, dS, g, dX, want, M, N, K)
        got = torch.full((M, N), 7.0, dtype=torch.float16, device="cuda")
        pkg.linear_static_scratch(dW, dS, g, dX, got, M, N, K)
        torch.cuda.synchronize()
        assert close(oracle, got.cpu().numpy(), want.cpu().numpy()), (M, N, K, g)
        assert close(oracle, got.cpu().numpy(), oracle.linear(W, ws, g, X)), (M, N, K, g)
    # no kernel of these calls gave up a bounded wait (the context-free counterpart of check_device_status)
    pkg.static_scratch_check_status()


def test_static_scratch_epilogue_and_per_token_mode(ctx, pkg, oracle):
    M, N, K, g = 12, 128, 1024, 256
    X, W, ws = synth.linear_case(61, M, N, K, g)
    R = np.random.default_rng(5).standard_normal((M, N)).astype(np.float16)
    dX, dW, dS, dR = dev(X), dev(W), dev(ws), dev(R)
    for kw in ({"epilogue": pkg.EPI_RESIDUAL, "residual": dR}, {"act_mode": pkg.ACT_PER_TOKEN}):
        want = torch.empty((M, N), dtype=torch.float16, device="cuda")
        got = torch.empty((M, N), dtype=torch.float16, device="cuda")
        ctx.linear(dW, dS, g, dX, want, M, N, K, **kw)
        pkg.linear_static_scratch(dW, dS, g, dX, got, M, N, K, **kw)
        torch.cuda.synchronize()
        assert close(oracle, got.cpu().numpy(), want.cpu().numpy()), list(kw)


def test_static_scratch_refuses_what_does_not_fit(pkg):
    M, N, K, g = 4096, 16, 9728, 64  # 38 MiB of codes alone
    Y = torch.full((8,), 3.0, dtype=torch.float16, device="cuda")
    dummy = torch.zeros(16, dtype=torch.int8, device="cuda")
    with pytest.raises(pkg.W8A8Error) as e:
        pkg.linear_static_scratch(dummy, dummy, g, dummy, Y, M, N, K)
    assert e.value.status == 5 and "built-in array holds" in str(e.value)
    torch.cuda.synchronize()
    assert (Y == 3.0).all(), "a refused call must launch nothing"
