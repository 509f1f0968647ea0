"""Generates tests/golden/w8a8_reference_kernels.npz by running the REFERENCE's own CUDA kernels
(oracle/_ref/libfishref.so, built from the reference checkout) on seeded inputs. Run on a GPU box:

    python tests/golden/make_golden.py [OUTPUT.npz]     (default: w8a8_reference_kernels.npz beside this script)

The fixtures hold, per case, the seed and shape (inputs are regenerated from the seed by
fish-audio-cpp_b200/synth.py) and the reference's int8 codes, fp32 activation scales and fp16
outputs. tests/test_golden_cpu.py checks the CPU oracle against them without a GPU.
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import __graft_entry__ as ge  # noqa: E402

ge.package()
from fish_audio_cpp_b200 import synth  # noqa: E402
from oracle import fishref  # noqa: E402

# (seed, M tokens, N rows, K, g): covers the reference's three branches (M == 1, M <= 4, M > 4),
# one group (g = 0), ragged last group, both headline group sizes.
CASES = [(1, 1, 64, 512, 256), (2, 1, 48, 512, 64), (3, 3, 40, 256, 64), (4, 4, 32, 1024, 256), (5, 8, 64, 512, 256),
         (6, 16, 48, 512, 64), (7, 5, 24, 100, 32), (8, 6, 16, 256, 0), (9, 2, 16, 72, 20), (10, 12, 32, 2560, 256)]


def main():
    out = {"cases": np.array(CASES, dtype=np.int64)}
    for (seed, M, N, K, g) in CASES:
        X, W, ws = synth.linear_case(seed, M, N, K, g)
        G = synth.num_groups(K, g)
        dX, dW, dS = (torch.from_numpy(a).cuda() for a in (X, W, ws))
        dY = torch.empty((M, N), dtype=torch.float16, device="cuda")
        fishref.int8_dequant_gemm_fp16(dW.data_ptr(), dS.data_ptr(), g, None, None, dX.data_ptr(), dY.data_ptr(), N,
                                       M, K)
        torch.cuda.synchronize()
        q = torch.empty((M, K), dtype=torch.int8, device="cuda")
        s = torch.empty((M, G), dtype=torch.float32, device="cuda")
        fishref.copy_workspace(0, q.data_ptr(), M * K)
        fishref.copy_workspace(1, s.data_ptr(), M * G * 4)
        out[f"codes_{seed}"] = q.cpu().numpy()
        out[f"scales_{seed}"] = s.cpu().numpy()
        out[f"y_{seed}"] = dY.cpu().numpy().view(np.uint16)
    # RMSNorm and the elementwise kernels on seeded inputs
    rng = np.random.default_rng(77)
    x = rng.standard_normal((6, 2560)).astype(np.float16)
    w = rng.uniform(0.5, 1.5, 2560).astype(np.float16)
    dx, dw = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    do = torch.empty_like(dx)
    fishref.rms_norm(dx.data_ptr(), dw.data_ptr(), do.data_ptr(), 6, 2560, 1e-6)
    a = (rng.standard_normal(4096) * 2).astype(np.float16)
    b = rng.standard_normal(4096).astype(np.float16)
    db = torch.from_numpy(b).cuda()
    outs = {}
    for name, fn in (("silu", lambda t: fishref.silu(t.data_ptr(), 4096)),
                     ("mul", lambda t: fishref.mul(t.data_ptr(), db.data_ptr(), 4096)),
                     ("add", lambda t: fishref.residual_add(t.data_ptr(), db.data_ptr(), 4096))):
        t = torch.from_numpy(a).cuda()
        fn(t)
        torch.cuda.synchronize()
        outs[name] = t.cpu().numpy().view(np.uint16)
    torch.cuda.synchronize()
    out.update(rms_x=x.view(np.uint16), rms_w=w.view(np.uint16), rms_out=do.cpu().numpy().view(np.uint16),
               elt_a=a.view(np.uint16), elt_b=b.view(np.uint16), elt_silu=outs["silu"], elt_mul=outs["mul"],
               elt_add=outs["add"])
    dst = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).resolve().parent / "w8a8_reference_kernels.npz"
    dst.parent.mkdir(parents=True, exist_ok=True)
    np.savez_compressed(dst, **out)
    print("wrote", dst, dst.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
