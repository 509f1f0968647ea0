"""Binding of _ref/libfishref.so: the reference's own CUDA kernels, compiled from the
reference checkout where it lies (see Makefile target `ref`). TEST INFRASTRUCTURE.

Needs a GPU to run. Arguments are device pointers (ints) in the reference's own order.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "_ref" / "libfishref.so"
_lib = None


def available() -> bool:
    return LIB_PATH.exists()


def reference_root_default() -> str | None:
    """The reference checkout: $FISH_REFERENCE_ROOT, else a directory named `reference` beside this repository."""
    cand = os.environ.get("FISH_REFERENCE_ROOT") or str(HERE.parent.parent / "reference")
    return cand if Path(cand, "src/kernels/int8_gemm.cu").exists() else None


def build(reference_root_dir: str | None = None) -> Path | None:
    """Compiles the harness when the reference checkout is present; otherwise keeps what is there."""
    reference_root = reference_root_dir or reference_root_default()
    if reference_root and Path(reference_root, "src/kernels/int8_gemm.cu").exists():
        subprocess.run(["make", "-C", str(HERE), "ref", f"REF={reference_root}"], check=True, capture_output=True)
    return LIB_PATH if LIB_PATH.exists() else None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not available():
            raise RuntimeError(f"{LIB_PATH} not built (needs the reference checkout at build time)")
        _lib = C.CDLL(str(LIB_PATH))
        P, I = C.c_void_p, C.c_int
        _lib.fishref_last_error.restype = C.c_char_p
        _lib.fishref_int8_dequant_gemm_fp16.argtypes = [P, P, I, P, P, P, P, I, I, I, P]
        _lib.fishref_workspace_ptr.restype = P
        _lib.fishref_workspace_ptr.argtypes = [I]
        _lib.fishref_copy_workspace.argtypes = [I, P, C.c_size_t]
        _lib.fishref_rms_norm.argtypes = [P, P, P, I, I, C.c_float, P]
        _lib.fishref_silu.argtypes = [P, I, P]
        _lib.fishref_mul.argtypes = [P, P, I, P]
        _lib.fishref_residual_add.argtypes = [P, P, I, P]
        _lib.fishref_rope_qk.argtypes = [P, P, P, I, I, I, I, I, I, P]
        _lib.fishref_paged_attention_decode.argtypes = [P, P, P, P, P, P, I, I, I, I, C.c_float, I, I, I, P]
    return _lib


def _check(rc):
    if rc != 0:
        raise RuntimeError("reference kernel failed: " + lib().fishref_last_error().decode())


def int8_dequant_gemm_fp16(W, scale, group_size, act_scale, smooth_inv, X, Y, M_out, N_tok, K, stream=None):
    _check(lib().fishref_int8_dequant_gemm_fp16(W, scale, group_size, act_scale, smooth_inv, X, Y, M_out, N_tok, K,
                                                stream))


def workspace_ptr(which: int) -> int:
    """0 codes [N_tok,K] int8 · 1 scales [N_tok,G] fp32 · 2 last group's int32 sums [N_tok][M_out] · 3 fp32 accum."""
    return lib().fishref_workspace_ptr(which)


def copy_workspace(which: int, dst: int, nbytes: int):
    """Device-to-device copy of workspace `which` (see workspace_ptr) into dst."""
    _check(lib().fishref_copy_workspace(which, dst, nbytes))


def rms_norm(x, w, out, n_tokens, dim, eps, stream=None):
    _check(lib().fishref_rms_norm(x, w, out, n_tokens, dim, eps, stream))


def silu(x, n, stream=None):
    _check(lib().fishref_silu(x, n, stream))


def mul(a, b, n, stream=None):
    _check(lib().fishref_mul(a, b, n, stream))


def residual_add(a, b, n, stream=None):
    _check(lib().fishref_residual_add(a, b, n, stream))


def rope_qk(q, k, freqs, batch, n_q, n_k, seq_len, head_dim, offset, stream=None):
    _check(lib().fishref_rope_qk(q, k, freqs, batch, n_q, n_k, seq_len, head_dim, offset, stream))


def paged_attention_decode(q, k_cache, v_cache, block_table, seq_lens, out, batch, n_heads, head_dim, max_blocks,
                           sm_scale, layer, n_layers, n_kv, stream=None):
    _check(lib().fishref_paged_attention_decode(q, k_cache, v_cache, block_table, seq_lens, out, batch, n_heads,
                                                head_dim, max_blocks, sm_scale, layer, n_layers, n_kv, stream))
