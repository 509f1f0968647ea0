"""numpy-facing binding of the C oracle (w8a8_oracle.c). TEST INFRASTRUCTURE, NOT PRODUCT.

fp16 arrays are numpy float16; they cross into C as their uint16 bit patterns.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "_build" / "libw8a8_oracle.so"

ACT_PER_TOKEN_GROUP, ACT_PER_TOKEN = 0, 1
PROMOTE_FMA, PROMOTE_MUL_ADD = 0, 1
EPI_NONE, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2

_lib = None


def build() -> Path:
    src = HERE / "w8a8_oracle.c"
    if not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < max(src.stat().st_mtime,
                                                               (HERE / "w8a8_oracle.h").stat().st_mtime):
        subprocess.run(["make", "-C", str(HERE), "oracle"], check=True, capture_output=True)
    return LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(str(LIB_PATH))
        _lib.w8a8o_timed_linear.restype = C.c_double
        _lib.w8a8o_half_to_float.restype = C.c_float
        _lib.w8a8o_half_to_float.argtypes = [C.c_uint16]
        _lib.w8a8o_float_to_half.restype = C.c_uint16
        _lib.w8a8o_float_to_half.argtypes = [C.c_float]
    return _lib


def _p(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def _h(a):
    """float16 array -> contiguous uint16 view."""
    if a is None:
        return None
    a = np.ascontiguousarray(a, dtype=np.float16)
    return a.view(np.uint16)


def num_groups(K: int, g: int) -> int:
    return lib().w8a8o_num_groups(K, g)


def quantize(X, g, smooth_inv=None, act_scale=None, act_mode=ACT_PER_TOKEN_GROUP):
    M, K = X.shape
    G = num_groups(K, g)
    Xq = np.empty((M, K), np.int8)
    Xs = np.empty((M, G), np.float32)
    rc = lib().w8a8o_quantize(_p(_h(X)), _p(_h(smooth_inv)), _p(_h(act_scale)), M, K, g, act_mode, _p(Xq), _p(Xs))
    assert rc == 0
    return Xq, Xs


def group_sums(W, Xq, g):
    N, K = W.shape
    M = Xq.shape[0]
    G = num_groups(K, g)
    P = np.empty((M, N, G), np.int32)
    rc = lib().w8a8o_group_sums(_p(np.ascontiguousarray(W)), _p(np.ascontiguousarray(Xq)), M, N, K, g, _p(P))
    assert rc == 0
    return P


def linear_q(W, ws, Xq, Xs, g, promote=PROMOTE_FMA, want_f32=False, want_f64=False):
    N, K = W.shape
    M = Xq.shape[0]
    Y = np.empty((M, N), np.uint16)
    Yf = np.empty((M, N), np.float32) if want_f32 else None
    Yd = np.empty((M, N), np.float64) if want_f64 else None
    rc = lib().w8a8o_linear_q(_p(np.ascontiguousarray(W)), _p(_h(ws)), _p(np.ascontiguousarray(Xq)),
                              _p(np.ascontiguousarray(Xs, dtype=np.float32)), M, N, K, g, promote, _p(Y), _p(Yf),
                              _p(Yd))
    assert rc == 0
    out = [Y.view(np.float16)]
    if want_f32:
        out.append(Yf)
    if want_f64:
        out.append(Yd)
    return out[0] if len(out) == 1 else tuple(out)


def linear(W, ws, g, X, act_scale=None, smooth_inv=None, act_mode=ACT_PER_TOKEN_GROUP, promote=PROMOTE_FMA,
           epilogue=EPI_NONE, residual=None):
    N, K = W.shape
    M = X.shape[0]
    outN = N // 2 if epilogue == EPI_SWIGLU else N
    Y = np.empty((M, outN), np.uint16)
    rc = lib().w8a8o_linear(_p(np.ascontiguousarray(W)), _p(_h(ws)), g, _p(_h(act_scale)), _p(_h(smooth_inv)),
                            _p(_h(X)), M, N, K, act_mode, promote, epilogue, _p(_h(residual)), _p(Y))
    assert rc == 0, rc
    return Y.view(np.float16)


def rms_norm(x, w, eps):
    T, D = x.shape
    out = np.empty((T, D), np.uint16)
    rc = lib().w8a8o_rms_norm(_p(_h(x)), _p(_h(w)), _p(out), T, D, C.c_float(eps))
    assert rc == 0
    return out.view(np.float16)


def _inplace(fn, a, b=None):
    out = _h(a).copy()
    if b is None:
        rc = fn(_p(out), C.c_long(out.size))
    else:
        rc = fn(_p(out), _p(_h(b)), C.c_long(out.size))
    assert rc == 0
    return out.view(np.float16).reshape(a.shape)


def silu(a):
    return _inplace(lib().w8a8o_silu, a)


def mul(a, b):
    return _inplace(lib().w8a8o_mul, a, b)


def residual_add(a, b):
    return _inplace(lib().w8a8o_residual_add, a, b)


def pack_gate_up(w_gate, s_gate, w_up, s_up):
    """numpy restatement of the block-16 interleave the SwiGLU epilogue expects."""
    inter, K = w_gate.shape
    assert inter % 8 == 0
    G = s_gate.reshape(inter, -1).shape[1]
    W = np.empty((2 * inter, K), np.int8)
    S = np.empty((2 * inter, G), np.float16)
    wg, wu = w_gate.reshape(inter // 8, 8, K), w_up.reshape(inter // 8, 8, K)
    W.reshape(inter // 8, 16, K)[:, :8] = wg
    W.reshape(inter // 8, 16, K)[:, 8:] = wu
    S.reshape(inter // 8, 16, G)[:, :8] = s_gate.reshape(inter // 8, 8, G)
    S.reshape(inter // 8, 16, G)[:, 8:] = s_up.reshape(inter // 8, 8, G)
    return W, (S if G > 1 else S.reshape(-1))


def pack_weight(W, S, g):
    """numpy restatement of the decode-time weight stream (see include/w8a8.h, w8a8_pack_weight):
    blocks of 16 rows x 256 K-bytes, rt-major then K; inside a block [4 chunks of 64 K-bytes]
    [row lane//4 | row lane//4 + 8][32 lanes][16 bytes at K offset chunk*64 + (lane%4)*16], then [16 rows][groups
    per block] fp16 scales. Rows past N are zeros."""
    N, K = W.shape
    g = K if g <= 0 or g > K else g
    assert K % 256 == 0 and K % g == 0 and (g in (64, 128) or g % 256 == 0)
    G = K // g
    S = np.ascontiguousarray(S, dtype=np.float16).reshape(N, G)
    gpb = 1 if g >= 256 else 256 // g
    tiles, kblocks = (N + 15) // 16, K // 256
    Wp = np.zeros((tiles * 16, K), np.int8)
    Wp[:N] = W
    Sp = np.zeros((tiles * 16, G), np.float16)
    Sp[:N] = S
    # [rt][r16][kb][ch][c][16] -> [rt][kb][ch][half][gq][c][16] with r16 = gq + 8*half, lane = gq*4 + c
    w = Wp.reshape(tiles, 2, 8, kblocks, 4, 4, 16)          # rt, half, gq, kb, ch, c, byte
    w = w.transpose(0, 3, 4, 1, 2, 5, 6).reshape(tiles, kblocks, 4096)
    if g >= 256:
        jidx = (np.arange(kblocks) * 256) // g               # group of each block
        s = Sp.reshape(tiles, 16, G)[:, :, jidx]             # rt, row, kb
        s = s.transpose(0, 2, 1).reshape(tiles, kblocks, 16, 1)
    else:
        s = Sp.reshape(tiles, 16, kblocks, gpb).transpose(0, 2, 1, 3)  # rt, kb, row, q
    s = np.ascontiguousarray(s).view(np.uint8).reshape(tiles, kblocks, 32 * gpb)
    return np.concatenate([w.view(np.uint8), s], axis=2).reshape(-1)


def rope_freqs(head_dim=128, base=1e6):
    """fp32 frequencies as the engine builds them on the host (dual_ar_engine.cc:161-167)."""
    i = np.arange(head_dim // 2, dtype=np.float32)
    return (np.float32(1.0) / np.power(np.float32(base), (np.float32(2.0) * i / np.float32(head_dim)))).astype(np.float32)


def qknorm_rope(x, w, eps, freqs, pos):
    """x fp16 [heads, D]: per-head rms_norm (w may be None), then interleaved-pair RoPE at `pos`
    (rms_norm.cu:10-58, rope.cu:36-45), every fp16 rounding of the reference chain kept."""
    h = x
    if w is not None:
        h = rms_norm(np.ascontiguousarray(x), w, eps)
    f = h.astype(np.float32)
    ang = (freqs.astype(np.float32) * np.float32(pos)).astype(np.float32)
    c, s = np.cos(ang.astype(np.float64)).astype(np.float32), np.sin(ang.astype(np.float64)).astype(np.float32)
    x0, x1 = f[:, 0::2], f[:, 1::2]
    out = np.empty_like(f)
    out[:, 0::2] = x0 * c - x1 * s
    out[:, 1::2] = x0 * s + x1 * c
    return out.astype(np.float16)


def paged_attention_decode(q, k_cache, v_cache, block_table, seq_lens, layer, sm_scale):
    """float64 restatement of paged_attention.cu:13-110. q fp16 [B, H, D]; caches fp16
    [blocks, layers, KvH, 16, D]; returns float64 [B, H, D] (callers compare at a tolerance)."""
    B, H, D = q.shape
    KvH = k_cache.shape[2]
    out = np.zeros((B, H, D), np.float64)
    for b in range(B):
        L = int(seq_lens[b])
        if L <= 0:
            continue
        nb = (L + 15) // 16
        phys = block_table[b, :nb]
        for h in range(H):
            kv = (h * KvH) // H
            K = k_cache[phys, layer, kv].reshape(-1, D)[:L].astype(np.float64)
            V = v_cache[phys, layer, kv].reshape(-1, D)[:L].astype(np.float64)
            sc = K @ q[b, h].astype(np.float64) * sm_scale
            p = np.exp(sc - sc.max())
            out[b, h] = (p / p.sum()) @ V
    return out


def host_threads() -> int:
    return lib().w8a8o_host_threads()


def timed_linear(W, ws, g, X, n_rows, threads):
    """Seconds the scalar oracle takes for the first n_rows output rows, on `threads` host threads."""
    N, K = W.shape
    M = X.shape[0]
    Y = np.empty((M, N), np.uint16)
    t = lib().w8a8o_timed_linear(_p(np.ascontiguousarray(W)), _p(_h(ws)), g, _p(_h(X)), M, N, K, n_rows, threads,
                                 _p(Y))
    assert t >= 0
    return t


def ulp_distance_fp16(a, b):
    """Distance in fp16 units-in-the-last-place between two float16 arrays (sign-aware)."""
    def key(x):
        u = np.ascontiguousarray(x, dtype=np.float16).view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return np.abs(key(a) - key(b))
