"""ctypes binding of include/w8a8.h. Pointers are plain integers (``tensor.data_ptr()``)."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

ACT_PER_TOKEN_GROUP, ACT_PER_TOKEN = 0, 1
EPI_NONE, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2
KERNEL_AUTO, KERNEL_GENERIC, KERNEL_GEMV, KERNEL_GEMM, KERNEL_GEMV_TMA, KERNEL_GEMV_PACKED = 0, 1, 2, 3, 4, 5
KERNEL_GEMM_SINGLE, KERNEL_GEMM_PAIR = 6, 7

_LIB = None


class W8A8Error(RuntimeError):
    def __init__(self, status: int, where: str, message: str):
        super().__init__(f"{where}: status {status}: {message}")
        self.status = status


class LinearOpts(C.Structure):
    _fields_ = [
        ("act_mode", C.c_int),
        ("epilogue", C.c_int),
        ("residual", C.c_void_p),
        ("dump_group_sums", C.c_void_p),
        ("kernel", C.c_int),
        ("split_k", C.c_int),
    ]


class Tail(C.Structure):
    """w8a8_tail of include/w8a8.h."""
    _fields_ = [("kind", C.c_int), ("x", C.c_void_p), ("norm_weight", C.c_void_p), ("eps", C.c_float),
                ("group_size", C.c_int), ("Xq", C.c_void_p), ("Xs", C.c_void_p), ("normed_out", C.c_void_p)]


TAIL_NONE, TAIL_ROWNORM, TAIL_GROUPQUANT = 0, 1, 2


class DecodeStack(C.Structure):
    """w8a8_decode_stack of include/w8a8.h."""
    _fields_ = [("n_layers", C.c_int), ("batch", C.c_int), ("dim", C.c_int), ("n_q_heads", C.c_int),
                ("n_kv_heads", C.c_int), ("head_dim", C.c_int), ("inter", C.c_int), ("group_size", C.c_int),
                ("eps", C.c_float), ("sm_scale", C.c_float), ("layers", C.c_void_p), ("final_norm", C.c_void_p),
                ("rope_freqs", C.c_void_p), ("positions", C.c_void_p), ("seq_lens", C.c_void_p),
                ("block_table", C.c_void_p), ("max_blocks_per_seq", C.c_int), ("k_cache", C.c_void_p),
                ("v_cache", C.c_void_p), ("x", C.c_void_p), ("out", C.c_void_p)]


DECODE_LAYER_POINTERS = 8  # w8a8_decode_layer: attn_norm, ffn_norm, q_norm, k_norm, packed[4]


def library_path() -> Path:
    """lib/libw8a8.so beside this file; $W8A8_LIBRARY names another build of the same library (diagnostic builds)."""
    import os

    alt = os.environ.get("W8A8_LIBRARY")
    return Path(alt) if alt else Path(__file__).resolve().parent / "lib" / "libw8a8.so"


def load_library() -> C.CDLL:
    """Loads libw8a8.so; raises if it has not been built (there is no fallback path)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not path.exists():
        raise W8A8Error(-1, "load_library", f"{path} is missing: run __graft_entry__.build() first")
    lib = C.CDLL(str(path))
    P, I, L, Z, F = C.c_void_p, C.c_int, C.c_long, C.c_size_t, C.c_float
    sigs = {
        "w8a8_status_string": (C.c_char_p, [I]),
        "w8a8_last_error": (C.c_char_p, []),
        "w8a8_create": (I, [C.POINTER(P), I, Z]),
        "w8a8_destroy": (I, [P]),
        "w8a8_workspace_bytes": (Z, [I, I, I, I]),
        "w8a8_ctx_workspace_bytes": (Z, [P]),
        "w8a8_check_device_status": (I, [P, P]),
        "w8a8_quantize": (I, [P, P, P, P, I, I, I, I, P, P, P]),
        "w8a8_rms_norm": (I, [P, P, P, P, I, I, F, P]),
        "w8a8_rmsnorm_quantize": (I, [P, P, P, P, F, P, P, I, I, I, I, P, P, P, P]),
        "w8a8_silu": (I, [P, P, L, P]),
        "w8a8_mul": (I, [P, P, P, L, P]),
        "w8a8_residual_add": (I, [P, P, P, L, P]),
        "w8a8_linear": (I, [P, P, P, I, P, P, P, P, I, I, I, C.POINTER(LinearOpts), P]),
        "w8a8_linear_q": (I, [P, P, P, I, P, P, P, I, I, I, C.POINTER(LinearOpts), P]),
        "w8a8_rmsnorm_linear": (I, [P, P, P, I, P, P, P, P, F, P, I, I, I, C.POINTER(LinearOpts), P, P, P]),
        "w8a8_linear_q_tail": (I, [P, P, P, I, P, P, P, I, I, I, C.POINTER(LinearOpts), C.POINTER(Tail), P]),
        "w8a8_debug_tail_counters": (I, [P, P, I, P]),
        "w8a8_pack_gate_up": (I, [P, P, P, P, P, I, I, I, P, P, P]),
        "w8a8_decode_stack_workspace_bytes": (Z, [C.POINTER(DecodeStack)]),
        "w8a8_decode_stack_step": (I, [P, C.POINTER(DecodeStack), P]),
        "w8a8_decode_stack_timeline": (I, [P, C.POINTER(DecodeStack), P, I, P]),
        "w8a8_qknorm_rope_kvwrite": (I, [P, P, P, P, F, P, P, P, I, P, P, I, I, I, I, I, I, P, P]),
        "w8a8_paged_attention_decode": (I, [P, P, P, P, P, P, P, I, I, I, I, F, I, I, I, I, P, P, I, P]),
        "w8a8_qkv_attention_decode": (I, [P, P, P, P, F, P, P, P, P, P, P, P, I, I, I, I, F, I, I, I, I, P, P, I, P]),
        "w8a8_tp_create": (I, [P, I, I, I, I, P]),
        "w8a8_tp_connect": (I, [P, P]),
        "w8a8_tp_allreduce_rmsnorm_quantize": (I, [P, P, P, P, F, P, P, I, I, I, I, P, P, P, P]),
        "w8a8_tp_linear_q": (I, [P, P, P, I, P, P, I, I, I, C.POINTER(LinearOpts), P]),
        "w8a8_packed_weight_bytes": (Z, [I, I, I]),
        "w8a8_pack_weight": (I, [P, P, P, I, I, I, P, P]),
        "w8a8_register_packed_weight": (I, [P, P, P, I, I, I]),
        "w8a8_static_scratch_check_status": (I, [P]),
        "w8a8_static_scratch_bytes": (Z, []),
        "w8a8_linear_static_scratch": (I, [P, P, I, P, P, P, P, I, I, I, C.POINTER(LinearOpts), P]),
        "fish_shim_int8_dequant_gemm_fp16": (I, [P, P, I, P, P, P, P, I, I, I, P, C.c_char_p, I]),
        "fish_shim_rms_norm": (I, [P, P, P, I, I, F, P, C.c_char_p, I]),
        "fish_shim_silu_forward": (I, [P, I, P, C.c_char_p, I]),
        "fish_shim_mul_forward": (I, [P, P, I, P, C.c_char_p, I]),
        "fish_shim_residual_add": (I, [P, P, I, P, C.c_char_p, I]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _LIB = lib
    return lib


EXPORTS = [
    "w8a8_status_string", "w8a8_last_error", "w8a8_create", "w8a8_destroy", "w8a8_workspace_bytes",
    "w8a8_ctx_workspace_bytes", "w8a8_check_device_status", "w8a8_quantize", "w8a8_rms_norm",
    "w8a8_rmsnorm_quantize", "w8a8_silu", "w8a8_mul", "w8a8_residual_add", "w8a8_linear", "w8a8_linear_q",
    "w8a8_rmsnorm_linear", "w8a8_linear_q_tail", "w8a8_debug_tail_counters", "w8a8_decode_stack_workspace_bytes", "w8a8_decode_stack_step",
    "w8a8_decode_stack_timeline",
    "w8a8_pack_gate_up", "w8a8_qknorm_rope_kvwrite", "w8a8_paged_attention_decode", "w8a8_qkv_attention_decode", "w8a8_tp_create", "w8a8_tp_connect",
    "w8a8_tp_linear_q", "w8a8_tp_allreduce_rmsnorm_quantize", "w8a8_packed_weight_bytes", "w8a8_pack_weight", "w8a8_register_packed_weight",
    "w8a8_static_scratch_bytes", "w8a8_linear_static_scratch", "w8a8_static_scratch_check_status",
]


def num_groups(K: int, group_size: int) -> int:
    g = K if group_size <= 0 or group_size > K else group_size
    return (K + g - 1) // g


def _ptr(x) -> int | None:
    if x is None:
        return None
    if isinstance(x, int):
        return x
    return x.data_ptr()


def _stream(stream) -> int | None:
    if stream is None:
        import torch

        return torch.cuda.current_stream().cuda_stream or None
    return stream or None


def static_scratch_bytes() -> int:
    return load_library().w8a8_static_scratch_bytes()


def linear_static_scratch(W, w_scale, group_size, X, Y, M, N, K, act_scale=None, smooth_inv=None,
                          act_mode=ACT_PER_TOKEN_GROUP, epilogue=EPI_NONE, residual=None, dump=None,
                          kernel=KERNEL_AUTO, split_k=0, stream=None):
    """w8a8_linear for callers that may not allocate: no context, scratch built into the library
    (one 8 MiB array per GPU, shared by all callers — do not overlap calls)."""
    lib = load_library()
    rc = lib.w8a8_linear_static_scratch(_ptr(W), _ptr(w_scale), group_size, _ptr(act_scale), _ptr(smooth_inv),
                                        _ptr(X), _ptr(Y), M, N, K,
                                        Context._opts(act_mode, epilogue, residual, dump, kernel, split_k),
                                        _stream(stream))
    if rc != 0:
        raise W8A8Error(rc, "w8a8_linear_static_scratch", lib.w8a8_last_error().decode())


def static_scratch_check_status(stream=None):
    """Raises W8A8Error(status 4) if a kernel launched by linear_static_scratch on the current device gave up a
    bounded wait since the last check; synchronises the stream."""
    lib = load_library()
    rc = lib.w8a8_static_scratch_check_status(_stream(stream))
    if rc != 0:
        raise W8A8Error(rc, "w8a8_static_scratch_check_status", lib.w8a8_last_error().decode())


class Context:
    """Owns one w8a8_ctx. Use one per stream."""

    def __init__(self, device: int = 0, workspace_bytes: int = 0):
        self.lib = load_library()
        h = C.c_void_p()
        self._check(self.lib.w8a8_create(C.byref(h), device, workspace_bytes), "w8a8_create")
        self.handle = h
        self.device = device

    def close(self):
        if getattr(self, "handle", None):
            self.lib.w8a8_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, status: int, where: str):
        if status != 0:
            raise W8A8Error(status, where, self.lib.w8a8_last_error().decode())

    @property
    def workspace_bytes(self) -> int:
        return self.lib.w8a8_ctx_workspace_bytes(self.handle)

    def check_device_status(self, stream=None):
        self._check(self.lib.w8a8_check_device_status(self.handle, _stream(stream)), "w8a8_check_device_status")

    def quantize(self, X, M, K, group_size, Xq, Xs, smooth_inv=None, act_scale=None,
                 act_mode=ACT_PER_TOKEN_GROUP, stream=None):
        self._check(self.lib.w8a8_quantize(self.handle, _ptr(X), _ptr(smooth_inv), _ptr(act_scale), M, K,
                                           group_size, act_mode, _ptr(Xq), _ptr(Xs), _stream(stream)),
                    "w8a8_quantize")

    def rms_norm(self, x, weight, out, tokens, dim, eps, stream=None):
        self._check(self.lib.w8a8_rms_norm(self.handle, _ptr(x), _ptr(weight), _ptr(out), tokens, dim, eps,
                                           _stream(stream)), "w8a8_rms_norm")

    def rmsnorm_quantize(self, x, weight, eps, M, K, group_size, Xq, Xs, residual=None, smooth_inv=None,
                         act_scale=None, act_mode=ACT_PER_TOKEN_GROUP, normed_out=None, stream=None):
        self._check(self.lib.w8a8_rmsnorm_quantize(self.handle, _ptr(x), _ptr(residual), _ptr(weight), eps,
                                                   _ptr(smooth_inv), _ptr(act_scale), M, K, group_size, act_mode,
                                                   _ptr(normed_out), _ptr(Xq), _ptr(Xs), _stream(stream)),
                    "w8a8_rmsnorm_quantize")

    def silu(self, a, n, stream=None):
        self._check(self.lib.w8a8_silu(self.handle, _ptr(a), n, _stream(stream)), "w8a8_silu")

    def mul(self, a, b, n, stream=None):
        self._check(self.lib.w8a8_mul(self.handle, _ptr(a), _ptr(b), n, _stream(stream)), "w8a8_mul")

    def residual_add(self, a, b, n, stream=None):
        self._check(self.lib.w8a8_residual_add(self.handle, _ptr(a), _ptr(b), n, _stream(stream)),
                    "w8a8_residual_add")

    @staticmethod
    def _opts(act_mode, epilogue, residual, dump, kernel, split_k):
        if (act_mode, epilogue, residual, dump, kernel, split_k) == (0, 0, None, None, 0, 0):
            return None
        return C.byref(LinearOpts(act_mode, epilogue, _ptr(residual), _ptr(dump), kernel, split_k))

    def linear(self, W, w_scale, group_size, X, Y, M, N, K, act_scale=None, smooth_inv=None,
               act_mode=ACT_PER_TOKEN_GROUP, epilogue=EPI_NONE, residual=None, dump=None, kernel=KERNEL_AUTO,
               split_k=0, stream=None):
        self._check(self.lib.w8a8_linear(self.handle, _ptr(W), _ptr(w_scale), group_size, _ptr(act_scale),
                                         _ptr(smooth_inv), _ptr(X), _ptr(Y), M, N, K,
                                         self._opts(act_mode, epilogue, residual, dump, kernel, split_k),
                                         _stream(stream)), "w8a8_linear")

    def linear_q(self, W, w_scale, group_size, Xq, Xs, Y, M, N, K, epilogue=EPI_NONE, residual=None, dump=None,
                 kernel=KERNEL_AUTO, split_k=0, stream=None):
        self._check(self.lib.w8a8_linear_q(self.handle, _ptr(W), _ptr(w_scale), group_size, _ptr(Xq), _ptr(Xs),
                                           _ptr(Y), M, N, K, self._opts(0, epilogue, residual, dump, kernel, split_k),
                                           _stream(stream)), "w8a8_linear_q")

    def linear_q_tail(self, W, w_scale, group_size, Xq, Xs, Y, M, N, K, tail_kind, tail_group_size, tail_Xq=None,
                      tail_Xs=None, x=None, norm_weight=None, eps=0.0, normed_out=None, epilogue=EPI_NONE, kernel=KERNEL_AUTO,
                      stream=None):
        """w8a8_linear_q followed, in the same launch where the decode kernel takes the shape, by the tail on its
        output: TAIL_ROWNORM (x += Y, RMSNorm, quantiser) or TAIL_GROUPQUANT (the quantiser alone)."""
        tail = Tail(tail_kind, _ptr(x), _ptr(norm_weight), eps, tail_group_size, _ptr(tail_Xq), _ptr(tail_Xs),
                    _ptr(normed_out))
        self._check(self.lib.w8a8_linear_q_tail(self.handle, _ptr(W), _ptr(w_scale), group_size, _ptr(Xq), _ptr(Xs),
                                                _ptr(Y), M, N, K, self._opts(0, epilogue, None, None, kernel, 0),
                                                C.byref(tail), _stream(stream)), "w8a8_linear_q_tail")

    def debug_tail_counters(self, count=256, stream=None):
        buf = (C.c_int * count)()
        self._check(self.lib.w8a8_debug_tail_counters(self.handle, buf, count, _stream(stream)), "w8a8_debug_tail_counters")
        return list(buf)

    def rmsnorm_linear(self, W, w_scale, group_size, x, norm_weight, eps, Y, M, N, K, residual=None, x_out=None,
                       epilogue=EPI_NONE, epi_residual=None, kernel=KERNEL_AUTO, act_mode=ACT_PER_TOKEN_GROUP,
                       codes_out=None, scales_out=None, stream=None):
        self._check(self.lib.w8a8_rmsnorm_linear(self.handle, _ptr(W), _ptr(w_scale), group_size, _ptr(x),
                                                 _ptr(residual), _ptr(x_out), _ptr(norm_weight), eps, _ptr(Y), M, N, K,
                                                 self._opts(act_mode, epilogue, epi_residual, None, kernel, 0),
                                                 _ptr(codes_out), _ptr(scales_out), _stream(stream)),
                    "w8a8_rmsnorm_linear")

    def decode_stack_workspace_bytes(self, desc: DecodeStack) -> int:
        return self.lib.w8a8_decode_stack_workspace_bytes(C.byref(desc))

    def decode_stack_step(self, desc: DecodeStack, stream=None):
        self._check(self.lib.w8a8_decode_stack_step(self.handle, C.byref(desc), _stream(stream)),
                    "w8a8_decode_stack_step")

    def decode_stack_timeline(self, desc: DecodeStack, stream=None):
        """Nanosecond stamps of the last one-launch step: start, then (phase end, barrier end) x 9 per layer, end."""
        n = 18 * desc.n_layers + 2
        buf = (C.c_ulonglong * n)()
        got = self.lib.w8a8_decode_stack_timeline(self.handle, C.byref(desc), buf, n, _stream(stream))
        if got < 0:
            raise W8A8Error(-got, "w8a8_decode_stack_timeline", self.lib.w8a8_last_error().decode())
        return list(buf)[:got]

    def pack_gate_up(self, w_gate, s_gate, w_up, s_up, inter, K, G, W_out, scale_out, stream=None):
        self._check(self.lib.w8a8_pack_gate_up(self.handle, _ptr(w_gate), _ptr(s_gate), _ptr(w_up), _ptr(s_up),
                                               inter, K, G, _ptr(W_out), _ptr(scale_out), _stream(stream)),
                    "w8a8_pack_gate_up")

    def qknorm_rope_kvwrite(self, qkv, q_norm_w, k_norm_w, eps, freqs, positions, block_table, max_blocks, k_cache,
                            v_cache, layer, n_layers, batch, n_q, n_kv, head_dim, q_out, stream=None):
        self._check(self.lib.w8a8_qknorm_rope_kvwrite(self.handle, _ptr(qkv), _ptr(q_norm_w), _ptr(k_norm_w), eps,
                                                      _ptr(freqs), _ptr(positions), _ptr(block_table), max_blocks,
                                                      _ptr(k_cache), _ptr(v_cache), layer, n_layers, batch, n_q, n_kv,
                                                      head_dim, _ptr(q_out), _stream(stream)),
                    "w8a8_qknorm_rope_kvwrite")

    def paged_attention_decode(self, q, k_cache, v_cache, block_table, seq_lens, out, batch, n_heads, head_dim,
                               max_blocks, sm_scale, layer, n_layers, n_kv, quant_group_size=0, Xq=None, Xs=None,
                               context_splits=0, stream=None):
        self._check(self.lib.w8a8_paged_attention_decode(self.handle, _ptr(q), _ptr(k_cache), _ptr(v_cache),
                                                         _ptr(block_table), _ptr(seq_lens), _ptr(out), batch, n_heads,
                                                         head_dim, max_blocks, sm_scale, layer, n_layers, n_kv,
                                                         quant_group_size, _ptr(Xq), _ptr(Xs), context_splits,
                                                         _stream(stream)), "w8a8_paged_attention_decode")

    def qkv_attention_decode(self, qkv, q_norm_w, k_norm_w, eps, freqs, positions, k_cache, v_cache, block_table,
                             seq_lens, out, batch, n_heads, head_dim, max_blocks, sm_scale, layer, n_layers, n_kv,
                             quant_group_size=0, Xq=None, Xs=None, context_splits=0, stream=None):
        self._check(self.lib.w8a8_qkv_attention_decode(self.handle, _ptr(qkv), _ptr(q_norm_w), _ptr(k_norm_w), eps,
                                                       _ptr(freqs), _ptr(positions), _ptr(k_cache), _ptr(v_cache),
                                                       _ptr(block_table), _ptr(seq_lens), _ptr(out), batch, n_heads,
                                                       head_dim, max_blocks, sm_scale, layer, n_layers, n_kv,
                                                       quant_group_size, _ptr(Xq), _ptr(Xs), context_splits,
                                                       _stream(stream)), "w8a8_qkv_attention_decode")

    def tp_create(self, rank, world, max_tokens, dim) -> bytes:
        """Allocates this rank's exchange buffer; returns its 64-byte IPC handle."""
        buf = C.create_string_buffer(64)
        self._check(self.lib.w8a8_tp_create(self.handle, rank, world, max_tokens, dim, buf), "w8a8_tp_create")
        return buf.raw

    def tp_connect(self, all_handles: bytes):
        self._check(self.lib.w8a8_tp_connect(self.handle, all_handles), "w8a8_tp_connect")

    def tp_linear_q(self, W, w_scale, group_size, Xq, Xs, M, N, K, kernel=KERNEL_AUTO, stream=None):
        """The row-parallel linear whose fp32 partial goes straight to every rank's exchange buffer."""
        self._check(self.lib.w8a8_tp_linear_q(self.handle, _ptr(W), _ptr(w_scale), group_size, _ptr(Xq), _ptr(Xs), M, N, K,
                                              self._opts(0, EPI_NONE, None, None, kernel, 0), _stream(stream)),
                    "w8a8_tp_linear_q")

    def tp_allreduce_rmsnorm_quantize(self, x, partial, weight, eps, M, K, group_size, Xq=None, Xs=None,
                                      smooth_inv=None, act_scale=None, act_mode=ACT_PER_TOKEN_GROUP, normed_out=None,
                                      stream=None):
        self._check(self.lib.w8a8_tp_allreduce_rmsnorm_quantize(self.handle, _ptr(x), _ptr(partial), _ptr(weight), eps,
                                                                _ptr(smooth_inv), _ptr(act_scale), M, K, group_size,
                                                                act_mode, _ptr(normed_out), _ptr(Xq), _ptr(Xs),
                                                                _stream(stream)), "w8a8_tp_allreduce_rmsnorm_quantize")

    def packed_weight_bytes(self, N, K, group_size) -> int:
        return self.lib.w8a8_packed_weight_bytes(N, K, group_size)

    def pack_weight(self, W, w_scale, N, K, group_size, packed_out, stream=None):
        self._check(self.lib.w8a8_pack_weight(self.handle, _ptr(W), _ptr(w_scale), N, K, group_size,
                                              _ptr(packed_out), _stream(stream)), "w8a8_pack_weight")

    def register_packed_weight(self, W, packed, N=0, K=0, group_size=0):
        """packed=None removes the entry; otherwise N, K, group_size are the shape the image was packed for."""
        self._check(self.lib.w8a8_register_packed_weight(self.handle, _ptr(W), _ptr(packed), N, K, group_size),
                    "w8a8_register_packed_weight")

    def _shim(self, name, *args, stream=None):
        buf = C.create_string_buffer(512)
        rc = getattr(self.lib, name)(*args, _stream(stream), buf, 512)
        if rc:
            raise RuntimeError(buf.value.decode())

    def shim_rms_norm(self, x, weight, out, n_tokens, dim, eps, stream=None):
        """fish::kernels::rms_norm with the reference's signature (src/kernels/kernels.h:10-19)."""
        self._shim("fish_shim_rms_norm", _ptr(x), _ptr(weight), _ptr(out), n_tokens, dim, eps, stream=stream)

    def shim_silu_forward(self, x, n, stream=None):
        self._shim("fish_shim_silu_forward", _ptr(x), n, stream=stream)

    def shim_mul_forward(self, a, b, n, stream=None):
        self._shim("fish_shim_mul_forward", _ptr(a), _ptr(b), n, stream=stream)

    def shim_residual_add(self, a, b, n, stream=None):
        self._shim("fish_shim_residual_add", _ptr(a), _ptr(b), n, stream=stream)

    def shim_int8_dequant_gemm_fp16(self, W, scale, group_size, act_scale, smooth_inv, X, Y, M_out, N_tok, K,
                                    stream=None):
        """Drives the C++ entry point with the reference's own signature and argument order."""
        buf = C.create_string_buffer(512)
        rc = self.lib.fish_shim_int8_dequant_gemm_fp16(_ptr(W), _ptr(scale), group_size, _ptr(act_scale),
                                                       _ptr(smooth_inv), _ptr(X), _ptr(Y), M_out, N_tok, K,
                                                       _stream(stream), buf, 512)
        if rc:
            raise RuntimeError(buf.value.decode())


# ---- native reader of the reference's .bin container (include/w8a8_container.h; host memory only) ----
class TensorInfo(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dtype", C.c_int), ("ndim", C.c_int), ("shape", C.c_int64 * 8),
                ("offset", C.c_uint64), ("nbytes", C.c_uint64), ("data", C.c_void_p)]


CONTAINER_EXPORTS = ["w8a8_container_open", "w8a8_container_close", "w8a8_container_count",
                     "w8a8_container_data_section_offset", "w8a8_container_tensor", "w8a8_container_find",
                     "w8a8_container_group_size", "w8a8_container_pin"]


def _check(rc, where):
    if rc != 0:
        raise W8A8Error(rc, where, load_library().w8a8_last_error().decode())


class NativeContainer:
    """The library's own reader of a ``.bin`` file (mapped read-only; ``bytes_of`` copies out of the mapping)."""

    def __init__(self, path):
        lib = load_library()
        P, I = C.c_void_p, C.c_int
        lib.w8a8_container_open.restype, lib.w8a8_container_open.argtypes = I, [C.c_char_p, C.POINTER(P)]
        lib.w8a8_container_close.restype, lib.w8a8_container_close.argtypes = I, [P]
        lib.w8a8_container_count.restype, lib.w8a8_container_count.argtypes = I, [P]
        lib.w8a8_container_data_section_offset.restype = C.c_uint64
        lib.w8a8_container_data_section_offset.argtypes = [P]
        lib.w8a8_container_tensor.restype, lib.w8a8_container_tensor.argtypes = I, [P, I, C.POINTER(TensorInfo)]
        lib.w8a8_container_find.restype, lib.w8a8_container_find.argtypes = I, [P, C.c_char_p]
        lib.w8a8_container_group_size.restype = I
        lib.w8a8_container_group_size.argtypes = [P, C.c_char_p, C.POINTER(I)]
        lib.w8a8_container_pin.restype, lib.w8a8_container_pin.argtypes = I, [P]
        self._lib, self._h = lib, P()
        _check(lib.w8a8_container_open(str(path).encode(), C.byref(self._h)), "w8a8_container_open")

    def close(self):
        if self._h:
            self._lib.w8a8_container_close(self._h)
            self._h = C.c_void_p()

    def __len__(self):
        return self._lib.w8a8_container_count(self._h)

    @property
    def data_section_offset(self):
        return self._lib.w8a8_container_data_section_offset(self._h)

    def tensor(self, index):
        info = TensorInfo()
        _check(self._lib.w8a8_container_tensor(self._h, index, C.byref(info)), "w8a8_container_tensor")
        return info

    def find(self, name):
        return self._lib.w8a8_container_find(self._h, name.encode())

    def group_size(self, weight):
        g = C.c_int()
        _check(self._lib.w8a8_container_group_size(self._h, weight.encode(), C.byref(g)), "w8a8_container_group_size")
        return g.value

    def pin(self):
        _check(self._lib.w8a8_container_pin(self._h), "w8a8_container_pin")

    def bytes_of(self, index):
        info = self.tensor(index)
        return C.string_at(info.data, info.nbytes)
