"""The reference's ``.bin`` checkpoint container, and a pre-packed sidecar for the decode kernels.

File layout (``src/model/tensor.h:53-67``, read by ``src/model/loader.cc:110-153``, written by
``tools/quant_utils.py:197-228``): magic ``FISH`` (u32 0x46495348), format version 1 (u32), tensor count
(u32), then one 344-byte header per tensor — zero-padded name[256], dtype u32 (0 fp32, 1 fp16, 2 bf16,
3 int8), ndim u32 (<= 8), shape i64[8], data offset u64 (from the start of the file, 256-byte aligned),
data size u64 — zero padding to the next multiple of 256, then the tensor data.

A W8A8 linear is the int8 tensor ``<name>`` plus ``<name>_scale`` (fp16 ``[N]`` or ``[N, G]``), and
optionally ``<name>_smooth_inv`` (fp16 ``[K]``) and ``<name>_act_scale`` (``dual_ar_engine.cc:240-275``);
the group size follows from the scale's shape exactly as ``infer_group_size_from_scale`` does
(``dual_ar_engine.cc:17-24``).

``write_packed_sidecar`` runs the library's pre-pack (``w8a8_pack_gate_up``, ``w8a8_pack_weight``) over every
W8A8 linear of a container and writes the images into a second container of the same format, so that a
loader can map them instead of packing at every start.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np

MAGIC = 0x46495348
FORMAT_VERSION = 1
HEADER_SIZE = 344
ALIGN = 256
DTYPE_FP32, DTYPE_FP16, DTYPE_BF16, DTYPE_INT8 = 0, 1, 2, 3
# bf16 has no numpy type: it is exposed as raw uint16
_NP_OF = {DTYPE_FP32: np.dtype("<f4"), DTYPE_FP16: np.dtype("<f2"), DTYPE_BF16: np.dtype("<u2"), DTYPE_INT8: np.dtype("i1")}
_CODE_OF = {np.dtype("<f4"): DTYPE_FP32, np.dtype("<f2"): DTYPE_FP16, np.dtype("i1"): DTYPE_INT8, np.dtype("u1"): DTYPE_INT8}
_HEADER = struct.Struct("<256sII8qQQ")
assert _HEADER.size == HEADER_SIZE


def align256(x: int) -> int:
    return (x + ALIGN - 1) // ALIGN * ALIGN


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype_val: int
    shape: Tuple[int, ...]
    data_offset: int
    data_size: int


class ContainerError(ValueError):
    """A file that the reference's loader would refuse, or that points outside itself."""


class Container:
    """Read-only view of a ``.bin`` file; tensors are numpy views of one memory map (no copies)."""

    def __init__(self, path):
        self.path = Path(path)
        self._map = np.memmap(self.path, dtype=np.uint8, mode="r")
        size = self._map.shape[0]
        if size < 12:
            raise ContainerError(f"{self.path}: shorter than the 12-byte preamble")
        magic, version, count = struct.unpack("<III", self._map[:12].tobytes())
        if magic != MAGIC:
            raise ContainerError(f"{self.path}: invalid magic 0x{magic:08X}, expected 0x{MAGIC:08X}")
        if version != FORMAT_VERSION:
            raise ContainerError(f"{self.path}: unsupported version {version}")
        if 12 + count * HEADER_SIZE > size:
            raise ContainerError(f"{self.path}: {count} headers do not fit in {size} bytes")
        self.entries: Dict[str, TensorEntry] = {}
        for i in range(count):
            raw = self._map[12 + i * HEADER_SIZE: 12 + (i + 1) * HEADER_SIZE].tobytes()
            name_b, dtype_val, ndim, *rest = _HEADER.unpack(raw)
            shape8, offset, nbytes = rest[:8], rest[8], rest[9]
            name = name_b.split(b"\0", 1)[0].decode("utf-8")
            if dtype_val not in _NP_OF:
                raise ContainerError(f"{name}: unknown dtype {dtype_val}")
            if ndim > 8:
                raise ContainerError(f"{name}: {ndim} dimensions")
            shape = tuple(int(s) for s in shape8[:ndim])
            if any(s < 0 for s in shape):
                raise ContainerError(f"{name}: negative extent in {shape}")
            numel = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if nbytes != numel * _NP_OF[dtype_val].itemsize:
                raise ContainerError(f"{name}: {nbytes} bytes for shape {shape}")
            if offset % ALIGN or offset + nbytes > size:
                raise ContainerError(f"{name}: data at {offset}+{nbytes} is unaligned or outside the file")
            self.entries[name] = TensorEntry(name, dtype_val, shape, offset, nbytes)
        self.data_section_offset = 12 + count * HEADER_SIZE

    def names(self) -> List[str]:
        return list(self.entries)

    def has(self, name: str) -> bool:
        return name in self.entries

    def get(self, name: str) -> np.ndarray:
        e = self.entries.get(name)
        if e is None:
            raise KeyError(f"Tensor not found: {name}")
        return self._map[e.data_offset: e.data_offset + e.data_size].view(_NP_OF[e.dtype_val]).reshape(e.shape)

    # ---- W8A8 conventions of the engine's loader ----
    def is_w8a8(self, weight: str) -> bool:
        e = self.entries.get(weight)
        return e is not None and e.dtype_val == DTYPE_INT8 and self.has(weight + "_scale")

    def group_size(self, weight: str) -> int:
        """K for a per-channel scale, else ceil(K / groups): ``infer_group_size_from_scale``."""
        w, s = self.entries[weight], self.entries[weight + "_scale"]
        K = int(np.prod(w.shape[1:], dtype=np.int64))
        if len(s.shape) <= 1 or s.shape[1] <= 1:
            return K
        return (K + s.shape[1] - 1) // s.shape[1]

    def linear(self, weight: str) -> "W8A8Linear":
        if not self.is_w8a8(weight):
            raise KeyError(f"{weight} is not an int8 tensor with a _scale")
        W = self.get(weight)
        opt = lambda suffix: self.get(weight + suffix) if self.has(weight + suffix) else None
        return W8A8Linear(weight, W.reshape(W.shape[0], -1), self.get(weight + "_scale"), self.group_size(weight),
                          opt("_smooth_inv"), opt("_act_scale"))

    def w8a8_linears(self) -> List[str]:
        return [n for n in self.entries if self.is_w8a8(n)]


@dataclass
class W8A8Linear:
    name: str
    W: np.ndarray                      # int8 [N, K]
    scale: np.ndarray                  # fp16 [N] or [N, G]
    group_size: int
    smooth_inv: Optional[np.ndarray]   # fp16 [K]
    act_scale: Optional[np.ndarray]

    @property
    def N(self) -> int:
        return self.W.shape[0]

    @property
    def K(self) -> int:
        return self.W.shape[1]

    @property
    def G(self) -> int:
        return (self.K + self.group_size - 1) // self.group_size


def write_container(path, tensors: Dict[str, np.ndarray], dtype_vals: Optional[Dict[str, int]] = None) -> None:
    """Writes the layout of ``tools/quant_utils.py:197-228``: headers, padding to 256, each tensor 256-aligned."""
    items = []
    offset = align256(12 + HEADER_SIZE * len(tensors))
    for name, arr in tensors.items():
        arr = np.ascontiguousarray(arr)
        code = (dtype_vals or {}).get(name)
        if code is None:
            if arr.dtype not in _CODE_OF:
                raise ContainerError(f"{name}: dtype {arr.dtype} has no container code")
            code = _CODE_OF[arr.dtype]
        if len(name.encode("utf-8")) > 255:
            raise ContainerError(f"Tensor name too long: {name}")
        if arr.ndim > 8:
            raise ContainerError(f"{name}: {arr.ndim} dimensions")
        items.append((name, code, arr, offset))
        offset = align256(offset + arr.nbytes)
    with open(path, "wb") as f:
        f.write(struct.pack("<III", MAGIC, FORMAT_VERSION, len(items)))
        for name, code, arr, off in items:
            shape8 = list(arr.shape) + [0] * (8 - arr.ndim)
            f.write(_HEADER.pack(name.encode("utf-8"), code, arr.ndim, *shape8, off, arr.nbytes))
        for name, code, arr, off in items:
            f.write(b"\0" * (off - f.tell()))
            f.write(arr.tobytes())


def fused_gate_up_names(c: Container) -> Iterable[Tuple[str, str, str]]:
    """(prefix, w1, w3) of every feed-forward whose gate and up may share one activation quantisation: both
    W8A8 with the same group size, and the same (or no) ``smooth_inv`` — the vector multiplies the activations
    before they are quantised, so two different vectors need two quantisations and the pair stays unfused."""
    for n in c.names():
        if not n.endswith("feed_forward.w1.weight"):
            continue
        w3 = n[: -len("w1.weight")] + "w3.weight"
        if not (c.is_w8a8(n) and c.is_w8a8(w3)) or c.group_size(n) != c.group_size(w3):
            continue
        a, b = c.linear(n), c.linear(w3)
        if a.W.shape != b.W.shape:
            continue
        if (a.smooth_inv is None) != (b.smooth_inv is None):
            continue
        if a.smooth_inv is not None and not np.array_equal(a.smooth_inv.view(np.uint16), b.smooth_inv.view(np.uint16)):
            continue
        yield n[: -len("w1.weight")], n, w3


PACKED_SUFFIX = "_packed"
META_SUFFIX = "_packed_meta"  # fp32 [3]: rows, K, group size of the packed image


def write_packed_sidecar(ctx, c: Container, out_path) -> Dict[str, Tuple[int, int, int]]:
    """Packs every W8A8 linear of ``c`` that the decode kernel can stream and writes the images to ``out_path``.

    ``ctx`` is a library context on the current CUDA device. Gate and up of a feed-forward that may share one
    activation quantisation (``fused_gate_up_names``) are interleaved first (``w8a8_pack_gate_up``) and stored
    as ``<prefix>w13.weight_packed``; every other linear as ``<name>_packed``. Beside each image goes
    ``<...>_packed_meta`` = (rows, K, group size). Shapes the kernel cannot stream (``w8a8_packed_weight_bytes``
    returns 0) are left out: such weights stay row-major. Returns {stored name: (rows, K, group size)}.
    """
    import torch

    def dev(a):
        return torch.from_numpy(np.array(a, order="C")).cuda()  # a copy: container views are read-only

    fused = {}
    for prefix, w1, w3 in fused_gate_up_names(c):
        lin = c.linear(w1)
        # a pair whose interleaved form cannot be streamed is not fused: w1 and w3 are then packed each on its own
        if lin.N % 8 == 0 and ctx.packed_weight_bytes(2 * lin.N, lin.K, lin.group_size) != 0:
            fused[w1] = (prefix, w3)
    second = {w3 for _, w3 in fused.values()}
    out: Dict[str, np.ndarray] = {}
    done: Dict[str, Tuple[int, int, int]] = {}
    for name in c.w8a8_linears():
        if name in second:
            continue
        lin = c.linear(name)
        N, K, g, G = lin.N, lin.K, lin.group_size, lin.G
        if name in fused:
            prefix, w3 = fused[name]
            up = c.linear(w3)
            dW = torch.empty((2 * N, K), dtype=torch.int8, device="cuda")
            dS = torch.empty((2 * N, G), dtype=torch.float16, device="cuda")
            ctx.pack_gate_up(dev(lin.W), dev(lin.scale.reshape(N, G)), dev(up.W), dev(up.scale.reshape(N, G)), N, K, G, dW, dS)
            rows, stored = 2 * N, prefix + "w13.weight"
        else:
            if ctx.packed_weight_bytes(N, K, g) == 0:
                continue
            dW, dS, rows, stored = dev(lin.W), dev(lin.scale), N, name
        image = torch.empty(ctx.packed_weight_bytes(rows, K, g), dtype=torch.uint8, device="cuda")
        ctx.pack_weight(dW, dS, rows, K, g, image)
        torch.cuda.synchronize()
        out[stored + PACKED_SUFFIX] = image.cpu().numpy().view(np.int8)
        out[stored + META_SUFFIX] = np.array([rows, K, g], dtype=np.float32)
        done[stored] = (rows, K, g)
    write_container(out_path, out)
    return done
