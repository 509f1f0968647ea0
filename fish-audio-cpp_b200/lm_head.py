"""The slow AR's LM head restricted to the rows its samplers read.

The reference computes logits for all 155 776 vocabulary rows (``dual_ar_engine.cc:663-665``) and its decode
sampler then reads the semantic range and the end-of-sequence row only (``sampling.cu:157-229``:
``abs_idx = (i == semantic_size) ? eos_id : semantic_start + i``). ``sampled_rows`` lists those rows in that
order; a loader gathers them once (``compact_head``), packs the 4097-row table with ``w8a8_pack_weight`` and runs
the same decode kernel over 10.5 MB instead of 399 MB. The compact logits buffer ``[M, size + 1]`` is then sampled
with ``semantic_start = 0``, ``eos_id = size``, ``total_vocab_size = size + 1``: a different logits-buffer
contract from the reference's, which is why this is a helper for the caller and not the default.
"""
from __future__ import annotations

import numpy as np

# src/model/dual_ar_config.h:33-35
SEMANTIC_BEGIN_ID = 151678
SEMANTIC_END_ID = 155773  # inclusive
EOS_ID = 151645


def sampled_rows(semantic_begin: int = SEMANTIC_BEGIN_ID, semantic_end: int = SEMANTIC_END_ID,
                 eos_id: int = EOS_ID) -> np.ndarray:
    """Vocabulary rows in the order of the compact logits buffer: the semantic range, then end-of-sequence."""
    if semantic_end < semantic_begin:
        raise ValueError(f"empty semantic range [{semantic_begin}, {semantic_end}]")
    return np.concatenate([np.arange(semantic_begin, semantic_end + 1, dtype=np.int64), np.array([eos_id], dtype=np.int64)])


def compact_head(W, w_scale, rows):
    """(W[rows], w_scale[rows]) for numpy arrays or torch tensors (int8 ``[vocab, K]``, fp16 ``[vocab, G]``)."""
    if hasattr(W, "index_select"):  # torch
        import torch

        idx = torch.as_tensor(np.asarray(rows), device=W.device, dtype=torch.long)
        return W.index_select(0, idx).contiguous(), w_scale.index_select(0, idx).contiguous()
    rows = np.asarray(rows)
    return np.ascontiguousarray(W[rows]), np.ascontiguousarray(w_scale[rows])


def expand_logits(compact, rows, vocab: int, fill=-np.inf):
    """The reference-shaped ``[M, vocab]`` buffer from compact logits (for callers that keep the old contract)."""
    out = np.full((compact.shape[0], vocab), fill, dtype=compact.dtype)
    out[:, np.asarray(rows)] = compact
    return out


# ---- column-parallel over the vocabulary (tensor parallelism) ----
# The reference runs on one GPU. Under tensor parallelism the head's rows are independent outputs (each has its own
# weight scales, and the activation codes are the same on every rank), so a rank computes the logits of its own row
# range with the same decode kernel and the ranges are concatenated. Codes, scales and per-group integer sums are
# those of the whole head; the fp16 logits agree with a one-launch head up to fp32 re-association (the decode kernel
# groups the sum along K by how many row tiles a CTA holds, which depends on the number of rows in the launch).

def vocab_shard(vocab: int, world: int, rank: int, unit: int = 16):
    """Row range ``[lo, hi)`` of rank ``rank``: whole units of ``unit`` rows (the packed decode stream's row tile),
    the first ``units % world`` ranks one unit longer; a ragged tail of fewer than ``unit`` rows goes to the last rank."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside a world of {world}")
    units = vocab // unit
    base, extra = divmod(units, world)
    lo = (rank * base + min(rank, extra)) * unit
    hi = ((rank + 1) * base + min(rank + 1, extra)) * unit
    if rank == world - 1:
        hi = vocab
    return lo, hi


def gather_logits(torch, dist, local, vocab: int, world: int, group=None):
    """``[M, vocab]`` logits on every rank from the ranks' ``[M, hi - lo]`` slices: one all-gather of equal-sized
    (padded) pieces — the ranges differ by at most one unit plus the ragged tail — then the padding is cut away."""
    bounds = [vocab_shard(vocab, world, r) for r in range(world)]
    widest = max(hi - lo for lo, hi in bounds)
    M = local.shape[0]
    padded = local
    if local.shape[1] != widest:
        padded = torch.zeros((M, widest), dtype=local.dtype, device=local.device)
        padded[:, : local.shape[1]] = local
    flat = torch.empty((world * M, widest), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, padded.contiguous(), group=group)
    pieces = flat.view(world, M, widest)
    return torch.cat([pieces[r, :, : hi - lo] for r, (lo, hi) in enumerate(bounds)], dim=1)
