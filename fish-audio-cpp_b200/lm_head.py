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
