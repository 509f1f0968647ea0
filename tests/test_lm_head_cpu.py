"""Rows of the LM head that the reference's decode sampler reads (sampling.cu:157-229), and the compact table."""
import numpy as np
import pytest

from fish_audio_cpp_b200 import lm_head as lmh


def test_rows_follow_the_sampler_index_rule():
    rows = lmh.sampled_rows()
    size = lmh.SEMANTIC_END_ID - lmh.SEMANTIC_BEGIN_ID + 1
    assert size == 4096 and len(rows) == size + 1
    for i in (0, 1, size - 1, size):  # abs_idx = (i == semantic_size) ? eos_id : semantic_start + i
        assert rows[i] == (lmh.EOS_ID if i == size else lmh.SEMANTIC_BEGIN_ID + i)
    assert len(np.unique(rows)) == len(rows)
    with pytest.raises(ValueError):
        lmh.sampled_rows(10, 9, 0)


def test_compact_head_and_expansion():
    rng = np.random.default_rng(0)
    W = rng.integers(-127, 128, (64, 32), dtype=np.int8)
    S = rng.uniform(1e-3, 5e-3, (64, 2)).astype(np.float16)
    rows = lmh.sampled_rows(40, 47, 3)
    Wc, Sc = lmh.compact_head(W, S, rows)
    assert Wc.shape == (9, 32) and Wc.flags["C_CONTIGUOUS"] and np.array_equal(Wc[8], W[3]) and np.array_equal(Wc[0], W[40])
    assert np.array_equal(Sc.view(np.uint16), S[rows].view(np.uint16))
    logits = rng.standard_normal((2, 9)).astype(np.float16)
    full = lmh.expand_logits(logits, rows, 64)
    assert full.shape == (2, 64) and np.array_equal(full[:, rows], logits)
    assert np.isneginf(np.delete(full, rows, axis=1)).all()


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("vocab", [155776, 4097, 160])
def test_vocab_shards_tile_the_rows_in_whole_row_tiles(world, vocab):
    """Column-parallel LM head: the ranks' row ranges tile [0, vocab) without gap or overlap, every range but the
    last is a whole number of 16-row tiles (what the packed decode stream needs), and they differ by at most one tile
    plus the ragged tail."""
    b = [lmh.vocab_shard(vocab, world, r) for r in range(world)]
    assert b[0][0] == 0 and b[-1][1] == vocab
    assert all(b[i][1] == b[i + 1][0] for i in range(world - 1))
    assert all((hi - lo) % 16 == 0 for lo, hi in b[:-1]) and all(lo % 16 == 0 for lo, _ in b)
    widths = [hi - lo for lo, hi in b]
    assert max(widths) - min(widths) <= 16 + vocab % 16
    with pytest.raises(ValueError):
        lmh.vocab_shard(vocab, world, world)
