"""Tensor-parallel sharding of the linear path, checked on CPU with world_size-2 gloo ranks and the
oracle as the arithmetic: column-parallel shards gather to exactly the full result; row-parallel shards
(K cut at quantisation-group boundaries) all-reduce to the full result up to fp32 re-association."""
import socket

import sys
from pathlib import Path

import pytest
import torch.multiprocessing as mp

sys.path.insert(0, str(Path(__file__).resolve().parent))

from fish_audio_cpp_b200 import stack as S

import _tp_worker


def test_shard_bounds():
    assert S.shard_bounds(38, 4) == [0, 10, 20, 29, 38]          # down at g256 over 4 ranks: 10/10/9/9
    assert S.shard_bounds(38, 8) == [0, 5, 10, 15, 20, 25, 30, 34, 38]
    assert S.shard_bounds(152, 8)[-1] == 152 and S.shard_bounds(16, 2) == [0, 8, 16]


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
@pytest.mark.parametrize("group", [256, 64])
def test_shard_plan_of_the_benchmark_stack(tp, group):
    """Every rank's shard of the 36-layer config keeps the shapes the decode kernels take: K of each linear a
    multiple of 256 (packable), whole quantisation groups, four query heads per kv head; the shards tile the
    intermediate channels without gap or overlap."""
    cfg = S.SlowARConfig(group=group)
    edges = []
    for r in range(tp):
        nq, nkv, qkv_n, attn_k, lo, hi = S.shard_plan(cfg, tp, r)
        assert nq == 4 * nkv and nkv >= 1 and qkv_n == (nq + 2 * nkv) * 128 and qkv_n % 16 == 0
        assert attn_k % 256 == 0 and attn_k % group == 0            # K of wo
        assert (hi - lo) % 256 == 0 and (hi - lo) % group == 0      # K of w2, and rows of w1 | w3 (x2, % 16)
        assert cfg.dim % 256 == 0                                   # K of wqkv and w1 | w3
        edges.append((lo, hi))
    assert edges[0][0] == 0 and edges[-1][1] == cfg.inter
    assert all(edges[i][1] == edges[i + 1][0] for i in range(tp - 1))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.timeout(120)
def test_row_and_column_parallel_with_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_tp_worker.worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=100) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    for rank, ok_col, ok_quant, ulp in res:
        assert ok_col, "column-parallel shards must gather to the full result bit for bit"
        assert ok_quant, "per-(token, group) quantisation must not depend on the shard"
        assert ulp <= 1, f"row-parallel all-reduce differs by {ulp} fp16 ulp"


@pytest.mark.timeout(120)
def test_column_parallel_lm_head_with_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_tp_worker.lm_head_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=100) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert sorted(b for _, _, b in res) == [(0, 112), (112, 213)]
    for rank, same, _ in res:
        assert same, f"rank {rank}: gathered logits must equal the whole head bit for bit"


@pytest.mark.timeout(120)
def test_benchmark_ranks_agree_on_the_top_up_step_count():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_tp_worker.top_up_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=100) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    # 0.2 s left on the slower clock, 2 ms per step on the slower rank: 101 steps on both; nobody has time left: none
    assert sorted(res) == [(0, 101, 0), (1, 101, 0)]
