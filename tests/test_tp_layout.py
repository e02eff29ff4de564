"""Tensor-parallel layout: shard arithmetic, and a two-rank gloo run in which every rank computes
its shard with the CPU oracle; column shards must concatenate and row shards must all-reduce to
the single-GPU result."""

import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_shard_bounds_cover_and_balance():
    from bas import tp

    for total, world in [(172, 8), (172, 4), (172, 2), (64, 8), (5, 8), (0, 2)]:
        edges = [tp.shard_bounds(total, world, r) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == total
        for (a0, a1), (b0, b1) in zip(edges, edges[1:]):
            assert a1 == b0
        sizes = [b - a for a, b in edges]
        assert max(sizes) - min(sizes) <= 1
    assert sorted({b - a for a, b in (tp.shard_bounds(172, 8, r) for r in range(8))}) == [21, 22]
    # gate/up column shards line up with down's input-block shards
    for world in (2, 4, 8):
        for r in range(world):
            n0, n1 = tp.column_shard(11008, world, r)
            b0, b1 = tp.row_shard_blocks(11008, world, r)
            assert (n0, n1) == (64 * b0, 64 * b1)
    with pytest.raises(ValueError):
        tp.shard_bounds(8, 2, 2)


def _rank_main(rank: int, world: int, port: int, out_dir: str) -> None:
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "towards-batched-activation-sparsity_b200"))
    import torch
    import torch.distributed as dist

    from bas import tp
    from oracle import bas_oracle as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    b, k, n = 5, 704, 320
    x = O.make_activations(b, k, seed=3)                      # replicated input
    w = O.make_weight(n, k, seed=3)
    ids = O.select_active_blocks(x, 0.4, O.SCORE_NORM)        # replicated mask: same on every rank
    gathered = [None] * world
    dist.all_gather_object(gathered, ids.tolist())
    assert all(g == gathered[0] for g in gathered)
    full = O.masked_gemm(x, w, ids)
    # column-parallel: own output columns
    n0, n1 = tp.column_shard(n, world, rank)
    y_col = O.masked_gemm(x, w[n0:n1], ids)
    parts = [None] * world
    dist.all_gather_object(parts, y_col)
    np.testing.assert_allclose(np.concatenate(parts, axis=1), full, rtol=0, atol=0)
    # row-parallel: own input blocks, partial sums all-reduced
    b0, b1 = tp.row_shard_blocks(k, world, rank)
    local = ids[(ids >= b0) & (ids < b1)] - b0
    y_row = O.masked_gemm(x[:, 64 * b0:64 * b1], w[:, 64 * b0:64 * b1], local)
    t = torch.from_numpy(y_row.astype(np.float64))
    dist.all_reduce(t)
    np.testing.assert_allclose(t.numpy(), full.astype(np.float64), rtol=1e-6, atol=1e-6)
    # selection from a K-SHARDED input (what the list kernel's sharded entries do over the exchange area): every
    # rank scores the blocks it holds, the scores are gathered, every rank ranks ALL of them and keeps its own
    # part - together the ranks hold exactly the unsharded top-k, and the row-parallel sum is the unsharded product
    mine = O.block_scores(x[:, 64 * b0:64 * b1], O.SCORE_NORM)
    assert np.array_equal(mine, O.block_scores(x, O.SCORE_NORM)[b0:b1])        # a block's score needs its own channels only
    shards = [None] * world
    dist.all_gather_object(shards, mine.tolist())
    everyone = np.concatenate([np.asarray(sc, dtype=np.float64) for sc in shards])
    global_ids = O.topk_ids(everyone, len(ids))
    assert np.array_equal(global_ids, ids)
    local2 = global_ids[(global_ids >= b0) & (global_ids < b1)] - b0
    assert np.array_equal(local2, local)
    kept = [None] * world
    dist.all_gather_object(kept, (local2 + b0).tolist())
    assert sorted(j for part in kept for j in part) == ids.tolist()
    Path(out_dir, f"ok{rank}").write_text("ok")
    dist.destroy_process_group()


def test_two_rank_gloo_sharding_matches_single_rank(tmp_path):
    torch = pytest.importorskip("torch")
    import torch.multiprocessing as mp

    port = 29600 + (os.getpid() % 200)
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
