"""Row-partitioned path on CPU ranks (gloo, world size 2 and 3): partition, column blocks, the
exchange schedule and the overlapped gather+SpMM orchestration, checked against the CPU oracle."""
from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import dense, random_csr, to_np, weights
from oracle import oracle as orc

from autosage_b200 import dist as asg_dist


def test_partition_matches_oracle_and_balances():
    crow, _ = random_csr(2000, 15, seed=3, hubs={100: 4000, 1500: 2500})
    for parts in (1, 2, 3, 4, 8):
        bounds = asg_dist.partition_rows(crow, parts)
        np.testing.assert_array_equal(bounds.numpy(), orc.partition_rows(to_np(crow), parts))
        assert bounds.dtype == torch.long and bounds[0] == 0 and bounds[-1] == 2000
    # degenerate: more parts than rows with edges
    crow = torch.tensor([0, 0, 5, 5])
    np.testing.assert_array_equal(asg_dist.partition_rows(crow, 4).numpy(), orc.partition_rows(to_np(crow), 4))


def test_column_blocks_reassemble_the_shard():
    crow, col = random_csr(300, 10, seed=9, hubs={5: 600})
    val = weights(col.numel(), 1)
    bounds = asg_dist.partition_rows(crow, 3)
    x = dense(300, 16, 2)
    exact = orc.spmm(to_np(crow), to_np(col), to_np(val), to_np(x))
    rows = []
    for rank in range(3):
        shard = asg_dist.shard_csr(crow, col, val, rank, 3, bounds)
        assert shard.n_global == 300 and shard.crow[0] == 0 and shard.crow.numel() == shard.n_local + 1
        total = 0
        acc = np.zeros((shard.n_local, 16))
        for block in shard.blocks:
            lo, hi = int(bounds[block.owner]), int(bounds[block.owner + 1])
            assert bool(((block.col >= lo) & (block.col < hi)).all())  # only the owner's columns
            total += block.col.numel()
            acc += orc.spmm(to_np(block.crow), to_np(block.col), to_np(block.val), to_np(x))
        assert total == shard.col.numel()
        rows.append(acc)
    np.testing.assert_allclose(np.concatenate(rows), exact, rtol=1e-12, atol=1e-12)


def test_exchange_schedule_is_a_perfect_matching_every_step():
    for world in (2, 3, 4, 8):
        for step in range(world - 1):
            sends = {r: asg_dist.exchange_schedule(r, world)[step][0] for r in range(world)}
            recvs = {r: asg_dist.exchange_schedule(r, world)[step][1] for r in range(world)}
            assert sorted(sends.values()) == list(range(world))
            for r in range(world):
                assert recvs[sends[r]] == r  # whoever I send to expects me
        for r in range(world):
            assert sorted(src for _, src in asg_dist.exchange_schedule(r, world)) == [k for k in range(world) if k != r]


def test_column_groups_follow_arrival_order():
    assert asg_dist.arrival_order(2, 4) == [2, 3, 0, 1]
    assert asg_dist.column_groups(2, 4) == [[2], [3], [0], [1]]
    assert asg_dist.column_groups(2, 4, 2) == [[2, 3], [0, 1]]
    assert asg_dist.column_groups(0, 8, 3) == [[0, 1, 2], [3, 4, 5], [6, 7]]
    assert asg_dist.column_groups(5, 8, 100) == [[k % 8] for k in range(5, 13)]
    assert asg_dist.column_groups(1, 3, 1) == [[1, 2, 0]]
    # grouped blocks still reassemble the shard and only hold their owners' columns
    crow, col = random_csr(240, 9, seed=4)
    val = weights(col.numel(), 2)
    x = dense(240, 8, 3)
    bounds = asg_dist.partition_rows(crow, 4)
    for groups in (1, 2, 3, 4):
        shard = asg_dist.shard_csr(crow, col, val, 1, 4, bounds, groups=groups)
        assert len(shard.blocks) == groups and shard.groups == asg_dist.column_groups(1, 4, groups)
        acc = np.zeros((shard.n_local, 8))
        for block, members in zip(shard.blocks, shard.groups):
            assert block.owner == members[-1]
            owners = torch.bucketize(block.col, bounds[1:-1], right=True)
            assert set(owners.tolist()) <= set(members)
            acc += orc.spmm(to_np(block.crow), to_np(block.col), to_np(block.val), to_np(x))
        exact = orc.spmm(to_np(shard.crow), to_np(shard.col), to_np(shard.val), to_np(x))
        np.testing.assert_allclose(acc, exact, rtol=1e-12, atol=1e-12)


def test_explicit_group_sizes():
    assert asg_dist.column_groups(2, 8, (1, 3, 3, 1)) == [[2], [3, 4, 5], [6, 7, 0], [1]]
    assert asg_dist.column_groups(0, 4, 2) == [[0, 1], [2, 3]]
    with pytest.raises(ValueError):
        asg_dist.column_groups(0, 8, (4, 3))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, overlap: bool, out_dir: str, groups=None, exchange=None, chunks=2):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        crow, col = random_csr(400, 9, seed=21, hubs={7: 900, 350: 300})
        val = weights(col.numel(), 4)
        x = dense(400, 24, 5)
        bounds = asg_dist.partition_rows(crow, world)
        shard = asg_dist.shard_csr(crow, col, val, rank, world, bounds, groups=groups)
        torch.manual_seed(0)
        layer = asg_dist.ShardedAutoSAGEConv(shard, 24, 8, exchange=exchange, chunks=chunks)
        assert layer.spmm.exchange == (exchange or "nccl")  # CPU ranks default to grouped send/recv
        layer.spmm.x_full.fill_(float("nan"))  # anything not received stays NaN and poisons the result
        with torch.no_grad():
            out = layer(x[shard.row_begin:shard.row_end], overlap=overlap)
            agg = layer.spmm.forward(overlap=overlap)
        torch.save({"out": out, "agg": agg, "begin": shard.row_begin, "end": shard.row_end,
                    "weight": layer.linear.weight.detach(), "bias": layer.linear.bias.detach()},
                   os.path.join(out_dir, f"rank{rank}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,overlap,groups,exchange,chunks", [
    (2, True, None, None, 2), (2, False, None, None, 2), (3, True, None, None, 2), (3, True, 2, None, 2),
    (2, True, None, "allgather", 1), (3, True, None, "allgather", 3)])
def test_sharded_conv_on_gloo_ranks(tmp_path, world, overlap, groups, exchange, chunks):
    mp.spawn(_worker, args=(world, _free_port(), overlap, str(tmp_path), groups, exchange, chunks), nprocs=world, join=True)
    crow, col = random_csr(400, 9, seed=21, hubs={7: 900, 350: 300})
    val = weights(col.numel(), 4)
    x = dense(400, 24, 5)
    exact = orc.spmm(to_np(crow), to_np(col), to_np(val), to_np(x))
    parts = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]
    assert parts[0]["begin"] == 0 and parts[-1]["end"] == 400
    agg = torch.cat([p["agg"] for p in parts]).numpy()
    ok, ratio = orc.within_tolerance(agg, exact, to_np(crow))
    assert ok, ratio
    weight, bias = parts[0]["weight"], parts[0]["bias"]
    for p in parts[1:]:
        assert torch.equal(p["weight"], weight)  # same seed, same layer on every rank
    expected = torch.from_numpy(exact).float() @ weight.t() + bias
    assert torch.allclose(torch.cat([p["out"] for p in parts]), expected, rtol=1e-4, atol=1e-4)


def _attention_worker(rank: int, world: int, port: int, out_dir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        crow, col = random_csr(300, 7, seed=13, hubs={5: 400})
        q, k, v = dense(300, 16, 1), dense(300, 16, 2), dense(300, 16, 3)
        bounds = asg_dist.partition_rows(crow, world)
        shard = asg_dist.shard_csr(crow, col, None, rank, world, bounds)
        mine = slice(shard.row_begin, shard.row_end)
        scores = asg_dist.ShardedSddmm(shard, 16).forward(q[mine], k[mine])
        out = asg_dist.ShardedAttention(shard, 16).forward(q[mine], k[mine], v[mine], scale=0.25)
        torch.save({"scores": scores, "out": out}, os.path.join(out_dir, f"rank{rank}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_sharded_sddmm_and_attention_on_gloo_ranks(tmp_path):
    """Q row-local, K and V gathered like X: the shards' results concatenate to the whole-graph ones."""
    world = 2
    mp.spawn(_attention_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    crow, col = random_csr(300, 7, seed=13, hubs={5: 400})
    q, k, v = dense(300, 16, 1), dense(300, 16, 2), dense(300, 16, 3)
    parts = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]
    exact_scores = orc.sddmm(to_np(crow), to_np(col), to_np(q), to_np(k))
    np.testing.assert_allclose(torch.cat([p["scores"] for p in parts]).numpy(), exact_scores, rtol=1e-4, atol=1e-4)
    exact_out = orc.attention(to_np(crow), to_np(col), to_np(q), to_np(k), to_np(v), 0.25)
    np.testing.assert_allclose(torch.cat([p["out"] for p in parts]).numpy(), exact_out, rtol=1e-4, atol=1e-4)


def _failing_worker(rank: int, world: int, port: int, out_dir: str):
    """Rank 1 leaves between steps (after a completed step, nothing in flight); rank 0 must get an
    error from its next exchange instead of waiting forever."""
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    crow, col = random_csr(120, 6, seed=2)
    x = dense(120, 8, 3)
    bounds = asg_dist.partition_rows(crow, world)
    shard = asg_dist.shard_csr(crow, col, None, rank, world, bounds)
    layer = asg_dist.ShardedAutoSAGEConv(shard, 8, 4)
    with torch.no_grad():
        layer(x[shard.row_begin:shard.row_end])       # one good step on both ranks
    dist.barrier()
    if rank == 1:
        dist.destroy_process_group()
        return                                           # the peer is gone
    outcome = "no error"
    try:
        with torch.no_grad():
            layer(x[shard.row_begin:shard.row_end])
    except Exception as exc:  # noqa: BLE001 - any error is the expected outcome
        outcome = f"error: {type(exc).__name__}"
    with open(os.path.join(out_dir, "rank0.txt"), "w") as handle:
        handle.write(outcome)


@pytest.mark.timeout(180)
def test_a_departed_rank_surfaces_as_an_error_on_the_host(tmp_path):
    mp.spawn(_failing_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "rank0.txt").read_text().startswith("error:")


def test_chunked_layout_places_every_row_once():
    """GatherLayout: positions are a bijection onto distinct buffer rows, own pieces are contiguous and
    chunk c of every owner is one contiguous slice (what one all-gather fills)."""
    bounds = torch.tensor([0, 5, 12, 12, 20])
    for chunks in (1, 2, 3, 7):
        layout = asg_dist.GatherLayout(bounds, chunks)
        rows = torch.arange(20)
        position = layout.position(rows)
        assert position.unique().numel() == 20 and int(position.max()) < layout.rows_total
        span = layout.world * layout.chunk_rows
        assert torch.equal(torch.div(position, span, rounding_mode="floor"), layout.chunk_of(rows))
        for rank in range(4):
            covered = 0
            for first, count, where in layout.local_pieces(rank):
                mine = torch.arange(int(bounds[rank]) + first, int(bounds[rank]) + first + count)
                assert torch.equal(layout.position(mine), torch.arange(where, where + count))
                covered += count
            assert covered == int(bounds[rank + 1] - bounds[rank])
        buffer = torch.arange(layout.rows_total)
        for c in range(layout.chunks):
            whole = layout.chunk_view(buffer, c)
            for rank in range(4):
                own = layout.own_view(buffer, c, rank)
                assert own.numel() == layout.chunk_rows and int(own[0]) == int(whole[rank * layout.chunk_rows])
