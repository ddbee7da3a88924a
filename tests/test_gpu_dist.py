"""Row-partitioned path on real GPUs (needs at least two; skipped otherwise): every exchange mode
must reproduce the single-GPU / oracle result."""
from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import dense, random_csr, to_np, weights

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from autosage_b200 import dist as asg_dist

        crow, col = random_csr(6000, 14, seed=21, hubs={7: 5000, 3500: 1200})
        val = weights(col.numel(), 4)
        x = dense(6000, 128, 5)
        bounds = asg_dist.partition_rows(crow, world)
        results = {}
        for name, kwargs, groups in (("peer_blocks", dict(exchange="peer"), None),
                                     ("peer_blocks_2streams", dict(exchange="peer", copy_streams=2), 1),
                                     ("peer_slabs2", dict(exchange="peer", slabs=2), 1),
                                     ("peer_slabs4", dict(exchange="peer", slabs=4, copy_streams=2), 1),
                                     ("nccl_blocks", dict(exchange="nccl"), None),
                                     ("allgather_1chunk", dict(exchange="allgather", chunks=1), None),
                                     ("allgather_3chunks", dict(exchange="allgather", chunks=3), None),
                                     ("push_2chunks", dict(exchange="push", chunks=2, push_ctas=8), None)):
            shard = asg_dist.shard_csr(crow, col, val, rank, world, bounds, device=device, groups=groups)
            torch.manual_seed(0)
            layer = asg_dist.ShardedAutoSAGEConv(shard, 128, 16, feature_tile=64, warps=4, threshold=1024,
                                                 **kwargs).to(device)
            layer.spmm.x_full.fill_(float("nan"))
            local = x[shard.row_begin:shard.row_end].to(device)
            with torch.no_grad():
                for _ in range(2):                      # twice: buffers and plans are reused
                    out = layer(local)
                agg = layer.spmm.forward()
            results[name] = {"agg": agg.cpu(), "out": out.cpu(), "mode": layer.spmm.exchange,
                             "slabs": layer.spmm.slabs}
            if name == "peer_blocks":
                replay = layer.capture()        # the whole step as one CUDA graph
                if replay is not None:
                    replay()
                    layer.spmm.x_local.mul_(2.0)    # new features in place: the graph reads the same buffers
                    doubled = replay().clone()
                    layer.spmm.x_local.mul_(0.5)
                    results["graph_replay"] = {"agg": agg.cpu(), "out": replay().cpu(), "doubled": doubled.cpu(),
                                               "mode": "graph", "slabs": 0}
            dist.barrier()
        # a graph whose first row holds most of the edges: some rank ends up with no rows at all
        e_crow, e_col = random_csr(40, 2, seed=1, hubs={0: 4000})
        e_x = dense(40, 64, 2)
        e_bounds = asg_dist.partition_rows(e_crow, world)
        e_shard = asg_dist.shard_csr(e_crow, e_col, None, rank, world, e_bounds, device=device)
        torch.manual_seed(0)
        e_layer = asg_dist.ShardedAutoSAGEConv(e_shard, 64, 8).to(device)
        with torch.no_grad():
            e_layer(e_x[e_shard.row_begin:e_shard.row_end].to(device))
            e_agg = e_layer.spmm.forward()
        results["empty_shard"] = {"agg": e_agg.cpu(), "rows": e_shard.n_local}
        dist.barrier()
        # SDDMM and fused attention over the shard: Q row-local, K and V gathered like X
        shard = asg_dist.shard_csr(crow, col, None, rank, world, bounds, device=device)
        mine = slice(shard.row_begin, shard.row_end)
        q, k = dense(6000, 128, 6), dense(6000, 128, 7)
        sddmm = asg_dist.ShardedSddmm(shard, 128)
        attention = asg_dist.ShardedAttention(shard, 128)
        for _ in range(2):
            scores = sddmm.forward(q[mine].to(device), k[mine].to(device))
            attended = attention.forward(q[mine].to(device), k[mine].to(device), x[mine].to(device), scale=128 ** -0.5)
        results["sddmm"] = {"scores": scores.cpu(), "attended": attended.cpu(), "mode": sddmm.keys.exchange}
        dist.barrier()
        torch.save({"results": results, "begin": int(bounds[rank]), "end": int(bounds[rank + 1])},
                   os.path.join(out_dir, f"rank{rank}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_sharded_layer_on_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    from oracle import oracle as orc

    world = min(torch.cuda.device_count(), 4)
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    crow, col = random_csr(6000, 14, seed=21, hubs={7: 5000, 3500: 1200})
    val = weights(col.numel(), 4)
    x = dense(6000, 128, 5)
    exact = orc.spmm(to_np(crow), to_np(col), to_np(val), to_np(x))
    parts = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]
    torch.manual_seed(0)
    linear = torch.nn.Linear(128, 16)       # the layers above draw their weights from the same seed
    expected_out = exact @ linear.weight.detach().double().numpy().T + linear.bias.detach().double().numpy()
    lopsided = [p["results"].pop("empty_shard") for p in parts]
    e_crow, e_col = random_csr(40, 2, seed=1, hubs={0: 4000})
    assert world < 3 or min(p["rows"] for p in lopsided) == 0
    ok, ratio = orc.within_tolerance(torch.cat([p["agg"] for p in lopsided]).numpy(),
                                     orc.spmm(to_np(e_crow), to_np(e_col), None, to_np(dense(40, 64, 2))), to_np(e_crow))
    assert ok, ("empty shard", ratio)
    sharded = [p["results"].pop("sddmm") for p in parts]
    q, k = dense(6000, 128, 6), dense(6000, 128, 7)
    ok, ratio = orc.within_tolerance(torch.cat([p["scores"] for p in sharded]).numpy(),
                                     orc.sddmm(to_np(crow), to_np(col), to_np(q), to_np(k)), to_np(crow), per_edge=True)
    assert ok, ("sddmm", ratio)
    ok, ratio = orc.within_tolerance(torch.cat([p["attended"] for p in sharded]).numpy(),
                                     orc.attention(to_np(crow), to_np(col), to_np(q), to_np(k), to_np(x), 128 ** -0.5),
                                     to_np(crow))
    assert ok, ("attention", ratio)
    for name in parts[0]["results"]:
        agg = torch.cat([p["results"][name]["agg"] for p in parts]).numpy()
        ok, ratio = orc.within_tolerance(agg, exact, to_np(crow))
        assert ok, (name, ratio)
        out = torch.cat([p["results"][name]["out"] for p in parts]).double().numpy()
        scale = np.abs(expected_out).max()
        assert np.abs(out - expected_out).max() <= 2e-5 * scale, name
    if "graph_replay" in parts[0]["results"]:
        bias = linear.bias.detach().double().numpy()
        doubled = torch.cat([p["results"]["graph_replay"]["doubled"] for p in parts]).double().numpy()
        assert np.abs(doubled - (2.0 * (expected_out - bias) + bias)).max() <= 4e-5 * scale
    assert parts[0]["results"]["peer_slabs2"]["slabs"] in (0, 2)   # 0 only if symmetric memory was unavailable
