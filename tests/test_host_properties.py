"""Property tests (hypothesis) of the host-side integer logic: row partition, column groups and
blocks, the probe's row sample and the COO -> CSR build, each against the CPU oracle or an
independent restatement."""
from __future__ import annotations

import numpy as np
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from helpers import to_np
from oracle import oracle as orc

from autosage_b200 import _auto
from autosage_b200 import dist as asg_dist
from autosage_b200.utils.csr import csr_with_order

FAST = settings(max_examples=40, deadline=None)


@st.composite
def csr_patterns(draw, max_rows=60, max_degree=12):
    rows = draw(st.integers(1, max_rows))
    degrees = draw(st.lists(st.integers(0, max_degree), min_size=rows, max_size=rows))
    seed = draw(st.integers(0, 2 ** 20))
    gen = torch.Generator().manual_seed(seed)
    crow = torch.zeros(rows + 1, dtype=torch.long)
    torch.cumsum(torch.tensor(degrees, dtype=torch.long), 0, out=crow[1:])
    col = torch.randint(0, rows, (int(crow[-1]),), generator=gen)
    return crow, col


@FAST
@given(csr_patterns(), st.integers(1, 9))
def test_partition_is_the_oracles(pattern, parts):
    crow, _ = pattern
    bounds = asg_dist.partition_rows(crow, parts)
    np.testing.assert_array_equal(bounds.numpy(), orc.partition_rows(to_np(crow), parts))
    assert bounds[0] == 0 and bounds[-1] == crow.numel() - 1 and bool((bounds[1:] >= bounds[:-1]).all())


@FAST
@given(st.integers(1, 8), st.data())
def test_column_groups_cover_the_arrival_order(world, data):
    rank = data.draw(st.integers(0, world - 1))
    groups = data.draw(st.one_of(st.none(), st.integers(1, world)))
    got = asg_dist.column_groups(rank, world, groups)
    flat = [owner for group in got for owner in group]
    assert flat == asg_dist.arrival_order(rank, world) and flat[0] == rank
    sizes = [len(g) for g in got]
    assert max(sizes) - min(sizes) <= 1 and all(sizes)
    assert asg_dist.column_groups(rank, world, sizes) == got          # explicit sizes give the same cut


@FAST
@given(csr_patterns(), st.integers(1, 4), st.data())
def test_blocks_partition_every_shard_edge(pattern, world, data):
    crow, col = pattern
    val = torch.arange(col.numel(), dtype=torch.float32)              # edge identity travels with the edge
    bounds = asg_dist.partition_rows(crow, world)
    groups = data.draw(st.one_of(st.none(), st.integers(1, world)))
    for rank in range(world):
        shard = asg_dist.shard_csr(crow, col, val, rank, world, bounds, groups=groups)
        seen = []
        for block, members in zip(shard.blocks, shard.groups):
            owners = torch.bucketize(block.col, bounds[1:-1], right=True) if world > 1 else torch.zeros_like(block.col)
            assert set(owners.tolist()) <= set(members)
            for r in range(shard.n_local):                            # order inside a (row, block) pair is kept
                segment = block.val[block.crow[r]:block.crow[r + 1]]
                assert bool((segment[1:] > segment[:-1]).all())
                lo, hi = shard.crow[r], shard.crow[r + 1]
                assert bool(((segment >= shard.val[lo]) & (segment <= shard.val[hi - 1])).all()) if hi > lo else segment.numel() == 0
            seen.append(block.val)
        together = torch.cat(seen) if seen else torch.zeros(0)
        assert sorted(together.tolist()) == sorted(shard.val.tolist())


@FAST
@given(csr_patterns(), st.floats(0.05, 1.0), st.integers(0, 1000))
def test_row_sample_is_a_row_slice(pattern, fraction, seed):
    crow, col = pattern
    val = torch.rand(col.numel())
    s_crow, s_col, s_val, rows = _auto._row_sample_csr(crow, col, val, fraction=fraction, minimum_rows=2, seed=seed)
    n = crow.numel() - 1
    assert rows.numel() == min(max(int(n * fraction), 2, 1), n)
    assert bool((rows[1:] > rows[:-1]).all()) if rows.numel() > 1 else True
    assert torch.equal(s_crow[1:] - s_crow[:-1], (crow[1:] - crow[:-1])[rows])
    for i, r in enumerate(rows.tolist()):
        assert torch.equal(s_col[s_crow[i]:s_crow[i + 1]], col[crow[r]:crow[r + 1]])
        assert torch.equal(s_val[s_crow[i]:s_crow[i + 1]], val[crow[r]:crow[r + 1]])


@FAST
@given(st.integers(1, 40), st.integers(0, 200), st.sampled_from(["dst", "src"]), st.integers(0, 2 ** 20))
def test_csr_build_matches_the_oracle(nodes, edges, rows_by, seed):
    gen = torch.Generator().manual_seed(seed)
    edge_index = torch.randint(0, nodes, (2, edges), generator=gen)
    weight = torch.rand(edges, generator=gen)
    crow, col, order, permuted = csr_with_order(edge_index, nodes, rows_by=rows_by, want_order=True, edge_weight=weight)
    o_crow, o_col, o_perm = orc.edge_index_to_csr(edge_index.numpy(), nodes, rows_by)
    np.testing.assert_array_equal(crow.numpy(), o_crow)
    np.testing.assert_array_equal(col.numpy(), o_col)
    np.testing.assert_array_equal(order.numpy(), o_perm)
    assert torch.equal(permuted, weight[order])
