"""GPU parity at the sizes of the benchmark configurations, against the float64 CPU oracle.

The graphs are the seeded power-law stand-ins the benchmark runs (232,965 rows / ~114.6 M nnz;
169,343 rows / ~2.48 M nnz; 2,449,029 rows / ~123.7 M nnz) with N(0, 1) dense operands.  The oracle is
evaluated row by row, so it is run on a subset of the rows: the 128 longest rows, a seeded sample of
384 rows of the hub class (degree >= the hub threshold of the call) and a seeded sample of 4,000 rows
of the whole graph.  Their edges are cut out of the device CSR, copied to the host and handed to the
oracle together with the full dense operand; the kernel's output rows (or edge scores) for the same
subset must lie within |y - y64| <= 1e-5*|y64| + 1e-5*sqrt(row degree).
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL = 1e-5
ATOL = 1e-5


@pytest.fixture(scope="module")
def asg():
    import autosage_b200

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    assert autosage_b200.load_native(), f"native library failed to load: {autosage_b200.ops.native_load_error()}"
    return autosage_b200


@pytest.fixture(scope="module")
def orc():
    from oracle import oracle

    return oracle


def _graph(name):
    from benchlib import synthetic as syn

    spec = {"c2": syn.REDDIT_LIKE, "c4": syn.ARXIV_LIKE, "c5": syn.PRODUCTS_LIKE}[name]
    crow, col, info = syn.powerlaw_csr(spec, seed=0, device=torch.device("cuda"))
    assert abs(info["nnz"] - spec.target_nnz) <= 0.005 * spec.target_nnz
    return crow, col, info


@pytest.fixture(scope="module")
def reddit_like():
    graph = _graph("c2")
    yield graph
    del graph
    torch.cuda.empty_cache()


@pytest.fixture(scope="module")
def arxiv_like():
    graph = _graph("c4")
    yield graph
    del graph
    torch.cuda.empty_cache()


@pytest.fixture(scope="module")
def products_like():
    graph = _graph("c5")
    yield graph
    del graph
    torch.cuda.empty_cache()


class RowSubset:
    """Rows picked for the oracle and their edges as a small host CSR (column ids unchanged)."""

    def __init__(self, crow: torch.Tensor, col: torch.Tensor, val, hub_threshold: int, seed: int = 11,
                 longest: int = 128, hubs: int = 384, anywhere: int = 4000) -> None:
        n = crow.numel() - 1
        degree = crow[1:] - crow[:-1]
        gen = torch.Generator().manual_seed(seed)
        picked = [torch.topk(degree, min(longest, n)).indices.cpu()]
        hub_rows = torch.nonzero(degree >= hub_threshold).flatten().cpu()
        if hub_rows.numel():
            picked.append(hub_rows[torch.randperm(hub_rows.numel(), generator=gen)[:hubs]])
        picked.append(torch.randperm(n, generator=gen)[:anywhere])
        rows = torch.unique(torch.cat(picked)).to(crow.device)            # ascending, no duplicates
        starts, counts = crow[rows], degree[rows]
        sub_crow = torch.zeros(rows.numel() + 1, dtype=torch.long, device=crow.device)
        torch.cumsum(counts, 0, out=sub_crow[1:])
        edges = torch.repeat_interleave(starts - sub_crow[:-1], counts) + torch.arange(int(sub_crow[-1]), device=crow.device)
        self.rows = rows
        self.edges = edges                       # positions of the subset's edges in the full col/val
        self.crow = sub_crow.cpu().numpy()
        self.col = col[edges].cpu().numpy()
        self.val = None if val is None else val[edges].cpu().numpy()
        self.n_hub_class = int(hub_rows.numel())

    def check_rows(self, orc, actual_rows: torch.Tensor, exact: np.ndarray, what: str) -> None:
        ok, ratio = orc.within_tolerance(actual_rows.cpu().numpy(), exact, self.crow, rtol=RTOL, atol=ATOL)
        assert ok, f"{what}: outside rtol {RTOL} / atol {ATOL}*sqrt(deg); worst error/bound = {ratio:.3f}"

    def check_edges(self, orc, actual_edges: torch.Tensor, exact: np.ndarray, what: str) -> None:
        ok, ratio = orc.within_tolerance(actual_edges.cpu().numpy(), exact, self.crow, per_edge=True, rtol=RTOL, atol=ATOL)
        assert ok, f"{what}: outside rtol {RTOL} / atol {ATOL}*sqrt(deg); worst error/bound = {ratio:.3f}"


def _dense_pair(n, f, seed):
    """The same N(0, 1) matrix on the host (for the oracle) and on the device."""
    from benchlib import synthetic as syn

    host = syn.dense(n, f, seed)
    return host, host.cuda()


# ------------------------------------------------------------------------- configuration 2: SpMM
@pytest.mark.parametrize("f", [64, 128, 256])
def test_c2_weighted_spmm_against_oracle(asg, orc, reddit_like, f):
    from benchlib import synthetic as syn

    crow, col, info = reddit_like
    val = syn.edge_values(info["nnz"], seed=0, device=crow.device)
    x_host, x = _dense_pair(info["rows"], f, 3)
    subset = RowSubset(crow, col, val, hub_threshold=1024)
    assert subset.n_hub_class > 1000                      # the CTA-per-hub path is exercised
    exact = orc.spmm(subset.crow, subset.col, subset.val, x_host.numpy())
    y = torch.ops.autosage.spmm_csr(crow, col, val, x)    # library defaults (tile 64, 4 warps, hubs from 1024)
    subset.check_rows(orc, y[subset.rows], exact, f"spmm_csr F={f}")
    del y
    y = torch.ops.autosage.spmm_csr_split(crow, col, val, x, 128, 8, 1024)
    subset.check_rows(orc, y[subset.rows], exact, f"spmm_csr_split(128, 8, 1024) F={f}")


def test_c2_scheduler_picks_the_kernels(asg, reddit_like, isolated_cache):
    from benchlib import synthetic as syn

    crow, col, info = reddit_like
    val = syn.edge_values(info["nnz"], seed=0, device=crow.device)
    x = syn.dense(info["rows"], 128, 3, crow.device)
    y, schedule = asg.spmm_csr_auto(crow, col, val, x)
    assert schedule["choice"] == "autosage", schedule
    assert schedule["candidate"] is not None and not schedule["from_cache"]
    again, replayed = asg.spmm_csr_auto(crow, col, val, x)
    assert replayed["from_cache"] and replayed["choice"] == "autosage"
    assert torch.equal(y, again)


# ------------------------------------------------------------------------ configuration 3: SDDMM
@pytest.mark.parametrize("f", [64, 128])
def test_c3_sddmm_against_oracle(asg, orc, reddit_like, f):
    crow, col, info = reddit_like
    q_host, q = _dense_pair(info["rows"], f, 1)
    k_host, k = _dense_pair(info["rows"], f, 2)
    subset = RowSubset(crow, col, None, hub_threshold=8192)
    # the oracle indexes queries by (subset) row and keys by column id: subset of Q, whole K
    exact = orc.sddmm(subset.crow, subset.col, q_host[subset.rows.cpu()].numpy(), k_host.numpy())
    out = torch.ops.autosage.sddmm_csr(crow, col, q, k)
    subset.check_edges(orc, out[subset.edges], exact, f"sddmm_csr F={f}")
    del out
    out = torch.ops.autosage.sddmm_csr_split(crow, col, q, k, 4, 1024)   # with a hub class
    subset.check_edges(orc, out[subset.edges], exact, f"sddmm_csr_split(4, 1024) F={f}")


# -------------------------------------------------------------------- configuration 4: attention
def test_c4_attention_against_oracle(asg, orc, arxiv_like, isolated_cache):
    crow, col, info = arxiv_like
    n, f = info["rows"], 128
    q_host, q = _dense_pair(n, f, 1)
    k_host, k = _dense_pair(n, f, 2)
    v_host, v = _dense_pair(n, f, 3)
    scale = f ** -0.5
    subset = RowSubset(crow, col, None, hub_threshold=512)
    exact = orc.attention(subset.crow, subset.col, q_host[subset.rows.cpu()].numpy(), k_host.numpy(), v_host.numpy(), scale)
    fused, info_f = asg.csr_attention_forward(crow, col, q, k, v, scale=scale, fused=True)
    subset.check_rows(orc, fused[subset.rows], exact, "fused attention")
    unfused, _ = asg.csr_attention_forward(crow, col, q, k, v, scale=scale, fused=False)
    subset.check_rows(orc, unfused[subset.rows], exact, "three-pass attention")
    # scheduled: the fused kernel must win the probe against the three-pass pipeline
    _, scheduled = asg.csr_attention_forward(crow, col, q, k, v, scale=scale)
    assert scheduled["attention"]["choice"] == "autosage", scheduled["attention"]


# ---------------------------------------------------------- configuration 5: SpMM and the layer
@pytest.mark.parametrize("f", [128, 256])
def test_c5_spmm_and_layer_against_oracle(asg, orc, products_like, f):
    from autosage_b200.conv import apply_linear

    crow, col, info = products_like
    n = info["rows"]
    x_host, x = _dense_pair(n, f, 3)
    subset = RowSubset(crow, col, None, hub_threshold=1024)
    assert subset.n_hub_class > 1000
    exact = orc.spmm(subset.crow, subset.col, None, x_host.numpy())
    y = torch.ops.autosage.spmm_csr_split(crow, col, None, x, 128, 4, 1024)   # the benchmark's parameters
    subset.check_rows(orc, y[subset.rows], exact, f"spmm_csr_split(128, 4, 1024) F={f}")
    # the layer's projection on the aggregated rows: Xavier weight, random bias, float64 reference
    torch.manual_seed(0)
    linear = torch.nn.Linear(f, 256).cuda()
    torch.nn.init.xavier_uniform_(linear.weight)
    torch.nn.init.normal_(linear.bias)
    with torch.no_grad():
        out = apply_linear(linear, y)
    w64 = linear.weight.detach().double().cpu().numpy()
    exact_out = exact @ w64.T + linear.bias.detach().double().cpu().numpy()
    # bound: the aggregation's bound carried through the projection (row of |W| sums to at most
    # sqrt(F) * ||w||_2 <= a few), plus the projection's own float32 rounding
    degree = np.maximum(subset.crow[1:] - subset.crow[:-1], 1).astype(np.float64)
    carried = (RTOL * np.abs(exact) + ATOL * np.sqrt(degree)[:, None]) @ np.abs(w64).T
    bound = carried + RTOL * np.abs(exact_out) + ATOL * np.sqrt(f)
    error = np.abs(out[subset.rows].double().cpu().numpy() - exact_out)
    assert bool((error <= bound).all()), f"layer F={f}: worst error/bound = {float((error / bound).max()):.3f}"
    del y, out
    if f == 128:
        # the one-kernel form of the layer (aggregated rows kept on chip) against the same float64 rows
        from autosage_b200 import _native

        fused = torch.empty(n, 256, device=x.device)
        ws = _native.conv_fused(crow, col, None, x, linear.weight.detach(), linear.bias.detach(), fused)
        assert _native.workspace_status(ws) == 0
        error = np.abs(fused[subset.rows].double().cpu().numpy() - exact_out)
        assert bool((error <= bound).all()), f"fused layer: worst error/bound = {float((error / bound).max()):.3f}"
        del fused, ws
    y = torch.ops.autosage.spmm_csr(crow, col, None, x)
    subset.check_rows(orc, y[subset.rows], exact, f"spmm_csr F={f}")


def test_c5_scheduler_picks_the_kernels(asg, products_like, isolated_cache):
    from benchlib import synthetic as syn

    crow, col, info = products_like
    x = syn.dense(info["rows"], 128, 3, crow.device)
    _, schedule = asg.spmm_csr_auto(crow, col, None, x)
    assert schedule["choice"] == "autosage", schedule
