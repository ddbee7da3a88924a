"""GPU parity of the fused aggregation + Linear kernel (asg_conv_fused) against float64.

Bound per output element: the aggregation's bound (rtol 1e-5, atol 1e-5 * sqrt(row degree)) carried
through the projection, plus the projection's own float32 rounding (rtol 1e-5, atol 1e-5 * sqrt(K)).
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import csr_from_counts, dense, random_csr, to_np, weights

pytestmark = pytest.mark.gpu

RTOL = 1e-5
ATOL = 1e-5


@pytest.fixture(scope="module")
def lib():
    import autosage_b200
    from autosage_b200 import _native

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    assert autosage_b200.load_native(), f"native library failed to load: {autosage_b200.ops.native_load_error()}"
    return _native


@pytest.fixture(scope="module")
def orc():
    from oracle import oracle

    return oracle


def layer_reference(orc, crow, col, val, x, weight, bias):
    """(A x) W^T + b in float64 and the error bound of a float32 implementation."""
    aggregated = orc.spmm(to_np(crow), to_np(col), to_np(val), x.numpy())
    w64 = weight.double().numpy()
    exact = aggregated @ w64.T + (0 if bias is None else bias.double().numpy())
    degree = np.maximum(np.diff(to_np(crow)), 1).astype(np.float64)
    carried = (RTOL * np.abs(aggregated) + ATOL * np.sqrt(degree)[:, None]) @ np.abs(w64).T
    return exact, carried + RTOL * np.abs(exact) + ATOL * np.sqrt(x.size(1))


def run_fused(lib, crow, col, val, x, weight, bias, threshold, guard_rows=3):
    dev = torch.device("cuda")
    n = crow.numel() - 1
    whole = torch.full((n + guard_rows, weight.size(0)), float("nan"), device=dev)
    ws = lib.conv_fused(crow.to(dev), col.to(dev), None if val is None else val.to(dev), x.to(dev), weight.to(dev),
                        None if bias is None else bias.to(dev), whole[:n], hub_threshold=threshold)
    torch.cuda.synchronize()
    if n:
        assert lib.workspace_status(ws) == 0
    assert bool(torch.isnan(whole[n:]).all())   # nothing written past the last row
    return whole[:n]


@pytest.mark.parametrize("rows,mean_degree,k,n,weighted,threshold", [
    (1, 5, 128, 256, False, 64), (127, 9, 128, 256, True, 64), (128, 9, 64, 32, True, 32), (129, 3, 64, 64, False, 64),
    (1000, 20, 128, 256, True, 64), (5000, 12, 128, 96, False, 32), (40001, 10, 64, 128, True, 128),
    (70000, 14, 128, 256, False, 256)])
def test_conv_fused_matches_float64(lib, orc, rows, mean_degree, k, n, weighted, threshold):
    hubs = {r: threshold + 37 * (i + 1) for i, r in enumerate(range(0, rows, max(rows // 9, 1)))}
    hubs.update({r: threshold - 1 for r in range(1, rows, max(rows // 7, 2))})      # just below the threshold
    crow, col = random_csr(rows, mean_degree, seed=rows + k, hubs=hubs)
    val = weights(col.numel(), 5) if weighted else None
    x = dense(rows, k, 6)
    gen = torch.Generator().manual_seed(n + k)
    weight = torch.randn(n, k, generator=gen) / k ** 0.5
    bias = torch.randn(n, generator=gen)
    out = run_fused(lib, crow, col, val, x, weight, bias, threshold)
    exact, bound = layer_reference(orc, crow, col, val, x, weight, bias)
    error = np.abs(out.double().cpu().numpy() - exact)
    assert bool((error <= bound).all()), f"worst error/bound = {float((error / bound).max()):.3f}"


def test_conv_fused_row_patterns(lib, orc):
    """Empty rows, whole groups of hub rows, rows of exactly 32 / 33 / 63 edges, a hub as the last row, no bias."""
    counts = [0, 0, 0, 0, 70, 80, 90, 100, 32, 33, 63, 1, 0, 64, 0, 5] * 17 + [0, 200]
    crow, col = csr_from_counts(counts, len(counts), seed=3)
    x = dense(len(counts), 128, 4)
    gen = torch.Generator().manual_seed(8)
    weight = torch.randn(64, 128, generator=gen) / 128 ** 0.5
    out = run_fused(lib, crow, col, None, x, weight, None, 64)
    exact, bound = layer_reference(orc, crow, col, None, x, weight, None)
    error = np.abs(out.double().cpu().numpy() - exact)
    assert bool((error <= bound).all()), f"worst error/bound = {float((error / bound).max()):.3f}"
    empty = np.diff(to_np(crow)) == 0
    assert bool((out.cpu().numpy()[empty] == 0).all())      # an empty row projects to the (absent) bias exactly


def test_conv_fused_rejects_other_sizes(lib):
    dev = torch.device("cuda")
    assert lib.conv_fused_supported(128, 256) and lib.conv_fused_supported(64, 32)
    assert not lib.conv_fused_supported(256, 256) and not lib.conv_fused_supported(128, 48)
    assert not lib.conv_fused_supported(128, 512)
    crow = torch.tensor([0, 1], device=dev)
    col = torch.tensor([0], device=dev)
    x, weight, out = torch.zeros(1, 256, device=dev), torch.zeros(256, 256, device=dev), torch.zeros(1, 256, device=dev)
    with pytest.raises(RuntimeError, match="64 or 128 input features"):
        lib.conv_fused(crow, col, None, x, weight, None, out)


def test_layer_takes_the_fused_kernel_when_asked(lib, monkeypatch):
    from autosage_b200.conv import AutoSAGEConv

    dev = torch.device("cuda")
    torch.manual_seed(0)
    gen = torch.Generator().manual_seed(1)
    nodes, edges = 20_000, 300_000
    edge_index = torch.randint(0, nodes, (2, edges), generator=gen)
    edge_index[1, :5000] = 7                                    # a hub destination
    edge_index = edge_index.to(dev)
    edge_weight = torch.rand(edges, generator=gen).to(dev)
    x = dense(nodes, 128, 2).to(dev)
    layer = AutoSAGEConv(128, 256, mode="native").to(dev)
    with torch.no_grad():
        plain, info = layer(x, edge_index, edge_weight, return_info=True)
        assert info["choice"] == "native"
        monkeypatch.setenv("AUTOSAGE_CONV_FUSED", "1")
        fused, info = layer(x, edge_index, edge_weight, return_info=True)
    assert info["choice"] == "fused" and info["operation"] == "conv_fused"
    scale = float(plain.abs().max())
    assert float((fused - plain).abs().max()) <= 2e-5 * scale + 2e-4
    # a gradient is wanted: the differentiable two-kernel route runs even with the variable set
    out, info = layer(x.requires_grad_(), edge_index, edge_weight, return_info=True)
    assert info["choice"] == "native"
    out.sum().backward()
    assert x.grad is not None


def test_conv_fused_bounded_wait_gives_up_and_reports(lib, orc):
    """Self-test flag: the MMA thread waits on a barrier nothing arrives on; the wait runs out after
    20 ms, every warp of the CTA leaves through the common exit and the status word says so.  The next
    call on the same workspace is complete and correct."""
    dev = torch.device("cuda")
    rows = 40_000                                            # more tiles than SMs: every CTA owns a second tile
    crow, col = random_csr(rows, 10, seed=11, hubs={5: 300, 20_000: 900})
    x = dense(rows, 128, 12)
    gen = torch.Generator().manual_seed(13)
    weight = torch.randn(256, 128, generator=gen) / 128 ** 0.5
    bias = torch.randn(256, generator=gen)
    args = (crow.to(dev), col.to(dev), None, x.to(dev), weight.to(dev), bias.to(dev))
    out = torch.zeros(rows, 256, device=dev)
    ws = lib.conv_fused(*args, out, extra_flags=lib.FLAG_SELFTEST_STALL)
    torch.cuda.synchronize()
    assert lib.workspace_status(ws) == 3
    ws = lib.conv_fused(*args, out, workspace=ws)
    torch.cuda.synchronize()
    assert lib.workspace_status(ws) == 0
    exact, bound = layer_reference(orc, crow, col, None, x, weight, bias)
    error = np.abs(out.double().cpu().numpy() - exact)
    assert bool((error <= bound).all())
