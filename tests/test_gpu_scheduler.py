"""The scheduler and the layer on a GPU: result dicts, cache replay, calibration, guardrail, and the
operator-level checks of the reference's own CUDA tests (tests/test_cuda.py:32-69)."""
from __future__ import annotations

import json

import numpy as np
import pytest
import torch

from helpers import dense, random_csr, to_np, weights

pytestmark = pytest.mark.gpu

SPMM_KEYS = {"operation", "schema_version", "choice", "candidate", "baseline", "guardrail", "configuration",
             "probe_rows", "probe_nonzeros", "sampling_ms", "probe_ms", "baseline_probe_ms", "autosage_probe_ms",
             "sampled_speedup", "candidates", "from_cache"}


@pytest.fixture(scope="module")
def asg():
    import autosage_b200

    assert torch.cuda.is_available()
    assert autosage_b200.load_native(), autosage_b200.ops.native_load_error()
    return autosage_b200


@pytest.fixture(scope="module")
def orc():
    from oracle import oracle

    return oracle


@pytest.fixture(scope="module")
def graph():
    crow, col = random_csr(20000, 24, seed=3, hubs={5: 9000, 777: 4000, 19999: 2500})
    val = weights(col.numel(), 4)
    x = dense(20000, 128, seed=5)
    return crow, col, val, x


@pytest.mark.parametrize("features", [32, 64, 113, 128, 256])
def test_operator_matches_torch_sparse(asg, features):
    gen = torch.Generator(device="cuda").manual_seed(0)
    counts = torch.randint(0, 25, (256,), generator=gen, device="cuda")
    crow = torch.cat((torch.zeros(1, device="cuda", dtype=torch.long), counts.cumsum(0)))
    col = torch.randint(0, 256, (int(crow[-1].item()),), generator=gen, device="cuda")
    x = torch.randn(256, features, device="cuda")
    values = torch.rand(col.numel(), device="cuda")
    expected = torch.sparse.mm(torch.sparse_csr_tensor(crow, col, values, size=(256, 256)), x)
    actual = torch.ops.autosage.spmm_csr(crow, col, values, x)
    assert torch.allclose(actual, expected, rtol=1e-4, atol=3e-3)
    assert torch.allclose(asg.spmm_csr(crow.int(), col.int(), values, x), expected, rtol=1e-4, atol=3e-3)


def test_split_operator_on_a_hub_graph_and_argument_checks(asg):
    rows = 512
    counts = torch.full((rows,), 8, device="cuda", dtype=torch.long)
    counts[0] = 400
    crow = torch.cat((torch.zeros(1, device="cuda", dtype=torch.long), counts.cumsum(0)))
    col = torch.randint(0, rows, (int(crow[-1].item()),), device="cuda")
    x = torch.randn(rows, 128, device="cuda")
    matrix = torch.sparse_csr_tensor(crow, col, torch.ones(col.numel(), device="cuda"), size=(rows, rows))
    expected = torch.sparse.mm(matrix, x)
    actual = torch.ops.autosage.spmm_csr_split(crow, col, None, x, 128, 8, 128)
    assert torch.allclose(actual, expected, rtol=1e-4, atol=3e-3)
    with pytest.raises(RuntimeError, match="feature_tile must be 64 or 128"):
        torch.ops.autosage.spmm_csr_split(crow, col, None, x, 96, 8, 128)
    with pytest.raises(RuntimeError, match="warps_per_block must be 2, 4, or 8"):
        torch.ops.autosage.spmm_csr_split(crow, col, None, x, 128, 3, 128)
    with pytest.raises(RuntimeError, match="hub_threshold must be positive"):
        torch.ops.autosage.spmm_csr_split(crow, col, None, x, 128, 8, 0)
    with pytest.raises(RuntimeError, match="torch.long"):
        torch.ops.autosage.spmm_csr(crow.int(), col, None, x)
    with pytest.raises(RuntimeError, match="N \\+ 1"):
        torch.ops.autosage.spmm_csr(crow[:-1], col, None, x)
    with pytest.raises(TypeError, match="float32 features only"):
        asg.spmm_csr(crow, col, None, x.double())


def test_sddmm_auto_matches_gather_dot(asg, isolated_cache):
    gen = torch.Generator(device="cuda").manual_seed(1)
    counts = torch.randint(0, 17, (128,), generator=gen, device="cuda")
    crow = torch.cat((torch.zeros(1, device="cuda", dtype=torch.long), counts.cumsum(0)))
    col = torch.randint(0, 128, (int(crow[-1].item()),), generator=gen, device="cuda")
    query, key = torch.randn(128, 64, device="cuda"), torch.randn(128, 64, device="cuda")
    actual, info = asg.sddmm_csr_auto(crow, col, query, key)
    rows = torch.repeat_interleave(torch.arange(128, device="cuda"), crow[1:] - crow[:-1])
    expected = (query[rows] * key[col]).sum(dim=1)
    assert torch.allclose(actual, expected, rtol=1e-4, atol=1e-4)
    assert info["operation"] == "sddmm" and info["choice"] in ("autosage", "baseline")


def test_spmm_auto_probe_then_cache_replay(asg, orc, graph, isolated_cache):
    crow, col, val, x = (t.cuda() for t in graph)
    exact = orc.spmm(to_np(crow), to_np(col), to_np(val), to_np(x))
    out, info = asg.spmm_csr_auto(crow, col, val, x)
    assert set(info) == SPMM_KEYS
    assert info["operation"] == "spmm" and info["schema_version"] == 3 and info["from_cache"] is False
    assert info["probe_rows"] == 20000 and info["guardrail"] == 0.95  # a graph this small is probed whole
    assert info["baseline"] == "torch.sparse.mm(csr)"
    assert 1 <= len(info["candidates"]) <= 7     # the shortlist of 6 plus the library default
    for entry in info["candidates"]:
        tile, warps, threshold = entry["candidate"]
        assert tile in (64, 128) and warps in (2, 4, 8) and threshold >= 1
        assert {"best_ms", "mean_ms", "std_ms", "iterations", "total_ms", "wall_ms"} <= set(entry)
    if info["choice"] == "autosage":
        assert info["candidate"] in [e["candidate"] for e in info["candidates"]]
        assert info["autosage_probe_ms"] <= 0.95 * info["baseline_probe_ms"]
    else:
        assert info["candidate"] is None
    ok, ratio = orc.within_tolerance(out.cpu().numpy(), exact, to_np(crow)) if info["choice"] == "autosage" else (
        torch.allclose(out.cpu(), torch.from_numpy(exact).float(), rtol=1e-4, atol=1e-3), 0.0)
    assert ok, ratio
    # the schedule is on disk in the reference's format and replays
    payload = json.loads((isolated_cache / "schedules.json").read_text())
    assert payload["schema_version"] == 1 and len(payload["records"]) == 1
    out2, info2 = asg.spmm_csr_auto(crow, col, val, x)
    assert info2["from_cache"] is True and info2["choice"] == info["choice"] and info2["candidate"] == info["candidate"]
    if info["choice"] == "autosage":
        assert torch.equal(out, out2)  # the sm_100a kernels sum in a fixed order
    else:  # the vendor baseline may reorder its sums between runs
        assert torch.allclose(out2.cpu(), torch.from_numpy(exact).float(), rtol=1e-4, atol=1e-3)


def test_replay_only_and_tuning_signature_mismatch(asg, graph, isolated_cache, monkeypatch):
    crow, col, val, x = (t.cuda() for t in graph)
    monkeypatch.setenv("AUTOSAGE_REPLAY_ONLY", "1")
    out, info = asg.spmm_csr_auto(crow, col, None, x)
    assert info == {"operation": "spmm", "schema_version": 3, "choice": "baseline",
                    "baseline": "torch.sparse.mm(csr)", "from_cache": False, "replay_only": True,
                    "reason": "cache miss"}
    assert not (isolated_cache / "schedules.json").exists()
    monkeypatch.delenv("AUTOSAGE_REPLAY_ONLY")
    _, first = asg.spmm_csr_auto(crow, col, None, x)
    assert first["from_cache"] is False
    monkeypatch.setenv("AUTOSAGE_PROBE_ITERS", "3")   # different tuning signature: probe again
    _, second = asg.spmm_csr_auto(crow, col, None, x)
    assert second["from_cache"] is False and second["configuration"]["probe_iterations"] == 3
    monkeypatch.setenv("AUTOSAGE_REPLAY_ONLY", "true")  # replay accepts any schema-3 record
    monkeypatch.setenv("AUTOSAGE_PROBE_ITERS", "5")
    _, third = asg.spmm_csr_auto(crow, col, None, x)
    assert third["from_cache"] is True


def test_pinned_parameters_and_disabled_hub_split(asg, orc, graph, isolated_cache, monkeypatch):
    crow, col, val, x = (t.cuda() for t in graph)
    monkeypatch.setenv("AUTOSAGE_FTILE", "64")
    monkeypatch.setenv("AUTOSAGE_WPB", "4")
    monkeypatch.setenv("AUTOSAGE_HUB_T", "1000")
    monkeypatch.setenv("AUTOSAGE_CACHE", "0")
    _, info = asg.spmm_csr_auto(crow, col, val, x)
    assert [e["candidate"] for e in info["candidates"]] == [[64, 4, 1000]]
    assert not (isolated_cache / "schedules.json").exists()
    monkeypatch.setenv("AUTOSAGE_HUB_CTA", "0")
    out, info = asg.spmm_csr_auto(crow, col, val, x)
    assert [e["candidate"] for e in info["candidates"]] == [None]
    monkeypatch.setenv("AUTOSAGE_VEC4", "0")          # scalar kernels
    out, _ = asg.spmm_csr_auto(crow, col, val, x)
    exact = orc.spmm(to_np(crow), to_np(col), to_np(val), to_np(x))
    assert torch.allclose(out.cpu(), torch.from_numpy(exact).float(), rtol=1e-4, atol=1e-3)


def test_calibrate_full_stores_a_full_graph_schedule(asg, graph, isolated_cache):
    crow, col, val, x = (t.cuda() for t in graph)
    choice, info = asg.calibrate_full(crow, col, val, x)
    assert choice in ("autosage", "baseline") and info["calibration"] == "full_graph"
    assert {"baseline_ms", "autosage_ms", "speedup", "candidates", "configuration"} <= set(info)
    assert all(set(e) == {"candidate", "best_ms"} for e in info["candidates"])
    _, replay = asg.spmm_csr_auto(crow, col, val, x)
    assert replay["from_cache"] is True and replay.get("calibration") == "full_graph"


def test_small_graphs_fall_back_to_the_baseline(asg, isolated_cache):
    """Fewer than 64 sampled rows / 512 sampled nonzeros is not enough work to trust a probe."""
    crow, col = random_csr(40, 3, seed=1)
    x = dense(40, 32, 2)
    out, info = asg.spmm_csr_auto(crow.cuda(), col.cuda(), None, x.cuda())
    assert info["choice"] == "baseline" and info["candidate"] is None and info["probe_rows"] == 40


def test_attention_forward_schedules_the_fused_kernel(asg, orc, isolated_cache):
    crow, col = random_csr(6000, 20, seed=8, hubs={3: 5000})
    q, k, v = dense(6000, 64, 1), dense(6000, 64, 2), dense(6000, 64, 3)
    exact = orc.attention(to_np(crow), to_np(col), to_np(q), to_np(k), to_np(v), 0.125)
    args = [t.cuda() for t in (crow, col, q, k, v)]
    out, info = asg.csr_attention_forward(*args, scale=0.125)
    assert {"sddmm", "spmm", "attention"} <= set(info)
    ok, ratio = orc.within_tolerance(out.cpu().numpy(), exact, to_np(crow), rtol=2e-5, atol=2e-5)
    assert ok, ratio
    out2, info2 = asg.csr_attention_forward(*args, scale=0.125)
    assert info2["attention"]["from_cache"] is True
    unfused, info3 = asg.csr_attention_forward(*args, scale=0.125, fused=False)
    assert set(info3) == {"sddmm", "spmm"}
    ok, ratio = orc.within_tolerance(unfused.cpu().numpy(), exact, to_np(crow), rtol=2e-5, atol=2e-5)
    assert ok, ratio


def test_convolution_on_gpu_matches_the_cpu_layer(asg, isolated_cache):
    torch.manual_seed(0)
    edge_index = torch.randint(0, 3000, (2, 60000))
    weight = torch.rand(60000)
    x = torch.randn(3000, 96)
    for mode in ("native", "auto"):
        layer = asg.AutoSAGEConv(96, 32, mode=mode)
        expected = layer(x, edge_index, weight)
        gpu_layer = layer.to("cuda")
        got, info = gpu_layer(x.cuda(), edge_index.cuda(), weight.cuda(), return_info=True)
        assert torch.allclose(got.cpu(), expected, rtol=1e-4, atol=1e-3)
        assert info["operation"] == "spmm"
        if mode == "native":
            assert info == {"operation": "spmm", "choice": "native", "from_cache": False}


def test_operators_are_differentiable(asg, isolated_cache):
    """Gradients of the operators against dense autograd (the reference registers no backward)."""
    crow, col = random_csr(300, 7, seed=12, hubs={4: 900})
    n = 300
    val = weights(col.numel(), 3).cuda().requires_grad_()
    x = dense(n, 48, 4).cuda().requires_grad_()
    crow_d, col_d = crow.cuda(), col.cuda()
    rows = torch.repeat_interleave(torch.arange(n, device="cuda"), crow_d[1:] - crow_d[:-1])

    def dense_adj(v):
        return torch.zeros(n, n, device="cuda").index_put((rows, col_d), v, accumulate=True)

    upstream = dense(n, 48, 5).cuda()
    for op in (lambda: torch.ops.autosage.spmm_csr(crow_d, col_d, val, x),
               lambda: torch.ops.autosage.spmm_csr_split(crow_d, col_d, val, x, 64, 4, 64)):
        val.grad = x.grad = None
        (op() * upstream).sum().backward()
        got_val, got_x = val.grad.clone(), x.grad.clone()
        val.grad = x.grad = None
        ((dense_adj(val) @ x) * upstream).sum().backward()
        assert torch.allclose(got_x, x.grad, rtol=1e-4, atol=1e-3)
        assert torch.allclose(got_val, val.grad, rtol=1e-4, atol=1e-3)
    # unweighted: only x gets a gradient
    x.grad = None
    (torch.ops.autosage.spmm_csr(crow_d, col_d, None, x) * upstream).sum().backward()
    ones = torch.ones(col.numel(), device="cuda")
    assert torch.allclose(x.grad, dense_adj(ones).t() @ upstream, rtol=1e-4, atol=1e-3)

    q = dense(n, 32, 6).cuda().requires_grad_()
    k = dense(n, 32, 7).cuda().requires_grad_()
    g = dense(col.numel(), 1, 8).flatten().cuda()
    (torch.ops.autosage.sddmm_csr(crow_d, col_d, q, k) * g).sum().backward()
    got_q, got_k = q.grad.clone(), k.grad.clone()
    q.grad = k.grad = None
    (((q[rows] * k[col_d]).sum(1)) * g).sum().backward()
    assert torch.allclose(got_q, q.grad, rtol=1e-4, atol=1e-3)
    assert torch.allclose(got_k, k.grad, rtol=1e-4, atol=1e-3)

    # the layer trains: loss goes through AutoSAGEConv on the GPU
    layer = asg.AutoSAGEConv(48, 8, mode="native").cuda()
    edge_index = torch.stack((col_d, rows))
    layer(x, edge_index).square().mean().backward()
    assert layer.linear.weight.grad is not None and torch.isfinite(layer.linear.weight.grad).all()


def test_fused_attention_backward_matches_the_three_pass_gradients(asg):
    """The fused kernel's backward (probabilities recomputed with the library's kernels) against the
    gradients torch's autograd takes through the reference formulation of the pipeline in float64:
    gather-dot scores, scatter softmax, index_add aggregation."""
    n, f, scale = 900, 64, 0.125
    crow, col = random_csr(n, 7, seed=41, hubs={3: 1400, 500: 90})
    dev = torch.device("cuda")
    crow_d, col_d = crow.to(dev), col.to(dev)
    rows = torch.repeat_interleave(torch.arange(n, device=dev), crow_d[1:] - crow_d[:-1])
    base = [dense(n, f, seed).to(dev) for seed in (51, 52, 53)]
    weight = dense(n, f, 54).to(dev)                      # d(loss)/d(out)

    q, k, v = (t.clone().requires_grad_() for t in base)
    out, info = asg.csr_attention_forward(crow_d, col_d, q, k, v, scale=scale, fused=True)
    assert "attention" in info                            # the fused path ran although gradients are wanted
    (out * weight).sum().backward()

    q64, k64, v64 = (t.double().clone().requires_grad_() for t in base)
    scores = (q64[rows] * k64[col_d]).sum(1) * scale
    peak = torch.full((n,), -torch.inf, dtype=torch.float64, device=dev).scatter_reduce(0, rows, scores, "amax")
    e = (scores - peak[rows]).exp()
    p = e / torch.zeros(n, dtype=torch.float64, device=dev).index_add(0, rows, e)[rows]
    out64 = torch.zeros(n, f, dtype=torch.float64, device=dev).index_add(0, rows, p[:, None] * v64[col_d])
    (out64 * weight.double()).sum().backward()
    assert torch.allclose(out.double(), out64, rtol=1e-4, atol=1e-5)
    for got, want, name in ((q.grad, q64.grad, "dQ"), (k.grad, k64.grad, "dK"), (v.grad, v64.grad, "dV")):
        scale_of = float(want.abs().max())
        assert float((got.double() - want).abs().max()) <= 2e-4 * scale_of + 1e-6, name
    # only one operand differentiable: the others' gradients are skipped, not wrong
    q2 = base[0].clone().requires_grad_()
    out2, _ = asg.csr_attention_forward(crow_d, col_d, q2, base[1], base[2], scale=scale, fused=True)
    (out2 * weight).sum().backward()
    assert torch.allclose(q2.grad, q.grad, rtol=1e-5, atol=1e-6)


def test_operators_replay_inside_a_cuda_graph(asg, orc):
    """Small graphs are launch-bound; the operators must be capturable (no allocation inside the
    library, no host synchronisation) so that a layer's steady state can be replayed as a CUDA graph."""
    crow, col = random_csr(4000, 10, seed=31, hubs={9: 3000})
    val = weights(col.numel(), 2)
    x = dense(4000, 64, 3)
    crow_d, col_d, val_d, x_d = (t.cuda() for t in (crow, col, val, x))
    q_d, k_d = dense(4000, 64, 4).cuda(), dense(4000, 64, 5).cuda()
    # warm up on a side stream (builds the plans, loads the kernels), then capture
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            torch.ops.autosage.spmm_csr_split(crow_d, col_d, val_d, x_d, 64, 4, 256)
            torch.ops.autosage.sddmm_csr_split(crow_d, col_d, q_d, k_d, 4, 256)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y = torch.ops.autosage.spmm_csr_split(crow_d, col_d, val_d, x_d, 64, 4, 256)
        s = torch.ops.autosage.sddmm_csr_split(crow_d, col_d, q_d, k_d, 4, 256)
    for trial in range(3):
        x_d.copy_(dense(4000, 64, 10 + trial))          # new inputs, same buffers
        graph.replay()
        torch.cuda.synchronize()
        exact = orc.spmm(to_np(crow), to_np(col), to_np(val), x_d.cpu().numpy())
        ok, ratio = orc.within_tolerance(y.cpu().numpy(), exact, to_np(crow))
        assert ok, ratio
    exact_s = orc.sddmm(to_np(crow), to_np(col), q_d.cpu().numpy(), k_d.cpu().numpy())
    ok, ratio = orc.within_tolerance(s.cpu().numpy(), exact_s, to_np(crow), per_edge=True)
    assert ok, ratio
    # The captured launches must not lean on the plan cache: evict every cached plan, let the freed
    # memory be recycled by other tensors, and replay once more.
    from autosage_b200 import _native

    _native.clear_plan_cache()
    torch.cuda.empty_cache()
    junk = [torch.full((1 << 20,), 0x7fffffff, device="cuda", dtype=torch.int32) for _ in range(16)]
    for other in range(20):  # more probe-sized entries than the cache holds
        other_crow = torch.arange(0, 5 * (300 + other) + 1, 5, device="cuda")
        torch.ops.autosage.spmm_csr(other_crow, torch.zeros(5 * (300 + other), dtype=torch.long, device="cuda"), None,
                                    torch.ones(300 + other, 8, device="cuda"))
    x_d.copy_(dense(4000, 64, 20))
    graph.replay()
    torch.cuda.synchronize()
    exact = orc.spmm(to_np(crow), to_np(col), to_np(val), x_d.cpu().numpy())
    ok, ratio = orc.within_tolerance(y.cpu().numpy(), exact, to_np(crow))
    assert ok, ratio
    del junk


def test_debug_index_check(monkeypatch):
    """AUTOSAGE_CHECK_INDICES=1 turns an out-of-range column into an error instead of a stray read."""
    import autosage_b200 as asg

    dev = torch.device("cuda")
    crow = torch.tensor([0, 2, 3], device=dev)
    col = torch.tensor([0, 1, 5], device=dev)      # 5 is outside a 2-row X
    x = torch.ones(2, 4, device=dev)
    monkeypatch.setenv("AUTOSAGE_CHECK_INDICES", "1")
    with pytest.raises(RuntimeError, match="col entries must lie in"):
        asg.spmm_csr(crow, col, None, x)
    good = torch.tensor([0, 1, 1], device=dev)
    assert torch.equal(asg.spmm_csr(crow, good, None, x), torch.tensor([[2.0] * 4, [1.0] * 4], device=dev))


def test_probe_on_row_sample_prefers_the_kernels(asg, isolated_cache, monkeypatch):
    """On a power-law graph the whole-row probe sample ranks the kernels ahead of the gather-dot
    baseline (SDDMM) and records a full-graph candidate; the induced sample stays selectable."""
    from benchlib import synthetic as syn

    dev = torch.device("cuda")
    crow, col, info = syn.powerlaw_csr(syn.ARXIV_LIKE, seed=0, device=dev)
    n = info["rows"]
    q, k = syn.dense(n, 64, 1, dev), syn.dense(n, 64, 2, dev)
    out, sched = asg.sddmm_csr_auto(crow, col, q, k)
    assert sched["choice"] == "autosage" and sched["candidate"] is not None
    assert sched["probe_rows"] == n and sched["probe_nonzeros"] == info["nnz"]   # 2.5 M edges: probed whole
    monkeypatch.setenv("AUTOSAGE_PROBE_EDGES", "500000")                         # force a row sample
    monkeypatch.setenv("AUTOSAGE_CACHE", "0")
    _, sampled = asg.sddmm_csr_auto(crow, col, q, k)
    assert sampled["choice"] == "autosage"
    assert 0.1 * info["nnz"] < sampled["probe_nonzeros"] < 0.4 * info["nnz"] and sampled["probe_rows"] < n
    rows = torch.repeat_interleave(torch.arange(n, device=dev), crow[1:] - crow[:-1])
    expected = (q[rows[:100000]] * k[col[:100000]]).sum(1)
    assert torch.allclose(out[:100000], expected, rtol=1e-4, atol=1e-4)
    monkeypatch.setenv("AUTOSAGE_PROBE_SAMPLE", "induced")
    monkeypatch.setenv("AUTOSAGE_CACHE", "0")
    _, sched = asg.sddmm_csr_auto(crow, col, q, k)
    assert sched["probe_nonzeros"] < 0.01 * info["nnz"]


def test_native_row_sample_is_bit_exact(asg):
    """asg_csr_row_sample against the torch formulation of the same sample (integer outputs bit-exact,
    weights copied verbatim), and its behaviour when the selected rows exceed the capacity."""
    from autosage_b200 import _auto, _native

    dev = torch.device("cuda")
    crow, col = random_csr(6000, 9, seed=77, hubs={5: 4000, 4100: 1500})
    val = weights(col.numel(), 3)
    crow_d, col_d, val_d = crow.to(dev), col.to(dev), val.to(dev)
    ref_crow, ref_col, ref_val, selected = _auto._row_sample_csr(crow_d, col_d, val_d, fraction=0.3, minimum_rows=8, seed=4)
    total = ref_col.numel()
    for weights_given in (True, False):
        s_crow, s_col, s_val, kept = _native.csr_row_sample(crow_d, col_d, val_d if weights_given else None, selected,
                                                            total + 100)
        assert kept.tolist() == [selected.numel(), total]
        assert torch.equal(s_crow, ref_crow) and torch.equal(s_col[:total], ref_col)
        assert (s_val is None) == (not weights_given)
        if weights_given:
            assert torch.equal(s_val[:total], ref_val)
    # capacity below the total: only the leading rows that fit are copied, the tail rows are empty
    capacity = int(ref_crow[selected.numel() // 2])
    s_crow, s_col, _, kept = _native.csr_row_sample(crow_d, col_d, None, selected, capacity)
    rows_kept, edges_kept = kept.tolist()
    assert edges_kept <= capacity and edges_kept == int(ref_crow[rows_kept])
    assert rows_kept == selected.numel() or int(ref_crow[rows_kept + 1]) > capacity
    assert torch.equal(s_crow[: rows_kept + 1], ref_crow[: rows_kept + 1])
    assert bool((s_crow[rows_kept:] == edges_kept).all())
    assert torch.equal(s_col[:edges_kept], ref_col[:edges_kept])
    # nothing selected
    empty = _native.csr_row_sample(crow_d, col_d, None, selected[:0], 16)
    assert empty[0].tolist() == [0] and empty[3].tolist() == [0, 0]


def test_scheduler_probe_uses_the_device_sample(asg, isolated_cache, monkeypatch):
    """Above the probe's edge target the sample is cut by the library; the schedule reports the
    sample's real sizes and the replayed call gives the same result as the plain operator."""
    from benchlib import synthetic as syn

    dev = torch.device("cuda")
    crow, col, info = syn.powerlaw_csr(syn.ARXIV_LIKE, seed=0, device=dev)
    n = info["rows"]
    x = syn.dense(n, 64, 3, dev)
    monkeypatch.setenv("AUTOSAGE_PROBE_EDGES", "600000")
    y, schedule = asg.spmm_csr_auto(crow, col, None, x)
    assert 0 < schedule["probe_rows"] < n and 0.1 * info["nnz"] < schedule["probe_nonzeros"] < 0.5 * info["nnz"]
    assert len(schedule["candidates"]) >= 2 and all(c["iterations"] >= 1 for c in schedule["candidates"])
    assert torch.allclose(y, torch.ops.autosage.spmm_csr(crow, col, None, x), rtol=1e-4, atol=1e-3)
