"""Host-side behaviour of the drop-in API on CPU: configuration, cache format, schedule keys,
shortlist, induced sample, CSR build and the CPU paths.  Integer outputs are compared bit-exactly
with values the reference produced (tests/golden/)."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import pytest
import torch

import autosage_b200 as asg
from autosage_b200 import _auto, _cache
from autosage_b200.config import SchedulerConfig
from autosage_b200.utils.csr import edge_index_to_csr

GOLDEN = Path(__file__).resolve().parent / "golden"
CASES = ["tiny", "ragged", "hub", "wide"]


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


# ---------------------------------------------------------------------------------- API surface
def test_public_names_match_the_reference_package():
    assert asg.__version__ == "0.1.0"
    assert sorted(asg.__all__) == sorted([
        "AutoSAGEConv", "__version__", "calibrate_full", "csr_attention_forward", "load_native",
        "native_available", "sddmm_csr_auto", "spmm_csr", "spmm_csr_auto"])
    import autosage  # the drop-in alias

    assert autosage.spmm_csr is asg.spmm_csr
    from autosage._auto import _spmm_candidates  # noqa: F401
    from autosage._cache import ScheduleCache  # noqa: F401
    from autosage.utils.csr import edge_index_to_csr as alias_fn

    assert alias_fn is edge_index_to_csr
    from autosage.ops import native_load_error, native_op  # noqa: F401


def test_spmm_rejects_fractional_indices():
    with pytest.raises(TypeError, match="integer indices"):
        asg.spmm_csr(torch.tensor([0.0, 1.0]), torch.tensor([0.0]), None, torch.ones(1, 1))
    with pytest.raises(TypeError, match="integer indices"):
        asg.sddmm_csr_auto(torch.tensor([0.0, 1.0]), torch.tensor([0.0]), torch.ones(1, 1), torch.ones(1, 1))


def test_validation_errors():
    crow, col = torch.tensor([0, 1, 2]), torch.tensor([1, 0])
    with pytest.raises(ValueError, match="N \\+ 1"):
        asg.spmm_csr(crow, col, None, torch.ones(3, 2))
    with pytest.raises(ValueError, match="one weight per nonzero"):
        asg.spmm_csr(crow, col, torch.ones(3), torch.ones(2, 2))
    with pytest.raises(TypeError, match="floating-point"):
        asg.spmm_csr(crow, col, None, torch.ones(2, 2, dtype=torch.long))
    with pytest.raises(ValueError, match="same \\[N, F\\] shape"):
        asg.sddmm_csr_auto(crow, col, torch.ones(2, 2), torch.ones(2, 3))
    with pytest.raises(ValueError, match="mode must be"):
        asg.AutoSAGEConv(2, 2, mode="fast")


def test_int32_indices_are_accepted():
    crow = torch.tensor([0, 2, 2, 3], dtype=torch.int32)
    col = torch.tensor([1, 2, 0], dtype=torch.int32)
    x = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])
    val = torch.tensor([0.5, 2.0, -1.0])
    out = asg.spmm_csr(crow, col, val, x)
    assert torch.allclose(out, torch.stack((0.5 * x[1] + 2.0 * x[2], torch.zeros(2), -x[0])))
    assert asg.spmm_csr(crow, col, val.double(), x.double()).dtype == torch.float64


def test_cpu_paths_report_the_baseline():
    crow, col = torch.tensor([0, 1, 2]), torch.tensor([1, 0])
    x = torch.randn(2, 4)
    out, info = asg.spmm_csr_auto(crow, col, None, x)
    assert out.shape == x.shape and info["choice"] == "baseline"
    assert info["reason"] == "AutoSAGE scheduling is CUDA-only" and info["schema_version"] == 3
    assert info["baseline"] == "torch CPU" and info["from_cache"] is False and info["operation"] == "spmm"
    scores, info = asg.sddmm_csr_auto(crow, col, x, x)
    assert info["choice"] == "baseline" and info["baseline"] == "gather-dot" and info["operation"] == "sddmm"
    choice, info = asg.calibrate_full(crow, col, None, x)
    assert choice == "baseline" and info["reason"] == "AutoSAGE scheduling is CUDA-only"


@pytest.mark.parametrize("case", CASES)
def test_cpu_pipeline_matches_reference_outputs(golden, case):
    vec, _ = golden
    crow, col, x, q, k, val = (t(vec[f"{case}.{n}"]) for n in ("crow", "col", "x", "q", "k", "val"))
    np.testing.assert_allclose(asg.spmm_csr(crow, col, val.double(), x.double()).numpy(),
                               vec[f"{case}.spmm_weighted"], rtol=1e-12, atol=1e-12)
    scores, _ = asg.sddmm_csr_auto(crow, col, q.double(), k.double())
    np.testing.assert_allclose(scores.numpy(), vec[f"{case}.sddmm"], rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(_auto._csr_row_softmax(crow, scores).numpy(), vec[f"{case}.softmax"], rtol=1e-12)
    out, info = asg.csr_attention_forward(crow, col, q.double(), k.double(), x.double())
    np.testing.assert_allclose(out.numpy(), vec[f"{case}.attention"], rtol=1e-10, atol=1e-12)
    assert set(info) == {"sddmm", "spmm"}
    # scale keyword: scaling the query is the same as scaling the scores
    scaled, _ = asg.csr_attention_forward(crow, col, q.double(), k.double(), x.double(), scale=0.25)
    manual, _ = asg.csr_attention_forward(crow, col, 0.25 * q.double(), k.double(), x.double())
    np.testing.assert_allclose(scaled.numpy(), manual.numpy(), rtol=1e-12)


def test_row_softmax_of_empty_input_is_a_clone():
    crow = torch.zeros(4, dtype=torch.long)
    scores = torch.zeros(0)
    out = _auto._csr_row_softmax(crow, scores)
    assert out.numel() == 0 and out.data_ptr() != scores.data_ptr() or out.numel() == 0


# -------------------------------------------------------------------------------- configuration
def test_environment_is_read_on_every_call(monkeypatch):
    monkeypatch.setenv("AUTOSAGE_FTILE", "64")
    monkeypatch.setenv("AUTOSAGE_WPB", "8")
    monkeypatch.setenv("AUTOSAGE_HUB_T", "16")
    first = SchedulerConfig.from_env()
    monkeypatch.setenv("AUTOSAGE_HUB_T", "32")
    second = SchedulerConfig.from_env()
    assert (first.feature_tile, first.warps_per_block, first.hub_threshold) == (64, 8, 16)
    assert second.hub_threshold == 32
    monkeypatch.setenv("AUTOSAGE_VEC4", "false")
    assert SchedulerConfig.from_env().tuning_signature()["vec4"] is False
    monkeypatch.setenv("AUTOSAGE_VEC4", "maybe")
    with pytest.raises(ValueError, match="AUTOSAGE_VEC4 must be a boolean"):
        SchedulerConfig.from_env()


def test_configuration_validation_and_signature(golden, monkeypatch):
    for name in ("AUTOSAGE_FTILE", "AUTOSAGE_WPB", "AUTOSAGE_HUB_T", "AUTOSAGE_VEC4", "AUTOSAGE_HUB_CTA",
                 "AUTOSAGE_PROBE_FRAC", "AUTOSAGE_PROBE_MIN_ROWS", "AUTOSAGE_PROBE_ITERS", "AUTOSAGE_PROBE_CAP_MS",
                 "AUTOSAGE_MIN_PROBE_ROWS", "AUTOSAGE_MIN_PROBE_NNZ"):
        monkeypatch.delenv(name, raising=False)
    _, keys = golden
    signature = SchedulerConfig.from_env().tuning_signature()
    assert signature == keys["tuning_signature"]
    assert list(signature) == ["guardrail", "probe_fraction", "probe_min_rows", "probe_iterations", "probe_cap_ms",
                               "minimum_probe_rows", "minimum_probe_nonzeros", "candidate_count", "hub_split", "vec4",
                               "feature_tile", "warps_per_block", "hub_threshold"]
    for bad in (dict(guardrail=0.0), dict(guardrail=1.5), dict(probe_fraction=0.0), dict(probe_min_rows=0),
                dict(probe_cap_ms=-1.0), dict(feature_tile=96), dict(warps_per_block=3), dict(hub_threshold=0)):
        with pytest.raises(ValueError):
            SchedulerConfig(**bad)


# ------------------------------------------------------------------------------ keys and cache
@pytest.mark.parametrize("case", CASES + ["long"])
def test_graph_signature_is_bit_exact(golden, case):
    vec, keys = golden
    crow, col = t(vec[f"{case}.crow"]), t(vec[f"{case}.col"])
    expected = keys["cases"][case]["graph_signature"]
    weighted = case != "long"
    got = _cache.graph_signature(crow, col, expected["feature_width"], "spmm", weighted=weighted, dtype=torch.float32)
    assert got == expected and len(got["structure_hash"]) == 24
    if case != "long":
        assert _cache.graph_signature(crow, col, expected["feature_width"], "sddmm", dtype=torch.float32) == \
            keys["cases"][case]["graph_signature_sddmm"]
    # memoised path returns the same dict
    assert _auto._SIGNATURES.signature(crow, col, expected["feature_width"], "spmm", weighted, torch.float32) == expected
    assert _auto._SIGNATURES.signature(crow, col, expected["feature_width"], "spmm", weighted, torch.float32) == expected


def test_quantiles_beyond_the_torch_quantile_limit(monkeypatch):
    values = torch.randint(0, 1000, (5001,), generator=torch.Generator().manual_seed(1))
    direct = _cache.rounded_quantiles(values, [0.5, 0.9, 0.99])
    monkeypatch.setattr(_cache, "_QUANTILE_LIMIT", 100)
    assert _cache.rounded_quantiles(values, [0.5, 0.9, 0.99]) == direct


def test_cache_key_and_file_interoperate_with_the_reference(golden, isolated_cache):
    _, keys = golden
    graph = keys["cases"]["hub"]["graph_signature"]
    assert _cache.ScheduleCache._key(keys["device"], graph) == keys["cache_key"]
    # a schedules.json written by the reference is readable here
    (isolated_cache / "schedules.json").write_text((GOLDEN / "reference_schedules.json").read_text())
    record = _cache.ScheduleCache().lookup(keys["device"], graph)
    assert record is not None and record["result"] == keys["stored_result"]
    assert _auto._cache_hit_allowed(record["result"], SchedulerConfig.from_env())
    # and what this implementation writes has the reference's layout
    cache = _cache.ScheduleCache()
    cache.store(keys["device"], {"operation": "spmm", "rows": 2}, {"choice": "baseline"})
    payload = json.loads((isolated_cache / "schedules.json").read_text())
    assert payload["schema_version"] == 1 and set(payload) == {"schema_version", "records"}
    assert len(payload["records"]) == 2
    for key, entry in payload["records"].items():
        assert set(entry) == {"timestamp", "device", "graph", "result"}
        assert key == json.dumps({"device": entry["device"], "graph": entry["graph"]}, sort_keys=True,
                                 separators=(",", ":"))
    assert _cache.cache_directory() == isolated_cache


def test_corrupt_or_foreign_cache_files_read_as_empty(isolated_cache):
    path = isolated_cache / "schedules.json"
    path.write_text("{not json")
    assert _cache.ScheduleCache().lookup({}, {}) is None
    path.write_text(json.dumps({"schema_version": 99, "records": {"k": {}}}))
    assert _cache.ScheduleCache()._records == {}
    path.write_text(json.dumps([1, 2, 3]))
    assert _cache.ScheduleCache()._records == {}


def test_probe_log_is_optional(isolated_cache, monkeypatch):
    monkeypatch.setenv("AUTOSAGE_LOG_PROBES", "1")
    _cache.log_probe({"a": 1})
    _cache.log_probe({"b": 2})
    lines = (isolated_cache / "probe_logs.jsonl").read_text().splitlines()
    assert [json.loads(line) for line in lines] == [{"a": 1}, {"b": 2}]
    monkeypatch.setenv("AUTOSAGE_LOG_PROBES", "0")
    _cache.log_probe({"c": 3})
    assert len((isolated_cache / "probe_logs.jsonl").read_text().splitlines()) == 2


def test_cache_hit_rules():
    config = SchedulerConfig.from_env()
    good = {"schema_version": 3, "configuration": config.tuning_signature()}
    assert _auto._cache_hit_allowed(good, config)
    assert not _auto._cache_hit_allowed({**good, "schema_version": 2}, config)
    assert not _auto._cache_hit_allowed({**good, "configuration": {"x": 1}}, config)
    replay = SchedulerConfig(replay_only=True)
    assert _auto._cache_hit_allowed({"schema_version": 3, "configuration": {"x": 1}}, replay)


# ------------------------------------------------------------------------------------ shortlist
@pytest.mark.parametrize("case", CASES + ["long"])
def test_shortlist_is_bit_exact(golden, case):
    vec, keys = golden
    crow = t(vec[f"{case}.crow"])
    expected = keys["cases"][case]
    assert list(_auto._degree_quantiles(crow)) == expected["degree_quantiles"]
    width = expected["graph_signature"]["feature_width"]
    assert [list(c) for c in _auto._spmm_candidates(crow, width, SchedulerConfig())] == expected["candidates_default"]
    if "candidates_k18" in expected:
        got = _auto._spmm_candidates(crow, width, SchedulerConfig(candidate_count=18))
        assert [list(c) for c in got] == expected["candidates_k18"]
        assert len(got) == len(set(got))
        assert all(tile in (64, 128) and warps in (2, 4, 8) and threshold > 0 for tile, warps, threshold in got)


def test_shortlist_honours_pinned_parameters():
    crow = torch.tensor([0, 1, 3, 3, 10])
    got = _auto._spmm_candidates(crow, 64, SchedulerConfig(feature_tile=64, warps_per_block=4, hub_threshold=5))
    assert got == [(64, 4, 5)]
    assert _auto._degree_quantiles(torch.zeros(1, dtype=torch.long)) == (1, 1, 1)


@pytest.mark.parametrize("case", CASES)
def test_induced_sample_is_bit_exact(golden, case):
    vec, _ = golden
    crow, col, val = t(vec[f"{case}.crow"]), t(vec[f"{case}.col"]), t(vec[f"{case}.val"])
    s_crow, s_col, s_val, rows = _auto._induced_sample_csr(crow, col, val, fraction=0.5, minimum_rows=4, seed=3)
    np.testing.assert_array_equal(s_crow.numpy(), vec[f"{case}.sample_crow"])
    np.testing.assert_array_equal(s_col.numpy(), vec[f"{case}.sample_col"])
    np.testing.assert_array_equal(s_val.numpy(), vec[f"{case}.sample_val"])
    np.testing.assert_array_equal(rows.numpy(), vec[f"{case}.sample_rows"])


def test_induced_sample_of_an_edgeless_graph():
    crow = torch.zeros(11, dtype=torch.long)
    s_crow, s_col, s_val, rows = _auto._induced_sample_csr(crow, torch.zeros(0, dtype=torch.long), torch.zeros(0),
                                                           fraction=0.5, minimum_rows=2, seed=0)
    assert s_crow.tolist() == [0] * 6 and s_col.numel() == 0 and s_val.numel() == 0 and rows.numel() == 5


def test_threshold_translation_matches_quantiles(golden):
    vec, _ = golden
    crow = t(vec["hub.crow"])
    sample = _auto._induced_sample_csr(crow, t(vec["hub.col"]), None, fraction=0.5, minimum_rows=4, seed=3)[0]
    mapping = _auto._threshold_translation(crow, sample, SchedulerConfig())
    assert list(mapping) == list(dict.fromkeys(_auto._degree_quantiles(crow)))
    assert _auto._threshold_translation(crow, sample, SchedulerConfig(hub_threshold=7)) == {7: 7}


# -------------------------------------------------------------------------------------- CSR/conv
def test_edge_index_to_csr_is_bit_exact(golden):
    vec, _ = golden
    edge_index = t(vec["coo.edge_index"])
    crow, col = edge_index_to_csr(edge_index, 40)
    np.testing.assert_array_equal(crow.numpy(), vec["coo.crow"])
    np.testing.assert_array_equal(col.numpy(), vec["coo.col"])
    crow, col = edge_index_to_csr(edge_index.to(torch.int32), 40, rows_by="src")
    np.testing.assert_array_equal(crow.numpy(), vec["coo.crow_src"])
    np.testing.assert_array_equal(col.numpy(), vec["coo.col_src"])
    assert crow.dtype == torch.long and col.dtype == torch.long
    with pytest.raises(ValueError, match=r"\[2, E\]"):
        edge_index_to_csr(torch.zeros(3, 4, dtype=torch.long), 4)
    with pytest.raises(ValueError, match="rows_by"):
        edge_index_to_csr(edge_index, 40, rows_by="both")
    crow, col = edge_index_to_csr(torch.zeros(2, 0, dtype=torch.long), 3)
    assert crow.tolist() == [0, 0, 0, 0] and col.numel() == 0
    # a row id outside [0, num_nodes) is an error (the reference's index_add_ raises IndexError on the CPU)
    with pytest.raises(IndexError):
        edge_index_to_csr(torch.tensor([[0, 1], [1, 5]]), 4)
    with pytest.raises((IndexError, RuntimeError)):
        edge_index_to_csr(torch.tensor([[0, 1], [1, -1]]), 4)


def test_layer_pickles_after_a_forward():
    """The CSR memo holds a weak reference; a layer must still pickle / deepcopy after it has run."""
    import copy
    import pickle

    torch.manual_seed(1)
    layer = asg.AutoSAGEConv(3, 2)
    x, edge_index = torch.randn(4, 3), torch.tensor([[0, 1, 2, 3], [1, 2, 3, 0]])
    expected = layer(x, edge_index)
    for clone in (pickle.loads(pickle.dumps(layer)), copy.deepcopy(layer)):
        assert torch.equal(clone(x, edge_index), expected)


def test_convolution_shapes_info_and_weight_order():
    edge_index = torch.tensor([[0, 1], [1, 0]])
    x = torch.randn(2, 3)
    layer = asg.AutoSAGEConv(3, 2)
    out = layer(x, edge_index)
    out2, info = layer(x, edge_index, return_info=True)
    assert out.shape == (2, 2) and torch.equal(out, out2) and info["choice"] == "baseline"
    # weights follow their edges into CSR order (reference tests/test_cpu.py:70-78)
    edge_index = torch.tensor([[2, 0, 1], [0, 1, 0]])
    layer = asg.AutoSAGEConv(1, 1, mode="native", bias=False)
    with torch.no_grad():
        layer.linear.weight.fill_(1.0)
    x = torch.tensor([[1.0], [2.0], [3.0]])
    weight = torch.tensor([10.0, 20.0, 30.0])
    assert torch.equal(layer(x, edge_index, weight), torch.tensor([[90.0], [20.0], [0.0]]))
    assert torch.equal(layer(x, edge_index, weight), torch.tensor([[90.0], [20.0], [0.0]]))  # memoised CSR
    edge_index[0, 0] = 1  # in-place change invalidates the memo
    assert torch.equal(layer(x, edge_index, weight), torch.tensor([[80.0], [20.0], [0.0]]))
    with pytest.raises(ValueError, match="one value per edge"):
        layer(x, edge_index, torch.ones(2))


def test_cuda_request_without_a_device_fails_loudly(monkeypatch):
    """There is no CPU fallback for the CUDA operators: calling one with CPU tensors raises."""
    if not asg.load_native():
        pytest.skip("library not built")
    crow, col = torch.tensor([0, 1, 2]), torch.tensor([1, 0])
    with pytest.raises(NotImplementedError):
        torch.ops.autosage.spmm_csr(crow, col, None, torch.ones(2, 4))
    with pytest.raises(NotImplementedError):
        torch.ops.autosage.sddmm_csr_split(crow, col, torch.ones(2, 4), torch.ones(2, 4), 8, 16)


def test_transposed_pattern_for_the_backward_pass():
    from autosage_b200.ops import _transposed_pattern

    crow, col = torch.tensor([0, 2, 2, 3, 6]), torch.tensor([1, 2, 0, 3, 1, 1])  # row 3 repeats column 1
    crow_t, col_t, perm = _transposed_pattern(crow, col)
    dense = torch.zeros(4, 4)
    rows = torch.repeat_interleave(torch.arange(4), crow[1:] - crow[:-1])
    dense.index_put_((rows, col), torch.ones(6), accumulate=True)
    rows_t = torch.repeat_interleave(torch.arange(4), crow_t[1:] - crow_t[:-1])
    dense_t = torch.zeros(4, 4).index_put_((rows_t, col_t), torch.ones(6), accumulate=True)
    assert torch.equal(dense_t, dense.t())
    assert torch.equal(col[perm], rows_t) and torch.equal(rows[perm], col_t)   # perm maps transpose edges back
    assert _transposed_pattern(crow, col)[0] is crow_t                           # memoised per tensor pair
    col[0] = 3                                                                   # in-place edit invalidates
    assert _transposed_pattern(crow, col)[0] is not crow_t


def test_linear_helper_matches_the_module_on_cpu():
    from autosage_b200.conv import apply_linear

    torch.manual_seed(0)
    layer = torch.nn.Linear(5, 3)
    x = torch.randn(7, 5)
    assert torch.equal(apply_linear(layer, x), layer(x))


def test_row_sample_keeps_whole_rows():
    """The probe's row sample: same selected rows as the induced sample, every edge of each kept."""
    from autosage_b200 import _auto

    gen = torch.Generator().manual_seed(5)
    degree = torch.randint(0, 9, (200,), generator=gen)
    crow = torch.cat((torch.zeros(1, dtype=torch.long), degree.cumsum(0)))
    col = torch.randint(0, 200, (int(crow[-1]),), generator=gen)
    val = torch.rand(col.numel(), generator=gen)
    s_crow, s_col, s_val, rows = _auto._row_sample_csr(crow, col, val, fraction=0.25, minimum_rows=4, seed=3)
    induced_rows = _auto._induced_sample_csr(crow, col, val, fraction=0.25, minimum_rows=4, seed=3)[3]
    assert torch.equal(rows, induced_rows) and rows.numel() == 50
    assert torch.equal(s_crow[1:] - s_crow[:-1], degree[rows])
    expected_col = torch.cat([col[crow[r]:crow[r + 1]] for r in rows.tolist()])
    expected_val = torch.cat([val[crow[r]:crow[r + 1]] for r in rows.tolist()])
    assert torch.equal(s_col, expected_col) and torch.equal(s_val, expected_val)
    empty = _auto._row_sample_csr(torch.zeros(11, dtype=torch.long), torch.zeros(0, dtype=torch.long), None,
                                  fraction=0.5, minimum_rows=2, seed=0)
    assert empty[0].tolist() == [0] * 6 and empty[1].numel() == 0 and empty[2] is None


def test_fused_layer_route_is_opt_in_and_cuda_only(monkeypatch):
    """The one-kernel form of the layer is taken only when AUTOSAGE_CONV_FUSED=1 and the input is a CUDA
    float32 tensor; on the CPU the layer keeps the reference's path whatever the variable says."""
    import torch
    from autosage_b200 import conv

    linear = torch.nn.Linear(128, 256)
    x = torch.zeros(4, 128)
    assert not conv._fused_forward_ok(linear, x, None)
    monkeypatch.setenv("AUTOSAGE_CONV_FUSED", "1")
    assert not conv._fused_forward_ok(linear, x, None)          # CPU tensor
    layer = conv.AutoSAGEConv(128, 256, mode="native")
    edge_index = torch.tensor([[0, 1, 2], [1, 2, 3]])
    out, info = layer(x, edge_index, return_info=True)
    assert info["choice"] == "baseline" and out.shape == (4, 256)
