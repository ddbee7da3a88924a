"""Pins the CPU oracle (oracle/csr_oracle.c) to the reference: golden vectors produced by running
the reference itself (tests/golden/generate.py) and the known answers of its own CPU tests."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import oracle as orc

CASES = ["tiny", "ragged", "hub", "wide"]


@pytest.mark.parametrize("case", CASES)
def test_spmm_matches_reference_float64(golden, case):
    vec, _ = golden
    crow, col, val, x = (vec[f"{case}.{n}"] for n in ("crow", "col", "val", "x"))
    np.testing.assert_allclose(orc.spmm(crow, col, val, x), vec[f"{case}.spmm_weighted"], rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(orc.spmm(crow, col, None, x), vec[f"{case}.spmm_unweighted"], rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("case", CASES)
def test_float32_port_matches_reference_float32(golden, case):
    vec, _ = golden
    crow, col, val, x = (vec[f"{case}.{n}"] for n in ("crow", "col", "val", "x"))
    mine = orc.spmm(crow, col, val, x, dtype=np.float32)
    ok, ratio = orc.within_tolerance(mine, vec[f"{case}.spmm_weighted"], crow)
    assert ok, ratio
    np.testing.assert_allclose(mine, vec[f"{case}.spmm_weighted_f32"], rtol=2e-5, atol=2e-5)
    torch_path = orc.spmm_reference_cpu(torch.from_numpy(crow), torch.from_numpy(col), torch.from_numpy(val),
                                        torch.from_numpy(x)).numpy()
    np.testing.assert_array_equal(torch_path, vec[f"{case}.spmm_weighted_f32"])


@pytest.mark.parametrize("case", CASES)
def test_sddmm_softmax_attention_match_reference(golden, case):
    vec, _ = golden
    crow, col, x, q, k = (vec[f"{case}.{n}"] for n in ("crow", "col", "x", "q", "k"))
    scores = orc.sddmm(crow, col, q, k)
    np.testing.assert_allclose(scores, vec[f"{case}.sddmm"], rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(orc.row_softmax(crow, vec[f"{case}.sddmm"]), vec[f"{case}.softmax"], rtol=1e-10,
                               atol=1e-300)
    np.testing.assert_allclose(orc.attention(crow, col, q, k, x, 1.0), vec[f"{case}.attention"], rtol=1e-9,
                               atol=1e-12)


def test_known_answers_of_the_reference_cpu_tests():
    # weights + an empty row (reference tests/test_cpu.py:25-32)
    crow, col = np.array([0, 2, 2, 3]), np.array([1, 2, 0])
    val = np.array([0.5, 2.0, -1.0], dtype=np.float32)
    x = np.array([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], dtype=np.float32)
    expected = np.stack((0.5 * x[1] + 2.0 * x[2], np.zeros(2), -x[0]))
    np.testing.assert_allclose(orc.spmm(crow, col, val, x), expected)
    # SDDMM known answer and softmax rows summing to one (tests/test_cpu.py:45-56)
    crow, col = np.array([0, 2, 3]), np.array([0, 1, 0])
    q = np.array([[1.0, 2.0], [3.0, 4.0]], dtype=np.float32)
    k = np.array([[2.0, 1.0], [1.0, 3.0]], dtype=np.float32)
    scores = orc.sddmm(crow, col, q, k)
    np.testing.assert_allclose(scores, [4.0, 7.0, 10.0])
    probs = orc.row_softmax(crow, scores)
    assert probs[:2].sum() == pytest.approx(1.0) and probs[2] == pytest.approx(1.0)
    # destination-row orientation (tests/test_cpu.py:16-22) and weight order (:70-78)
    crow, col, perm = orc.edge_index_to_csr(np.array([[0, 1, 2, 3], [1, 2, 3, 0]]), 4)
    x = np.arange(12, dtype=np.float32).reshape(4, 3)
    y = orc.spmm(crow, col, None, x)
    np.testing.assert_array_equal(y[0], x[3])
    np.testing.assert_array_equal(y[1], x[0])
    crow, col, perm = orc.edge_index_to_csr(np.array([[2, 0, 1], [0, 1, 0]]), 3)
    w = np.array([10.0, 20.0, 30.0], dtype=np.float32)[perm]
    y = orc.spmm(crow, col, w, np.array([[1.0], [2.0], [3.0]], dtype=np.float32))
    np.testing.assert_array_equal(y, [[90.0], [20.0], [0.0]])


def test_coo_to_csr_matches_reference(golden):
    vec, _ = golden
    crow, col, perm = orc.edge_index_to_csr(vec["coo.edge_index"], 40)
    np.testing.assert_array_equal(crow, vec["coo.crow"])
    np.testing.assert_array_equal(col, vec["coo.col"])
    np.testing.assert_array_equal(perm, vec["coo.weight_order"])
    crow, col, _ = orc.edge_index_to_csr(vec["coo.edge_index"], 40, rows_by="src")
    np.testing.assert_array_equal(crow, vec["coo.crow_src"])
    np.testing.assert_array_equal(col, vec["coo.col_src"])


def test_row_split_and_plan_order_are_consistent(golden):
    vec, _ = golden
    crow = vec["hub.crow"]
    deg = crow[1:] - crow[:-1]
    for threshold in (0, 1, 4, 9, 150, 151):
        hubs, lights = orc.hub_split(crow, threshold)
        want = np.nonzero(deg >= threshold)[0] if threshold > 0 else np.array([], dtype=np.int64)
        np.testing.assert_array_equal(hubs, want)  # the reference's nonzero(deg >= T), ascending
        assert np.array_equal(np.sort(np.concatenate([hubs, lights])), np.arange(deg.size))
        order, n_hub, n_light = orc.plan_order(crow, threshold)
        assert (n_hub, n_light) == (hubs.size, lights.size)
        np.testing.assert_array_equal(np.sort(order[:n_hub]), hubs)
        np.testing.assert_array_equal(np.sort(order[n_hub:]), lights)
        for part in (order[:n_hub], order[n_hub:]):
            buckets = np.floor(np.log2(np.maximum(deg[part], 1))).astype(int) + (deg[part] > 0)
            assert np.all(np.diff(buckets) <= 0)  # descending degree class
            same = np.diff(buckets) == 0
            assert np.all(np.diff(part)[same] > 0)  # ascending row id inside a class


def test_partition_rows_balances_nonzeros():
    rng = np.random.default_rng(0)
    deg = rng.integers(0, 50, size=1000)
    deg[123] = 5000
    crow = np.concatenate([[0], np.cumsum(deg)])
    for parts in (1, 2, 3, 4, 8):
        bounds = orc.partition_rows(crow, parts)
        assert bounds[0] == 0 and bounds[-1] == 1000 and np.all(np.diff(bounds) >= 0)
        expected = np.searchsorted(crow, (np.arange(parts + 1) * crow[-1]) // parts, side="left")
        expected[0], expected[-1] = 0, 1000
        np.testing.assert_array_equal(bounds, expected)
        shares = np.diff(crow[bounds])
        assert shares.max() <= crow[-1] / parts + 5000


def test_tolerance_rule():
    crow = np.array([0, 4, 4, 5])
    exact = np.ones((3, 2))
    # bounds: row 0 (degree 4) 1e-5*1 + 1e-5*2 = 3e-5; rows 1 and 2 (degree 0 and 1) 2e-5
    ok, _ = orc.within_tolerance(exact + 2.5e-5, exact, crow)
    assert not ok
    ok, ratio = orc.within_tolerance(exact + np.array([[2.9e-5], [1.9e-5], [1.9e-5]]), exact, crow)
    assert ok and ratio < 1.0
    ok, _ = orc.within_tolerance(np.full((3, 2), np.nan), exact, crow)
    assert not ok
