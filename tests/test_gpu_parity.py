"""GPU parity: the sm_100a kernels, called through the C ABI, against the CPU oracle.

Tolerance for float32 results, from the project's acceptance rule: against the float64 oracle,
|y - y64| <= 1e-5*|y64| + 1e-5*sqrt(row degree); integer outputs must be bit-exact.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import csr_from_counts, dense, misaligned_copy, random_csr, to_np, weights

pytestmark = pytest.mark.gpu

RTOL = 1e-5
ATOL = 1e-5  # multiplied by sqrt(row degree)


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


def assert_close(orc, actual: torch.Tensor, exact: np.ndarray, crow, per_edge=False):
    ok, ratio = orc.within_tolerance(actual.detach().cpu().numpy(), exact, to_np(crow), per_edge=per_edge,
                                     rtol=RTOL, atol=ATOL)
    assert ok, f"outside rtol {RTOL} / atol {ATOL}*sqrt(deg): worst error/bound = {ratio:.3f}"


def run_spmm(lib, crow, col, val, x, *, tile=128, warps=8, threshold=64, flags=0, y=None, ws=None):
    dev = torch.device("cuda")
    crow_d, col_d, x_d = crow.to(dev), col.to(dev), x if x.is_cuda else x.to(dev)
    val_d = None if val is None else val.to(dev)
    n = crow.numel() - 1
    if y is None:
        y = torch.full((n, x.size(1)), float("nan"), device=dev)
    if ws is None:
        ws = torch.empty(lib.workspace_bytes(n), dtype=torch.uint8, device=dev)
    lib.spmm(crow_d, col_d, val_d, x_d, y, feature_tile=tile, warps=warps, threshold=threshold, flags=flags,
             workspace=ws)
    torch.cuda.synchronize()
    assert lib.workspace_status(ws) == 0
    return y


# ------------------------------------------------------------------------------------------ plan
@pytest.mark.parametrize("rows,threshold", [(1, 1), (31, 4), (1024, 9), (1025, 9), (5000, 1), (5000, 0), (70000, 33)])
def test_plan_order_is_bit_exact(lib, orc, rows, threshold):
    crow, _ = random_csr(rows, 8, seed=rows, hubs={0: 700, rows // 2: 40})
    ws = torch.empty(lib.workspace_bytes(rows), dtype=torch.uint8, device="cuda")
    lib.plan_build(crow.cuda(), threshold, ws)
    order, counts = lib.plan_export(ws, rows)
    expected, n_hub, n_light = orc.plan_order(to_np(crow), threshold)
    assert counts.cpu().tolist() == [n_hub, n_light]
    assert np.array_equal(order.cpu().numpy(), expected)
    # the hub set is the reference's nonzero(deg >= T), which is ascending
    hubs, lights = orc.hub_split(to_np(crow), threshold)
    assert np.array_equal(np.sort(order.cpu().numpy()[:n_hub]), hubs)
    assert np.array_equal(np.sort(order.cpu().numpy()[n_hub:]), lights)


# ------------------------------------------------------------------------------------------ SpMM
@pytest.mark.parametrize("features", [1, 3, 4, 32, 64, 100, 113, 128, 192, 256, 512])
@pytest.mark.parametrize("weighted", [False, True])
def test_spmm_feature_widths(lib, orc, features, weighted):
    crow, col = random_csr(300, 12, seed=features, hubs={7: 900, 150: 64})
    x = dense(300, features, seed=1)
    val = weights(col.numel(), 2) if weighted else None
    exact = orc.spmm(to_np(crow), to_np(col), to_np(val), to_np(x))
    for tile in (64, 128):
        y = run_spmm(lib, crow, col, val, x, tile=tile, warps=8, threshold=64)
        assert_close(orc, y, exact, crow)


@pytest.mark.parametrize("features", [3, 32, 64, 100, 128, 256, 512])
@pytest.mark.parametrize("weighted", [False, True])
def test_spmm_packed_short_rows(lib, orc, features, weighted):
    """ASG_FLAG_PACK_SHORT_ROWS: rows under 32 edges one per lane group - every degree from 0 to 31 (and
    so every lane-group fill), with and without accumulation into an existing output."""
    rows = 520
    counts = torch.arange(rows) % 32
    counts[5], counts[300] = 700, 45
    crow, col = csr_from_counts(counts, rows, seed=features)
    x = dense(rows, features, seed=2)
    val = weights(col.numel(), 3) if weighted else None
    exact = orc.spmm(to_np(crow), to_np(col), to_np(val), to_np(x))
    for tile in (64, 128):
        y = run_spmm(lib, crow, col, val, x, tile=tile, warps=4, threshold=256, flags=lib.FLAG_PACK_SHORT_ROWS)
        assert_close(orc, y, exact, crow)
        start = dense(rows, features, seed=9).cuda()
        y = run_spmm(lib, crow, col, val, x, tile=tile, warps=4, threshold=256,
                     flags=lib.FLAG_PACK_SHORT_ROWS | lib.FLAG_ACCUMULATE, y=start.clone())
        assert_close(orc, y, exact + start.double().cpu().numpy(), crow)


def test_bounded_wait_gives_up_and_reports(lib, orc, monkeypatch):
    """The give-up path of the hub staging: with ASG_FLAG_SELFTEST_STALL every stage announces 16 bytes that
    never arrive, so the wait runs out after its (shortened) limit; the kernel must return, leave status 1
    in the workspace, still produce the light rows, and the next ordinary call on the same workspace must
    be clean.  AUTOSAGE_CHECK_STATUS=1 turns the status into an exception."""
    crow, col = random_csr(600, 6, seed=12, hubs={17: 3000, 400: 1500})
    x = dense(600, 64, seed=4)
    dev = torch.device("cuda")
    crow_d, col_d, x_d = crow.to(dev), col.to(dev), x.to(dev)
    ws = torch.empty(lib.workspace_bytes(600), dtype=torch.uint8, device=dev)
    y = torch.full((600, 64), float("nan"), device=dev)
    lib.spmm(crow_d, col_d, None, x_d, y, feature_tile=64, warps=4, threshold=1024, flags=lib.FLAG_SELFTEST_STALL,
             workspace=ws)
    torch.cuda.synchronize()
    assert lib.workspace_status(ws) == 1
    exact = orc.spmm(to_np(crow), to_np(col), None, to_np(x))
    light = torch.ones(600, dtype=torch.bool)
    light[[17, 400]] = False
    assert np.abs(y.cpu().numpy()[light.numpy()] - exact[light.numpy()]).max() < 1e-3   # light rows were computed
    assert bool(torch.isnan(y[17]).all()) and bool(torch.isnan(y[400]).all())             # hub rows were not
    monkeypatch.setenv("AUTOSAGE_CHECK_STATUS", "1")
    with pytest.raises(RuntimeError, match="gave up a bounded wait"):
        lib.spmm(crow_d, col_d, None, x_d, y, feature_tile=64, warps=4, threshold=1024, flags=lib.FLAG_SELFTEST_STALL,
                 workspace=ws)
    monkeypatch.delenv("AUTOSAGE_CHECK_STATUS")
    y = run_spmm(lib, crow, col, None, x, tile=64, warps=4, threshold=1024, ws=ws)      # asserts status == 0
    assert_close(orc, y, exact, crow)


@pytest.mark.parametrize("tile", [32, 64, 128, 256])
@pytest.mark.parametrize("warps", [2, 4, 8, 16])
def test_spmm_tile_and_warp_grid(lib, orc, tile, warps):
    crow, col = random_csr(257, 20, seed=tile + warps, hubs={0: 3000, 100: 1500, 256: 700})
    x = dense(257, 200, seed=3)
    val = weights(col.numel(), 4)
    exact = orc.spmm(to_np(crow), to_np(col), to_np(val), to_np(x))
    y = run_spmm(lib, crow, col, val, x, tile=tile, warps=warps, threshold=500)
    assert_close(orc, y, exact, crow)


@pytest.mark.parametrize("flags_name", ["default", "no_vec4", "no_bulk", "no_vec4_no_bulk"])
def test_spmm_code_paths(lib, orc, flags_name):
    flags = {"default": 0, "no_vec4": lib.FLAG_NO_VEC4, "no_bulk": lib.FLAG_NO_BULK_STAGE,
             "no_vec4_no_bulk": lib.FLAG_NO_VEC4 | lib.FLAG_NO_BULK_STAGE}[flags_name]
    crow, col = random_csr(400, 10, seed=9, hubs={3: 5000, 399: 2049})
    x = dense(400, 128, seed=5)
    val = weights(col.numel(), 6)
    exact = orc.spmm(to_np(crow), to_np(col), to_np(val), to_np(x))
    y = run_spmm(lib, crow, col, val, x, threshold=100, flags=flags)
    assert_close(orc, y, exact, crow)
    y = run_spmm(lib, crow, col, None, x, threshold=100, flags=flags)
    assert_close(orc, y, orc.spmm(to_np(crow), to_np(col), None, to_np(x)), crow)


def test_spmm_degrees_at_bin_and_chunk_edges(lib, orc):
    # 32-edge batches, the 4-edge staging alignment, and the 128*warps staging chunk
    degrees = [0, 1, 2, 3, 4, 5, 7, 8, 9, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 256, 257, 511, 512, 513,
               1023, 1024, 1025, 1026, 1027, 2047, 2048, 2049, 4095, 4096, 4097, 0, 0, 6]
    crow, col = csr_from_counts(degrees, len(degrees), seed=77)
    x = dense(len(degrees), 96, seed=8)
    val = weights(col.numel(), 9)
    exact = orc.spmm(to_np(crow), to_np(col), to_np(val), to_np(x))
    for threshold in (1, 32, 33, 1024, 100000):
        for warps in (2, 8):
            y = run_spmm(lib, crow, col, val, x, tile=64, warps=warps, threshold=threshold)
            assert_close(orc, y, exact, crow)


def test_spmm_empty_shapes(lib, orc):
    # all rows empty
    crow = torch.zeros(50, dtype=torch.long)
    col = torch.zeros(0, dtype=torch.long)
    x = dense(49, 64, seed=1)
    y = run_spmm(lib, crow, col, None, x)
    assert torch.equal(y.cpu(), torch.zeros(49, 64))
    # zero rows / zero features: nothing to launch, status OK
    lib.check(lib.library().asg_spmm_csr_ex(None, None, None, None, None, 0, 0, 64, 64, 8, 16, 0, None, 0, None))
    lib.check(lib.library().asg_spmm_csr_ex(None, None, None, None, None, 10, 0, 0, 64, 8, 16, 0, None, 0, None))


def test_spmm_misaligned_operands_take_scalar_path(lib, orc):
    crow, col = random_csr(200, 9, seed=31, hubs={5: 1200})
    x = dense(200, 128, seed=2)
    val = weights(col.numel(), 3)
    exact = orc.spmm(to_np(crow), to_np(col), to_np(val), to_np(x))
    x_off = misaligned_copy(x.cuda())          # 4-byte offset: neither 16- nor 32-byte aligned
    assert x_off.data_ptr() % 16 != 0
    y = run_spmm(lib, crow, col, val, x_off, threshold=100)
    assert_close(orc, y, exact, crow)
    x16 = misaligned_copy(x.cuda(), 4)         # 16-byte aligned only: 128-bit loads
    assert x16.data_ptr() % 32 != 0 and x16.data_ptr() % 16 == 0
    y = run_spmm(lib, crow, col, val, x16, threshold=100)
    assert_close(orc, y, exact, crow)
    # misaligned col/val force the plain-load staging of hub rows
    col_off = misaligned_copy(col.cuda())
    val_off = misaligned_copy(val.cuda())
    assert col_off.data_ptr() % 16 != 0
    y = run_spmm(lib, crow, col_off, val_off, x, threshold=100)
    assert_close(orc, y, exact, crow)


def test_spmm_accumulate_and_plan_reuse(lib, orc):
    crow, col = random_csr(500, 14, seed=41, hubs={10: 2500})
    x = dense(500, 160, seed=4)
    val = weights(col.numel(), 5)
    exact = orc.spmm(to_np(crow), to_np(col), to_np(val), to_np(x))
    ws = torch.empty(lib.workspace_bytes(500), dtype=torch.uint8, device="cuda")
    y = run_spmm(lib, crow, col, val, x, threshold=200, ws=ws)
    assert_close(orc, y, exact, crow)
    # same workspace, plan kept: three more launches, the last two accumulating
    y2 = run_spmm(lib, crow, col, val, x, threshold=200, ws=ws, flags=lib.FLAG_PLAN_READY)
    assert torch.equal(y, y2)
    y3 = run_spmm(lib, crow, col, val, x, threshold=200, ws=ws, flags=lib.FLAG_PLAN_READY | lib.FLAG_ACCUMULATE, y=y2)
    assert_close(orc, y3, 2 * exact, crow)


def test_spmm_rectangular_column_space(lib, orc):
    """Rows of a shard index a taller X (the multi-GPU layout): 64 rows, 1000 columns."""
    counts = torch.randint(0, 40, (64,), generator=torch.Generator().manual_seed(2))
    counts[3] = 700
    crow, col = csr_from_counts(counts, 1000, seed=5)
    x = dense(1000, 128, seed=6)
    val = weights(col.numel(), 7)
    exact = orc.spmm(to_np(crow), to_np(col), to_np(val), to_np(x))
    y = run_spmm(lib, crow, col, val, x, threshold=128)
    assert_close(orc, y, exact, crow)


def test_spmm_entry_points_agree(lib, orc):
    crow, col = random_csr(350, 11, seed=51, hubs={1: 2600})
    x = dense(350, 128, seed=7).cuda()
    val = weights(col.numel(), 8).cuda()
    crow_d, col_d = crow.cuda(), col.cuda()
    exact = orc.spmm(to_np(crow), to_np(col), to_np(val), to_np(x))
    ws = torch.empty(lib.workspace_bytes(350), dtype=torch.uint8, device="cuda")
    y_plain = torch.empty_like(x)
    lib.spmm_plain(crow_d, col_d, val, x, y_plain, ws)
    y_split = torch.empty_like(x)
    lib.spmm_split_strict(crow_d, col_d, val, x, y_split, 64, 4, 300, ws)
    torch.cuda.synchronize()
    assert_close(orc, y_plain, exact, crow)
    assert_close(orc, y_split, exact, crow)
    with pytest.raises(RuntimeError, match="hub_threshold must be positive"):
        lib.spmm_split_strict(crow_d, col_d, val, x, y_split, 64, 4, 0, ws)
    with pytest.raises(RuntimeError, match="workspace"):
        lib.spmm_plain(crow_d, col_d, val, x, y_plain, ws[:128])


# ----------------------------------------------------------------------------------------- SDDMM
def run_sddmm(lib, crow, col, q, k, *, warps=8, threshold=64, flags=0):
    dev = torch.device("cuda")
    out = torch.full((col.numel(),), float("nan"), device=dev)
    ws = torch.empty(lib.workspace_bytes(crow.numel() - 1), dtype=torch.uint8, device=dev)
    q_d = q if q.is_cuda else q.to(dev)
    k_d = k if k.is_cuda else k.to(dev)
    lib.sddmm(crow.to(dev), col.to(dev), q_d, k_d, out, warps=warps, threshold=threshold, flags=flags, workspace=ws)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("features", [1, 3, 4, 32, 64, 100, 113, 128, 192, 256, 512, 640, 1024])
def test_sddmm_feature_widths(lib, orc, features):
    crow, col = random_csr(260, 10, seed=features + 1, hubs={9: 1100, 200: 65})
    q, k = dense(260, features, 11), dense(260, features, 12)
    exact = orc.sddmm(to_np(crow), to_np(col), to_np(q), to_np(k))
    for warps, threshold in ((8, 64), (2, 1), (4, 100000)):
        out = run_sddmm(lib, crow, col, q, k, warps=warps, threshold=threshold)
        ok, ratio = orc.within_tolerance(out.cpu().numpy(), exact, to_np(crow), per_edge=True, rtol=RTOL, atol=ATOL)
        assert ok, f"worst error/bound {ratio:.3f}"


def test_sddmm_scalar_and_misaligned_paths(lib, orc):
    crow, col = random_csr(180, 8, seed=61, hubs={4: 800})
    q, k = dense(180, 128, 13), dense(180, 128, 14)
    exact = orc.sddmm(to_np(crow), to_np(col), to_np(q), to_np(k))
    for out in (run_sddmm(lib, crow, col, q, k, flags=lib.FLAG_NO_VEC4),
                run_sddmm(lib, crow, col, misaligned_copy(q.cuda()), k),
                run_sddmm(lib, crow, col, q, misaligned_copy(k.cuda(), 4))):
        ok, ratio = orc.within_tolerance(out.cpu().numpy(), exact, to_np(crow), per_edge=True, rtol=RTOL, atol=ATOL)
        assert ok, f"worst error/bound {ratio:.3f}"


def test_sddmm_batch_edges(lib, orc):
    degrees = [0, 1, 31, 32, 33, 63, 64, 65, 255, 256, 257, 0, 1023, 1024, 1025, 2]
    crow, col = csr_from_counts(degrees, len(degrees), seed=3)
    q, k = dense(len(degrees), 64, 15), dense(len(degrees), 64, 16)
    exact = orc.sddmm(to_np(crow), to_np(col), to_np(q), to_np(k))
    for warps, threshold in ((2, 32), (8, 33), (16, 1), (4, 5000)):
        out = run_sddmm(lib, crow, col, q, k, warps=warps, threshold=threshold)
        ok, ratio = orc.within_tolerance(out.cpu().numpy(), exact, to_np(crow), per_edge=True, rtol=RTOL, atol=ATOL)
        assert ok, f"worst error/bound {ratio:.3f}"


# --------------------------------------------------------------------------- softmax & attention
def test_row_softmax_matches_oracle(lib, orc):
    degrees = [0, 1, 2, 31, 32, 33, 700, 5, 0, 3000, 64]
    crow, _ = csr_from_counts(degrees, 11, seed=1)
    scores = 11.0 * dense(int(crow[-1]), 1, 17).flatten()   # peaked rows, like unscaled F=128 scores
    exact = orc.row_softmax(to_np(crow), to_np(scores).astype(np.float64))
    for warps, threshold in ((8, 512), (2, 1), (4, 100000)):
        probs = torch.empty_like(scores, device="cuda")
        ws = torch.empty(lib.workspace_bytes(11), dtype=torch.uint8, device="cuda")
        lib.row_softmax(crow.cuda(), scores.cuda(), probs, warps=warps, threshold=threshold, flags=0, workspace=ws)
        torch.cuda.synchronize()
        np.testing.assert_allclose(probs.cpu().numpy(), exact, rtol=2e-5, atol=1e-7)
        sums = torch.segment_reduce(probs.cpu(), "sum", lengths=torch.tensor(degrees))
        nonempty = torch.tensor(degrees) > 0
        assert torch.allclose(sums[nonempty], torch.ones(int(nonempty.sum())), atol=1e-5)


@pytest.mark.parametrize("features", [4, 32, 64, 100, 128, 256, 512])
@pytest.mark.parametrize("scale", [1.0, None])
def test_fused_attention_matches_three_pass_oracle(lib, orc, features, scale):
    crow, col = random_csr(220, 9, seed=features, hubs={2: 1500, 100: 66})
    q, k, v = dense(220, features, 21), dense(220, features, 22), dense(220, features, 23)
    s = float(features) ** -0.5 if scale is None else scale
    exact = orc.attention(to_np(crow), to_np(col), to_np(q), to_np(k), to_np(v), s)
    for warps, threshold in ((8, 64), (2, 1), (4, 100000)):
        out = torch.full((220, features), float("nan"), device="cuda")
        ws = torch.empty(lib.workspace_bytes(220), dtype=torch.uint8, device="cuda")
        lib.attention(crow.cuda(), col.cuda(), q.cuda(), k.cuda(), v.cuda(), out, scale=s, warps=warps,
                      threshold=threshold, flags=0, workspace=ws)
        torch.cuda.synchronize()
        assert_close(orc, out, exact, crow)


@pytest.mark.parametrize("features", [32, 64, 128, 256, 512])
def test_fused_attention_splits_mega_rows_and_packs_short_rows(lib, orc, features):
    """Rows of 4,096 edges or more are cut into segments that different CTAs process and merge (with the
    larger workspace; one CTA per row with the small one); rows of fewer than 32 edges - every degree
    from 0 to 31, so every lane-group fill of the packed short-row kernel - share warps."""
    rows = 700
    counts = torch.arange(rows) % 32                      # all short degrees, including empty rows
    counts[3], counts[250], counts[699], counts[40] = 9000, 4096, 5000, 4095
    crow, col = csr_from_counts(counts, rows, seed=features)
    q, k, v = dense(rows, features, 31), dense(rows, features, 32), dense(rows, features, 33)
    scale = float(features) ** -0.5
    exact = orc.attention(to_np(crow), to_np(col), to_np(q), to_np(k), to_np(v), scale)
    sizes = (lib.workspace_bytes(rows) + lib.attention_extra_bytes(rows), lib.workspace_bytes(rows))
    assert sizes[0] > sizes[1]
    for size in sizes:
        for warps, threshold in ((8, 512), (4, 2048), (2, 100000)):
            out = torch.full((rows, features), float("nan"), device="cuda")
            ws = torch.empty(size, dtype=torch.uint8, device="cuda")
            for _ in range(2):                            # twice: the completion counters are reset per call
                lib.attention(crow.cuda(), col.cuda(), q.cuda(), k.cuda(), v.cuda(), out, scale=scale, warps=warps,
                              threshold=threshold, flags=0, workspace=ws)
            torch.cuda.synchronize()
            assert_close(orc, out, exact, crow)


def test_fused_attention_rejects_wide_rows(lib):
    crow, col = random_csr(8, 2, seed=1)
    t = torch.zeros(8, 516, device="cuda")
    ws = torch.empty(lib.workspace_bytes(8), dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError, match="512 features"):
        lib.attention(crow.cuda(), col.cuda(), t, t, t, torch.empty_like(t), scale=1.0, warps=8, threshold=64,
                      flags=0, workspace=ws)


# ----------------------------------------------------------------------------- golden fixtures
@pytest.mark.parametrize("case", ["tiny", "ragged", "hub", "wide"])
def test_kernels_match_reference_outputs(lib, orc, golden, case):
    """Outputs of the reference itself (float64 CPU run) are the expected values here."""
    vec, _ = golden
    crow, col = torch.from_numpy(vec[f"{case}.crow"]), torch.from_numpy(vec[f"{case}.col"])
    x, q, k = (torch.from_numpy(vec[f"{case}.{n}"]) for n in ("x", "q", "k"))
    val = torch.from_numpy(vec[f"{case}.val"])
    y = run_spmm(lib, crow, col, val, x, threshold=32)
    assert_close(orc, y, vec[f"{case}.spmm_weighted"], crow)
    y = run_spmm(lib, crow, col, None, x, threshold=32)
    assert_close(orc, y, vec[f"{case}.spmm_unweighted"], crow)
    out = run_sddmm(lib, crow, col, q, k, threshold=32)
    ok, ratio = orc.within_tolerance(out.cpu().numpy(), vec[f"{case}.sddmm"], to_np(crow), per_edge=True)
    assert ok, ratio
    att = torch.empty(x.shape, device="cuda")
    ws = torch.empty(lib.workspace_bytes(crow.numel() - 1), dtype=torch.uint8, device="cuda")
    lib.attention(crow.cuda(), col.cuda(), q.cuda(), k.cuda(), x.cuda(), att, scale=1.0, warps=8, threshold=32,
                  flags=0, workspace=ws)
    torch.cuda.synchronize()
    assert_close(orc, att, vec[f"{case}.attention"], crow)


# ------------------------------------------------------------------------- size-independent checks
def test_full_size_spmm_properties():
    """The Reddit-sized graph at full size (232,965 rows, ~114.6 M nnz): properties that need no
    oracle run. With X = ones, Y[i, :] is the sum of the row's weights; SpMM is linear in X."""
    import autosage_b200
    from benchlib import synthetic as syn

    assert autosage_b200.load_native()
    dev = torch.device("cuda")
    crow, col, info = syn.powerlaw_csr(syn.REDDIT_LIKE, device=dev)
    assert abs(info["nnz"] - syn.REDDIT_LIKE.target_nnz) <= 0.005 * syn.REDDIT_LIKE.target_nnz
    val = syn.edge_values(info["nnz"], device=dev)
    n = info["rows"]
    degree = crow[1:] - crow[:-1]
    row_sum = torch.segment_reduce(val.double(), "sum", lengths=degree)
    ones = torch.ones(n, 128, device=dev)
    y = torch.ops.autosage.spmm_csr_split(crow, col, val, ones, 128, 8, 1566)
    err = (y.double() - row_sum[:, None]).abs()
    bound = 1e-5 * row_sum[:, None].abs() + 1e-5 * degree.double().sqrt()[:, None]
    assert bool((err <= bound).all()), float((err / bound).max())
    assert bool((y == y[:, :1]).all())  # every feature column saw the same arithmetic
    # linearity: A(2a - b) == 2 A a - A b within rounding of the three results
    a, b = syn.dense(n, 64, 5, dev), syn.dense(n, 64, 6, dev)
    lhs = torch.ops.autosage.spmm_csr(crow, col, val, 2 * a - b)
    rhs = 2 * torch.ops.autosage.spmm_csr(crow, col, val, a) - torch.ops.autosage.spmm_csr(crow, col, val, b)
    scale = degree.double().sqrt()[:, None]
    assert float(((lhs - rhs).abs().double() / (scale * 1e-4 + 1e-4 * rhs.abs().double())).max()) <= 1.0
    # SDDMM: with Q = K = ones every edge scores F; softmax of equal scores is 1/degree
    scores = torch.ops.autosage.sddmm_csr_split(crow, col, ones, ones, 8, 1566)
    assert bool((scores == 128.0).all())
    probs = autosage_b200._auto._csr_row_softmax(crow, scores)
    expect = torch.repeat_interleave(1.0 / degree.double(), degree)
    assert float((probs.double() - expect).abs().max()) <= 1e-6


def test_full_size_attention_properties():
    """The ogbn-arxiv-sized graph (169,343 rows, ~2.48 M nnz, F = 128): with V constant per column the
    output of a softmax-weighted average is that constant; fused equals the three-pass pipeline."""
    import autosage_b200
    from benchlib import synthetic as syn

    dev = torch.device("cuda")
    crow, col, info = syn.powerlaw_csr(syn.ARXIV_LIKE, device=dev)
    n = info["rows"]
    q, k = syn.dense(n, 128, 1, dev), syn.dense(n, 128, 2, dev)
    v = torch.arange(128, device=dev, dtype=torch.float32).repeat(n, 1)
    scale = 128 ** -0.5
    fused, _ = autosage_b200.csr_attention_forward(crow, col, q, k, v, scale=scale, fused=True)
    nonempty = (crow[1:] - crow[:-1]) > 0
    assert torch.allclose(fused[nonempty], v[nonempty], rtol=1e-5, atol=1e-4)
    v2 = syn.dense(n, 128, 3, dev)
    fused, info_f = autosage_b200.csr_attention_forward(crow, col, q, k, v2, scale=scale, fused=True)
    unfused, info_u = autosage_b200.csr_attention_forward(crow, col, q, k, v2, scale=scale, fused=False)
    degree = (crow[1:] - crow[:-1]).double().clamp_min(1).sqrt()[:, None]
    err = (fused.double() - unfused.double()).abs()
    assert bool((err <= 2e-5 * unfused.abs().double() + 2e-5 * degree).all())
    assert set(info_f) >= {"sddmm", "spmm"} and set(info_u) >= {"sddmm", "spmm"}


def test_offsets_beyond_32_bits(lib):
    """N*F above 2^31 elements: the reference multiplies 32-bit ints when it indexes X and Y
    (csrc/spmm_csr_vec4.cu:47,49); these kernels must not.  Few edges, so the check itself is cheap."""
    n, f = 1_100_000, 2048                      # 2.25e9 elements per dense operand (9 GB each)
    free, _ = torch.cuda.mem_get_info()
    if free < 24 * 2**30:
        pytest.skip("needs 24 GB of free device memory")
    dev = torch.device("cuda")
    rows = torch.tensor([0, 1, n // 2, n - 2, n - 1], device=dev)
    cols = torch.tensor([n - 1, n - 1, 7, n // 2 + 3, n - 1], device=dev)
    counts = torch.zeros(n, dtype=torch.long, device=dev)
    counts[rows] = 1
    crow = torch.zeros(n + 1, dtype=torch.long, device=dev)
    torch.cumsum(counts, 0, out=crow[1:])
    x = torch.zeros(n, f, device=dev)
    for c in cols.unique().tolist():
        x[c] = torch.arange(f, device=dev, dtype=torch.float32) + float(c % 1000)
    y = torch.full((n, f), float("nan"), device=dev)
    ws = torch.empty(lib.workspace_bytes(n), dtype=torch.uint8, device=dev)
    lib.spmm(crow, cols, None, x, y, feature_tile=128, warps=8, threshold=64, flags=0, workspace=ws)
    torch.cuda.synchronize()
    for r, c in zip(rows.tolist(), cols.tolist()):
        assert torch.equal(y[r], x[c]), (r, c)
    assert float(y[3].abs().max()) == 0.0 and float(y[n - 3].abs().max()) == 0.0   # empty rows are zeroed
    out = torch.empty(5, device=dev)
    lib.sddmm(crow, cols, x, x, out, warps=8, threshold=64, flags=0, workspace=ws)
    torch.cuda.synchronize()
    expected = torch.stack([(x[r].double() * x[c].double()).sum() for r, c in zip(rows.tolist(), cols.tolist())])
    assert torch.allclose(out.double(), expected, rtol=1e-5)


def test_row_bias_epilogue(lib):
    for rows, cols, offset in ((1000, 256, 0), (333, 100, 0), (77, 5, 0), (64, 64, 1)):
        out = dense(rows, cols, 1).cuda()
        bias = dense(1, cols + offset, 2).flatten().cuda()[offset:]   # offset 1: misaligned -> scalar path
        expected = out + bias
        lib.add_row_bias(out, bias.contiguous() if offset == 0 else bias)
        torch.cuda.synchronize()
        assert torch.equal(out, expected)
    lib.check(lib.library().asg_add_row_bias(None, None, 0, 16, None))


def test_sddmm_feature_passes_on_a_large_key_matrix(lib, orc):
    """K above 64 MB switches SDDMM to one launch per 64-feature tile with partial sums kept in the
    output; the result must match the oracle and the single-launch form."""
    n, f = 140_000, 128                                  # K = 71.7 MB
    gen = torch.Generator().manual_seed(5)
    counts = torch.randint(0, 5, (n,), generator=gen)
    counts[100], counts[70_000], counts[139_999] = 3000, 900, 40   # a hub, two medium rows
    crow, col = csr_from_counts(counts, n, seed=6)
    q, k = dense(n, f, 7), dense(n, f, 8)
    exact = orc.sddmm(to_np(crow), to_np(col), to_np(q), to_np(k))
    tiled = run_sddmm(lib, crow, col, q, k, warps=8, threshold=1024)
    single = run_sddmm(lib, crow, col, q, k, warps=8, threshold=1024, flags=lib.FLAG_NO_TILE_PASSES)
    for out in (tiled, single):
        ok, ratio = orc.within_tolerance(out.cpu().numpy(), exact, to_np(crow), per_edge=True, rtol=RTOL, atol=ATOL)
        assert ok, f"worst error/bound {ratio:.3f}"
    assert not torch.isnan(tiled).any()


def test_spmm_feature_range(lib, orc):
    """Only a band of output columns is computed; the rest of y is left untouched."""
    crow, col = random_csr(500, 12, seed=3, hubs={4: 2000})
    x = dense(500, 192, 1)
    val = weights(col.numel(), 2)
    exact = orc.spmm(to_np(crow), to_np(col), to_np(val), to_np(x))
    dev = torch.device("cuda")
    crow_d, col_d, val_d, x_d = crow.to(dev), col.to(dev), val.to(dev), x.to(dev)
    ws = torch.empty(lib.workspace_bytes(500), dtype=torch.uint8, device=dev)
    y = torch.full((500, 192), float("nan"), device=dev)
    for begin, count, tile in ((64, 64, 64), (0, 64, 32), (128, 64, 64)):
        lib.spmm_range(crow_d, col_d, val_d, x_d, y, feature_begin=begin, feature_count=count, feature_tile=tile,
                       warps=4, threshold=256, flags=0, workspace=ws)
    torch.cuda.synchronize()
    assert_close(orc, y, exact, crow)
    y2 = torch.full((500, 192), float("nan"), device=dev)
    lib.spmm_range(crow_d, col_d, val_d, x_d, y2, feature_begin=128, feature_count=64, feature_tile=64, warps=4,
                   threshold=256, flags=0, workspace=ws)
    torch.cuda.synchronize()
    assert bool(torch.isnan(y2[:, :128]).all()) and not bool(torch.isnan(y2[:, 128:]).any())
    with pytest.raises(RuntimeError, match="feature_tile boundary"):
        lib.spmm_range(crow_d, col_d, val_d, x_d, y2, feature_begin=32, feature_count=64, feature_tile=64, warps=4,
                       threshold=256, flags=0, workspace=ws)
    # pitched copy of a band of columns
    dst = torch.zeros(500, 192, device=dev)
    lib.copy_columns(dst, x_d, 64, 32)
    torch.cuda.synchronize()
    assert torch.equal(dst[:, 64:96], x_d[:, 64:96]) and float(dst[:, :64].abs().sum()) == 0.0


@pytest.mark.parametrize("rows,k,n,with_bias", [(1, 128, 256, True), (127, 128, 256, True), (129, 64, 16, True),
                                                 (1000, 100, 36, False), (5000, 256, 256, True), (0, 128, 256, True)])
def test_linear_bias_matches_float64(lib, rows, k, n, with_bias):
    """The tensor-core Linear keeps float32 accuracy (rtol 1e-5, atol 1e-5 * sqrt(in_features) against float64)."""
    dev = torch.device("cuda")
    gen = torch.Generator().manual_seed(rows * 7 + k)
    x = torch.randn(rows, k, generator=gen).to(dev)
    weight = (torch.randn(n, k, generator=gen) / k ** 0.5).to(dev)
    bias = torch.randn(n, generator=gen).to(dev) if with_bias else None
    out = torch.full((rows, n), float("nan"), device=dev)
    lib.linear_bias(x, weight, bias, out)
    torch.cuda.synchronize()
    exact = x.double() @ weight.double().t()
    if with_bias:
        exact = exact + bias.double()
    if rows:
        err = (out.double() - exact).abs()
        bound = 1e-5 * exact.abs() + 1e-5 * k ** 0.5
        assert bool((err <= bound).all()), float((err / bound).max())
        # at least as close to float64 as the float32 library product
        library = torch.mm(x, weight.t()) + (bias if with_bias else 0)
        assert float(err.max()) <= 2.0 * float((library.double() - exact).abs().max()) + 1e-7


@pytest.mark.parametrize("rows,k,n,with_bias", [(1, 128, 256, True), (127, 128, 256, True), (128, 64, 32, True),
                                                 (129, 64, 32, False), (1000, 128, 64, True), (5000, 256, 256, True),
                                                 (70001, 192, 96, True), (0, 128, 256, True)])
def test_linear_bias_umma_matches_float64(lib, rows, k, n, with_bias):
    """The hand-written tcgen05 Linear: rtol 1e-5, atol 1e-5 * sqrt(in_features) against float64, rows
    past the last full 128-row tile untouched, status word clear."""
    dev = torch.device("cuda")
    gen = torch.Generator().manual_seed(rows * 7 + k + n)
    x = torch.randn(rows, k, generator=gen).to(dev)
    weight = (torch.randn(n, k, generator=gen) / k ** 0.5).to(dev)
    bias = torch.randn(n, generator=gen).to(dev) if with_bias else None
    guard_rows = 3
    whole = torch.full((rows + guard_rows, n), float("nan"), device=dev)
    out = whole[:rows]
    ws = lib.linear_bias_umma(x, weight, bias, out)
    torch.cuda.synchronize()
    if rows:
        assert lib.workspace_status(ws) == 0
    assert bool(torch.isnan(whole[rows:]).all())          # nothing written past the last row
    exact = x.double() @ weight.double().t()
    if with_bias:
        exact = exact + bias.double()
    if rows:
        err = (out.double() - exact).abs()
        bound = 1e-5 * exact.abs() + 1e-5 * k ** 0.5
        # all six piece products go into one tensor-memory accumulator (the tensor core truncates each
        # accumulation), which costs a few more ulps than cuBLAS SGEMM: still a quarter of the bound
        assert bool((err <= 0.25 * bound).all()), float((err / bound).max())
    # a second call with the same workspace and different operands (the ring phases start afresh)
    if rows:
        x2 = torch.randn(rows, k, generator=gen).to(dev)
        lib.linear_bias_umma(x2, weight, bias, out, ws)
        exact2 = x2.double() @ weight.double().t() + (bias.double() if with_bias else 0)
        err2 = (out.double() - exact2).abs()
        assert bool((err2 <= 1e-5 * exact2.abs() + 1e-5 * k ** 0.5).all())


def test_linear_bias_umma_rejects_other_sizes(lib):
    dev = torch.device("cuda")
    assert lib.linear_umma_supported(128, 256) and lib.linear_umma_supported(64, 32)
    assert not lib.linear_umma_supported(100, 256) and not lib.linear_umma_supported(128, 36)
    assert not lib.linear_umma_supported(128, 512)
    x, weight, out = torch.zeros(8, 100, device=dev), torch.zeros(36, 100, device=dev), torch.zeros(8, 36, device=dev)
    with pytest.raises(RuntimeError, match="multiples of 64"):
        lib.linear_bias_umma(x, weight, None, out)


def test_linear_bias_umma_bounded_wait_gives_up_and_reports(lib):
    """Self-test flag: the MMA thread's wait before its second tile is pointed at a barrier nothing arrives
    on; it runs out after 20 ms, every warp leaves through the common exit (tensor memory freed, copies in
    flight waited for) and the status word is 2.  The next call on the same workspace is complete."""
    dev = torch.device("cuda")
    rows, k, n = 50_000, 128, 256                         # more tiles than SMs: every CTA owns a second tile
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(rows, k, generator=gen).to(dev)
    weight = (torch.randn(n, k, generator=gen) / k ** 0.5).to(dev)
    bias = torch.randn(n, generator=gen).to(dev)
    out = torch.zeros(rows, n, device=dev)
    ws = lib.linear_bias_umma(x, weight, bias, out, flags=lib.FLAG_SELFTEST_STALL)
    torch.cuda.synchronize()
    assert lib.workspace_status(ws) == 2
    lib.linear_bias_umma(x, weight, bias, out, ws)
    torch.cuda.synchronize()
    assert lib.workspace_status(ws) == 0
    exact = x.double() @ weight.double().t() + bias.double()
    assert bool(((out.double() - exact).abs() <= 1e-5 * exact.abs() + 1e-5 * k ** 0.5).all())


def test_linear_bias_rejects_unaligned_sizes(lib):
    dev = torch.device("cuda")
    x, weight, out = torch.zeros(8, 6, device=dev), torch.zeros(4, 6, device=dev), torch.zeros(8, 4, device=dev)
    with pytest.raises(RuntimeError, match="multiples of 4"):
        lib.linear_bias(x, weight, None, out)


def test_layer_linear_uses_tensor_core_path(lib, monkeypatch):
    """apply_linear: same result through the tensor-core route and the cuBLAS route."""
    from autosage_b200 import conv

    dev = torch.device("cuda")
    torch.manual_seed(0)
    linear = torch.nn.Linear(128, 256).to(dev)
    x = dense(3000, 128, 9).to(dev)
    with torch.no_grad():
        fast = conv.apply_linear(linear, x)
        monkeypatch.setenv("AUTOSAGE_LINEAR", "cublas")
        plain = conv.apply_linear(linear, x)
    assert torch.allclose(fast, plain, rtol=1e-5, atol=1e-5 * 128 ** 0.5)
    monkeypatch.delenv("AUTOSAGE_LINEAR")
    monkeypatch.setenv("AUTOSAGE_LINEAR_KERNEL", "cutlass")
    with torch.no_grad():
        other = conv.apply_linear(linear, x.detach())
    assert torch.allclose(fast, other, rtol=1e-5, atol=1e-5 * 128 ** 0.5)
    monkeypatch.delenv("AUTOSAGE_LINEAR_KERNEL")
    y = conv.apply_linear(linear, x.requires_grad_())          # gradient wanted: differentiable route
    y.sum().backward()
    assert x.grad is not None and linear.weight.grad is not None


@pytest.mark.parametrize("nodes,edges,rows_by,dtype", [(1, 5, "dst", torch.long), (7, 0, "dst", torch.long),
                                                       (100, 1000, "dst", torch.int32), (257, 5000, "src", torch.long),
                                                       (5000, 200_000, "dst", torch.long),
                                                       (300_000, 1_500_000, "dst", torch.long)])
def test_device_csr_build_is_bit_exact(lib, monkeypatch, nodes, edges, rows_by, dtype):
    """The device COO -> CSR build returns the integers of the torch formulation (stable within a row),
    the edge ordering, and the permuted weights."""
    from autosage_b200.utils import csr as csr_utils

    gen = torch.Generator().manual_seed(nodes + edges)
    edge_index = torch.randint(0, nodes, (2, edges), generator=gen).to(dtype)
    if edges > 10:
        edge_index[1, : edges // 3] = edge_index[1, 0]      # a hub destination and many duplicates
    weight = torch.rand(edges, generator=gen)
    monkeypatch.setenv("AUTOSAGE_CSR_BUILD", "torch")
    want = csr_utils.csr_with_order(edge_index, nodes, rows_by=rows_by, want_order=True, edge_weight=weight)
    monkeypatch.setenv("AUTOSAGE_CSR_BUILD", "native")
    got = csr_utils.csr_with_order(edge_index.cuda(), nodes, rows_by=rows_by, want_order=True, edge_weight=weight.cuda())
    for a, b in zip(got, want):
        assert a.dtype == b.dtype and torch.equal(a.cpu(), b)
    crow, col = csr_utils.edge_index_to_csr(edge_index.cuda(), nodes, rows_by=rows_by)
    assert torch.equal(crow.cpu(), want[0]) and torch.equal(col.cpu(), want[1])
    from oracle import oracle as orc

    o_crow, o_col, o_perm = orc.edge_index_to_csr(edge_index.long().numpy(), nodes, rows_by)
    assert np.array_equal(got[2].cpu().numpy(), o_perm)
    assert np.array_equal(crow.cpu().numpy(), o_crow) and np.array_equal(col.cpu().numpy(), o_col)


def test_layer_forward_with_device_csr_build(lib):
    """AutoSAGEConv from an edge list (weighted and unweighted) against the dense formulation."""
    from autosage_b200 import AutoSAGEConv

    dev = torch.device("cuda")
    gen = torch.Generator().manual_seed(11)
    n, e = 2000, 30000
    edge_index = torch.randint(0, n, (2, e), generator=gen)
    weight = torch.rand(e, generator=gen)
    x = torch.randn(n, 64, generator=gen)
    torch.manual_seed(0)
    layer = AutoSAGEConv(64, 32, mode="native").to(dev)
    dense_a = torch.zeros(n, n, dtype=torch.float64)
    dense_a.index_put_((edge_index[1], edge_index[0]), weight.double(), accumulate=True)
    expected = (dense_a @ x.double()) @ layer.linear.weight.detach().cpu().double().t() + layer.linear.bias.detach().cpu().double()
    with torch.no_grad():
        out = layer(x.to(dev), edge_index.to(dev), weight.to(dev))
        again = layer(x.to(dev), edge_index.to(dev), weight.to(dev))
    assert torch.allclose(out.cpu().double(), expected, rtol=1e-4, atol=1e-3)
    assert torch.equal(out, again)
