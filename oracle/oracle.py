"""numpy front end of the C oracle (``csr_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import
this module; the product path (``autosage_b200``) never does.  Every function states the reference
code it restates (paths inside the AutoSAGE repository); parity of this oracle with the reference
itself is pinned by ``tests/golden/`` (vectors produced by running the reference, see
``tests/golden/generate.py``) and by the known answers of the reference's ``tests/test_cpu.py``.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "_ref" / "liboracle.so"

_LIB = None

_I64P = np.ctypeslib.ndpointer(dtype=np.int64, flags="C_CONTIGUOUS")
_I32P = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
_F32P = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_F64P = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")


def build(force: bool = False) -> Path:
    """Compile csr_oracle.c into oracle/_ref/liboracle.so (gcc, via the Makefile beside it)."""
    source = HERE / "csr_oracle.c"
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < source.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B", "all"], check=True, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT)
    return LIB_PATH


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        build()
        _LIB = ctypes.CDLL(str(LIB_PATH))
        _LIB.orc_threads.restype = ctypes.c_int
        _LIB.orc_set_threads.argtypes = [ctypes.c_int]
    return _LIB


def threads() -> int:
    return int(lib().orc_threads())


def set_threads(n: int) -> None:
    lib().orc_set_threads(int(n))


def _i64(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a), dtype=np.int64)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a), dtype=np.float32)


def spmm(crow, col, val, x, *, dtype=np.float64) -> np.ndarray:
    """Y = A X with A in CSR (autosage/ops.py:124-143, torch.sparse.mm on a CSR tensor).
    dtype float64 accumulates in double (accuracy oracle); float32 is the reference's CPU arithmetic."""
    crow, col, x = _i64(crow), _i64(col), _f32(x)
    n, f = crow.size - 1, x.shape[1]
    y = np.empty((n, f), dtype=dtype)
    fn = lib().orc_spmm_f64 if dtype == np.float64 else lib().orc_spmm_f32
    fn.argtypes = [_I64P, _I64P, ctypes.c_void_p, _F32P, _F64P if dtype == np.float64 else _F32P,
                   ctypes.c_int64, ctypes.c_int64]
    keep = None if val is None else _f32(val)
    fn(crow, col, None if keep is None else keep.ctypes.data_as(ctypes.c_void_p), x, y, n, f)
    return y


def sddmm(crow, col, q, k, *, dtype=np.float64) -> np.ndarray:
    """out[e] = <q[row(e)], k[col[e]]> (autosage/_auto.py:79-92, the gather-dot baseline)."""
    crow, col, q, k = _i64(crow), _i64(col), _f32(q), _f32(k)
    out = np.empty(col.size, dtype=dtype)
    fn = lib().orc_sddmm_f64 if dtype == np.float64 else lib().orc_sddmm_f32
    fn.argtypes = [_I64P, _I64P, _F32P, _F32P, _F64P if dtype == np.float64 else _F32P, ctypes.c_int64,
                   ctypes.c_int64]
    fn(crow, col, q, k, out, crow.size - 1, q.shape[1])
    return out


def row_softmax(crow, scores) -> np.ndarray:
    """Per-row softmax over CSR segments in double (autosage/_auto.py:744-759)."""
    crow = _i64(crow)
    scores = np.ascontiguousarray(np.asarray(scores), dtype=np.float64)
    probs = np.zeros_like(scores)
    fn = lib().orc_row_softmax_f64
    fn.argtypes = [_I64P, _F64P, _F64P, ctypes.c_int64]
    fn(crow, scores, probs, crow.size - 1)
    return probs


def attention(crow, col, q, k, v, scale: float = 1.0) -> np.ndarray:
    """softmax_row(scale * SDDMM(q, k)) applied to v, in double (autosage/_auto.py:762-780; the
    reference has no scale, i.e. scale = 1)."""
    crow, col, q, k, v = _i64(crow), _i64(col), _f32(q), _f32(k), _f32(v)
    n, f = crow.size - 1, q.shape[1]
    out = np.empty((n, f), dtype=np.float64)
    fn = lib().orc_attention_f64
    fn.argtypes = [_I64P, _I64P, _F32P, _F32P, _F32P, ctypes.c_double, _F64P, ctypes.c_int64, ctypes.c_int64]
    fn(crow, col, q, k, v, float(scale), out, n, f)
    return out


def hub_split(crow, threshold: int) -> tuple[np.ndarray, np.ndarray]:
    """(hub rows, light rows), each ascending - nonzero(deg >= T) and its complement
    (csrc/launcher_spmm.cu:49-59)."""
    crow = _i64(crow)
    n = crow.size - 1
    hubs, lights = np.empty(n, dtype=np.int32), np.empty(n, dtype=np.int32)
    counts = np.zeros(2, dtype=np.int64)
    fn = lib().orc_hub_split
    fn.argtypes = [_I64P, ctypes.c_int64, ctypes.c_int64, _I32P, _I32P, _I64P]
    fn(crow, n, int(threshold), hubs, lights, counts)
    return hubs[: counts[0]].copy(), lights[: counts[1]].copy()


def plan_order(crow, threshold: int) -> tuple[np.ndarray, int, int]:
    """Processing order of the degree-binned plan and (n_hub, n_light)."""
    crow = _i64(crow)
    n = crow.size - 1
    order = np.empty(n, dtype=np.int32)
    counts = np.zeros(2, dtype=np.int64)
    fn = lib().orc_plan_order
    fn.argtypes = [_I64P, ctypes.c_int64, ctypes.c_int64, _I32P, _I64P]
    fn(crow, n, int(threshold), order, counts)
    return order, int(counts[0]), int(counts[1])


def partition_rows(crow, parts: int) -> np.ndarray:
    """Row boundaries of an nnz-balanced partition into ``parts`` contiguous row ranges."""
    crow = _i64(crow)
    bounds = np.zeros(parts + 1, dtype=np.int64)
    fn = lib().orc_partition_rows
    fn.argtypes = [_I64P, ctypes.c_int64, ctypes.c_int64, _I64P]
    fn(crow, crow.size - 1, int(parts), bounds)
    return bounds


def edge_index_to_csr(edge_index, num_nodes: int, rows_by: str = "dst"):
    """(crow, col, perm): stable COO->CSR keyed by destination or source (autosage/utils/csr.py:6-26)."""
    edge_index = _i64(edge_index)
    src, dst = edge_index[0].copy(), edge_index[1].copy()
    rows, cols = (dst, src) if rows_by == "dst" else (src, dst)
    crow = np.zeros(num_nodes + 1, dtype=np.int64)
    col = np.empty(rows.size, dtype=np.int64)
    perm = np.empty(rows.size, dtype=np.int64)
    fn = lib().orc_coo_to_csr
    fn.argtypes = [_I64P, _I64P, ctypes.c_int64, ctypes.c_int64, _I64P, _I64P, _I64P]
    fn(rows, cols, rows.size, num_nodes, crow, col, perm)
    return crow, col, perm


def row_degrees(crow) -> np.ndarray:
    crow = _i64(crow)
    return crow[1:] - crow[:-1]


def within_tolerance(actual, exact, crow, *, per_edge: bool = False, rtol: float = 1e-5, atol: float = 1e-5):
    """The acceptance rule for float32 results against the float64 oracle:
    |a - e| <= rtol*|e| + atol*sqrt(degree(row)).  Returns (ok, worst ratio of error to bound)."""
    actual = np.asarray(actual, dtype=np.float64)
    exact = np.asarray(exact, dtype=np.float64)
    deg = np.maximum(row_degrees(crow), 1).astype(np.float64)
    if per_edge:
        scale = np.repeat(np.sqrt(deg), row_degrees(crow))
    else:
        scale = np.sqrt(deg)[:, None]
    bound = rtol * np.abs(exact) + atol * scale
    err = np.abs(actual - exact)
    bad = ~(err <= bound)  # catches NaN as well
    ratio = float(np.max(err / np.maximum(bound, 1e-300))) if err.size else 0.0
    return (not bool(bad.any())), ratio


def spmm_reference_cpu(crow, col, val, x):
    """The reference's CPU SpMM exactly as it runs it (autosage/ops.py:124-143): build a
    torch.sparse_csr_tensor (all-ones weights when val is None) and call torch.sparse.mm.  Takes and
    returns torch CPU tensors; the arithmetic is PyTorch's own multi-threaded CPU kernel.  Used as
    the timed CPU baseline and to cross-check ``spmm`` above."""
    import torch

    weights = torch.ones(col.numel(), dtype=x.dtype) if val is None else val.to(x.dtype)
    matrix = torch.sparse_csr_tensor(crow, col, weights, size=(crow.numel() - 1, x.size(0)), dtype=x.dtype)
    return torch.sparse.mm(matrix, x)


def sddmm_reference_cpu(crow, col, query, key):
    """The reference's CPU SDDMM exactly as it runs it (the gather-dot baseline its scheduler falls
    back to on CPU tensors, autosage/_auto.py:79-92): expand the row id of every edge, gather both
    operands, multiply and sum over the feature axis.  torch CPU tensors in and out; ``query`` holds one
    row per CSR row, ``key`` is indexed by column id.  Used as a timed CPU baseline."""
    import torch

    counts = (crow[1:] - crow[:-1]).to(torch.long)
    rows = torch.repeat_interleave(torch.arange(crow.numel() - 1, dtype=torch.long), counts)
    return (query.index_select(0, rows) * key.index_select(0, col)).sum(dim=1)


def row_softmax_reference_cpu(crow, scores):
    """The reference's CSR row softmax (autosage/_auto.py:744-759): scatter amax, exp of the shifted
    scores, scatter add, divide."""
    import torch

    row_count = crow.numel() - 1
    counts = (crow[1:] - crow[:-1]).to(torch.long)
    rows = torch.repeat_interleave(torch.arange(row_count, dtype=torch.long), counts)
    if scores.numel() == 0:
        return scores.clone()
    maxima = torch.full((row_count,), -torch.inf, dtype=scores.dtype)
    maxima.scatter_reduce_(0, rows, scores, reduce="amax", include_self=True)
    exponentials = (scores - maxima.index_select(0, rows)).exp()
    denominators = torch.zeros_like(maxima).scatter_add_(0, rows, exponentials)
    return exponentials / denominators.index_select(0, rows)


def attention_reference_cpu(crow, col, query, key, value, scale: float = 1.0):
    """The reference's attention pipeline on CPU tensors (autosage/_auto.py:762-780 with every stage on
    its CPU path): gather-dot SDDMM of the (scaled) queries, CSR row softmax, torch.sparse.mm with the
    probabilities as edge weights.  ``query`` holds one row per CSR row; ``key``/``value`` are indexed
    by column id."""
    import torch

    scores = sddmm_reference_cpu(crow, col, query * scale if scale != 1.0 else query, key)
    weights = row_softmax_reference_cpu(crow, scores)
    matrix = torch.sparse_csr_tensor(crow, col, weights, size=(crow.numel() - 1, value.size(0)), dtype=value.dtype)
    return torch.sparse.mm(matrix, value)
