"""Operator boundary: library loading, the ``torch.ops.autosage`` operators and ``spmm_csr``.

Mirrors the reference module ``autosage/ops.py`` (load_native :31-61, native_op :64-71,
native_available :74-75, native_load_error :78-79, _validate_csr :82-103, _normalize_csr :106-121,
_cpu_spmm :124-143, spmm_csr :146-164) and the operator schemas of ``csrc/spmm_binding.cpp:65-75`` and
``csrc/sddmm_csr_op.cu:191-201``.  The differences are behind the boundary: the operators are
defined from Python with ``torch.library`` and implemented by calls into the C ABI of
``libautosage_b200.so``; CUDA tensors never take a PyTorch or CPU fallback.
"""
from __future__ import annotations

import os
import weakref
from typing import Optional

import torch

from . import _native

# defaults of the plain operators, from the B200 sweeps (see the C entry points asg_spmm_csr / asg_sddmm_csr)
DEFAULT_WARPS = 4
DEFAULT_HUB_THRESHOLD = 1024
DEFAULT_TILE = 64
SDDMM_WARPS = 8
SDDMM_HUB_THRESHOLD = 8192

_ATTEMPTED = False
_ERROR: Optional[BaseException] = None
_LIBRARY_HANDLES: list = []  # keeps torch.library.Library objects alive


def _env_vec4_enabled() -> bool:
    """The reference launchers read AUTOSAGE_VEC4 on every call (csrc/spmm_csr_vec4.cu:135-143):
    anything but 0/false/no/off keeps vector loads on."""
    return os.getenv("AUTOSAGE_VEC4", "1").strip().lower() not in {"0", "false", "no", "off"}


def _base_flags() -> int:
    return 0 if _env_vec4_enabled() else _native.FLAG_NO_VEC4


# ------------------------------------------------------------------------------------------------
# Operator implementations (CUDA dispatch key).  Checks and messages follow the reference
# bindings: csrc/spmm_binding.cpp:9-29,40-61 and csrc/sddmm_csr_op.cu:85-106,136-150.
# ------------------------------------------------------------------------------------------------
def _require(condition: bool, message: str) -> None:
    if not condition:
        raise RuntimeError(message)


def _debug_check_columns(crow, col, bound: int) -> None:
    """AUTOSAGE_CHECK_INDICES=1: verify the index arrays before a launch (synchronises; the reference
    never checks ``col`` and an out-of-range entry there reads foreign memory)."""
    if os.getenv("AUTOSAGE_CHECK_INDICES") != "1" or col.numel() == 0:
        return
    low, high = int(col.min().item()), int(col.max().item())
    _require(low >= 0 and high < bound, f"col entries must lie in [0, {bound}); found [{low}, {high}]")
    _require(int(crow[0].item()) == 0 and int(crow[-1].item()) == col.numel(), "crow must run from 0 to nnz")
    _require(bool((crow[1:] >= crow[:-1]).all().item()), "crow must be non-decreasing")


def _check_spmm_inputs(crow, col, val, x) -> None:
    _require(crow.is_cuda and col.is_cuda and x.is_cuda, "crow, col, and x must be CUDA tensors")
    _require(crow.dtype == torch.long and col.dtype == torch.long, "crow and col must use torch.long indices")
    _require(crow.dim() == 1 and col.dim() == 1, "crow and col must be one-dimensional")
    _require(x.dim() == 2 and x.is_contiguous(), "x must be contiguous with shape [N, F]")
    _require(x.dtype == torch.float32, "x must be float32")
    _require(crow.is_contiguous() and col.is_contiguous(), "crow and col must be contiguous")
    _require(crow.device == x.device and col.device == x.device, "crow, col, and x must be on the same CUDA device")
    _require(crow.numel() == x.size(0) + 1, "crow must contain N + 1 entries")
    if val is not None:
        _require(val.is_cuda and val.device == x.device, "val must be on the same CUDA device as x")
        _require(val.dtype == torch.float32 and val.is_contiguous(), "val must be contiguous float32")
        _require(val.numel() == col.numel(), "val must contain one weight per nonzero")
    _debug_check_columns(crow, col, x.size(0))


def _check_sddmm_inputs(crow, col, query, key) -> None:
    _require(crow.is_cuda and col.is_cuda and query.is_cuda and key.is_cuda, "all SDDMM inputs must be CUDA tensors")
    _require(crow.dtype == torch.long and col.dtype == torch.long, "crow and col must use torch.long indices")
    _require(query.dtype == torch.float32 and key.dtype == torch.float32, "query and key must be float32")
    _require(query.dim() == 2 and query.shape == key.shape, "query and key must have the same [N, F] shape")
    _require(crow.numel() == query.size(0) + 1, "crow must contain N + 1 entries")
    _require(crow.device == query.device and col.device == query.device and key.device == query.device,
             "all SDDMM inputs must be on the same CUDA device")
    _require(crow.is_contiguous() and col.is_contiguous() and query.is_contiguous() and key.is_contiguous(),
             "all SDDMM inputs must be contiguous")
    _require(query.size(0) <= 2**31 - 1 and query.size(1) <= 2**31 - 1, "SDDMM dimensions exceed the kernel index range")
    _debug_check_columns(crow, col, key.size(0))


def _op_spmm_csr(crow, col, val, x):
    _check_spmm_inputs(crow, col, val, x)
    y = torch.empty_like(x)
    if x.numel() == 0:
        return y
    workspace, ready = _native.planned_workspace(crow, DEFAULT_HUB_THRESHOLD)
    _native.spmm(crow, col, val, x, y, feature_tile=DEFAULT_TILE, warps=DEFAULT_WARPS, threshold=DEFAULT_HUB_THRESHOLD,
                 flags=_base_flags() | ready, workspace=workspace)
    return y


def _op_spmm_csr_split(crow, col, val, x, feature_tile, warps_per_block, hub_threshold):
    _check_spmm_inputs(crow, col, val, x)
    _require(feature_tile in (64, 128), "feature_tile must be 64 or 128")
    _require(warps_per_block in (2, 4, 8), "warps_per_block must be 2, 4, or 8")
    _require(hub_threshold > 0, "hub_threshold must be positive")
    y = torch.empty_like(x)
    if x.numel() == 0:
        return y
    workspace, ready = _native.planned_workspace(crow, hub_threshold)
    _native.spmm(crow, col, val, x, y, feature_tile=feature_tile, warps=warps_per_block, threshold=hub_threshold,
                 flags=_base_flags() | ready, workspace=workspace)
    return y


def _op_sddmm_csr(crow, col, query, key):
    _check_sddmm_inputs(crow, col, query, key)
    out = torch.empty(col.numel(), dtype=query.dtype, device=query.device)
    if query.size(0) == 0 or col.numel() == 0:
        return out
    workspace, ready = _native.planned_workspace(crow, SDDMM_HUB_THRESHOLD)
    _native.sddmm(crow, col, query, key, out, warps=SDDMM_WARPS, threshold=SDDMM_HUB_THRESHOLD,
                  flags=_base_flags() | ready, workspace=workspace)
    return out


def _op_sddmm_csr_split(crow, col, query, key, warps_per_block, hub_threshold):
    _check_sddmm_inputs(crow, col, query, key)
    _require(warps_per_block in (2, 4, 8), "warps_per_block must be 2, 4, or 8")
    _require(0 < hub_threshold <= 2**31 - 1, "hub_threshold must be a positive 32-bit integer")
    out = torch.empty(col.numel(), dtype=query.dtype, device=query.device)
    if query.size(0) == 0 or col.numel() == 0:
        return out
    workspace, ready = _native.planned_workspace(crow, hub_threshold)
    _native.sddmm(crow, col, query, key, out, warps=warps_per_block, threshold=hub_threshold,
                  flags=_base_flags() | ready, workspace=workspace)
    return out


_SCHEMAS = (
    ("spmm_csr", "(Tensor crow, Tensor col, Tensor? val, Tensor x) -> Tensor", _op_spmm_csr),
    ("spmm_csr_split",
     "(Tensor crow, Tensor col, Tensor? val, Tensor x, int feature_tile, int warps_per_block, int hub_threshold) -> Tensor",
     _op_spmm_csr_split),
    ("sddmm_csr", "(Tensor crow, Tensor col, Tensor query, Tensor key) -> Tensor", _op_sddmm_csr),
    ("sddmm_csr_split",
     "(Tensor crow, Tensor col, Tensor query, Tensor key, int warps_per_block, int hub_threshold) -> Tensor",
     _op_sddmm_csr_split),
)


# ------------------------------------------------------------------------------------------------
# Autograd.  The reference registers no backward for its operators (its CUDA path is forward-only);
# here the four operators are differentiable in val / x and query / key, each gradient being one of
# the same kernels:
#   Y = A X          dX = A^T dY (SpMM over the transposed pattern),  dval[e] = <dY[row e], X[col e]> (SDDMM)
#   s[e] = <Q_r,K_c> dQ = A(ds) K (SpMM with the edge gradients as weights),  dK = A(ds)^T Q
# ------------------------------------------------------------------------------------------------
_TRANSPOSES: dict[tuple, tuple] = {}


def _transposed_pattern(crow: torch.Tensor, col: torch.Tensor):
    """(crow_t, col_t, perm) of the transposed square pattern; perm[i] is the position in the original
    edge order of the i-th edge of the transpose.  Memoised per (crow, col) tensor pair."""
    key = (crow.data_ptr(), col.data_ptr(), crow.numel(), col.numel())
    hit = _TRANSPOSES.get(key)
    if hit is not None and hit[0]() is crow and hit[1]() is col and hit[2] == (crow._version, col._version):
        return hit[3]
    n = crow.numel() - 1
    rows = torch.repeat_interleave(torch.arange(n, device=col.device, dtype=torch.long), crow[1:] - crow[:-1])
    perm = torch.argsort(col, stable=True)
    crow_t = torch.zeros(n + 1, dtype=torch.long, device=col.device)
    if col.numel():
        torch.cumsum(torch.bincount(col, minlength=n)[:n], 0, out=crow_t[1:])
    value = (crow_t, rows[perm].contiguous(), perm)
    if len(_TRANSPOSES) > 16:
        _TRANSPOSES.clear()
    _TRANSPOSES[key] = (weakref.ref(crow), weakref.ref(col), (crow._version, col._version), value)
    return value


def _spmm_setup(ctx, inputs, output) -> None:
    crow, col, val, x = inputs[:4]
    ctx.extra = tuple(inputs[4:])  # (feature_tile, warps_per_block, hub_threshold) for the split operator
    ctx.save_for_backward(crow, col, val, x)


def _spmm_backward(ctx, grad_y):
    crow, col, val, x = ctx.saved_tensors
    grad_y = grad_y.contiguous()
    run = (lambda c, k, v, d: torch.ops.autosage.spmm_csr_split(c, k, v, d, *ctx.extra)) if ctx.extra else \
        torch.ops.autosage.spmm_csr
    grad_x = grad_val = None
    if ctx.needs_input_grad[3]:
        crow_t, col_t, perm = _transposed_pattern(crow, col)
        grad_x = run(crow_t, col_t, None if val is None else val.detach()[perm].contiguous(), grad_y)
    if val is not None and ctx.needs_input_grad[2]:
        grad_val = torch.ops.autosage.sddmm_csr(crow, col, grad_y, x.detach())
    return (None, None, grad_val, grad_x) + (None,) * len(ctx.extra)


def _sddmm_setup(ctx, inputs, output) -> None:
    crow, col, query, key = inputs[:4]
    ctx.save_for_backward(crow, col, query, key)


def _sddmm_backward(ctx, grad_out):
    crow, col, query, key = ctx.saved_tensors
    grad_out = grad_out.contiguous()
    grad_q = grad_k = None
    if ctx.needs_input_grad[2]:
        grad_q = torch.ops.autosage.spmm_csr(crow, col, grad_out, key.detach())
    if ctx.needs_input_grad[3]:
        crow_t, col_t, perm = _transposed_pattern(crow, col)
        grad_k = torch.ops.autosage.spmm_csr(crow_t, col_t, grad_out[perm].contiguous(), query.detach())
    return (None, None, grad_q, grad_k) + (None,) * (len(ctx.needs_input_grad) - 4)


def _register_operators() -> None:
    definitions = torch.library.Library("autosage", "FRAGMENT")
    for name, schema, function in _SCHEMAS:
        definitions.define(name + schema)
        definitions.impl(name, function, "CUDA")
    for name in ("spmm_csr", "spmm_csr_split"):
        torch.library.register_autograd(f"autosage::{name}", _spmm_backward, setup_context=_spmm_setup, lib=definitions)
    for name in ("sddmm_csr", "sddmm_csr_split"):
        torch.library.register_autograd(f"autosage::{name}", _sddmm_backward, setup_context=_sddmm_setup,
                                        lib=definitions)
    _LIBRARY_HANDLES.append(definitions)


# ------------------------------------------------------------------------------------------------
# Loading
# ------------------------------------------------------------------------------------------------
def native_op(name: str):
    namespace = getattr(torch.ops, "autosage", None)
    if namespace is None:
        return None
    try:
        return getattr(namespace, name)
    except (AttributeError, RuntimeError):
        return None


def native_available() -> bool:
    return native_op("spmm_csr") is not None


def native_load_error() -> Optional[BaseException]:
    return _ERROR


def load_native() -> bool:
    """Load ``libautosage_b200.so`` once per process and register the four operators."""
    global _ATTEMPTED, _ERROR
    if native_available():
        return True
    if _ATTEMPTED:
        return False
    _ATTEMPTED = True
    failures: list[BaseException] = []
    for path in _native.candidate_libraries():
        if not path.is_file():
            continue
        try:
            _native.set_library(_native.bind(str(path)), str(path))
            _register_operators()
            return native_available()
        except (OSError, RuntimeError) as exc:
            failures.append(exc)
    _ERROR = failures[-1] if failures else FileNotFoundError(
        "libautosage_b200.so was not found. Build it with `python -m autosage_b200.build`."
    )
    return False


# ------------------------------------------------------------------------------------------------
# spmm_csr
# ------------------------------------------------------------------------------------------------
_INDEX_DTYPES = (torch.int32, torch.int64)


def _validate_csr(crow, col, val, x) -> None:
    if crow.ndim != 1 or col.ndim != 1:
        raise ValueError("crow and col must be one-dimensional")
    if crow.dtype != torch.long or col.dtype != torch.long:
        raise TypeError("crow and col must use torch.long indices")
    if x.ndim != 2:
        raise ValueError("x must have shape [N, F]")
    if not x.is_floating_point():
        raise TypeError("x must use a floating-point dtype")
    if crow.numel() != x.size(0) + 1:
        raise ValueError("crow must contain N + 1 entries")
    if val is not None and (val.ndim != 1 or val.numel() != col.numel()):
        raise ValueError("val must contain one weight per nonzero")
    if not (crow.device == col.device == x.device):
        raise ValueError("crow, col, and x must be on the same device")
    if val is not None and val.device != x.device:
        raise ValueError("val and x must be on the same device")


def _normalize_csr(crow, col, val, x):
    """int32/int64 indices -> contiguous int64; weights -> x's dtype; then validate."""
    if crow.dtype not in _INDEX_DTYPES or col.dtype not in _INDEX_DTYPES:
        raise TypeError("crow and col must use integer indices")
    crow = crow.to(torch.long).contiguous()
    col = col.to(torch.long).contiguous()
    x = x.contiguous()
    if val is not None:
        val = val.to(x.dtype).contiguous()
    _validate_csr(crow, col, val, x)
    return crow, col, val, x


def _cpu_spmm(crow, col, val, x):
    """CPU tensors keep the reference behaviour: torch.sparse.mm over a CSR tensor, any float dtype."""
    weights = torch.ones(col.numel(), dtype=x.dtype, device=x.device) if val is None else val.to(x.dtype)
    n = x.size(0)
    matrix = torch.sparse_csr_tensor(crow, col, weights, size=(n, n), dtype=x.dtype, device=x.device)
    return torch.sparse.mm(matrix, x)


def spmm_csr(crow: torch.Tensor, col: torch.Tensor, val: Optional[torch.Tensor], x: torch.Tensor) -> torch.Tensor:
    """``Y = A @ X`` for a square CSR matrix; float32 CUDA tensors run the sm_100a kernels."""
    crow, col, val, x = _normalize_csr(crow, col, val, x)
    if not x.is_cuda:
        return _cpu_spmm(crow, col, val, x)
    if x.dtype != torch.float32:
        raise TypeError("AutoSAGE CUDA kernels currently support float32 features only")
    if not load_native():
        detail = f": {_ERROR}" if _ERROR else ""
        raise RuntimeError(f"AutoSAGE CUDA extension is unavailable{detail}")
    op = native_op("spmm_csr")
    if op is None:
        raise RuntimeError("native operator autosage::spmm_csr is not registered")
    return op(crow, col, val, x)


def spmm_csr_auto(*args, **kwargs):
    from ._auto import spmm_csr_auto as implementation

    return implementation(*args, **kwargs)


__all__ = [
    "load_native",
    "native_available",
    "native_load_error",
    "native_op",
    "spmm_csr",
    "spmm_csr_auto",
]
