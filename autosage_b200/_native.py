"""ctypes binding of ``libautosage_b200.so`` (the C ABI declared in ``include/autosage_b200.h``).

Nothing here computes: every function forwards device pointers and sizes to the CUDA library and
turns a negative status code into ``RuntimeError`` (the reference's ``TORCH_CHECK`` failures surface
as ``RuntimeError`` too).  There is deliberately no CPU or PyTorch fallback: if the library cannot
be loaded the callers raise.
"""
from __future__ import annotations

import ctypes
import os
import weakref
from collections import OrderedDict
from pathlib import Path
from typing import Optional

import torch

LIB_NAMES = ("libautosage_b200.so",)

FLAG_ACCUMULATE = 1
FLAG_NO_VEC4 = 2
FLAG_PLAN_READY = 4
FLAG_NO_BULK_STAGE = 8
FLAG_NO_TILE_PASSES = 16
FLAG_PACK_SHORT_ROWS = 32
FLAG_SELFTEST_STALL = 64

_P = ctypes.c_void_p
_I64 = ctypes.c_int64
_INT = ctypes.c_int
_U32 = ctypes.c_uint
_SZ = ctypes.c_size_t
_F32 = ctypes.c_float

# name -> (restype, argtypes); kept in the order of the header
SIGNATURES = {
    "asg_version": (_INT, []),
    "asg_last_error_string": (ctypes.c_char_p, []),
    "asg_workspace_bytes": (_SZ, [_I64]),
    "asg_plan_build": (_INT, [_P, _I64, _I64, _P, _SZ, _P]),
    "asg_plan_export": (_INT, [_P, _I64, _P, _P, _P]),
    "asg_spmm_csr": (_INT, [_P, _P, _P, _P, _P, _I64, _I64, _I64, _P, _SZ, _P]),
    "asg_spmm_csr_split": (_INT, [_P, _P, _P, _P, _P, _I64, _I64, _I64, _INT, _INT, _I64, _P, _SZ, _P]),
    "asg_spmm_csr_ex": (_INT, [_P, _P, _P, _P, _P, _I64, _I64, _I64, _INT, _INT, _I64, _U32, _P, _SZ, _P]),
    "asg_spmm_csr_range": (_INT, [_P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _INT, _INT, _I64, _U32, _P, _SZ, _P]),
    "asg_sddmm_csr": (_INT, [_P, _P, _P, _P, _P, _I64, _I64, _I64, _P, _SZ, _P]),
    "asg_sddmm_csr_split": (_INT, [_P, _P, _P, _P, _P, _I64, _I64, _I64, _INT, _I64, _P, _SZ, _P]),
    "asg_sddmm_csr_ex": (_INT, [_P, _P, _P, _P, _P, _I64, _I64, _I64, _INT, _I64, _U32, _P, _SZ, _P]),
    "asg_csr_row_softmax": (_INT, [_P, _P, _P, _I64, _I64, _INT, _I64, _U32, _P, _SZ, _P]),
    "asg_attention_workspace_bytes": (_SZ, [_I64]),
    "asg_csr_attention": (_INT, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _F32, _INT, _I64, _U32, _P, _SZ, _P]),
    "asg_add_row_bias": (_INT, [_P, _P, _I64, _I64, _P]),
    "asg_csr_build_workspace_bytes": (_SZ, [_I64, _I64]),
    "asg_csr_from_edges": (_INT, [_P, _P, _P, _I64, _I64, _P, _P, _P, _P, _P, _SZ, _P]),
    "asg_row_sample_workspace_bytes": (_SZ, [_I64]),
    "asg_csr_row_sample": (_INT, [_P, _P, _P, _P, _I64, _I64, _P, _P, _P, _P, _P, _SZ, _P]),
    "asg_linear_available": (_INT, []),
    "asg_linear_bias": (_INT, [_P, _P, _P, _P, _I64, _I64, _I64, _P]),
    "asg_linear_workspace_bytes": (_SZ, [_I64, _I64]),
    "asg_linear_supported": (_INT, [_I64, _I64]),
    "asg_linear_bias_umma": (_INT, [_P, _P, _P, _P, _I64, _I64, _I64, _P, _SZ, _P]),
    "asg_linear_bias_umma_ex": (_INT, [_P, _P, _P, _P, _I64, _I64, _I64, _U32, _P, _SZ, _P]),
    "asg_conv_fused_supported": (_INT, [_I64, _I64]),
    "asg_conv_fused_workspace_bytes": (_SZ, [_I64, _I64, _I64, _I64, _I64]),
    "asg_conv_fused": (_INT, [_P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _INT, _U32, _P, _SZ, _P, _SZ, _P]),
    "asg_copy_2d": (_INT, [_P, _SZ, _P, _SZ, _SZ, _SZ, _P]),
    "asg_push_to_peers": (_INT, [_P, _P, _INT, _SZ, _INT, _P]),
    "asg_workspace_status": (_INT, [_P, _P, _P]),
    "asg_spmm_csr_split_noalloc": (_INT, [_P, _P, _P, _P, _P, _I64, _I64, _I64, _INT, _INT, _I64, _P]),
    "asg_static_max_rows": (_I64, []),
    "asg_static_status": (_INT, [_P, _P, _P]),
}

_LIB: Optional[ctypes.CDLL] = None
_LIB_PATH: Optional[str] = None


def candidate_libraries() -> list[Path]:
    """Search order, mirroring the reference loader (autosage/ops.py:14-28): the explicit
    ``AUTOSAGE_NATIVE_PATH``, then ``<repo>/build/``, then the package's ``lib/`` directory."""
    package = Path(__file__).resolve().parent
    paths: list[Path] = []
    explicit = os.getenv("AUTOSAGE_NATIVE_PATH")
    if explicit:
        paths.append(Path(explicit).expanduser())
    for directory in (package.parent / "build", package / "lib"):
        paths.extend(directory / name for name in LIB_NAMES)
    return paths


def bind(path: str) -> ctypes.CDLL:
    """Load the shared library at ``path`` and attach the prototypes; raises ``OSError`` if the file
    cannot be loaded and ``RuntimeError`` if it lacks a declared symbol."""
    lib = ctypes.CDLL(path)
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise RuntimeError(f"{path} does not export {name}") from exc
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


def set_library(lib: ctypes.CDLL, path: str) -> None:
    global _LIB, _LIB_PATH
    _LIB = lib
    _LIB_PATH = path


def library() -> ctypes.CDLL:
    if _LIB is None:
        raise RuntimeError("libautosage_b200.so is not loaded; call autosage_b200.load_native() first")
    return _LIB


def library_path() -> Optional[str]:
    return _LIB_PATH


def check(code: int) -> None:
    if code != 0:
        message = library().asg_last_error_string()
        text = message.decode("utf-8", "replace") if message else ""
        raise RuntimeError(f"{text} (autosage_b200 status {code})")


def _ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    return None if tensor is None else tensor.data_ptr()


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


# --------------------------------------------------------------------------------------------
# Workspaces.  The C ABI never allocates; scratch comes from torch's caching allocator so it
# follows torch's stream semantics.  One scratch buffer per (device, stream) is kept for calls that
# rebuild the plan, and a small LRU of buffers holding finished plans is keyed by the crow tensor.
# --------------------------------------------------------------------------------------------
_SCRATCH: dict[tuple[int, int], torch.Tensor] = {}
_PLANS: "OrderedDict[tuple, list]" = OrderedDict()   # key -> [crow weakref, crow version, buffer, plan built?]
_UNBUILT: dict[int, list] = {}                       # buffer address -> entry whose plan no kernel has built yet
PLAN_CACHE_ENTRIES = 16


def workspace_bytes(n_rows: int) -> int:
    return int(library().asg_workspace_bytes(int(n_rows)))


def _capturing() -> bool:
    return torch.cuda.is_current_stream_capturing()


def scratch(device: torch.device, n_rows: int, extra_bytes: int = 0) -> torch.Tensor:
    need = workspace_bytes(n_rows) + int(extra_bytes)
    if _capturing():
        # a captured launch keeps the raw pointer: the buffer has to come from the graph's own pool
        # (and so live as long as the graph), not from a cache that may replace it later
        return torch.empty(max(need, 256), dtype=torch.uint8, device=device)
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream(device))
    buffer = _SCRATCH.get(key)
    if buffer is None or buffer.numel() < need:
        buffer = torch.empty(max(need, 1 << 16), dtype=torch.uint8, device=device)
        _SCRATCH[key] = buffer
    return buffer


def attention_extra_bytes(n_rows: int) -> int:
    """Bytes beyond ``workspace_bytes`` that let the fused attention kernel split very long rows."""
    return int(library().asg_attention_workspace_bytes(int(n_rows))) - workspace_bytes(n_rows)


def planned_workspace(crow: torch.Tensor, threshold: int, extra_bytes: int = 0) -> tuple[torch.Tensor, int]:
    """Workspace holding the degree-binned plan of ``crow`` for ``threshold``.

    Returns ``(buffer, flags)`` where flags is ``FLAG_PLAN_READY`` when the buffer already holds
    the plan (same tensor object, same version counter, and an earlier call that built it returned
    without error) and 0 when the callee must build it.

    While the current stream is being captured into a CUDA graph the cache is bypassed: the graph
    records raw pointers, and a cached buffer can be evicted (or its plan replaced) long before the
    graph is replayed.  The buffer is then allocated inside the capture, so it belongs to the graph's
    memory pool, and the plan is rebuilt by the captured launches themselves.
    """
    if _capturing() or os.getenv("AUTOSAGE_PLAN_CACHE", "1") in ("0", "false", "off", "no"):
        return scratch(crow.device, crow.numel() - 1, extra_bytes), 0
    key = (crow.data_ptr(), crow.numel(), int(threshold), crow.device.index, _stream(crow.device), int(extra_bytes))
    entry = _PLANS.get(key)
    if entry is not None:
        ref, version, buffer, built = entry
        if ref() is crow and version == crow._version:
            _PLANS.move_to_end(key)
            return buffer, (FLAG_PLAN_READY if built else 0)
        _forget(key)
    buffer = torch.empty(max(workspace_bytes(crow.numel() - 1), 256) + int(extra_bytes), dtype=torch.uint8,
                         device=crow.device)
    entry = [weakref.ref(crow), crow._version, buffer, False]
    _PLANS[key] = entry
    _UNBUILT[buffer.data_ptr()] = entry
    while len(_PLANS) > PLAN_CACHE_ENTRIES:
        _forget(next(iter(_PLANS)))
    return buffer, 0


def _forget(key) -> None:
    entry = _PLANS.pop(key, None)
    if entry is not None:
        _UNBUILT.pop(entry[2].data_ptr(), None)


def _plan_was_built(workspace: torch.Tensor) -> None:
    """Called after a launch that (re)builds the plan returned without error."""
    entry = _UNBUILT.pop(workspace.data_ptr(), None) if _UNBUILT else None
    if entry is not None:
        entry[3] = True
    if os.getenv("AUTOSAGE_CHECK_STATUS") == "1" and not _capturing():
        # debugging aid (synchronises): a kernel whose bounded wait gave up leaves a status word in
        # the workspace header and returns with rows unwritten; turn that into an error here
        status = workspace_status(workspace)
        if status != 0:
            raise RuntimeError(f"a kernel gave up a bounded wait (status {status}); its output is incomplete")


def clear_plan_cache() -> None:
    _PLANS.clear()
    _UNBUILT.clear()
    _SCRATCH.clear()


# --------------------------------------------------------------------------------------------
# Thin wrappers (tensors in, status checked).  Inputs must already be validated and contiguous.
# --------------------------------------------------------------------------------------------
def plan_build(crow: torch.Tensor, threshold: int, workspace: torch.Tensor) -> None:
    check(library().asg_plan_build(crow.data_ptr(), crow.numel() - 1, int(threshold), workspace.data_ptr(),
                                   workspace.numel(), _stream(crow.device)))
    _plan_was_built(workspace)


def plan_export(workspace: torch.Tensor, n_rows: int) -> tuple[torch.Tensor, torch.Tensor]:
    order = torch.empty(n_rows, dtype=torch.int32, device=workspace.device)
    counts = torch.empty(2, dtype=torch.int32, device=workspace.device)
    check(library().asg_plan_export(workspace.data_ptr(), n_rows, order.data_ptr(), counts.data_ptr(),
                                    _stream(workspace.device)))
    return order, counts


def spmm(crow, col, val, x, y, *, feature_tile: int, warps: int, threshold: int, flags: int,
         workspace: torch.Tensor) -> None:
    check(library().asg_spmm_csr_ex(crow.data_ptr(), col.data_ptr(), _ptr(val), x.data_ptr(), y.data_ptr(),
                                    y.size(0), col.numel(), x.size(1), int(feature_tile), int(warps),
                                    int(threshold), int(flags), workspace.data_ptr(), workspace.numel(),
                                    _stream(x.device)))
    _plan_was_built(workspace)


def spmm_range(crow, col, val, x, y, *, feature_begin: int, feature_count: int, feature_tile: int, warps: int,
               threshold: int, flags: int, workspace: torch.Tensor) -> None:
    """SpMM restricted to the output columns [feature_begin, feature_begin + feature_count)."""
    check(library().asg_spmm_csr_range(crow.data_ptr(), col.data_ptr(), _ptr(val), x.data_ptr(), y.data_ptr(),
                                       y.size(0), col.numel(), x.size(1), int(feature_begin), int(feature_count),
                                       int(feature_tile), int(warps), int(threshold), int(flags),
                                       workspace.data_ptr(), workspace.numel(), _stream(x.device)))
    _plan_was_built(workspace)


def copy_columns(dst: torch.Tensor, src: torch.Tensor, column_begin: int, column_count: int) -> None:
    """dst[:, c0:c0+n] = src[:, c0:c0+n] for two row-major 2-D tensors of equal shape, as one pitched
    copy on the current stream (copy engines; src may be a peer-mapped tensor of another GPU)."""
    item = dst.element_size()
    offset = int(column_begin) * item
    check(library().asg_copy_2d(dst.data_ptr() + offset, dst.stride(0) * item, src.data_ptr() + offset,
                                src.stride(0) * item, int(column_count) * item, dst.size(0), _stream(dst.device)))


def spmm_split_strict(crow, col, val, x, y, feature_tile: int, warps: int, threshold: int,
                      workspace: torch.Tensor) -> None:
    check(library().asg_spmm_csr_split(crow.data_ptr(), col.data_ptr(), _ptr(val), x.data_ptr(), y.data_ptr(),
                                       y.size(0), col.numel(), x.size(1), int(feature_tile), int(warps),
                                       int(threshold), workspace.data_ptr(), workspace.numel(), _stream(x.device)))
    _plan_was_built(workspace)


def spmm_plain(crow, col, val, x, y, workspace: torch.Tensor) -> None:
    check(library().asg_spmm_csr(crow.data_ptr(), col.data_ptr(), _ptr(val), x.data_ptr(), y.data_ptr(),
                                 y.size(0), col.numel(), x.size(1), workspace.data_ptr(), workspace.numel(),
                                 _stream(x.device)))
    _plan_was_built(workspace)


def sddmm(crow, col, query, key, out, *, warps: int, threshold: int, flags: int, workspace: torch.Tensor) -> None:
    check(library().asg_sddmm_csr_ex(crow.data_ptr(), col.data_ptr(), query.data_ptr(), key.data_ptr(),
                                     out.data_ptr(), query.size(0), col.numel(), query.size(1), int(warps),
                                     int(threshold), int(flags), workspace.data_ptr(), workspace.numel(),
                                     _stream(query.device)))
    _plan_was_built(workspace)


def sddmm_split_strict(crow, col, query, key, out, warps: int, threshold: int, workspace: torch.Tensor) -> None:
    check(library().asg_sddmm_csr_split(crow.data_ptr(), col.data_ptr(), query.data_ptr(), key.data_ptr(),
                                        out.data_ptr(), query.size(0), col.numel(), query.size(1), int(warps),
                                        int(threshold), workspace.data_ptr(), workspace.numel(),
                                        _stream(query.device)))
    _plan_was_built(workspace)


def sddmm_plain(crow, col, query, key, out, workspace: torch.Tensor) -> None:
    check(library().asg_sddmm_csr(crow.data_ptr(), col.data_ptr(), query.data_ptr(), key.data_ptr(),
                                  out.data_ptr(), query.size(0), col.numel(), query.size(1),
                                  workspace.data_ptr(), workspace.numel(), _stream(query.device)))
    _plan_was_built(workspace)


def row_softmax(crow, scores, probs, *, warps: int, threshold: int, flags: int, workspace: torch.Tensor) -> None:
    check(library().asg_csr_row_softmax(crow.data_ptr(), scores.data_ptr(), probs.data_ptr(), crow.numel() - 1,
                                        scores.numel(), int(warps), int(threshold), int(flags),
                                        workspace.data_ptr(), workspace.numel(), _stream(scores.device)))
    _plan_was_built(workspace)


def attention(crow, col, query, key, value, out, *, scale: float, warps: int, threshold: int, flags: int,
              workspace: torch.Tensor) -> None:
    check(library().asg_csr_attention(crow.data_ptr(), col.data_ptr(), query.data_ptr(), key.data_ptr(),
                                      value.data_ptr(), out.data_ptr(), query.size(0), col.numel(),
                                      query.size(1), float(scale), int(warps), int(threshold), int(flags),
                                      workspace.data_ptr(), workspace.numel(), _stream(query.device)))
    _plan_was_built(workspace)


def add_row_bias(out: torch.Tensor, bias: torch.Tensor) -> None:
    """out[r, :] += bias, in place (contiguous float32 CUDA tensors)."""
    check(library().asg_add_row_bias(out.data_ptr(), bias.data_ptr(), out.size(0), out.size(1), _stream(out.device)))


def csr_from_edges(row_of_edge: torch.Tensor, col_of_edge: torch.Tensor, values: Optional[torch.Tensor],
                   n_rows: int, want_order: bool):
    """Stable COO -> CSR on the device (contiguous int64 CUDA ids, float32 values or None).
    Returns (crow, col, order or None, permuted values or None)."""
    device = row_of_edge.device
    n_edges = row_of_edge.numel()
    crow = torch.empty(n_rows + 1, dtype=torch.long, device=device)
    col = torch.empty(n_edges, dtype=torch.long, device=device)
    order = torch.empty(n_edges, dtype=torch.long, device=device) if want_order else None
    permuted = torch.empty(n_edges, dtype=torch.float32, device=device) if values is not None else None
    need = int(library().asg_csr_build_workspace_bytes(n_edges, n_rows))
    if need == 0:
        raise RuntimeError("asg_csr_build_workspace_bytes could not size the sort scratch")
    workspace = torch.empty(need, dtype=torch.uint8, device=device)
    check(library().asg_csr_from_edges(row_of_edge.data_ptr(), col_of_edge.data_ptr(),
                                       None if values is None else values.data_ptr(), n_edges, n_rows,
                                       crow.data_ptr(), col.data_ptr(), None if order is None else order.data_ptr(),
                                       None if permuted is None else permuted.data_ptr(), workspace.data_ptr(),
                                       workspace.numel(), _stream(device)))
    return crow, col, order, permuted


def csr_row_sample(crow: torch.Tensor, col: torch.Tensor, val: Optional[torch.Tensor], rows: torch.Tensor,
                   capacity: int):
    """Cut the rows ``rows`` (ascending int64, on the device) out of a CSR, all their edges kept.
    Returns (sample_crow[k + 1], sample_col[capacity], sample_val[capacity] or None, kept[2]) without
    synchronising; ``kept`` = (rows kept, edges kept) is a device tensor."""
    device = crow.device
    k = rows.numel()
    out_crow = torch.empty(k + 1, dtype=torch.long, device=device)
    out_col = torch.empty(capacity, dtype=torch.long, device=device)
    out_val = None if val is None else torch.empty(capacity, dtype=torch.float32, device=device)
    kept = torch.empty(2, dtype=torch.long, device=device)
    need = int(library().asg_row_sample_workspace_bytes(k))
    if need == 0:
        raise RuntimeError("asg_row_sample_workspace_bytes could not size the scan scratch")
    workspace = torch.empty(need, dtype=torch.uint8, device=device)
    check(library().asg_csr_row_sample(crow.data_ptr(), col.data_ptr(), _ptr(val), rows.data_ptr(), k, int(capacity),
                                       out_crow.data_ptr(), out_col.data_ptr(), _ptr(out_val), kept.data_ptr(),
                                       workspace.data_ptr(), workspace.numel(), _stream(device)))
    return out_crow, out_col, out_val, kept


def linear_bias(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out = x @ weight^T + bias on the tensor cores at float32 accuracy (contiguous float32 CUDA tensors)."""
    check(library().asg_linear_bias(x.data_ptr(), weight.data_ptr(), None if bias is None else bias.data_ptr(),
                                    out.data_ptr(), x.size(0), x.size(1), weight.size(0), _stream(x.device)))


def linear_umma_supported(in_features: int, out_features: int) -> bool:
    return bool(library().asg_linear_supported(int(in_features), int(out_features)))


def linear_bias_umma(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                     workspace: Optional[torch.Tensor] = None, flags: int = 0) -> torch.Tensor:
    """out = x @ weight^T + bias from the hand-written tcgen05 kernel; returns the workspace used (its
    header carries the kernel's status word)."""
    if workspace is None:
        workspace = torch.empty(int(library().asg_linear_workspace_bytes(x.size(1), weight.size(0))), dtype=torch.uint8,
                                device=x.device)
    check(library().asg_linear_bias_umma_ex(x.data_ptr(), weight.data_ptr(), None if bias is None else bias.data_ptr(),
                                            out.data_ptr(), x.size(0), x.size(1), weight.size(0), int(flags),
                                            workspace.data_ptr(), workspace.numel(), _stream(x.device)))
    return workspace


def conv_fused_supported(in_features: int, out_features: int) -> bool:
    return bool(library().asg_conv_fused_supported(int(in_features), int(out_features)))


CONV_FUSED_HUB_THRESHOLD = 64   # best of 32 ... 1024 on the 2.45 M-row power-law graph
CONV_FUSED_HUB_WARPS = 4


def conv_fused(crow: torch.Tensor, col: torch.Tensor, val: Optional[torch.Tensor], x: torch.Tensor, weight: torch.Tensor,
               bias: Optional[torch.Tensor], out: torch.Tensor, hub_threshold: int = CONV_FUSED_HUB_THRESHOLD,
               hub_warps: int = CONV_FUSED_HUB_WARPS, workspace: Optional[torch.Tensor] = None,
               extra_flags: int = 0) -> torch.Tensor:
    """out = (A x) @ weight^T + bias in one pass: the aggregated rows stay in shared memory (hub rows, of
    ``hub_threshold`` edges or more, take a first launch into a compact side buffer).  Returns the
    workspace used; its header carries the kernel's status word."""
    n_rows, nnz = crow.numel() - 1, col.numel()
    need = int(library().asg_conv_fused_workspace_bytes(n_rows, nnz, x.size(1), weight.size(0), int(hub_threshold)))
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    plan, flags = planned_workspace(crow, int(hub_threshold))
    check(library().asg_conv_fused(crow.data_ptr(), col.data_ptr(), None if val is None else val.data_ptr(), x.data_ptr(),
                                   weight.data_ptr(), None if bias is None else bias.data_ptr(), out.data_ptr(), n_rows,
                                   nnz, x.size(1), weight.size(0), int(hub_threshold), int(hub_warps),
                                   flags | int(extra_flags),
                                   plan.data_ptr(), plan.numel(), workspace.data_ptr(), workspace.numel(),
                                   _stream(x.device)))
    _plan_was_built(plan)
    return workspace


def push_to_peers(src: torch.Tensor, destinations: list[torch.Tensor], n_ctas: int = 32) -> None:
    """Store the contiguous tensor ``src`` into every tensor of ``destinations`` (same shape; peer-mapped
    memory of other GPUs) from ``n_ctas`` CTAs on the current stream."""
    if not destinations or src.numel() == 0:
        return
    pointers = (ctypes.c_void_p * len(destinations))(*[d.data_ptr() for d in destinations])
    check(library().asg_push_to_peers(src.data_ptr(), pointers, len(destinations), src.numel() * src.element_size(),
                                      int(n_ctas), _stream(src.device)))


def workspace_status(workspace: torch.Tensor) -> int:
    """Synchronising read of the status word kernels set when a bounded wait expired."""
    host = ctypes.c_int32(0)
    check(library().asg_workspace_status(workspace.data_ptr(), ctypes.byref(host), _stream(workspace.device)))
    torch.cuda.current_stream(workspace.device).synchronize()
    return int(host.value)
