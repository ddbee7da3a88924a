"""``edge_index`` ([2, E], COO) to CSR, rows keyed by destination (default) or source.

Behaviour of the reference ``autosage/utils/csr.py:6-26``: edges of one row keep their original
relative order (stable sort by row id), row pointers are int64.  CUDA inputs run the library's
device build (one 32-bit radix sort over the bits a row id can have, one gather pass); CPU inputs and
sizes beyond 2^31 run the reference's torch formulation.  Both produce the same integers.
"""
from __future__ import annotations

import os
from typing import Optional

import torch


def _torch_build(row_of_edge, col_of_edge, num_nodes: int, device):
    permutation = torch.argsort(row_of_edge, stable=True)
    counts = torch.bincount(row_of_edge, minlength=num_nodes) if row_of_edge.numel() else torch.zeros(
        num_nodes, dtype=torch.long, device=device)
    if counts.numel() > num_nodes:  # the reference's index_add_ raises here as well
        raise IndexError(f"edge_index holds a row id outside [0, {num_nodes})")
    crow = torch.zeros(num_nodes + 1, dtype=torch.long, device=device)
    torch.cumsum(counts, 0, out=crow[1:])
    return crow.contiguous(), col_of_edge[permutation].contiguous(), permutation


def _debug_check_row_ids(row_of_edge: torch.Tensor, num_nodes: int) -> None:
    """AUTOSAGE_CHECK_INDICES=1: the device build sorts only the bits a valid row id can have, so an id
    outside [0, num_nodes) would silently corrupt the CSR; check the range first (synchronises)."""
    if os.getenv("AUTOSAGE_CHECK_INDICES") != "1" or row_of_edge.numel() == 0:
        return
    low, high = int(row_of_edge.min().item()), int(row_of_edge.max().item())
    if low < 0 or high >= num_nodes:
        raise IndexError(f"edge_index holds a row id outside [0, {num_nodes}): found [{low}, {high}]")


def _native_build_ok(row_of_edge: torch.Tensor, num_nodes: int) -> bool:
    if not row_of_edge.is_cuda or os.getenv("AUTOSAGE_CSR_BUILD", "native") != "native":
        return False
    if row_of_edge.numel() >= 2 ** 31 or num_nodes >= 2 ** 31 or num_nodes < 1:
        return False
    from ..ops import load_native, native_load_error

    if not load_native():
        # no silent torch fallback on the GPU path: a CUDA call without the library is an error, as it
        # is for the operators (AUTOSAGE_CSR_BUILD=torch selects the torch formulation explicitly)
        raise RuntimeError(f"AutoSAGE CUDA extension is unavailable: {native_load_error()}")
    return True


def csr_with_order(edge_index: torch.Tensor, num_nodes: int, *, rows_by: str = "dst", want_order: bool = False,
                   edge_weight: Optional[torch.Tensor] = None):
    """(crow, col, order, permuted_weight): ``order`` is the stable ordering of the edges by row id
    (None unless asked for), ``permuted_weight`` is ``edge_weight[order]`` (None without weights)."""
    if edge_index.ndim != 2 or edge_index.size(0) != 2:
        raise ValueError("edge_index must have shape [2, E]")
    if rows_by not in ("dst", "src"):
        raise ValueError("rows_by must be 'dst' or 'src'")
    src, dst = edge_index[0].to(torch.long), edge_index[1].to(torch.long)
    row_of_edge, col_of_edge = (dst, src) if rows_by == "dst" else (src, dst)
    if _native_build_ok(row_of_edge, num_nodes):
        from .. import _native

        _debug_check_row_ids(row_of_edge, num_nodes)

        values = None
        if edge_weight is not None and edge_weight.dtype == torch.float32 and not (
                torch.is_grad_enabled() and edge_weight.requires_grad):
            values = edge_weight.detach().contiguous()
        need_order = want_order or (edge_weight is not None and values is None)
        crow, col, order, permuted = _native.csr_from_edges(row_of_edge.contiguous(), col_of_edge.contiguous(), values,
                                                            int(num_nodes), need_order)
        if edge_weight is not None and permuted is None:
            permuted = edge_weight.index_select(0, order)  # differentiable / non-float32 weights
        return crow, col, order, permuted
    crow, col, order = _torch_build(row_of_edge, col_of_edge, num_nodes, edge_index.device)
    permuted = None if edge_weight is None else edge_weight.index_select(0, order)
    return crow, col, (order if want_order else None), permuted


def edge_index_to_csr(edge_index: torch.Tensor, num_nodes: int, *, rows_by: str = "dst") -> tuple[torch.Tensor, torch.Tensor]:
    crow, col, _, _ = csr_with_order(edge_index, num_nodes, rows_by=rows_by)
    return crow, col


__all__ = ["edge_index_to_csr", "csr_with_order"]
