"""``edge_index`` ([2, E], COO) to CSR, rows keyed by destination (default) or source.

Behaviour of the reference ``autosage/utils/csr.py:6-26``: edges of one row keep their original
relative order (stable sort by row id), row pointers are int64.
"""
from __future__ import annotations

import torch


def edge_index_to_csr(edge_index: torch.Tensor, num_nodes: int, *, rows_by: str = "dst") -> tuple[torch.Tensor, torch.Tensor]:
    if edge_index.ndim != 2 or edge_index.size(0) != 2:
        raise ValueError("edge_index must have shape [2, E]")
    if rows_by not in ("dst", "src"):
        raise ValueError("rows_by must be 'dst' or 'src'")
    src, dst = edge_index[0].to(torch.long), edge_index[1].to(torch.long)
    row_of_edge, col_of_edge = (dst, src) if rows_by == "dst" else (src, dst)
    permutation = torch.argsort(row_of_edge, stable=True)
    counts = torch.bincount(row_of_edge, minlength=num_nodes) if row_of_edge.numel() else torch.zeros(
        num_nodes, dtype=torch.long, device=edge_index.device)
    crow = torch.zeros(num_nodes + 1, dtype=torch.long, device=edge_index.device)
    torch.cumsum(counts[:num_nodes], 0, out=crow[1:])
    return crow.contiguous(), col_of_edge[permutation].contiguous()


__all__ = ["edge_index_to_csr"]
