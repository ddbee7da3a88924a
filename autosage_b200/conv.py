"""``AutoSAGEConv``: neighbourhood aggregation (CSR SpMM over destination rows) + ``nn.Linear``.

Interface of the reference layer (``autosage/conv.py:13-56``): ``AutoSAGEConv(in_channels,
out_channels, *, mode="auto"|"native", bias=True)`` and ``forward(x, edge_index, edge_weight=None,
*, return_info=False)``.  The CSR build is memoised per ``edge_index`` tensor, so repeated forwards
over one graph do not re-sort the edges (the reference re-sorts on every call, ``conv.py:36,44``).
"""
from __future__ import annotations

import weakref
from typing import Optional

import torch
from torch import nn

from ._auto import spmm_csr_auto
from .ops import spmm_csr
from .utils.csr import edge_index_to_csr


def apply_linear(linear: nn.Linear, aggregated: torch.Tensor) -> torch.Tensor:
    """``linear(aggregated)``.  On CUDA float32 the product and the bias are issued separately
    (matmul, then an in-place add): cuBLAS's fused-bias SGEMM measured twice as slow as the plain one
    at these shapes on B200 (2.45 M x 128 -> 256: 6.1 ms against 3.2 ms), and the extra pass over the
    output (a copy-speed kernel of the library when no gradient is needed) costs far less than that.
    Same parameters, same float32 arithmetic, TF32 stays off."""
    if aggregated.is_cuda and aggregated.dtype == torch.float32 and aggregated.dim() == 2:
        out = torch.mm(aggregated, linear.weight.t())
        if linear.bias is None:
            return out
        if torch.is_grad_enabled() and (out.requires_grad or linear.bias.requires_grad):
            return out.add_(linear.bias)  # differentiable path
        from . import _native
        from .ops import load_native

        if load_native() and linear.bias.dtype == torch.float32:
            _native.add_row_bias(out, linear.bias.contiguous())
            return out
        return out.add_(linear.bias)
    return linear(aggregated)


class _CsrMemo:
    """Last (edge_index -> crow, col, edge permutation) conversion, valid while the same tensor object
    is passed again unmodified."""

    def __init__(self) -> None:
        self._ref = None
        self._version = -1
        self._nodes = -1
        self._value = None

    def get(self, edge_index: torch.Tensor, num_nodes: int, need_order: bool):
        same = (self._ref is not None and self._ref() is edge_index and self._version == edge_index._version
                and self._nodes == num_nodes)
        if not same:
            crow, col = edge_index_to_csr(edge_index, num_nodes, rows_by="dst")
            self._ref, self._version, self._nodes = weakref.ref(edge_index), edge_index._version, num_nodes
            self._value = [crow, col, None]
        if need_order and self._value[2] is None:
            self._value[2] = edge_index[1].to(torch.long).argsort(stable=True)
        return self._value


class AutoSAGEConv(nn.Module):
    def __init__(self, in_channels: int, out_channels: int, *, mode: str = "auto", bias: bool = True) -> None:
        super().__init__()
        if mode not in ("auto", "native"):
            raise ValueError("mode must be 'auto' or 'native'")
        self.linear = nn.Linear(in_channels, out_channels, bias=bias)
        self.mode = mode
        self._csr = _CsrMemo()

    def forward(self, x: torch.Tensor, edge_index: torch.Tensor, edge_weight: Optional[torch.Tensor] = None, *,
                return_info: bool = False):
        if edge_weight is not None:
            if edge_weight.ndim != 1 or edge_weight.numel() != edge_index.size(1):
                raise ValueError("edge_weight must contain one value per edge")
            if edge_weight.device != edge_index.device:
                raise ValueError("edge_weight and edge_index must be on the same device")
        crow, col, order = self._csr.get(edge_index, x.size(0), edge_weight is not None)
        weights = None if edge_weight is None else edge_weight.index_select(0, order)
        if self.mode == "auto":
            aggregated, info = spmm_csr_auto(crow, col, weights, x)
        else:
            aggregated = spmm_csr(crow, col, weights, x)
            info = {"operation": "spmm", "choice": "native" if x.is_cuda else "baseline", "from_cache": False}
        output = apply_linear(self.linear, aggregated)
        return (output, info) if return_info else output
