"""``AutoSAGEConv``: neighbourhood aggregation (CSR SpMM over destination rows) + ``nn.Linear``.

Interface of the reference layer (``autosage/conv.py:13-56``): ``AutoSAGEConv(in_channels,
out_channels, *, mode="auto"|"native", bias=True)`` and ``forward(x, edge_index, edge_weight=None,
*, return_info=False)``.  The CSR build is memoised per ``edge_index`` tensor, so repeated forwards
over one graph do not re-sort the edges (the reference re-sorts on every call, ``conv.py:36,44``).
"""
from __future__ import annotations

import os
import weakref
from typing import Optional

import torch
from torch import nn

from ._auto import spmm_csr_auto
from .ops import spmm_csr
from .utils.csr import csr_with_order, edge_index_to_csr  # noqa: F401  (edge_index_to_csr: re-exported as in the reference)


def _tensor_core_linear_ok(linear: nn.Linear, aggregated: torch.Tensor) -> bool:
    if os.getenv("AUTOSAGE_LINEAR", "tensor") != "tensor":
        return False
    if torch.is_grad_enabled() and (aggregated.requires_grad or any(p.requires_grad for p in linear.parameters())):
        return False
    weight, bias = linear.weight, linear.bias
    # the kernel moves 16-byte vectors: a parameter that is a view into a flat buffer may start elsewhere
    aligned = all(t is None or t.data_ptr() % 16 == 0 for t in (aggregated, weight, bias))
    return (aligned and weight.dtype == torch.float32 and weight.is_cuda and weight.device == aggregated.device
            and (bias is None or bias.dtype == torch.float32)
            and aggregated.size(1) % 4 == 0 and weight.size(0) % 4 == 0 and aggregated.size(0) < 2 ** 31)


def apply_linear(linear: nn.Linear, aggregated: torch.Tensor) -> torch.Tensor:
    """``linear(aggregated)`` for the layer's projection.

    CUDA float32, no gradient wanted: the library's tensor-core Linear (float32 operands split into
    three bfloat16 pieces each, piece products summed in float32, bias in the epilogue).  It keeps
    float32 accuracy - no TF32 rounding.  in_features a multiple of 64 and out_features a multiple of
    32 up to 256 run the hand-written tcgen05 kernel (1.05 ms at 2.45 M x 128 -> 256 on B200), other
    sizes the CUTLASS instantiation (1.5 ms there; ``AUTOSAGE_LINEAR_KERNEL=cutlass`` forces it); cuBLAS
    SGEMM plus a bias pass takes 3.3 ms.  ``AUTOSAGE_LINEAR=cublas`` selects the cuBLAS route below.

    Otherwise on CUDA float32 the product and the bias are issued separately (matmul, then an in-place
    add): cuBLAS's fused-bias SGEMM measured twice as slow as the plain one at these shapes (6.1 ms
    against 3.2 ms).  Same parameters, same float32 arithmetic, TF32 stays off."""
    if aggregated.is_cuda and aggregated.dtype == torch.float32 and aggregated.dim() == 2:
        from . import _native
        from .ops import load_native

        native = load_native()
        if native and _tensor_core_linear_ok(linear, aggregated):
            x = aggregated if aggregated.is_contiguous() else aggregated.contiguous()
            out = torch.empty(x.size(0), linear.out_features, dtype=torch.float32, device=x.device)
            bias = None if linear.bias is None else linear.bias.detach().contiguous()
            weight = linear.weight.detach().contiguous()
            if (os.getenv("AUTOSAGE_LINEAR_KERNEL", "umma") == "umma"
                    and _native.linear_umma_supported(x.size(1), linear.out_features)):
                _native.linear_bias_umma(x.detach(), weight, bias, out)   # the hand-written tcgen05 kernel
                return out
            if _native.library().asg_linear_available():
                _native.linear_bias(x.detach(), weight, bias, out)        # other sizes: the CUTLASS instantiation
                return out
        out = torch.mm(aggregated, linear.weight.t())
        if linear.bias is None:
            return out
        if torch.is_grad_enabled() and (out.requires_grad or linear.bias.requires_grad):
            return out.add_(linear.bias)  # differentiable path
        if native and linear.bias.dtype == torch.float32:
            _native.add_row_bias(out, linear.bias.contiguous())
            return out
        return out.add_(linear.bias)
    return linear(aggregated)


def _fused_forward_ok(linear: nn.Linear, x: torch.Tensor, weights: Optional[torch.Tensor]) -> bool:
    """The one-kernel form of the layer (aggregation and Linear fused, ``AUTOSAGE_CONV_FUSED=1``): CUDA
    float32, no gradient wanted, 64 or 128 input features, output features a multiple of 32 up to 256."""
    if os.getenv("AUTOSAGE_CONV_FUSED", "0") != "1" or not x.is_cuda or x.dtype != torch.float32 or x.dim() != 2:
        return False
    tensors = [x, linear.weight, linear.bias] + ([] if weights is None else [weights])
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors):
        return False
    from . import _native
    from .ops import load_native

    if not load_native() or not _native.conv_fused_supported(x.size(1), linear.out_features):
        return False
    return (x.is_contiguous() and x.data_ptr() % 32 == 0 and linear.weight.dtype == torch.float32
            and linear.weight.device == x.device and (linear.bias is None or linear.bias.dtype == torch.float32)
            and (weights is None or weights.dtype == torch.float32) and x.size(0) < 2 ** 31 - 2048)


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
            crow, col, order, _ = csr_with_order(edge_index, num_nodes, rows_by="dst", want_order=need_order)
            self._ref, self._version, self._nodes = weakref.ref(edge_index), edge_index._version, num_nodes
            self._value = [crow, col, order]
        if need_order and self._value[2] is None:
            self._value[2] = csr_with_order(edge_index, num_nodes, rows_by="dst", want_order=True)[2]
        return self._value

    def __reduce__(self):
        # the memo is a cache keyed by a weak reference: a pickled / saved / spawned layer starts without it
        return (_CsrMemo, ())


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
        if _fused_forward_ok(self.linear, x, weights):
            # Opt-in: it measured slower than the two kernels below on the large benchmark graph (the
            # gather inside the fused kernel runs with one CTA per SM), so it is not scheduled by default.
            from . import _native

            output = torch.empty(x.size(0), self.linear.out_features, dtype=torch.float32, device=x.device)
            bias = None if self.linear.bias is None else self.linear.bias.detach().contiguous()
            _native.conv_fused(crow, col, None if weights is None else weights.contiguous(), x,
                               self.linear.weight.detach().contiguous(), bias, output)
            info = {"operation": "conv_fused", "choice": "fused", "from_cache": False,
                    "hub_threshold": _native.CONV_FUSED_HUB_THRESHOLD}
            return (output, info) if return_info else output
        if self.mode == "auto":
            aggregated, info = spmm_csr_auto(crow, col, weights, x)
        else:
            aggregated = spmm_csr(crow, col, weights, x)
            info = {"operation": "spmm", "choice": "native" if x.is_cuda else "baseline", "from_cache": False}
        output = apply_linear(self.linear, aggregated)
        return (output, info) if return_info else output
