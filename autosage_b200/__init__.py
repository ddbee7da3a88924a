"""autosage_b200 - the sparse hot path of AutoSAGE rebuilt for NVIDIA B200 (sm_100a).

Same public names as the reference package (``autosage/__init__.py:7-17``); the CUDA side is
``libautosage_b200.so``, reached through a C ABI (``include/autosage_b200.h``).
"""
from ._auto import calibrate_full, csr_attention_forward, sddmm_csr_auto, spmm_csr_auto
from ._version import __version__
from .conv import AutoSAGEConv
from .ops import load_native, native_available, spmm_csr

__all__ = [
    "AutoSAGEConv",
    "__version__",
    "calibrate_full",
    "csr_attention_forward",
    "load_native",
    "native_available",
    "sddmm_csr_auto",
    "spmm_csr",
    "spmm_csr_auto",
]
