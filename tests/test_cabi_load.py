"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols() -> list[str]:
    text = (ROOT / "include" / "autosage_b200.h").read_text(encoding="utf-8")
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(asg_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for required in ("asg_spmm_csr", "asg_spmm_csr_split", "asg_sddmm_csr", "asg_sddmm_csr_split",
                     "asg_csr_row_softmax", "asg_csr_attention", "asg_plan_build", "asg_last_error_string",
                     "asg_version", "asg_workspace_bytes"):
        assert required in names


def test_library_exports_every_declared_symbol(native_library):
    lib = ctypes.CDLL(str(native_library))
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_binding_table_matches_header(native_library):
    from autosage_b200 import _native

    assert sorted(_native.SIGNATURES) == declared_symbols()
    lib = _native.bind(str(native_library))
    assert lib.asg_version() == 100
    assert lib.asg_workspace_bytes(0) >= 256
    small, large = lib.asg_workspace_bytes(1000), lib.asg_workspace_bytes(1_000_000)
    assert small % 256 == 0 and large > small + 4 * 999_000


def test_argument_errors_need_no_gpu(native_library):
    """Validation happens before any CUDA call, so bad arguments are reported on a CPU-only host."""
    from autosage_b200 import _native

    lib = _native.bind(str(native_library))
    rc = lib.asg_spmm_csr_split(None, None, None, None, None, 4, 0, 8, 48, 8, 16, None, 0, None)
    assert rc == -1 and b"feature_tile must be 64 or 128" in lib.asg_last_error_string()
    rc = lib.asg_spmm_csr_split(None, None, None, None, None, 4, 0, 8, 64, 3, 16, None, 0, None)
    assert rc == -1 and b"warps_per_block must be 2, 4, or 8" in lib.asg_last_error_string()
    rc = lib.asg_spmm_csr_split(None, None, None, None, None, 4, 0, 8, 64, 4, 0, None, 0, None)
    assert rc == -1 and b"hub_threshold must be positive" in lib.asg_last_error_string()
    rc = lib.asg_sddmm_csr_split(None, None, None, None, None, 4, 4, 8, 4, 0, None, 0, None)
    assert rc == -1 and b"hub_threshold" in lib.asg_last_error_string()
    rc = lib.asg_spmm_csr(None, None, None, None, None, 4, 0, 8, None, 0, None)
    assert rc == -1  # null crow/x/y
    rc = lib.asg_plan_build(None, -1, 4, None, 0, None)
    assert rc == -1
