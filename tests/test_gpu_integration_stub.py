"""The reference-side binding printed in INTEGRATION.md, executed as written.

The stub (`autosage/_b200.py` in that document) registers the four ``torch.ops.autosage`` operators on
top of the C ABI from inside the reference package.  This test cuts the stub's code block out of the
document, runs it in a fresh interpreter that never imports this repository's Python package (both
would define the same operator names) and drives it with the cases the reference's own CUDA tests use
(``tests/test_cuda.py:32-69``: SpMM against torch.sparse.mm for F in {32, 64, 113, 128, 256}, the split
operator on a 512-row graph with one 400-edge hub, SDDMM against the gather-dot) and with the hub graph
of ``scripts/sweep_hubs.py:15-26`` (20,000 rows, one 12,000-edge hub, its tile/warp/threshold grid).
"""
from __future__ import annotations

import re
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent

DRIVER = '''
import itertools, sys, torch
sys.path.insert(0, {stub_dir!r})
import _b200
assert "autosage_b200" not in sys.modules
keep = _b200.bind_b200({library!r})
ops = torch.ops.autosage

def random_csr(rows, degree, seed=0):
    g = torch.Generator(device="cuda"); g.manual_seed(seed)
    counts = torch.randint(0, 2 * degree + 1, (rows,), generator=g, device="cuda")
    crow = torch.cat((torch.zeros(1, device="cuda", dtype=torch.long), counts.cumsum(0)))
    col = torch.randint(0, rows, (int(crow[-1].item()),), generator=g, device="cuda")
    return crow, col

torch.manual_seed(0)
for features in (32, 64, 113, 128, 256):                      # tests/test_cuda.py:32-40
    crow, col = random_csr(256, 12)
    x = torch.randn(256, features, device="cuda")
    values = torch.rand(col.numel(), device="cuda")
    expected = torch.sparse.mm(torch.sparse_csr_tensor(crow, col, values, size=(256, 256)), x)
    assert torch.allclose(ops.spmm_csr(crow, col, values, x), expected, rtol=1e-4, atol=3e-3), features

rows = 512                                                     # tests/test_cuda.py:43-57
counts = torch.full((rows,), 8, device="cuda", dtype=torch.long); counts[0] = 400
crow = torch.cat((torch.zeros(1, device="cuda", dtype=torch.long), counts.cumsum(0)))
col = torch.randint(0, rows, (int(crow[-1].item()),), device="cuda")
x = torch.randn(rows, 128, device="cuda")
expected = torch.sparse.mm(torch.sparse_csr_tensor(crow, col, torch.ones(col.numel(), device="cuda"), size=(rows, rows)), x)
assert torch.allclose(ops.spmm_csr_split(crow, col, None, x, 128, 8, 128), expected, rtol=1e-4, atol=3e-3)

crow, col = random_csr(128, 8)                                 # tests/test_cuda.py:60-69
query, key = torch.randn(128, 64, device="cuda"), torch.randn(128, 64, device="cuda")
pairs = torch.repeat_interleave(torch.arange(128, device="cuda"), crow[1:] - crow[:-1])
expected = (query[pairs] * key[col]).sum(dim=1)
assert torch.allclose(ops.sddmm_csr(crow, col, query, key), expected, rtol=1e-4, atol=1e-4)
assert torch.allclose(ops.sddmm_csr_split(crow, col, query, key, 4, 8), expected, rtol=1e-4, atol=1e-4)

g = torch.Generator(device="cuda"); g.manual_seed(0)           # scripts/sweep_hubs.py:15-26
rows = 20000
degrees = torch.full((rows,), 8, device="cuda", dtype=torch.long); degrees[0] = 12000
crow = torch.cat((torch.zeros(1, device="cuda", dtype=torch.long), degrees.cumsum(0)))
col = torch.randint(0, rows, (int(crow[-1].item()),), generator=g, device="cuda")
x = torch.randn(rows, 128, device="cuda")
expected = torch.sparse.mm(torch.sparse_csr_tensor(crow, col, torch.ones(col.numel(), device="cuda"), size=(rows, rows)), x)
for tile, warps, threshold in itertools.product((64, 128), (2, 4, 8), (256, 512, 1024, 2048)):
    actual = ops.spmm_csr_split(crow, col, None, x, tile, warps, threshold)
    assert torch.allclose(actual, expected, rtol=1e-4, atol=3e-3), (tile, warps, threshold)
torch.cuda.synchronize()
print("STUB-OK")
'''


def _stub_source() -> str:
    text = (ROOT / "INTEGRATION.md").read_text(encoding="utf-8")
    blocks = re.findall(r"```python\n(.*?)```", text, flags=re.S)
    stubs = [b for b in blocks if "def bind_b200" in b]
    assert len(stubs) == 1, "INTEGRATION.md must hold exactly one bind_b200 stub"
    return stubs[0]


def test_integration_stub_runs_the_reference_cuda_cases(tmp_path):
    from autosage_b200 import build as builder

    native_library = builder.library_path()   # the prebuilt file: a GPU box does not recompile
    assert native_library.is_file(), "libautosage_b200.so has not been built"
    (tmp_path / "_b200.py").write_text(_stub_source(), encoding="utf-8")
    script = tmp_path / "drive_stub.py"
    script.write_text(textwrap.dedent(DRIVER.format(stub_dir=str(tmp_path), library=str(native_library))), encoding="utf-8")
    done = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=240, cwd=str(tmp_path))
    assert done.returncode == 0 and "STUB-OK" in done.stdout, done.stdout[-2000:] + done.stderr[-4000:]
