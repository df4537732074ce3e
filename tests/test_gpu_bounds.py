"""The checked build (-DELFA_BOUNDS, selected with ELFA_BOUNDS=1): kernels run clean through it on ordinary shapes, and its
index test records a violation in the status word without touching memory. Runs in child processes because the variant is
chosen when the package is imported."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu

_CHILD = r"""
import torch
from elfa_b200 import native
from elfa_b200.native import lib, stream_ptr
from elfa_b200.ops.gemm import gemm
from elfa_b200.ops.gemm_mxfp8 import gemm_mxfp8, quantize_mxfp8
from elfa_b200.ops.attention import attention
dev = torch.device("cuda", 0)
want = int(__import__("os").environ.get("ELFA_BOUNDS", "0") == "1")
assert lib.raw("elfa_bounds_enabled")() == want
torch.manual_seed(0)
a = torch.randn(512, 384, device=dev).to(torch.bfloat16)
b = torch.randn(384, 640, device=dev).to(torch.bfloat16)
y = gemm(a, b, b_mn=True)
ref = a.float() @ b.float()
assert (y.float() - ref).abs().max().item() <= 2.0 ** -7 * ref.abs().max().item()
aq, _ = quantize_mxfp8(torch.randn(256, 512, device=dev).to(torch.bfloat16))
bq, _ = quantize_mxfp8(torch.randn(320, 512, device=dev).to(torch.bfloat16), right=True)
gemm_mxfp8(aq, bq)
qkv = torch.randn(256, 2, 3, 4, 64, device=dev).to(torch.bfloat16).requires_grad_(True)
o = attention(qkv, causal=True)
o.float().sum().backward()
torch.cuda.synchronize()
assert native.status() == 0, "ordinary shapes must not trip the index test"
lib.call("elfa_bounds_selftest", stream_ptr(a))
st = native.status()
assert st == (native.ST_BOUNDS if want else 0), hex(st)
lib.call("elfa_bounds_selftest", stream_ptr(a))
if want:
    try:
        native.check_status()
        raise SystemExit("check_status did not report the violation")
    except native.NativeError:
        pass
print("BOUNDS_OK", want)
"""


@pytest.mark.parametrize("bounds", ["1", "0"])
def test_checked_build_runs_clean_and_reports(cuda_device, bounds):
    env = dict(os.environ, ELFA_BOUNDS=bounds)
    r = subprocess.run([sys.executable, "-c", _CHILD], capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert f"BOUNDS_OK {bounds}" in r.stdout
