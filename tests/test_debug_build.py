"""The -DAXB_DEBUG flavour of the native library: device-side index checks record the first index that falls
outside its buffer, the kernel still takes its skip / clamp path (nothing faults), and the host reads the record."""
import ctypes
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_both_flavours_exist_and_say_what_they_are():
    from axon_b200 import _native
    _native.build()
    _native.build(debug=True)
    rel, dbg = ctypes.CDLL(str(_native._SO)), ctypes.CDLL(str(_native._SO_DEBUG))
    assert rel.axb_debug_build() == 0 and dbg.axb_debug_build() == 1
    out = (ctypes.c_int * 4)()
    assert rel.axb_debug_status(out, None, 0) == 0           # the release flavour never reports


_CHILD = r"""
import torch
from axon_b200 import _native
from axon_b200.ops import _common as C
from axon_b200.ops import activation as A
assert _native.debug_requested() and C.lib().axb_debug_build() == 1
table = torch.randn(64, 256, device="cuda").to(torch.bfloat16)
ids = torch.tensor([3, 7, 63, 0], dtype=torch.int32, device="cuda")
out = A.embedding_fwd(ids, table)
C.check_status()                                   # indices inside the table: clean
assert torch.equal(out, table[ids.long()])
bad = torch.tensor([3, 64 + 5, 1, 2], dtype=torch.int32, device="cuda")      # 69 is outside a 64-row table
out = A.embedding_fwd(bad, table)
torch.cuda.synchronize()
assert torch.equal(out[1], table[63]) and torch.equal(out[0], table[3])      # clamped, other rows untouched
try:
    C.check_status()
except C.NativeKernelError as e:
    msg = str(e)
    assert "elementwise.cu" in msg and "value 69" in msg and "limit 64" in msg, msg
    print("RECORDED", msg)
else:
    raise SystemExit("the out-of-range index was not recorded")
C.check_status()                                   # reading the record cleared it
print("CLEAN")
"""


@pytest.mark.gpu
def test_debug_flavour_records_an_out_of_range_index_without_faulting():
    env = dict(os.environ, AXON_NATIVE_DEBUG="1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-c", _CHILD], capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RECORDED" in r.stdout and "CLEAN" in r.stdout
