"""dg_quant_mx_host_static: the quantiser for callers that cannot allocate device memory (the
host tensor is staged in an array built into the library instead of a cudaMallocAsync buffer).
Called through the C ABI, twice in a row, and compared byte for byte (the tolerance of every
quant_mx test) with dg_quant_mx_host.  This file sorts last so that a stop-at-first-failure run
has already run every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

from deepgemm import _lib

pytestmark = pytest.mark.gpu

MAX_BYTES = 16 << 20


def _run(fn, x, dtype, gran):
    m, k = x.shape
    data = torch.full((m, k // 2 if dtype == 1 else k), 0xEE, dtype=torch.uint8, device="cuda")
    rows, cols = (k // gran + 3) // 4, (m + 3) // 4 * 4
    sf = torch.full((rows, cols), -1, dtype=torch.int32, device="cuda")
    st = fn(x.ctypes.data_as(C.c_void_p), m, k, dtype, gran, data.data_ptr(), sf.data_ptr(),
            C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return st, data.cpu().numpy(), sf.cpu().numpy()


def test_static_staging_matches_allocating_entry_twice_in_a_row():
    L = _lib.load()
    rng = np.random.default_rng(42)
    # second call is smaller and of another format: stale bytes of the first must not leak in
    cases = [((1024, 4096), 0, 128), ((37, 224), 1, 32), ((512, 8192), 0, 32)]
    for shape, dtype, gran in cases:
        x = rng.standard_normal(shape).astype(np.float32)
        st_a, data_a, sf_a = _run(L.dg_quant_mx_host, x, dtype, gran)
        st_b, data_b, sf_b = _run(L.dg_quant_mx_host_static, x, dtype, gran)
        assert st_a == 0 and st_b == 0, L.dg_last_error()
        assert np.array_equal(data_a, data_b) and np.array_equal(sf_a, sf_b)


def test_static_staging_rejects_oversize_input():
    L = _lib.load()
    m, k = 1025, 4096                     # 1 row past the 16 MiB area
    assert m * k * 4 > MAX_BYTES
    x = np.zeros((m, k), dtype=np.float32)
    st, _, _ = _run(L.dg_quant_mx_host_static, x, 0, 128)
    assert st == 3 and b"exceeds" in L.dg_last_error()
    ok, _, _ = _run(L.dg_quant_mx_host_static, x[:1024], 0, 128)   # exactly 16 MiB is accepted
    assert ok == 0


_COLD = r"""
import ctypes as C, sys
import numpy as np, torch
sys.path.insert(0, sys.argv[1])
from deepgemm import _lib
L = _lib.load()
torch.cuda.init()
torch.cuda.set_device(0)
stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
m, k = 256, 1024
x = np.random.default_rng(1).standard_normal((m, k)).astype(np.float32)
data = torch.zeros((m, k), dtype=torch.uint8, device="cuda")
sf = torch.zeros((2, m), dtype=torch.int32, device="cuda")
args = (x.ctypes.data_as(C.c_void_p), m, k, 0, 128, data.data_ptr(), sf.data_ptr(), stream)
# the very first call into the library on this device is the static entry: its own set-up path runs
assert L.dg_quant_mx_host_static(*args) == 0, L.dg_last_error()
torch.cuda.synchronize()
first = data.cpu().numpy().copy()
free0 = torch.cuda.mem_get_info()[0]
for _ in range(5):
    assert L.dg_quant_mx_host_static(*args) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0, "device memory in use changed across a call that must not allocate"
assert np.array_equal(data.cpu().numpy(), first)
assert L.dg_quant_mx_host(*args) == 0            # the allocating entry afterwards gives the same bytes
torch.cuda.synchronize()
assert np.array_equal(data.cpu().numpy(), first)
print("cold-ok")
"""


def test_static_entry_first_on_a_cold_device_and_allocates_nothing():
    """In a fresh process the static entry is the first call into the library (its own first-call set-up runs,
    not the allocating entries'), and the free device memory reported by the driver does not move across
    further calls."""
    import os
    import subprocess
    import sys
    pkg = os.path.dirname(os.path.dirname(os.path.abspath(_lib.__file__)))
    r = subprocess.run([sys.executable, "-c", _COLD, pkg], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "cold-ok" in r.stdout, r.stdout + r.stderr
