"""The benchmark's ceiling probes (libhtree_b200_probes.so, a library of its own beside the operator's) return plausible
bandwidths and refuse bad arguments."""
from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_probes_report_bandwidths():
    from htree_b200 import build
    L = ctypes.CDLL(build.PROBES_LIB)
    vp = ctypes.c_void_p
    for fn in (L.htree_probe_gather, L.htree_probe_reduction):
        fn.restype = ctypes.c_int
        fn.argtypes = [vp, ctypes.c_int64, ctypes.c_int32, ctypes.POINTER(ctypes.c_float), vp]
    buf = torch.zeros(32 << 20, dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    val = ctypes.c_float()
    assert L.htree_probe_gather(buf.data_ptr(), buf.numel(), 2, ctypes.byref(val), st) == 0
    assert 500.0 < val.value < 1.0e6          # GB/s: well above HBM for an L2-resident table
    assert L.htree_probe_reduction(buf.data_ptr(), buf.numel(), 2, ctypes.byref(val), st) == 0
    assert 200.0 < val.value < 1.0e6
    torch.cuda.synchronize()
    assert L.htree_probe_gather(None, 1 << 20, 1, ctypes.byref(val), st) != 0
    assert L.htree_probe_gather(buf.data_ptr(), 128, 1, ctypes.byref(val), st) != 0
    assert L.htree_probe_reduction(buf.data_ptr(), buf.numel(), 0, ctypes.byref(val), st) != 0
