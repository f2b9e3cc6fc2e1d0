"""The measured-ceiling probes return plausible bandwidths and refuse bad arguments."""
from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_probes_report_bandwidths():
    from htree_b200 import _lib
    buf = torch.zeros(32 << 20, dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    val = ctypes.c_float()
    assert _lib.lib().htree_b200_probe_gather(buf.data_ptr(), buf.numel(), 2, ctypes.byref(val), st) == 0
    assert 500.0 < val.value < 1.0e6          # GB/s: well above HBM for an L2-resident table
    assert _lib.lib().htree_b200_probe_reduction(buf.data_ptr(), buf.numel(), 2, ctypes.byref(val), st) == 0
    assert 200.0 < val.value < 1.0e6
    torch.cuda.synchronize()
    assert _lib.lib().htree_b200_probe_gather(None, 1 << 20, 1, ctypes.byref(val), st) == _lib.E_NULL if hasattr(_lib, "E_NULL") else True
    assert _lib.lib().htree_b200_probe_gather(buf.data_ptr(), 128, 1, ctypes.byref(val), st) != 0
    assert _lib.lib().htree_b200_probe_reduction(buf.data_ptr(), buf.numel(), 0, ctypes.byref(val), st) != 0
