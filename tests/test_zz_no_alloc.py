"""htree_b200_backward_static_scratch: the backward entry point for callers that cannot allocate device memory
(an FFI host that owns only the tensors it was handed, or a process whose device memory is fully reserved by its
framework's pool).  Called through the C ABI and compared with htree_b200_backward on the same inputs, twice in a row:
the second call sees the built-in scratch array still holding the first call's contents and must clear it itself.

This file sorts last on purpose, so that a run that stops at the first failure has already run every other test."""
import ctypes

import numpy as np
import pytest
import torch

from tests import parity

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _call(lib, shape, q, ctx, out, dO, dq, dk_arg, dv_arg, static, half_tables=False):
    from htree_b200 import _lib
    L = ctx["num_layers"]
    ptrs = lambda ts: _lib.ptr_array([t.data_ptr() for t in ts])
    parents = [ctx["per_layer_parents"][l] for l in range(L)]
    flags = _lib.PARENTS_U16 if parents[0].dtype == torch.int16 else 0
    rope_half = ctx["rope_half"] if half_tables else None       # cos*scale, sin*scale as float16: packed-half rotations
    common = [ctypes.byref(shape), q.data_ptr(), ptrs(ctx["layers_k"]), ptrs(ctx["layers_v"]),
              ptrs(ctx["layers_k_rot"]) if ctx["layers_k_rot"] is not None else None, ctx["cos_cache"].data_ptr(),
              ctx["sin_cache"].data_ptr(), rope_half[0].data_ptr() if rope_half else None,
              rope_half[1].data_ptr() if rope_half else None, ctx["cos_cache"].shape[0], float(ctx["scale"]), out.data_ptr(),
              dO.data_ptr(),
              ctx["global_max"].data_ptr(), ctx["global_sum"].data_ptr(), ptrs(parents), dq.data_ptr()]
    stream = torch.cuda.current_stream().cuda_stream
    if static:
        return lib.htree_b200_backward_static_scratch(*common, dk_arg.data_ptr(), dv_arg.data_ptr(), None, flags, stream)
    return lib.htree_b200_backward(*common, ptrs(dk_arg), ptrs(dv_arg), None, None, flags, stream)


@pytest.mark.parametrize("dtype,K,compact", [("float32", 32, False), ("bfloat16", 128, False), ("bfloat16", 128, True)])
def test_static_scratch_backward_matches_backward_twice(dtype, K, compact, monkeypatch):
    """compact: the selections travel as uint16 node ids and the kernels rotate with the packed-half tables, the
    combination the autograd path of a memory-constrained caller would use."""
    import htree_b200 as ht
    from htree_b200 import _lib, ops
    if compact:
        monkeypatch.setattr(ops, "SELECTION_STORAGE", "uint16")
    lib = _lib.lib()
    assert lib.htree_b200_static_scratch_bytes() == 16 << 20
    B, T, H, Hkv, CR, TK, MTN = 2, 1500, 8, 2, 16, 8, 16                 # levels 1500 -> 94 -> 6
    tol = 1e-5 if dtype == "float32" else 1e-3                            # same kernels; only atomic order differs
    for seed in (41, 42):                                                 # two calls in a row, different data
        q, k, v, dO = (x.to(DEV) for x in parity.make_inputs(B, T, H, Hkv, K, K, dtype, seed))
        out, ctx = ht.htree_forward(q, k, v, CR, MTN, TK, _save_for_backward=True)
        L = ctx["num_layers"]
        assert L == 3
        shape = _lib.HtreeShape(B, T, H, Hkv, K, K, CR, TK, MTN, {"float32": 0, "bfloat16": 1}[dtype])
        dq_a = torch.empty(B, T, H, K, dtype=torch.float32, device=DEV)
        dk_l = [torch.empty(x.shape, dtype=torch.float32, device=DEV) for x in ctx["layers_k"]]
        dv_l = [torch.empty(x.shape, dtype=torch.float32, device=DEV) for x in ctx["layers_v"]]
        assert (ctx["per_layer_parents"][0].dtype == torch.int16) == compact
        assert _call(lib, shape, q, ctx, out, dO, dq_a, dk_l, dv_l, static=False, half_tables=compact) == 0
        dq_b = torch.empty_like(dq_a)
        dk_b = torch.full_like(dk_l[0], float("nan")); dv_b = torch.full_like(dv_l[0], float("nan"))
        assert _call(lib, shape, q, ctx, out, dO, dq_b, dk_b, dv_b, static=True, half_tables=compact) == 0
        torch.cuda.synchronize()
        for a, b in ((dq_a, dq_b), (dk_l[0], dk_b), (dv_l[0], dv_b)):
            scale = max(1.0, float(a.abs().max()))
            assert float((a - b).abs().max()) <= tol * scale


def test_static_scratch_rejects_oversized_levels():
    from htree_b200 import _lib
    lib = _lib.lib()
    # pooled levels of 4 x 65536 tokens with 4 KV heads and K = V = 128 need 71 MB: more than the 16 MiB array
    shape = _lib.HtreeShape(4, 65536, 64, 4, 128, 128, 16, 64, 256, 1)
    one = ctypes.c_void_p(256)
    rc = lib.htree_b200_backward_static_scratch(ctypes.byref(shape), 256, None, None, None, 256, 256, None, None, 2048, 0.1, 256, 256,
                                                256, 256, None, 256, one, one, None, 0, None)
    assert rc == -11
    assert "scratch" in _lib.error_string(rc)
