"""The C ABI: the library loads without a GPU, exports every symbol include/htree_b200.h declares, and rejects bad
arguments before anything is launched (no compute happens in these tests)."""
import ctypes
import os
import re

import pytest

from htree_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "htree_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(htree_b200_\w+)\s*\(", text)))


def test_header_and_binding_list_agree():
    assert declared_symbols() == sorted(_lib.SYMBOLS)


def test_library_exports_every_declared_symbol():
    lib = _lib.lib()
    for name in declared_symbols():
        assert hasattr(lib, name), name
    assert lib.htree_b200_version() == 3      # HTREE_B200_VERSION of the header


def test_level_sizes_follow_the_reference_loop():
    # pooling continues while the level is longer than max_top_nodes (src/parallel.py:941-945)
    assert _lib.level_sizes(2048, 16, 64) == [2048, 128, 8]
    assert _lib.level_sizes(2048, 16, 512) == [2048, 128]
    assert _lib.level_sizes(32768, 16, 128) == [32768, 2048, 128]
    assert _lib.level_sizes(65536, 16, 256) == [65536, 4096, 256]
    assert _lib.level_sizes(524288, 16, 512) == [524288, 32768, 2048, 128]
    assert _lib.level_sizes(12000, 16, 8192) == [12000, 750]
    assert _lib.level_sizes(300, 4, 32) == [300, 75, 19]
    assert _lib.level_sizes(64, 4, 64) == [64]


def _shape(**kw):
    d = dict(B=1, T=256, H=4, H_kv=2, K=16, V=16, compression_rate=4, top_k=8, max_top_nodes=32, dtype=0)
    d.update(kw)
    return _lib.HtreeShape(*[d.get(n, 0) for n, _ in _lib.HtreeShape._fields_])


def _fwd(shape, q=16, lk=None, n_pos=2048):
    lib = _lib.lib()
    dummy = (ctypes.c_void_p * 12)(*[ctypes.c_void_p(4096)] * 12)
    return lib.htree_b200_forward(ctypes.byref(shape), q, lk if lk is not None else dummy, dummy, None, None, None, 4096, 4096, None, None, n_pos,
                                  0.25, 4096, 4096, 4096, None, None, None, 0, None)


def test_argument_errors_are_reported_before_any_launch():
    assert _fwd(_shape(H=5)) == -2                      # H % H_kv
    assert _fwd(_shape(K=15)) == -2                     # odd K
    assert _fwd(_shape(dtype=7)) == -3
    assert _fwd(_shape(T=100000, max_top_nodes=1, compression_rate=2)) == -4      # too many levels
    assert _fwd(_shape(max_top_nodes=200)) == -5        # single level of 256 nodes > top_k*CR = 32
    assert _fwd(_shape(K=20, V=20)) == -7               # rows not 16-byte multiples
    assert _fwd(_shape(), q=None) == -1
    assert _fwd(_shape(), n_pos=8) == -6
    assert _fwd(_shape(), q=4100) == -7                 # misaligned pointer
    assert _fwd(_shape(T_q=100, t_offset=200)) == -10   # window runs past the sequence
    for code in (-1, -2, -3, -4, -5, -6, -7, -8, -9, -10):
        assert "unknown htree_b200 error" not in _lib.error_string(code)


def test_python_entry_points_refuse_cpu_tensors():
    import torch
    from htree_b200 import htree_forward
    q = torch.zeros(1, 8, 2, 16); k = torch.zeros(1, 8, 1, 16); v = torch.zeros(1, 8, 1, 16)
    with pytest.raises(RuntimeError, match="CUDA"):
        htree_forward(q, k, v, 4, 8, 2)
    with pytest.raises(ValueError):
        htree_forward(q[0], k, v, 4, 8, 2)


def test_compact_selection_storage_host_rules():
    """uint16 selections: refused when a pooled level has more than 65535 nodes; decoding restores the int32 layout."""
    import torch
    from htree_b200 import ops
    small = [torch.empty(1, 70000, 1, 8), torch.empty(1, 4375, 1, 8)]
    large = [torch.empty(1, 1, 1, 8).expand(1, 2 ** 21, 1, 8), torch.empty(1, 1, 1, 8).expand(1, 2 ** 17, 1, 8)]   # no memory behind them
    assert ops._parents_dtype(small, 64) is torch.int32
    ops.SELECTION_STORAGE = "uint16"
    try:
        assert ops._parents_dtype(small, 64) is torch.int16
        with pytest.raises(ValueError):
            ops._parents_dtype(large, 64)
        ops.SELECTION_STORAGE = "int8"
        with pytest.raises(ValueError):
            ops._parents_dtype(small, 64)
    finally:
        ops.SELECTION_STORAGE = "int32"
    stored = torch.tensor([0, 5, 40000, 65534, 65535], dtype=torch.int32).to(torch.int16)
    assert ops.decode_parents(stored).tolist() == [0, 5, 40000, 65534, -1]
    same = torch.tensor([3, -1], dtype=torch.int32)
    assert ops.decode_parents(same) is same


def test_per_kernel_shims_check_their_arguments_without_a_gpu():
    """htree_b200.compat: level index from layer_power, and CPU tensors are refused before anything is launched."""
    import torch
    from htree_b200 import compat
    assert compat._level_of(1, 16) == 0 and compat._level_of(256, 16) == 2 and compat._level_of(8, 8) == 1
    with pytest.raises(ValueError):
        compat._level_of(24, 16)
    x = torch.zeros(1, 16, 1, 8)
    with pytest.raises(RuntimeError):
        compat.htree_build_kernel[(1, 1)](x, x, x[:, :4], x[:, :4], N_child=16, N_parent=4, B=1, H_kv=1, K=8, V=8,
                                          COMPRESSION_RATE=4, BLOCK_SIZE=8)
    with pytest.raises(RuntimeError):
        compat.htree_merge_to_global_kernel[(16, 1)](x[..., 0], x[..., 0], x, x[..., 0], x[..., 0], x, B=1, T=16, H=1, V=8)
    assert "htree_select_accumulate_gqa_kernel" in repr(compat.htree_select_accumulate_gqa_kernel)


def test_topk_runner_refuses_cpu_tensors():
    import torch
    from htree_b200 import topk_bench
    with pytest.raises(ValueError):
        topk_bench.topk(torch.zeros(2, 64), 8)
    assert set(topk_bench.METHODS) == {"threshold_search", "radix_select", "bitonic"}
