"""Per-kernel call surface of the reference (src/parallel.py of skywong14/htree), for code that drives the levels one by one.

The reference exposes its Triton kernels as module-level objects launched as ``kernel[grid](tensors..., NAME=value...)``;
its parity harness (correctness_test.py:105-347) builds the tree and runs the forward level by level through them so
that it can record the per-level state.  The objects below accept the same call form -- the same positional tensors and
the same keyword names -- and run the CUDA kernels of this library through its C ABI.  The launch grid and the Triton
tuning constants (BLOCK_SIZE, G_PAD, TILE_P, LOG_N, N_DIMS_TOPK, DROP_BLOCK, NEG_INF, SCORE_VALID_THRESHOLD) are
accepted and ignored: the library sizes its own launches.

    htree_build_kernel                   src/parallel.py:88-165     one mean-pooling step child level -> parent level
    htree_select_accumulate_gqa_kernel   src/parallel.py:537-867    one level above the leaves: score, Top-K, accumulate
    htree_bottom_accumulate_gqa_kernel   src/parallel.py:369-530    the leaf level: score and accumulate everything
    htree_merge_to_global_kernel         src/parallel.py:248-313    online-softmax merge of a level into the global state
    htree_final_normalize_kernel         src/parallel.py:316-363    output = global_output / global_sum

The per-level kernels compute in fp32 arithmetic (the library's general kernels); the fused tensor-core path is reached
through ``htree_forward`` only.
"""
from __future__ import annotations

import ctypes
from typing import Callable

import torch

from . import _lib
from .ops import _DTYPES, _status, _stream


class KernelShim:
    """``shim[grid](...)`` calls the wrapped launcher; the grid is ignored."""

    def __init__(self, name: str, fn: Callable):
        self.__name__ = name
        self._fn = fn

    def __getitem__(self, grid):
        return self._fn

    def __call__(self, *a, **kw):
        return self._fn(*a, **kw)

    def __repr__(self):
        return f"<htree_b200 kernel shim {self.__name__}>"


def _need_cuda(*tensors):
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("htree_b200 kernels run on CUDA tensors only")
        if not t.is_contiguous():
            raise ValueError("htree_b200 kernels take contiguous tensors")


def _level_of(layer_power: int, compression_rate: int) -> int:
    level, p = 0, 1
    while p < layer_power:
        p *= compression_rate
        level += 1
    if p != layer_power:
        raise ValueError(f"layer_power {layer_power} is not a power of COMPRESSION_RATE {compression_rate}")
    return level


def _build(child_k, child_v, parent_k, parent_v, *, N_child, N_parent, B, H_kv, K, V, COMPRESSION_RATE, BLOCK_SIZE=None):
    _need_cuda(child_k, child_v, parent_k, parent_v)
    if N_parent != (N_child + COMPRESSION_RATE - 1) // COMPRESSION_RATE:
        raise ValueError("N_parent must be ceil(N_child / COMPRESSION_RATE)")
    if child_k.dtype not in _DTYPES:
        raise TypeError(f"unsupported dtype {child_k.dtype}")
    # a two-level tree whose leaves are the child level
    shape = _lib.HtreeShape(B, N_child, H_kv, H_kv, K, V, COMPRESSION_RATE, 1, max(N_parent, 1), _DTYPES[child_k.dtype],
                            N_child, 0)
    if N_child <= N_parent:      # N_child == 1: nothing to pool
        parent_k.copy_(child_k)
        parent_v.copy_(child_v)
        return
    with torch.cuda.device(child_k.device):
        _lib.check(_lib.lib().htree_b200_build_tree(
            ctypes.byref(shape), _lib.ptr_array([child_k.data_ptr(), parent_k.data_ptr()]),
            _lib.ptr_array([child_v.data_ptr(), parent_v.data_ptr()]), None, None, None, None, None, _stream()), "htree_build_kernel")


def _level(q, k_layer, v_layer, prev_selected_parents, cos_cache, sin_cache, layer_max, layer_sum, layer_output,
           next_selected_parents=None, *, layer_power, B, T, H, H_kv, K, V, N_layer, COMPRESSION_RATE, TOP_K, scale,
           NUM_GROUPS=None, **_tuning):
    tensors = [q, k_layer, v_layer, prev_selected_parents, cos_cache, sin_cache, layer_max, layer_sum, layer_output]
    if next_selected_parents is not None:
        tensors.append(next_selected_parents)
    _need_cuda(*tensors)
    if q.dtype not in _DTYPES:
        raise TypeError(f"unsupported dtype {q.dtype}")
    if prev_selected_parents.dtype != torch.int32:
        raise TypeError("parent lists are int32")
    for t in (cos_cache, sin_cache, layer_max, layer_sum, layer_output):
        if t.dtype != torch.float32:
            raise TypeError("rotary tables and level state are float32")
    if NUM_GROUPS is not None and NUM_GROUPS != H // H_kv:
        raise ValueError("NUM_GROUPS must be H // H_kv")
    level = _level_of(int(layer_power), int(COMPRESSION_RATE))
    shape = _lib.HtreeShape(B, T, H, H_kv, K, V, COMPRESSION_RATE, TOP_K, TOP_K * COMPRESSION_RATE, _DTYPES[q.dtype], T, 0)
    with torch.cuda.device(q.device):
        _lib.check(_lib.lib().htree_b200_level_forward(
            ctypes.byref(shape), level, int(N_layer), q.data_ptr(), k_layer.data_ptr(), v_layer.data_ptr(),
            prev_selected_parents.data_ptr(), cos_cache.data_ptr(), sin_cache.data_ptr(), cos_cache.shape[0],
            float(scale), layer_max.data_ptr(), layer_sum.data_ptr(), layer_output.data_ptr(),
            next_selected_parents.data_ptr() if next_selected_parents is not None else None,
            _status(q.device).data_ptr(), _stream()), "level_forward")


def _select(q, k_layer, v_layer, prev_selected_parents, cos_cache, sin_cache, layer_max, layer_sum, layer_output,
            next_selected_parents, **kw):
    if _level_of(int(kw["layer_power"]), int(kw["COMPRESSION_RATE"])) == 0:
        raise ValueError("htree_select_accumulate_gqa_kernel runs above the leaf level (layer_power > 1)")
    _level(q, k_layer, v_layer, prev_selected_parents, cos_cache, sin_cache, layer_max, layer_sum, layer_output,
           next_selected_parents, **kw)


def _bottom(q, k_layer, v_layer, prev_selected_parents, cos_cache, sin_cache, layer_max, layer_sum, layer_output, **kw):
    if int(kw["layer_power"]) != 1:
        raise ValueError("htree_bottom_accumulate_gqa_kernel runs at the leaf level (layer_power == 1)")
    _level(q, k_layer, v_layer, prev_selected_parents, cos_cache, sin_cache, layer_max, layer_sum, layer_output, None, **kw)


def _merge(layer_max, layer_sum, layer_output, global_max, global_sum, global_output, *, B, T, H, V):
    _need_cuda(layer_max, layer_sum, layer_output, global_max, global_sum, global_output)
    with torch.cuda.device(layer_max.device):
        _lib.check(_lib.lib().htree_b200_merge_to_global(
            layer_max.data_ptr(), layer_sum.data_ptr(), layer_output.data_ptr(), global_max.data_ptr(),
            global_sum.data_ptr(), global_output.data_ptr(), B * T * H, V, _stream()), "merge_to_global")


def _normalize(global_output, global_sum, output, *, B, T, H, V):
    _need_cuda(global_output, global_sum, output)
    if output.dtype not in _DTYPES:
        raise TypeError(f"unsupported dtype {output.dtype}")
    with torch.cuda.device(output.device):
        _lib.check(_lib.lib().htree_b200_final_normalize(
            global_output.data_ptr(), global_sum.data_ptr(), output.data_ptr(), _DTYPES[output.dtype], B * T * H, V,
            _stream()), "final_normalize")


htree_build_kernel = KernelShim("htree_build_kernel", _build)
htree_select_accumulate_gqa_kernel = KernelShim("htree_select_accumulate_gqa_kernel", _select)
htree_bottom_accumulate_gqa_kernel = KernelShim("htree_bottom_accumulate_gqa_kernel", _bottom)
htree_merge_to_global_kernel = KernelShim("htree_merge_to_global_kernel", _merge)
htree_final_normalize_kernel = KernelShim("htree_final_normalize_kernel", _normalize)
