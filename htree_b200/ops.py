"""Host side of the htree operator: the reference's Python entry points over the C ABI of libhtree_b200.

Same names, keyword arguments, tensor layouts and return values as the reference (skywong14/htree):
    htree_forward                  src/parallel.py:874-1159
    htree_backward                 src/backward.py:941-1119
    HTreeTritonFunction            src/backward.py:1126-1193   (alias of HTreeFunction here)
    htree_forward_triton_autograd  src/backward.py:1196-1208
    LayerTrace                     src/naive.py:13-19
PyTorch supplies device memory and the current stream only; all arithmetic runs in the CUDA library.  There is no
CPU path: tensors must live on a CUDA device and the library must have been built.

Differences from the reference that callers can rely on:
  * `max_top_nodes` may be smaller than `top_k_per_layer * compression_rate` (the reference asserts equality).  The
    additional top levels then hold at most top_k nodes, every candidate is kept and nothing is accumulated there, so
    the result equals the reference called with max_top_nodes = top_k_per_layer * compression_rate.
  * sizes need not be powers of two, and top_k_per_layer need not be a multiple of 64 or of compression_rate.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from . import _lib

HTREE_SCORE_NEG_INF: float = -1.0e10                                  # src/parallel.py:75
HTREE_SCORE_VALID_THRESHOLD: float = HTREE_SCORE_NEG_INF * 0.9         # src/parallel.py:81

_DTYPES = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}

# Keep the per-level selections from the forward for the backward of the autograd function (True), or rebuild them
# in the backward with the selection-only pass like the reference does (False; saves L*B*T*H_kv*top_k*4 bytes).
SAVE_SELECTIONS_FOR_BACKWARD = True

# Storage of the per-level selections (bwd_ctx["per_layer_parents"]): "int32" is the reference's layout
# (src/parallel.py:1044, -1 = none); "uint16" halves that memory (torch.int16 tensors holding the unsigned bit
# pattern, 0xFFFF = none; decode_parents() converts) and needs every pooled level to have at most 65535 nodes.
SELECTION_STORAGE = "int32"

# Largest temporary the forward may allocate for handing selections from its selection kernel to its accumulation
# kernel when the caller does not keep them (see htree_forward); above it the fused single-kernel forward runs.
SPLIT_FORWARD_MAX_BYTES = 4 << 30


def _parents_dtype(layers_k, top_k: int):
    if SELECTION_STORAGE == "int32":
        return torch.int32
    if SELECTION_STORAGE != "uint16":
        raise ValueError(f"SELECTION_STORAGE must be 'int32' or 'uint16', not {SELECTION_STORAGE!r}")
    if top_k > 65535 or any(x.shape[1] > 65535 for x in layers_k[1:]):
        raise ValueError("SELECTION_STORAGE='uint16' needs pooled levels of at most 65535 nodes")
    return torch.int16


def _parents_flag(parents) -> int:
    first = parents[0] if parents is not None else None
    return _lib.PARENTS_U16 if first is not None and first.dtype == torch.int16 else 0


def decode_parents(t: torch.Tensor) -> torch.Tensor:
    """Selections in the reference's layout (int32, -1 = none) from either storage format."""
    if t.dtype == torch.int32:
        return t
    x = t.to(torch.int32) & 0xFFFF
    return torch.where(x == 0xFFFF, torch.full_like(x, -1), x)


@dataclass
class LayerTrace:
    layer_idx: int
    selected_parents: Optional[torch.Tensor]
    layer_max: torch.Tensor
    layer_sum: torch.Tensor
    layer_output: torch.Tensor


_rope_tables: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor]] = {}
_status_words: Dict[torch.device, torch.Tensor] = {}


def rope_cache(k_dim: int, cache_size: int, rope_base: float, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables [cache_size, k_dim/2] fp32 (src/parallel.py:983-988), built once per configuration.

    The tables are evaluated with torch's CPU float32 kernels and copied to the device: the angle pos*inv_freq is
    rounded to float32 before the cosine, so results only match the reference's CPU oracle bit for bit when
    inv_freq comes out of the same pow implementation."""
    key = (int(k_dim), int(cache_size), float(rope_base), torch.device(device))
    hit = _rope_tables.get(key)
    if hit is None:
        inv_freq = 1.0 / (rope_base ** (torch.arange(0, k_dim, 2, dtype=torch.float32) / k_dim))
        freqs = torch.outer(torch.arange(cache_size, dtype=torch.float32), inv_freq)
        hit = (freqs.cos().to(device).contiguous(), freqs.sin().to(device).contiguous())
        _rope_tables[key] = hit
    return hit


_rope_half: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor]] = {}


def rope_cache_half(k_dim: int, cache_size: int, rope_base: float, scale: float, device):
    """cos*scale and sin*scale as float16 tables (same shape as rope_cache), for the packed-half query rotation of the
    tensor-core kernels in the passes that do not decide the Top-K."""
    key = (int(k_dim), int(cache_size), float(rope_base), float(scale), torch.device(device))
    hit = _rope_half.get(key)
    if hit is None:
        c, s = rope_cache(k_dim, cache_size, rope_base, device)
        hit = ((c * float(scale)).to(torch.float16).contiguous(), (s * float(scale)).to(torch.float16).contiguous())
        _rope_half[key] = hit
    return hit


def _status(device) -> torch.Tensor:
    device = torch.device(device)
    w = _status_words.get(device)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[device] = w
    return w


def check_status(device=None) -> None:
    """Synchronise and raise if a kernel flagged a problem since the last check: an out-of-range node index (bits 0-3), or a
    bounded wait of the pipelined forward that ran out (bit 4)."""
    device = torch.device(device if device is not None else torch.cuda.current_device())
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    w = _status_words.get(device)
    if w is not None:
        v = int(w.item())
        if v:
            w.zero_()
            what = []
            if v & 0xF:
                what.append("a node index outside its tree level (clamped)")
            if v & 16:
                what.append("an asynchronous operand copy of the pipelined forward did not complete within its bounded wait "
                            "(the affected outputs were not written)")
            raise RuntimeError(f"htree_b200 kernels reported device-side status 0x{v:x}: " + "; ".join(what or ["unknown bits"]))


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _validate(q, k, v, compression_rate, max_top_nodes, top_k_per_layer, q_offset=None):
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("q/k/v must be rank-4 tensors")          # src/naive.py:141-142
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("htree_b200 runs on CUDA tensors only; there is no CPU implementation")
    B, T_q, H, K = q.shape
    T = T_q if q_offset is None else k.shape[1]
    H_kv, V = k.shape[2], v.shape[-1]
    assert H % H_kv == 0, f"H ({H}) must be divisible by H_kv ({H_kv})"                      # src/parallel.py:912
    assert k.shape[2] == v.shape[2], "K and V must have same number of heads"                # src/parallel.py:914
    assert tuple(k.shape[:2]) == (B, T) and tuple(v.shape[:2]) == (B, T) and k.shape[3] == K  # src/naive.py:146
    if q_offset is not None:
        assert 0 <= q_offset and q_offset + T_q <= T, "query window must lie inside the key/value sequence"
    assert q.dtype == k.dtype == v.dtype and q.dtype in _DTYPES, "q, k, v must share one of fp32/bf16/fp16"
    assert max_top_nodes <= top_k_per_layer * compression_rate, (
        f"max_top_nodes ({max_top_nodes}) must not exceed top_k_per_layer*compression_rate "
        f"({top_k_per_layer}*{compression_rate})")                                            # cf. src/parallel.py:917-920
    return _lib.HtreeShape(B, T, H, H_kv, K, V, int(compression_rate), int(top_k_per_layer), int(max_top_nodes),
                           _DTYPES[q.dtype], 0 if q_offset is None else T_q, 0 if q_offset is None else int(q_offset))


def _ptrs(tensors) -> ctypes.Array:
    return _lib.ptr_array([t.data_ptr() if t is not None else None for t in tensors])


def build_tree(k: torch.Tensor, v: torch.Tensor, compression_rate: int, max_top_nodes: int,
               rope_base: Optional[float] = None):
    """Mean-pool tree (src/parallel.py:941-976).  Returns (layers_k, layers_v); level 0 are k and v themselves.

    With `rope_base` given, (layers_k, layers_v, layers_k_rot, layers_v_blk) is returned; the last two are the operand
    copies the tensor-core kernels read (None where no such kernel exists: fp32, or head sizes / compression rates they
    do not cover): the keys of every level rotated by their child index (node % compression_rate), float16 for bf16
    inputs too (one rounding of the rotated value, with half's finer significand), and the values of every level grouped
    per parent in the order the kernel's lanes consume them ([B, ceil(N/CR)*CR, H_kv, V], rows past N zero)."""
    k = k.contiguous(); v = v.contiguous()
    B, T, H_kv, K = k.shape
    V = v.shape[-1]
    sizes = _lib.level_sizes(T, compression_rate, max_top_nodes)
    layers_k, layers_v = [k], [v]
    for n in sizes[1:]:
        layers_k.append(torch.empty(B, n, H_kv, K, dtype=k.dtype, device=k.device))
        layers_v.append(torch.empty(B, n, H_kv, V, dtype=v.dtype, device=v.device))
    want_rot = rope_base is not None and _rotatable(k.dtype, K, V, compression_rate)
    layers_kr = [_rotated_like(x) for x in layers_k] if want_rot else None
    want_blk = want_rot and _blockable(V, compression_rate)
    layers_vb = [_blocked_like(x, compression_rate) for x in layers_v] if want_blk else None
    want_kblk = want_blk and _pipelined(k.dtype, K, compression_rate)
    layers_kb = [_blocked_like(x, compression_rate) for x in layers_kr] if want_kblk else None
    if len(sizes) > 1 or want_rot:
        shape = _lib.HtreeShape(B, T, H_kv, H_kv, K, V, int(compression_rate), 1, int(max_top_nodes),
                                _DTYPES[k.dtype])   # H and top_k play no role in the tree
        cos_c = sin_c = None
        if want_rot:
            cos_c, sin_c = rope_cache(K, max(int(compression_rate), 16), rope_base, k.device)
        with torch.cuda.device(k.device):
            _lib.check(_lib.lib().htree_b200_build_tree(
                ctypes.byref(shape), _ptrs(layers_k), _ptrs(layers_v), _ptrs(layers_kr) if want_rot else None,
                _ptrs(layers_kb) if want_kblk else None, _ptrs(layers_vb) if want_blk else None,
                cos_c.data_ptr() if want_rot else None, sin_c.data_ptr() if want_rot else None, _stream()),
                "build_tree")
    if rope_base is not None:
        return layers_k, layers_v, layers_kr, OperandBlocks(layers_vb, layers_kb) if layers_vb is not None else None
    return layers_k, layers_v


class OperandBlocks(list):
    """The blocked values of every level (the list itself) together with the blocked keys of every level (`.keys`, or
    None where the pipelined kernels do not apply): the per-parent operand copies of the tensor-core forward."""

    def __init__(self, values, keys=None):
        super().__init__(values)
        self.keys = keys


def _pipelined(dtype, K: int, compression_rate: int) -> bool:
    """Shapes with a pipelined forward (operand blocks streamed through shared memory): 16-bit types, 128-wide heads,
    16 children per parent."""
    return dtype != torch.float32 and K == 128 and int(compression_rate) == 16


def build_tree_into(k: torch.Tensor, v: torch.Tensor, out_k, out_v, compression_rate: int, max_top_nodes: int) -> None:
    """Mean-pool tree of (k, v) with the pooled levels written into caller-provided tensors out_k[i], out_v[i]
    (level i+1; contiguous, shaped [B, N_{i+1}, H_kv, *]).  Sequence-sharded runs pool their slice of the leaves straight
    into their slot of the buffers that the all-gather then completes."""
    B, T, H_kv, K = k.shape
    V = v.shape[-1]
    sizes = _lib.level_sizes(T, compression_rate, max_top_nodes)
    assert len(out_k) == len(out_v) == len(sizes) - 1
    layers_k, layers_v = [k] + list(out_k), [v] + list(out_v)
    for x, n in zip(layers_k, sizes):
        assert x.is_contiguous() and x.shape[1] == n, "level tensors must be contiguous and of the level's length"
    for x in layers_v:
        assert x.is_contiguous()
    if len(sizes) == 1:
        return
    shape = _lib.HtreeShape(B, T, H_kv, H_kv, K, V, int(compression_rate), 1, int(max_top_nodes), _DTYPES[k.dtype])
    with torch.cuda.device(k.device):
        _lib.check(_lib.lib().htree_b200_build_tree(ctypes.byref(shape), _ptrs(layers_k), _ptrs(layers_v), None, None, None, None,
                                                    None, _stream()), "build_tree")


def _split_half(dtype, K: int, V: int, compression_rate: int) -> bool:
    """fp32 storage on the tensor cores (operands carried as hi + lo half planes): 64-wide heads only."""
    return dtype == torch.float32 and K == 64 and V == 64 and int(compression_rate) in (8, 16)


def _rotatable(dtype, K: int, V: int, compression_rate: int) -> bool:
    return (dtype != torch.float32 and K % 16 == 0) or _split_half(dtype, K, V, compression_rate)


def _rotated_like(x: torch.Tensor) -> torch.Tensor:
    """K' buffer of one level: float16, for fp32 storage two planes (hi, lo)."""
    shape = ((2,) if x.dtype == torch.float32 else ()) + tuple(x.shape)
    return torch.empty(shape, dtype=torch.float16, device=x.device)


def _blockable(V: int, compression_rate: int) -> bool:
    return V in (64, 128) and int(compression_rate) in (8, 16)


def _blocked_like(x: torch.Tensor, compression_rate: int) -> torch.Tensor:
    B, N, H_kv, V = x.shape
    cr = int(compression_rate)
    if x.dtype == torch.float32:      # split-half planes (hi, lo) of float16
        return torch.empty(2, B, (N + cr - 1) // cr * cr, H_kv, V, dtype=torch.float16, device=x.device)
    return torch.empty(B, (N + cr - 1) // cr * cr, H_kv, V, dtype=x.dtype, device=x.device)


def block_values(layers_v, compression_rate: int, max_top_nodes: int, layers_k_rot=None):
    """Blocked copies of existing value levels (see build_tree) and, given the K' levels, of the keys where the pipelined
    forward applies; None for shapes the tensor-core forward does not cover."""
    v = layers_v[0]
    B, T, H_kv, V = v.shape
    if not _blockable(V, compression_rate) or (v.dtype == torch.float32 and V != 64):
        return None
    out = [_blocked_like(x, compression_rate) for x in layers_v]
    shape = _lib.HtreeShape(B, T, H_kv, H_kv, V, V, int(compression_rate), 1, int(max_top_nodes), _DTYPES[v.dtype])
    keys = None
    with torch.cuda.device(v.device):
        _lib.check(_lib.lib().htree_b200_block_values(ctypes.byref(shape), _ptrs(layers_v), _ptrs(out), _stream()), "block_values")
        if layers_k_rot is not None and _pipelined(v.dtype, layers_k_rot[0].shape[-1], compression_rate):
            keys = [_blocked_like(x, compression_rate) for x in layers_k_rot]
            _lib.check(_lib.lib().htree_b200_block_keys(ctypes.byref(shape), _ptrs(layers_k_rot), _ptrs(keys), _stream()), "block_keys")
    return OperandBlocks(out, keys)


def rotate_keys(layers_k, compression_rate: int, max_top_nodes: int, rope_base: float):
    """K' levels (keys rotated by their child index) for existing tree levels; None where no tensor-core kernel reads them
    (K % 16 != 0, or fp32 storage with heads other than 64 wide)."""
    k = layers_k[0]
    B, T, H_kv, K = k.shape
    if not _rotatable(k.dtype, K, K, compression_rate):
        return None
    out = [_rotated_like(x) for x in layers_k]
    shape = _lib.HtreeShape(B, T, H_kv, H_kv, K, K, int(compression_rate), 1, int(max_top_nodes), _DTYPES[k.dtype])
    cos_c, sin_c = rope_cache(K, max(int(compression_rate), 16), rope_base, k.device)
    with torch.cuda.device(k.device):
        _lib.check(_lib.lib().htree_b200_rotate_keys(ctypes.byref(shape), _ptrs(layers_k), _ptrs(out),
                                                     cos_c.data_ptr(), sin_c.data_ptr(), _stream()), "rotate_keys")
    return out


def _run_forward(shape, q, layers_k, layers_v, cos_cache, sin_cache, scale, out, gmax, gsum, parents, trace, flags,
                 layers_kr=None, half_tables=None, layers_vb=None):
    with torch.cuda.device(q.device):
        rc = _lib.lib().htree_b200_forward(
            ctypes.byref(shape), q.data_ptr(), _ptrs(layers_k), _ptrs(layers_v),
            _ptrs(layers_kr) if layers_kr is not None else None,
            _ptrs(layers_vb.keys) if getattr(layers_vb, "keys", None) is not None else None,
            _ptrs(layers_vb) if layers_vb is not None else None,
            cos_cache.data_ptr(), sin_cache.data_ptr(),
            half_tables[0].data_ptr() if half_tables else None, half_tables[1].data_ptr() if half_tables else None,
            cos_cache.shape[0], float(scale),
            out.data_ptr() if out is not None else None, gmax.data_ptr() if gmax is not None else None,
            gsum.data_ptr() if gsum is not None else None, _ptrs(parents) if parents is not None else None,
            ctypes.byref(trace) if trace is not None else None, _status(q.device).data_ptr(), flags, _stream())
    _lib.check(rc, "forward")


def htree_forward(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
    compression_rate: int = 16, max_top_nodes: int = 8192, top_k_per_layer: int = 512,
    scale: Optional[float] = None, rope_base: float = 10000.0,
    _save_for_backward: bool = False, _save_parents: bool = True,
    return_trace: bool = False, _force_generic: bool = False, _q_offset: Optional[int] = None, _layers=None,
    _fused: bool = False, _tiled: bool = False, _no_pipeline: bool = False,
):
    """htree forward.  q [B,T,H,K], k [B,T,H_kv,K], v [B,T,H_kv,V] -> out [B,T,H,V] in q's dtype.

    Returns `out`, or `(out, bwd_ctx)` with `_save_for_backward` (the reference's contract, src/parallel.py:1139-1159),
    with a third element — {"num_layers", "num_groups", "layers": {l: LayerTrace}} — when `return_trace` is set
    (the shape of htree_forward_naive's trace, src/naive.py:225-234).

    Sequence sharding: with `_q_offset` = t0, q holds only the query positions t0 .. t0+q.shape[1]-1 while k, v (or the
    prebuilt tree `_layers` = (layers_k, layers_v)) cover the whole sequence; outputs have q's length."""
    shape = _validate(q, k, v, compression_rate, max_top_nodes, top_k_per_layer, _q_offset)
    B, T, H, K = q.shape
    H_kv, V = k.shape[2], v.shape[-1]
    if scale is None:
        scale = K ** -0.5
    q = q.contiguous(); k = k.contiguous(); v = v.contiguous()
    dev = q.device
    if _layers is not None:
        layers_k, layers_v = _layers[0], _layers[1]
        layers_kr = _layers[2] if len(_layers) > 2 else None
        layers_vb = _layers[3] if len(_layers) > 3 else None
        if layers_kr is not None and layers_vb is None:
            layers_vb = block_values(layers_v, compression_rate, max_top_nodes, layers_kr)
    else:
        layers_k, layers_v, layers_kr, layers_vb = build_tree(k, v, compression_rate, max_top_nodes, rope_base)
    if layers_vb is None:
        layers_kr = None          # the tensor-core forward needs both operand copies
    L = len(layers_k)
    cos_cache, sin_cache = rope_cache(K, top_k_per_layer * compression_rate + 1024, rope_base, dev)
    out = torch.empty(B, T, H, V, dtype=q.dtype, device=dev)
    gmax = torch.empty(B, T, H, dtype=torch.float32, device=dev)
    gsum = torch.empty(B, T, H, dtype=torch.float32, device=dev)
    want_parents = (_save_for_backward and _save_parents) or return_trace
    # The tensor-core forward is faster as selection kernel + accumulation kernel, which hand the selections over in
    # buffers of L * B * T * H_kv * top_k ids (cfg3: 805 MB as int32; 2.1 GB per level at the reference's default top_k of
    # 512 with the same shape).  A caller who does not keep the selections gets them only as temporaries, in int32
    # whatever SELECTION_STORAGE says, and only up to SPLIT_FORWARD_MAX_BYTES: beyond it the single fused kernel runs,
    # which needs no buffers and gives identical results.
    split_forward = layers_kr is not None and not (_force_generic or return_trace or _fused)
    if want_parents:
        pdt = _parents_dtype(layers_k, top_k_per_layer)
    else:
        pdt = torch.int32
        if split_forward and L * B * q.shape[1] * H_kv * top_k_per_layer * 4 > SPLIT_FORWARD_MAX_BYTES:
            split_forward = False
    parents = [torch.empty(B, q.shape[1], H_kv, top_k_per_layer, dtype=pdt, device=dev) for _ in range(L)] \
        if (want_parents or split_forward) else None
    trace = tr = None
    if return_trace:
        tr = (torch.empty(L, B, T, H, dtype=torch.float32, device=dev),
              torch.empty(L, B, T, H, dtype=torch.float32, device=dev),
              torch.empty(L, B, T, H, V, dtype=torch.float32, device=dev))
        trace = _lib.HtreeTrace(tr[0].data_ptr(), tr[1].data_ptr(), tr[2].data_ptr())
    flags = _lib.FWD_GENERIC if (_force_generic or return_trace) else (_lib.FWD_FUSED if _fused else 0)
    if _tiled:
        flags |= _lib.FWD_TILED
    if _no_pipeline:
        flags |= _lib.FWD_NO_PIPELINE
    flags |= _parents_flag(parents)
    half_tables = rope_cache_half(K, cos_cache.shape[0], rope_base, scale, dev) if layers_kr is not None else None
    _run_forward(shape, q, layers_k, layers_v, cos_cache, sin_cache, scale, out, gmax, gsum, parents, trace, flags,
                 layers_kr, half_tables, layers_vb)
    if not (_save_for_backward or return_trace):
        return out
    result = [out]
    if _save_for_backward:
        G = H // H_kv
        result.append(dict(
            global_max=gmax, global_sum=gsum,
            per_layer_parents={l: parents[l] for l in range(L)} if (_save_parents and want_parents) else None,
            layers_k=layers_k, layers_v=layers_v, layers_k_rot=layers_kr, layers_v_blk=layers_vb,
            cos_cache=cos_cache, sin_cache=sin_cache,
            rope_half=half_tables,
            num_layers=L, rope_base=rope_base,
            compression_rate=compression_rate, top_k_per_layer=top_k_per_layer, max_top_nodes=max_top_nodes,
            scale=scale, NUM_GROUPS=G,
            # tuning constants of the reference's Triton kernels; kept so that code reading them keeps working
            G_PAD=max(16, 1 << (G - 1).bit_length()), TILE_P=4, DROP_BLOCK=64,
        ))
    if return_trace:
        check_status(dev)
        layers = {l: LayerTrace(l, decode_parents(parents[l - 1]) if l > 0 else None, tr[0][l], tr[1][l], tr[2][l])
                  for l in range(L)}
        result.append({"num_layers": L, "num_groups": H // H_kv, "selection_mode": "parallel_importance",
                       "layers": layers})
    return tuple(result)


def recompute_parents(q, layers_k, layers_v, cos_cache, sin_cache, compression_rate, top_k_per_layer,
                      max_top_nodes, scale, layers_k_rot=None, _force_generic=False, layers_v_blk=None) -> Dict[int, torch.Tensor]:
    """Selection-only replay of the forward (the reference's _recompute_parents, src/backward.py:881-934)."""
    B, T, H, K = q.shape
    H_kv, V = layers_k[0].shape[2], layers_v[0].shape[-1]
    shape = _lib.HtreeShape(B, T, H, H_kv, K, V, int(compression_rate), int(top_k_per_layer), int(max_top_nodes),
                            _DTYPES[q.dtype])
    L = len(layers_k)
    parents = [torch.empty(B, T, H_kv, top_k_per_layer, dtype=_parents_dtype(layers_k, top_k_per_layer), device=q.device)
               for _ in range(L)]
    _run_forward(shape, q.contiguous(), layers_k, layers_v, cos_cache, sin_cache, scale, None, None, None, parents,
                 None, _lib.FWD_SELECT_ONLY | (_lib.FWD_GENERIC if _force_generic else 0) | _parents_flag(parents),
                 layers_k_rot, None, layers_v_blk)
    return {l: parents[l] for l in range(L)}


def htree_backward(dO: torch.Tensor, q: torch.Tensor, output: torch.Tensor, bwd_ctx: dict, _force_generic: bool = False,
                   _typed: bool = False, _window: Optional[dict] = None):
    """Backward given the forward context; returns fp32 (dq, dk, dv) with the shapes of q, k, v
    (src/backward.py:941-1119).  If bwd_ctx['per_layer_parents'] is None the selections are rebuilt first.

    `_typed=True` returns the three gradients in q's dtype instead, rounded once inside the kernels: what the
    reference's autograd function produces by casting the fp32 results afterwards (src/backward.py:1193), without the
    fp32 dq tensor and the extra passes over memory.
    dO must have q's dtype (the kernels read it in the storage type; the reference up-casts both to fp32,
    src/backward.py:966): a wider dO is refused rather than rounded silently.

    `_window` runs the backward over consecutive query windows that share the dK/dV accumulators (what the host-buffer
    pipeline does to overlap transfers with kernels): {"t0": first position of this window, "first": bool, "last": bool,
    "acc": dict kept by the caller across the windows of one backward}.  q, dO, output and bwd_ctx then belong to the
    window (a forward called with `_q_offset`); dq is returned for the window, dk and dv only with the last window
    (None before)."""
    B, T, H, K = q.shape
    layers_k, layers_v = bwd_ctx["layers_k"], bwd_ctx["layers_v"]
    H_kv, V = layers_k[0].shape[2], layers_v[0].shape[-1]
    L = bwd_ctx["num_layers"]
    CR, TK, MTN = bwd_ctx["compression_rate"], bwd_ctx["top_k_per_layer"], bwd_ctx["max_top_nodes"]
    scale = bwd_ctx["scale"]
    cos_cache, sin_cache = bwd_ctx["cos_cache"], bwd_ctx["sin_cache"]
    layers_kr = bwd_ctx.get("layers_k_rot")
    half_tables = bwd_ctx.get("rope_half")
    dev = q.device
    q = q.contiguous()
    if dO.dtype != q.dtype:
        raise ValueError(f"dO has dtype {dO.dtype} but q has {q.dtype}: pass the output gradient in the operator's storage "
                         "type (cast it explicitly if the loss of precision is acceptable)")
    dO = dO.contiguous()
    output = output.contiguous()
    parents = bwd_ctx.get("per_layer_parents")
    if parents is None:
        parents = recompute_parents(q, layers_k, layers_v, cos_cache, sin_cache, CR, TK, MTN, scale,
                                    bwd_ctx.get("layers_k_rot"), layers_v_blk=bwd_ctx.get("layers_v_blk"))
    flags = 0
    if _window is None:
        shape = _lib.HtreeShape(B, T, H, H_kv, K, V, int(CR), int(TK), int(MTN), _DTYPES[q.dtype])
        dk_levels = [torch.empty(x.shape, dtype=torch.float32, device=dev) for x in layers_k]
        dv_levels = [torch.empty(x.shape, dtype=torch.float32, device=dev) for x in layers_v]
    else:
        T_full = layers_k[0].shape[1]
        shape = _lib.HtreeShape(B, T_full, H, H_kv, K, V, int(CR), int(TK), int(MTN), _DTYPES[q.dtype], T, int(_window["t0"]))
        acc = _window["acc"]
        if _window["first"]:
            acc["dk"] = [torch.empty(x.shape, dtype=torch.float32, device=dev) for x in layers_k]
            acc["dv"] = [torch.empty(x.shape, dtype=torch.float32, device=dev) for x in layers_v]
        dk_levels, dv_levels = acc["dk"], acc["dv"]
        flags |= (0 if _window["first"] else _lib.BWD_KEEP_ACCUM) | (0 if _window["last"] else _lib.BWD_NO_FOLD)
    final = _window is None or _window["last"]
    typed = None
    if _typed:
        dq = torch.empty(B, T, H, K, dtype=q.dtype, device=dev)
        # before the last window the leaf gradients are not written; the struct still wants valid pointers
        dk_t = torch.empty(layers_k[0].shape if final else (8,), dtype=q.dtype, device=dev)
        dv_t = torch.empty(layers_v[0].shape if final else (8,), dtype=q.dtype, device=dev)
        typed = _lib.HtreeTypedGrads(dq.data_ptr(), dk_t.data_ptr(), dv_t.data_ptr())
    else:
        dq = torch.empty(B, T, H, K, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().htree_b200_backward(
            ctypes.byref(shape), q.data_ptr(), _ptrs(layers_k), _ptrs(layers_v),
            _ptrs(layers_kr) if layers_kr is not None else None, cos_cache.data_ptr(), sin_cache.data_ptr(),
            half_tables[0].data_ptr() if half_tables else None, half_tables[1].data_ptr() if half_tables else None,
            cos_cache.shape[0], float(scale), output.data_ptr(), dO.data_ptr(),
            bwd_ctx["global_max"].data_ptr(), bwd_ctx["global_sum"].data_ptr(),
            _ptrs([parents[l] for l in range(L)]), None if _typed else dq.data_ptr(), _ptrs(dk_levels), _ptrs(dv_levels),
            ctypes.byref(typed) if typed is not None else None, _status(dev).data_ptr(),
            flags | (_lib.FWD_GENERIC if _force_generic else 0) | _parents_flag([parents[l] for l in range(L)]), _stream())
    _lib.check(rc, "backward")
    if not final:
        return dq, None, None
    if _typed:
        return dq, dk_t, dv_t
    return dq, dk_levels[0], dv_levels[0]


class HTreeFunction(torch.autograd.Function):
    """Differentiable htree attention (the reference's HTreeTritonFunction, src/backward.py:1126-1193)."""

    @staticmethod
    def forward(ctx, q, k, v, compression_rate, max_top_nodes, top_k_per_layer, scale, rope_base):
        save = SAVE_SELECTIONS_FOR_BACKWARD
        output, bwd_ctx = htree_forward(q, k, v, compression_rate=compression_rate, max_top_nodes=max_top_nodes,
                                        top_k_per_layer=top_k_per_layer, scale=scale, rope_base=rope_base,
                                        _save_for_backward=True, _save_parents=save)
        ctx.save_for_backward(q, k, v, output, bwd_ctx["global_max"], bwd_ctx["global_sum"])
        ctx.bwd_ctx = bwd_ctx
        if not save:   # like the reference: drop the pooled levels and rebuild them in backward
            bwd_ctx["layers_k"] = bwd_ctx["layers_v"] = bwd_ctx["layers_k_rot"] = bwd_ctx["layers_v_blk"] = None
        return output

    @staticmethod
    def backward(ctx, dO):
        q, k, v, output, gmax, gsum = ctx.saved_tensors
        c = dict(ctx.bwd_ctx)
        if c["layers_k"] is None:
            c["layers_k"], c["layers_v"], c["layers_k_rot"], c["layers_v_blk"] = build_tree(
                k, v, c["compression_rate"], c["max_top_nodes"], c["rope_base"])
        dq, dk, dv = htree_backward(dO.to(q.dtype), q, output, c, _typed=True)    # gradients come back in the input dtype
        return dq, dk, dv, None, None, None, None, None


HTreeTritonFunction = HTreeFunction   # drop-in name of the reference


def htree_forward_autograd(q, k, v, compression_rate: int = 16, max_top_nodes: int = 8192,
                           top_k_per_layer: int = 512, scale: Optional[float] = None, rope_base: float = 10000.0):
    """Differentiable forward (signature of htree_forward_triton_autograd, src/backward.py:1196-1208)."""
    if scale is None:
        scale = q.shape[-1] ** -0.5
    return HTreeFunction.apply(q.contiguous(), k.contiguous(), v.contiguous(), compression_rate, max_top_nodes,
                               top_k_per_layer, scale, rope_base)


htree_forward_triton_autograd = htree_forward_autograd   # drop-in name of the reference

__all__ = [
    "decode_parents", "HTREE_SCORE_NEG_INF", "HTREE_SCORE_VALID_THRESHOLD", "LayerTrace", "build_tree", "rope_cache",
    "rotate_keys", "block_values",
    "htree_forward", "htree_backward", "recompute_parents", "HTreeFunction", "HTreeTritonFunction",
    "htree_forward_autograd", "htree_forward_triton_autograd", "check_status",
]
