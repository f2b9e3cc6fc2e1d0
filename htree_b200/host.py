"""Host-buffer entry points: inputs and results live in (pinned) host memory, the device only holds a window of them.

The reference has no counterpart (its scripts create tensors on the device, speed_test.py:66-69).  These functions are
what a caller with host-resident activations uses: the batch dimension is cut into chunks, and three CUDA streams
overlap the host->device copy of chunk i+1, the kernels of chunk i and the device->host copy of chunk i-1.  Chunks are
independent because every batch element is (htree_forward/htree_backward never mix batch elements)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib, ops


_stream_cache = {}


def _streams(dev):
    """Three streams per device, created once: the caching allocator keeps one pool per stream, so fresh streams on
    every call would mean fresh cudaMalloc calls (which synchronise the device) on every call."""
    key = (dev.type, dev.index)
    if key not in _stream_cache:
        _stream_cache[key] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev))
    return _stream_cache[key]


def _copy_unit(dst: torch.Tensor, src: torch.Tensor, stream) -> None:
    """dst <- src for two views of shape [1, T, heads, D] whose rows (one position: heads * D elements) are contiguous;
    either side may be a slice of a larger [B, T, H, D] tensor (rows a fixed pitch apart) in pinned host memory."""
    assert dst.shape == src.shape and dst.dtype == src.dtype
    T, es = dst.shape[1], dst.element_size()
    width = dst.shape[2] * dst.shape[3] * es
    for x in (dst, src):
        assert x.stride(3) == 1 and x.stride(2) == x.shape[3], "rows must be contiguous"
    _lib.check(_lib.lib().htree_b200_copy_rows(dst.data_ptr(), dst.stride(1) * es, src.data_ptr(), src.stride(1) * es, width, T,
                                               stream.cuda_stream), "copy_rows")


def forward_backward_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, dO: Optional[torch.Tensor],
                          compression_rate: int = 16, max_top_nodes: int = 8192, top_k_per_layer: int = 512,
                          scale: Optional[float] = None, rope_base: float = 10000.0, chunk: int = 1,
                          device=None, outputs: Optional[Tuple[torch.Tensor, ...]] = None):
    """htree forward (and backward when dO is given) for HOST tensors q [B,T,H,K], k, v [B,T,H_kv,*], dO [B,T,H,V].

    Returns host tensors (out,) or (out, dq, dk, dv) in the input dtype; pass `outputs` (pinned, same shapes) to reuse
    buffers.  `chunk` batch elements are resident on the device at a time (two chunks in flight).  The call returns
    after everything has arrived in host memory.  chunk="unit" moves and computes one (batch, KV head) unit at a time
    (strided copies of that head group's slices): the units are independent too, and the smaller the piece the less of
    the first upload and the last download is left outside the overlap."""
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    B = q.shape[0]
    bwd = dO is not None
    if outputs is None:
        pin = q.is_pinned()
        outs = [torch.empty((B,) + tuple(q.shape[1:3]) + (v.shape[-1],), dtype=q.dtype, pin_memory=pin)]
        if bwd:
            outs += [torch.empty(q.shape, dtype=q.dtype, pin_memory=pin), torch.empty(k.shape, dtype=k.dtype, pin_memory=pin),
                     torch.empty(v.shape, dtype=v.dtype, pin_memory=pin)]
    else:
        outs = list(outputs)
    s_in, s_run, s_out = _streams(dev)
    s_in.wait_stream(torch.cuda.current_stream(dev))
    if chunk == "unit":
        return _by_units(q, k, v, dO, outs, dev, (s_in, s_run, s_out), compression_rate, max_top_nodes, top_k_per_layer, scale,
                         rope_base)
    keep = []                      # device tensors stay referenced until the final synchronisation
    for b0 in range(0, B, chunk):
        b1 = min(B, b0 + chunk)
        with torch.cuda.stream(s_in):
            dev_in = [x[b0:b1].to(dev, non_blocking=True) for x in ((q, k, v, dO) if bwd else (q, k, v))]
            ready = torch.cuda.Event(); ready.record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(ready)
            if bwd:
                o, ctx = ops.htree_forward(dev_in[0], dev_in[1], dev_in[2], compression_rate, max_top_nodes,
                                           top_k_per_layer, scale, rope_base, _save_for_backward=True)
                dq, dk, dv = ops.htree_backward(dev_in[3], dev_in[0], o, ctx, _typed=True)
                res = [o, dq, dk, dv]
                del ctx
            else:
                res = [ops.htree_forward(dev_in[0], dev_in[1], dev_in[2], compression_rate, max_top_nodes,
                                         top_k_per_layer, scale, rope_base)]
            done = torch.cuda.Event(); done.record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            for h, r in zip(outs, res):
                h[b0:b1].copy_(r, non_blocking=True)
        for t in dev_in + res:     # the caching allocator must not hand these blocks to another stream early
            t.record_stream(s_run); t.record_stream(s_out)
        keep.append((dev_in, res))
        if len(keep) > 2:
            keep.pop(0)
    s_out.synchronize(); s_run.synchronize(); s_in.synchronize()
    return tuple(outs)


def _by_units(q, k, v, dO, outs, dev, streams, compression_rate, max_top_nodes, top_k_per_layer, scale, rope_base):
    """One (batch, KV head) unit at a time: q/dO/out/dq slices [1,T,G,D] and k/v/dk/dv slices [1,T,1,D]."""
    s_in, s_run, s_out = streams
    B, T, H, K = q.shape
    H_kv, V = k.shape[2], v.shape[-1]
    G = H // H_kv
    bwd = dO is not None
    if scale is None:
        scale = K ** -0.5
    keep = []
    with torch.cuda.device(dev):
        for b in range(B):
            for hk in range(H_kv):
                hs = slice(hk * G, (hk + 1) * G)
                srcs = [q[b:b + 1, :, hs], k[b:b + 1, :, hk:hk + 1], v[b:b + 1, :, hk:hk + 1]] + ([dO[b:b + 1, :, hs]] if bwd else [])
                dsts = [outs[0][b:b + 1, :, hs]] + ([outs[1][b:b + 1, :, hs], outs[2][b:b + 1, :, hk:hk + 1],
                                                     outs[3][b:b + 1, :, hk:hk + 1]] if bwd else [])
                # the forward starts as soon as q, k, v are there (dO follows), and its output leaves while the backward runs
                with torch.cuda.stream(s_in):
                    dev_in = [torch.empty(x.shape, dtype=x.dtype, device=dev) for x in srcs]
                    for d, x in zip(dev_in[:3], srcs[:3]):
                        _copy_unit(d, x, s_in)
                    ready = torch.cuda.Event(); ready.record(s_in)
                    if bwd:
                        _copy_unit(dev_in[3], srcs[3], s_in)
                        ready_bwd = torch.cuda.Event(); ready_bwd.record(s_in)
                with torch.cuda.stream(s_run):
                    s_run.wait_event(ready)
                    if bwd:
                        o, ctx = ops.htree_forward(dev_in[0], dev_in[1], dev_in[2], compression_rate, max_top_nodes,
                                                   top_k_per_layer, scale, rope_base, _save_for_backward=True)
                        fwd_done = torch.cuda.Event(); fwd_done.record(s_run)
                        s_run.wait_event(ready_bwd)
                        dq, dk, dv = ops.htree_backward(dev_in[3], dev_in[0], o, ctx, _typed=True)
                        res = [o, dq, dk, dv]
                        del ctx
                    else:
                        res = [ops.htree_forward(dev_in[0], dev_in[1], dev_in[2], compression_rate, max_top_nodes,
                                                 top_k_per_layer, scale, rope_base)]
                        fwd_done = torch.cuda.Event(); fwd_done.record(s_run)
                    done = torch.cuda.Event(); done.record(s_run)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(fwd_done)
                    _copy_unit(dsts[0], res[0], s_out)
                    if bwd:
                        s_out.wait_event(done)
                        for h, r in zip(dsts[1:], res[1:]):
                            _copy_unit(h, r, s_out)
                for t in dev_in + res:
                    t.record_stream(s_run); t.record_stream(s_out)
                keep.append((dev_in, res))
                if len(keep) > 2:
                    keep.pop(0)
    s_out.synchronize(); s_run.synchronize(); s_in.synchronize()
    return tuple(outs)
