"""Multi-GPU sharding of the htree operator: one process per GPU, torch.distributed for the plumbing.

The reference (skywong14/htree) is single-GPU; both modes below are new.  They rest on one property of the operator:
given the tree, every (batch, query position, KV head) group is independent (src/naive.py:180-213 loops over them).

Mode A — units.  A unit is one (batch, KV head) pair: it reads q[b, :, hk*G:(hk+1)*G], k[b, :, hk], v[b, :, hk] and
writes the same slices of out / dq / dk / dv.  Units are dealt round-robin to ranks; a rank runs its units as a batch
of independent single-KV-head problems.  Forward and backward need no communication at all.

Mode B — query positions of one long sequence.  Rank r owns the query range [r*T/n, (r+1)*T/n); k and v are
replicated inputs.  Each rank pools only its own slice of every tree level and one all_gather per pooled level puts
the complete coarse levels into local HBM before the attention kernel starts; the kernels only ever read local
memory.  Requires T/n to be a multiple of compression_rate^(levels-1) so that no pooled node straddles two ranks.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import configs


# ---------------------------------------------------------------- mode A: (batch, KV head) units

def unit_partition(n_units: int, world_size: int, rank: int) -> List[int]:
    """Units owned by `rank`: round-robin, so every rank gets floor or ceil of n_units/world_size of them."""
    if not (0 <= rank < world_size):
        raise ValueError(f"rank {rank} outside world of {world_size}")
    return list(range(rank, n_units, world_size))


def unit_of(b: int, hk: int, H_kv: int) -> int:
    return b * H_kv + hk


def gather_units(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, units: Sequence[int], extra: Sequence[torch.Tensor] = ()):
    """Slices of the full tensors for `units`, as a batch of single-KV-head problems.

    q [B,T,H,K] -> [U,T,G,K];  k, v [B,T,H_kv,*] -> [U,T,1,*];  every tensor in `extra` is sliced like q."""
    B, T, H, _ = q.shape
    H_kv = k.shape[2]
    G = H // H_kv

    def heads(x, u):
        b, hk = divmod(u, H_kv)
        return x[b, :, hk * G:(hk + 1) * G]

    ql = torch.stack([heads(q, u) for u in units]).contiguous()
    kl = torch.stack([k[u // H_kv, :, u % H_kv:u % H_kv + 1] for u in units]).contiguous()
    vl = torch.stack([v[u // H_kv, :, u % H_kv:u % H_kv + 1] for u in units]).contiguous()
    el = [torch.stack([heads(x, u) for u in units]).contiguous() for x in extra]
    return (ql, kl, vl, *el)


def scatter_units(local: torch.Tensor, full: torch.Tensor, units: Sequence[int], H_kv: int) -> None:
    """Inverse of gather_units for a q-shaped ([U,T,G,*] -> [B,T,H,*]) or k-shaped ([U,T,1,*] -> [B,T,H_kv,*]) tensor."""
    per = local.shape[2]
    for i, u in enumerate(units):
        b, hk = divmod(u, H_kv)
        full[b, :, hk * per:(hk + 1) * per] = local[i]


# ---------------------------------------------------------------- mode B: query positions

def query_range(T: int, world_size: int, rank: int, compression_rate: int, n_levels: int) -> Tuple[int, int]:
    """[t0, t1) owned by `rank`.  Raises if the split would cut a node of the coarsest pooled level."""
    if T % world_size:
        raise ValueError(f"T={T} is not divisible by world_size={world_size}")
    span = T // world_size
    grain = compression_rate ** (n_levels - 1)
    if span % grain:
        raise ValueError(f"T/world_size={span} must be a multiple of compression_rate^(levels-1)={grain}")
    return rank * span, (rank + 1) * span


def build_tree_sequence_parallel(k: torch.Tensor, v: torch.Tensor, compression_rate: int, max_top_nodes: int,
                                 group=None, _build=None):
    """Tree build for mode B: pool the local leaf range, all-gather every pooled level.

    k, v are the full (replicated) leaves [B,T,H_kv,*].  Returns full-length (layers_k, layers_v) in local memory.
    `_build(k, v, compression_rate, max_top_nodes)` replaces the CUDA tree build in host-only tests."""
    import torch.distributed as dist
    if _build is None:
        from .ops import build_tree as _build
    build_tree = _build

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    B, T, H_kv, K = k.shape
    sizes = configs.level_sizes(T, compression_rate, max_top_nodes)
    L = len(sizes)
    if world == 1 or L == 1:
        return build_tree(k, v, compression_rate, max_top_nodes)
    t0, t1 = query_range(T, world, rank, compression_rate, L)
    # pool the local slice to the same depth: its top level is this rank's share of the global top level
    lk, lv = build_tree(k[:, t0:t1].contiguous(), v[:, t0:t1].contiguous(), compression_rate, sizes[-1] // world)
    assert len(lk) == L
    layers_k, layers_v = [k], [v]
    for l in range(1, L):
        for src, dst in ((lk[l], layers_k), (lv[l], layers_v)):
            n_loc = src.shape[1]
            assert n_loc * world == sizes[l]
            gathered = torch.empty((world * B,) + tuple(src.shape[1:]), dtype=src.dtype, device=src.device)
            dist.all_gather_into_tensor(gathered, src.contiguous(), group=group)   # rank-major along dim 0
            # [world, B, n_loc, H_kv, D] -> [B, world*n_loc, H_kv, D]
            gathered = gathered.view(world, B, n_loc, H_kv, src.shape[-1])
            dst.append(gathered.permute(1, 0, 2, 3, 4).reshape(B, sizes[l], H_kv, src.shape[-1]).contiguous())
    return layers_k, layers_v


def htree_forward_sequence_parallel(q_local: torch.Tensor, k: torch.Tensor, v: torch.Tensor, compression_rate: int = 16,
                                    max_top_nodes: int = 8192, top_k_per_layer: int = 512, scale: Optional[float] = None,
                                    rope_base: float = 10000.0, group=None) -> torch.Tensor:
    """Mode B forward: q_local holds this rank's query positions [B, T/world, H, K]; k, v are the full sequence.
    Returns out_local [B, T/world, H, V]."""
    import torch.distributed as dist
    from .ops import htree_forward

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    T = k.shape[1]
    L = len(configs.level_sizes(T, compression_rate, max_top_nodes))
    t0, t1 = query_range(T, world, rank, compression_rate, L) if world > 1 else (0, T)
    assert q_local.shape[1] == t1 - t0
    from .ops import rotate_keys
    layers_k, layers_v = build_tree_sequence_parallel(k, v, compression_rate, max_top_nodes, group)
    layers_kr = rotate_keys(layers_k, compression_rate, max_top_nodes, rope_base)   # local work on the gathered levels
    return htree_forward(q_local, k, v, compression_rate, max_top_nodes, top_k_per_layer, scale, rope_base,
                         _q_offset=t0, _layers=(layers_k, layers_v, layers_kr))
