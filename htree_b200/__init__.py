"""htree_b200: hierarchical tree sparse attention (the algorithm of skywong14/htree) as hand-written sm_100a CUDA
kernels behind a C ABI (include/htree_b200.h), with the reference's Python entry points on top (htree_b200.ops)."""
from .ops import (  # noqa: F401
    HTREE_SCORE_NEG_INF, HTREE_SCORE_VALID_THRESHOLD, HTreeFunction, HTreeTritonFunction, LayerTrace, build_tree,
    check_status, decode_parents, htree_backward, htree_forward, htree_forward_autograd, htree_forward_triton_autograd,
    recompute_parents, rope_cache,
)

__version__ = "0.1.0"
