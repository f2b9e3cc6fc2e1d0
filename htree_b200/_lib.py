"""ctypes binding of libhtree_b200.so (the C ABI declared in include/htree_b200.h).

There is no CPU or PyTorch fallback: if the library has not been built, loading raises with the build command.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("HTREE_B200_LIB") or os.path.join(_HERE, "libhtree_b200.so")   # override: another build of the same ABI

MAX_LEVELS = 12
F32, BF16, F16 = 0, 1, 2
FWD_SELECT_ONLY = 1
FWD_GENERIC = 2
FWD_FUSED = 4
FWD_TILED = 8
PARENTS_U16 = 16
FWD_NO_PIPELINE = 128
BWD_KEEP_ACCUM = 32
BWD_NO_FOLD = 64

# every exported symbol of include/htree_b200.h; tests check that the library exports all of them
SYMBOLS = (
    "htree_b200_version",
    "htree_b200_error_string",
    "htree_b200_launch_count",
    "htree_b200_num_levels",
    "htree_b200_level_sizes",
    "htree_b200_build_tree",
    "htree_b200_rotate_keys",
    "htree_b200_block_values",
    "htree_b200_block_keys",
    "htree_b200_forward",
    "htree_b200_level_forward",
    "htree_b200_merge_to_global",
    "htree_b200_final_normalize",
    "htree_b200_topk",
    "htree_b200_copy_rows",
    "htree_b200_backward",
    "htree_b200_static_scratch_bytes",
    "htree_b200_backward_static_scratch",
)


class HtreeShape(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in
                ("B", "T", "H", "H_kv", "K", "V", "compression_rate", "top_k", "max_top_nodes", "dtype", "T_q",
                 "t_offset")]


class HtreeTypedGrads(ctypes.Structure):
    _fields_ = [("dq", ctypes.c_void_p), ("dk", ctypes.c_void_p), ("dv", ctypes.c_void_p)]


class HtreeTrace(ctypes.Structure):
    _fields_ = [("layer_max", ctypes.c_void_p), ("layer_sum", ctypes.c_void_p), ("layer_out", ctypes.c_void_p)]


class HtreeError(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"htree_b200 {what} failed with code {code}: {error_string(code)}")
        self.code = code


_lib = None


def lib() -> ctypes.CDLL:
    """Load the shared library once.  Raises if it is missing: the CUDA extension is the only implementation."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m htree_b200.build` (nvcc, sm_100a). "
                "htree_b200 has no fallback implementation.")
        L = ctypes.CDLL(LIB_PATH)
        vp, i32, u32, f32 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_uint32, ctypes.c_float
        L.htree_b200_version.restype = ctypes.c_int
        L.htree_b200_error_string.restype = ctypes.c_char_p
        L.htree_b200_error_string.argtypes = [ctypes.c_int]
        L.htree_b200_launch_count.restype = ctypes.c_uint64
        L.htree_b200_num_levels.restype = ctypes.c_int
        L.htree_b200_num_levels.argtypes = [i32, i32, i32]
        L.htree_b200_level_sizes.restype = ctypes.c_int
        L.htree_b200_level_sizes.argtypes = [i32, i32, i32, ctypes.POINTER(i32), i32]
        L.htree_b200_build_tree.restype = ctypes.c_int
        L.htree_b200_build_tree.argtypes = [ctypes.POINTER(HtreeShape), vp, vp, vp, vp, vp, vp, vp, vp]
        L.htree_b200_rotate_keys.restype = ctypes.c_int
        L.htree_b200_rotate_keys.argtypes = [ctypes.POINTER(HtreeShape), vp, vp, vp, vp, vp]
        L.htree_b200_block_values.restype = ctypes.c_int
        L.htree_b200_block_values.argtypes = [ctypes.POINTER(HtreeShape), vp, vp, vp]
        L.htree_b200_block_keys.restype = ctypes.c_int
        L.htree_b200_block_keys.argtypes = [ctypes.POINTER(HtreeShape), vp, vp, vp]
        L.htree_b200_forward.restype = ctypes.c_int
        L.htree_b200_forward.argtypes = [ctypes.POINTER(HtreeShape), vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, f32, vp, vp, vp, vp,
                                         ctypes.POINTER(HtreeTrace), vp, u32, vp]
        L.htree_b200_level_forward.restype = ctypes.c_int
        L.htree_b200_level_forward.argtypes = [ctypes.POINTER(HtreeShape), i32, i32, vp, vp, vp, vp, vp, vp, i32, f32, vp, vp, vp, vp,
                                               vp, vp]
        L.htree_b200_merge_to_global.restype = ctypes.c_int
        L.htree_b200_merge_to_global.argtypes = [vp, vp, vp, vp, vp, vp, ctypes.c_int64, i32, vp]
        L.htree_b200_final_normalize.restype = ctypes.c_int
        L.htree_b200_final_normalize.argtypes = [vp, vp, vp, i32, ctypes.c_int64, i32, vp]
        L.htree_b200_copy_rows.restype = ctypes.c_int
        L.htree_b200_copy_rows.argtypes = [vp, ctypes.c_int64, vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, vp]
        L.htree_b200_topk.restype = ctypes.c_int
        L.htree_b200_topk.argtypes = [vp, vp, vp, i32, i32, i32, i32, vp, vp, vp, vp, vp]
        L.htree_b200_backward.restype = ctypes.c_int
        L.htree_b200_backward.argtypes = [ctypes.POINTER(HtreeShape), vp, vp, vp, vp, vp, vp, vp, vp, i32, f32, vp, vp, vp, vp, vp,
                                          vp, vp, vp, ctypes.POINTER(HtreeTypedGrads), vp, u32, vp]
        L.htree_b200_static_scratch_bytes.restype = ctypes.c_size_t
        L.htree_b200_backward_static_scratch.restype = ctypes.c_int
        L.htree_b200_backward_static_scratch.argtypes = [ctypes.POINTER(HtreeShape), vp, vp, vp, vp, vp, vp, vp, vp, i32, f32, vp,
                                                         vp, vp, vp, vp, vp, vp, vp, vp, u32, vp]
        _lib = L
    return _lib


def launch_count() -> int:
    return int(lib().htree_b200_launch_count())


def error_string(code: int) -> str:
    return lib().htree_b200_error_string(int(code)).decode()


def check(code: int, what: str) -> None:
    if code != 0:
        raise HtreeError(code, what)


def level_sizes(T: int, compression_rate: int, max_top_nodes: int):
    buf = (ctypes.c_int32 * MAX_LEVELS)()
    n = lib().htree_b200_level_sizes(int(T), int(compression_rate), int(max_top_nodes), buf, MAX_LEVELS)
    if n < 0:
        raise HtreeError(n, "level_sizes")
    return [int(buf[i]) for i in range(n)]


def ptr_array(ptrs):
    """A C array of void* from a list of integer addresses (None -> NULL)."""
    return (ctypes.c_void_p * len(ptrs))(*[ctypes.c_void_p(p) if p else None for p in ptrs])
