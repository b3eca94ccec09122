"""ctypes binding of libmoba_b200.so (the C ABI declared in include/moba_b200.h).

The library is the product; there is no Python or CPU fallback.  Importing this
module never compiles anything: a missing library is an error that names the
build command.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

#: MOBA_B200_LIB selects another build of the same library (A/B runs of kernel variants)
LIB_PATH = Path(os.environ.get("MOBA_B200_LIB") or Path(__file__).resolve().parent / "libmoba_b200.so")

ATTEND_TCGEN05 = 0
ATTEND_MMA_SYNC = 1

#: every symbol include/moba_b200.h declares
SYMBOLS = (
    "moba_b200_abi_version", "moba_b200_strerror", "moba_problem_check", "moba_problem_dims",
    "moba_workspace_size", "moba_workspace_size_min", "moba_forward", "moba_forward_events", "moba_forward_cached", "moba_workspace_size_host", "moba_forward_host",
    "moba_chunk_metadata", "moba_chunk_means", "moba_gate_topk", "moba_gate_topk_stats", "moba_compact_routes",
    "moba_attend", "moba_merge", "moba_attend_tile_rows", "moba_attend_tile_rows_for", "moba_problem_tile_rows", "moba_route_static",
    "moba_backward_workspace_size", "moba_backward",
    "moba_cp_workspace_size", "moba_cp_forward", "moba_cp_poll", "moba_cp_abort", "moba_selftest_bounded_wait",
)


class Problem(C.Structure):
    """struct moba_problem"""
    _fields_ = [
        ("total_tokens", C.c_int64), ("batch", C.c_int32), ("num_q_heads", C.c_int32),
        ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("max_seqlen", C.c_int32),
        ("chunk_size", C.c_int32), ("topk", C.c_int32), ("attend_impl", C.c_int32),
        ("q_stride_token", C.c_int64), ("q_stride_head", C.c_int64),
        ("k_stride_token", C.c_int64), ("k_stride_head", C.c_int64),
        ("v_stride_token", C.c_int64), ("v_stride_head", C.c_int64),
        ("o_stride_token", C.c_int64), ("o_stride_head", C.c_int64),
        ("q_token_begin", C.c_int64), ("q_tokens", C.c_int64),
        ("dtype", C.c_int32), ("reserved", C.c_int32),
    ]


class Dims(C.Structure):
    """struct moba_dims"""
    _fields_ = [
        ("chunks_per_seq", C.c_int32), ("slots", C.c_int32), ("hist", C.c_int32),
        ("partials", C.c_int32), ("rows", C.c_int64), ("lists", C.c_int64),
    ]


class MobaError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"moba_b200 error {code}: {message}")
        self.code = code


_lib = None


def lib() -> C.CDLL:
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m baselinebenchmark_b200.build` "
                "(nvcc, sm_100a).  There is no fallback implementation.")
        handle = C.CDLL(str(LIB_PATH))
        handle.moba_b200_strerror.restype = C.c_char_p
        handle.moba_b200_strerror.argtypes = [C.c_int]
        vp, i32p, sz = C.c_void_p, C.c_void_p, C.c_size_t
        pp = C.POINTER(Problem)
        handle.moba_problem_check.argtypes = [pp]
        handle.moba_problem_dims.argtypes = [pp, C.POINTER(Dims)]
        handle.moba_workspace_size.argtypes = [pp, C.POINTER(sz)]
        handle.moba_workspace_size_host.argtypes = [pp, C.POINTER(sz)]
        handle.moba_workspace_size_min.argtypes = [pp, C.POINTER(sz)]
        handle.moba_forward.argtypes = [pp, vp, vp, vp, i32p, vp, vp, i32p, vp, sz, vp]
        handle.moba_forward_events.argtypes = [pp, vp, vp, vp, i32p, vp, vp, i32p, vp, sz, vp, C.POINTER(C.c_void_p)]
        handle.moba_forward_cached.argtypes = [pp, vp, vp, vp, i32p, vp, vp, i32p, vp, C.c_int32, vp, sz, vp]
        handle.moba_forward_host.argtypes = [pp, vp, vp, vp, i32p, vp, vp, i32p, vp, sz, vp]
        handle.moba_chunk_metadata.argtypes = [pp, i32p, i32p, i32p, vp, vp]
        handle.moba_chunk_means.argtypes = [pp, vp, i32p, vp, vp]
        handle.moba_gate_topk.argtypes = [pp, vp, vp, i32p, i32p, i32p, vp]
        handle.moba_gate_topk_stats.argtypes = [pp, vp, vp, i32p, i32p, i32p, i32p, C.c_int32, vp]
        handle.moba_compact_routes.argtypes = [pp, i32p, i32p, i32p, i32p, i32p, i32p, i32p, vp, C.c_int32, vp]
        handle.moba_attend.argtypes = [pp, vp, vp, vp, i32p, i32p, i32p, i32p, i32p, vp, vp, i32p, vp]
        handle.moba_merge.argtypes = [pp, vp, vp, i32p, vp, vp, vp]
        handle.moba_attend_tile_rows.argtypes = [C.c_int]
        handle.moba_attend_tile_rows_for.argtypes = [C.c_int, C.c_int]
        handle.moba_problem_tile_rows.argtypes = [pp]
        handle.moba_route_static.argtypes = [pp, vp, vp, i32p, i32p, vp]
        handle.moba_backward_workspace_size.argtypes = [pp, C.POINTER(sz)]
        handle.moba_backward.argtypes = [pp, vp, vp, vp, i32p, vp, vp, i32p, vp, vp, vp, vp, vp, sz, vp]
        handle.moba_cp_workspace_size.argtypes = [pp, C.POINTER(sz)]
        handle.moba_cp_forward.argtypes = [pp, vp, C.c_int32, C.c_int32, C.POINTER(C.c_int64), vp, vp, vp, i32p, vp, vp,
                                           i32p, vp, sz, vp, vp, C.POINTER(C.c_void_p)]
        handle.moba_cp_poll.argtypes = [vp, C.POINTER(C.c_int32)]
        handle.moba_cp_abort.argtypes = [vp]
        handle.moba_selftest_bounded_wait.argtypes = [i32p, C.c_uint32, vp]
        _lib = handle
    return _lib


def check(code: int) -> None:
    if code != 0:
        raise MobaError(code, lib().moba_b200_strerror(code).decode())
