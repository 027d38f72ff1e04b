"""ctypes binding of libfaws.so (include/faws.h).  No fallback: if the library is
missing or does not load, importing the operators raises."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libfaws.so")

FP16, BF16 = 0, 1
SCORES_F32, SCORES_INPUT = 0, 1
BACKEND_AUTO, BACKEND_GENERIC, BACKEND_TCGEN05 = 0, 1, 2
ETOOLARGE = -6
NOALLOC_SCRATCH_BYTES = 8 << 20
BACKENDS = {None: BACKEND_AUTO, "auto": BACKEND_AUTO, "generic": BACKEND_GENERIC, "tcgen05": BACKEND_TCGEN05}

OP_ATTENTION, OP_SCORES, OP_ROW_SUM, OP_COL_SUM, OP_COL_SUM_SEQUENTIAL = 0, 1, 2, 3, 4
OP_SOFTMAX_COL_SUM, OP_CROSS_QK_SUM, OP_CROSS_SOFTMAX_SUM, OP_CROSS_SOFTMAX_SUM_BUFFERED = 5, 6, 7, 8
OP_TOTAL_ATTENTION = 9
OP_ATTENTION_BACKWARD = 10
OP_ATTENTION_SPLIT_KV = 11

# every symbol include/faws.h declares
EXPORTS = [
    "faws_attention", "faws_attention_with_scores", "faws_compute_attention_scores", "faws_split_kv_plan",
    "faws_attention_split_kv", "faws_attention_with_row_sum",
    "faws_attention_with_col_sum", "faws_attention_with_col_sum_noalloc",
    "faws_attention_with_col_sum_sequential",
    "faws_attention_with_softmax_col_sum", "faws_attention_cross_token_qk_sum",
    "faws_attention_cross_token_softmax_sum", "faws_attention_cross_token_softmax_sum_buffered",
    "faws_total_attention", "faws_attention_backward", "faws_workspace_bytes", "faws_reduce_ranks", "faws_device_status",
    "faws_selftest_wait_give_up", "faws_last_backend",
    "faws_launch_count", "faws_strerror", "faws_version",
]


class Tensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_h", C.c_int64), ("stride_s", C.c_int64)]


class Problem(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hk", C.c_int32), ("M", C.c_int32), ("N", C.c_int32), ("D", C.c_int32),
        ("dtype", C.c_int32), ("causal", C.c_int32), ("sm_scale", C.c_float),
        ("m_begin", C.c_int32), ("m_end", C.c_int32),
        ("q", Tensor), ("k", Tensor), ("v", Tensor), ("out", Tensor),
        ("log_normalizer", C.c_void_p),
        ("backend", C.c_int32), ("dropout_p", C.c_float), ("dropout_scale", C.c_float), ("reserved", C.c_int32),
        ("philox_seed", C.c_uint64), ("philox_offset", C.c_uint64),
    ]


class Grads(C.Structure):
    _fields_ = [("dout", Tensor), ("dq", Tensor), ("dk", Tensor), ("dv", Tensor)]


_lib = None


def load():
    """dlopen libfaws.so once and declare the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m flash_attn_with_score_b200.build` "
            "(needs nvcc with sm_100a support). There is no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    PP = C.POINTER(Problem)
    vp, i32, u32, sz = C.c_void_p, C.c_int32, C.c_uint32, C.c_size_t
    protos = {
        "faws_attention": (i32, [PP, vp]),
        "faws_attention_with_scores": (i32, [PP, vp, i32, u32, vp]),
        "faws_compute_attention_scores": (i32, [PP, vp, i32, vp]),
        "faws_split_kv_plan": (i32, [PP]),
        "faws_attention_split_kv": (i32, [PP, i32, vp, sz, vp]),
        "faws_attention_with_row_sum": (i32, [PP, vp, vp]),
        "faws_attention_with_col_sum": (i32, [PP, vp, i32, vp, sz, vp]),
        "faws_attention_with_col_sum_noalloc": (i32, [PP, vp, i32, vp]),
        "faws_attention_with_col_sum_sequential": (i32, [PP, vp, i32, vp, sz, vp]),
        "faws_attention_with_softmax_col_sum": (i32, [PP, vp, i32, vp, sz, vp]),
        "faws_attention_cross_token_qk_sum": (i32, [PP, i32, vp, i32, vp, sz, vp]),
        "faws_attention_cross_token_softmax_sum": (i32, [PP, i32, vp, i32, vp, sz, vp]),
        "faws_attention_cross_token_softmax_sum_buffered": (i32, [PP, i32, vp, i32, vp, sz, vp]),
        "faws_total_attention": (i32, [PP, vp, vp]),
        "faws_attention_backward": (i32, [PP, C.POINTER(Grads), vp, sz, vp]),
        "faws_workspace_bytes": (sz, [i32, PP, i32]),
        "faws_reduce_ranks": (i32, [vp, i32, C.c_int64, vp, vp]),
        "faws_device_status": (i32, [i32]),
        "faws_selftest_wait_give_up": (i32, [vp]),
        "faws_last_backend": (i32, []),
        "faws_launch_count": (C.c_int64, []),
        "faws_strerror": (C.c_char_p, [i32]),
        "faws_version": (i32, []),
    }
    for name, (res, args) in protos.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int, what: str):
    if status != 0:
        msg = load().faws_strerror(status).decode()
        raise RuntimeError(f"{what}: libfaws status {status}: {msg}")
