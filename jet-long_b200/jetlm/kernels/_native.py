"""ctypes binding of libjetlong_b200.so (the C ABI declared in include/jetlong_b200.h).

There is no fallback: if the shared library is missing, or a call returns a non-zero status, an
exception is raised.  Build the library with `python jet-long_b200/build.py`.
"""
from __future__ import annotations

import ctypes as C
import os

JL_MAX_CLASSES = 3
JL_MAX_SEGMENTS = 4
JL_MAX_PARTS = 16

JL_OK, JL_ERR_BAD_ARG, JL_ERR_UNSUPPORTED, JL_ERR_LAUNCH, JL_ERR_ARCH, JL_ERR_WORKSPACE = range(6)
JL_MAP_BAND, JL_MAP_CHUNK = 0, 1

LIB_NAME = "libjetlong_b200.so"
LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), LIB_NAME)


class PosMap(C.Structure):
    _fields_ = [("kind", C.c_int32), ("n_classes", C.c_int32), ("near_span", C.c_int64), ("chunk", C.c_int64)]


class PrefillArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p * JL_MAX_CLASSES), ("k", C.c_void_p * JL_MAX_CLASSES), ("v", C.c_void_p),
        ("out", C.c_void_p), ("lse", C.c_void_p),
        ("q_stride_b", C.c_int64), ("q_stride_s", C.c_int64), ("q_stride_h", C.c_int64),
        ("k_stride_b", C.c_int64), ("k_stride_s", C.c_int64), ("k_stride_h", C.c_int64),
        ("v_stride_b", C.c_int64), ("v_stride_s", C.c_int64), ("v_stride_h", C.c_int64),
        ("o_stride_b", C.c_int64), ("o_stride_s", C.c_int64), ("o_stride_h", C.c_int64),
        ("batch", C.c_int32), ("seqlen_q", C.c_int32), ("seqlen_k", C.c_int32),
        ("heads", C.c_int32), ("kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("q_pos0", C.c_int64), ("k_pos0", C.c_int64), ("k_block", C.c_int64), ("k_block_stride", C.c_int64),
        ("softmax_scale", C.c_float), ("map", PosMap), ("impl", C.c_int32),
        ("q_block", C.c_int64), ("q_block_stride", C.c_int64),
        ("remap_far_in_kernel", C.c_int32), ("group_size", C.c_int32), ("inv_freq", C.c_void_p),
        ("q_batch_first", C.c_int32), ("q_batch_wrap", C.c_int32), ("q_pos0_batch_step", C.c_int64),
    ]


class KvSegment(C.Structure):
    _fields_ = [
        ("k", C.c_void_p), ("v", C.c_void_p),
        ("k_stride_b", C.c_int64), ("k_stride_s", C.c_int64), ("k_stride_h", C.c_int64),
        ("v_stride_b", C.c_int64), ("v_stride_s", C.c_int64), ("v_stride_h", C.c_int64),
        ("len_dev", C.c_void_p), ("pos0", C.c_int64),
        ("len", C.c_int32), ("q_class", C.c_int32), ("rotate", C.c_int32), ("reserved", C.c_int32),
        ("pos_block", C.c_int64), ("pos_block_stride", C.c_int64), ("row0_dev", C.c_void_p),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p * JL_MAX_CLASSES), ("q_stride_b", C.c_int64), ("q_stride_h", C.c_int64),
        ("seg", KvSegment * JL_MAX_SEGMENTS), ("n_segments", C.c_int32),
        ("batch", C.c_int32), ("heads", C.c_int32), ("kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("num_splits", C.c_int32), ("softmax_scale", C.c_float),
        ("inv_freq", C.c_void_p), ("group_size", C.c_int32), ("reserved", C.c_int32),
        ("out", C.c_void_p), ("lse", C.c_void_p), ("o_stride_b", C.c_int64), ("o_stride_h", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class MergeArgs(C.Structure):
    _fields_ = [
        ("o", C.c_void_p * JL_MAX_PARTS), ("lse", C.c_void_p * JL_MAX_PARTS), ("n_parts", C.c_int32),
        ("batch", C.c_int32), ("seqlen", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32),
        ("round_like_reference", C.c_int32), ("out", C.c_void_p), ("lse_out", C.c_void_p),
    ]


class RotateArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("out", C.c_void_p),
        ("x_stride_b", C.c_int64), ("x_stride_s", C.c_int64), ("x_stride_h", C.c_int64),
        ("o_stride_b", C.c_int64), ("o_stride_s", C.c_int64), ("o_stride_h", C.c_int64),
        ("batch", C.c_int32), ("seqlen", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32),
        ("pos0", C.c_int64), ("div", C.c_int64), ("div_mul", C.c_int64), ("mod", C.c_int64),
        ("mod_mul", C.c_int64), ("add", C.c_int64), ("t_max", C.c_int64), ("inv_freq", C.c_void_p),
        ("pos_block", C.c_int64), ("pos_block_stride", C.c_int64),
    ]


class NormRopeArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("weight", C.c_void_p), ("out_base", C.c_void_p), ("out_group", C.c_void_p),
        ("x_stride_b", C.c_int64), ("x_stride_s", C.c_int64), ("x_stride_h", C.c_int64),
        ("b_stride_b", C.c_int64), ("b_stride_s", C.c_int64), ("b_stride_h", C.c_int64),
        ("g_stride_b", C.c_int64), ("g_stride_s", C.c_int64), ("g_stride_h", C.c_int64),
        ("batch", C.c_int32), ("seqlen", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32),
        ("eps", C.c_float), ("group_size", C.c_int32),
        ("pos0", C.c_int64), ("pos_block", C.c_int64), ("pos_block_stride", C.c_int64), ("inv_freq", C.c_void_p),
    ]


class RmsNormArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("residual", C.c_void_p), ("weight", C.c_void_p), ("sum_out", C.c_void_p),
                ("out", C.c_void_p), ("rows", C.c_int64), ("hidden", C.c_int32), ("eps", C.c_float)]


class SiluMulArgs(C.Structure):
    _fields_ = [("gate", C.c_void_p), ("up", C.c_void_p), ("out", C.c_void_p), ("count", C.c_int64)]


JL_STEP_STATE_WORDS = 6


class StepAdvanceArgs(C.Structure):
    _fields_ = [("state", C.c_void_p), ("lens", C.c_void_p), ("batch", C.c_int32), ("rank", C.c_int32),
                ("world", C.c_int32), ("reserved", C.c_int32), ("block", C.c_int64), ("w_0", C.c_int64)]


class DecodeAppendArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("q_stride_b", C.c_int64), ("q_stride_h", C.c_int64), ("k_stride_b", C.c_int64), ("k_stride_h", C.c_int64),
        ("v_stride_b", C.c_int64), ("v_stride_h", C.c_int64),
        ("q_weight", C.c_void_p), ("k_weight", C.c_void_p), ("q_eps", C.c_float), ("k_eps", C.c_float),
        ("q_base", C.c_void_p), ("q_group", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("kc_stride_b", C.c_int64), ("kc_stride_s", C.c_int64), ("kc_stride_h", C.c_int64),
        ("vc_stride_b", C.c_int64), ("vc_stride_s", C.c_int64), ("vc_stride_h", C.c_int64),
        ("batch", C.c_int32), ("heads", C.c_int32), ("kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("group_size", C.c_int32), ("reserved", C.c_int32), ("cache_rows", C.c_int64),
        ("inv_freq", C.c_void_p), ("state", C.c_void_p),
        ("k_group_cache", C.c_void_p), ("pos0", C.c_int64), ("pos_block", C.c_int64), ("pos_block_stride", C.c_int64),
    ]


class PeerMergeArgs(C.Structure):
    _fields_ = [("part_o", C.c_void_p), ("part_lse", C.c_void_p), ("peer_buf", C.c_void_p * JL_MAX_PARTS),
                ("buffer_bytes", C.c_size_t), ("rank", C.c_int32), ("world", C.c_int32),
                ("batch", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32), ("wait_limit_ms", C.c_int32),
                ("epoch_base_dev", C.c_void_p), ("epoch_stride", C.c_int64), ("epoch_offset", C.c_int64),
                ("out", C.c_void_p), ("lse_out", C.c_void_p), ("status", C.c_void_p)]


# Every symbol include/jetlong_b200.h declares: (name, restype, argtypes)
EXPORTS = [
    ("jl_version", C.c_int, []),
    ("jl_status_string", C.c_char_p, [C.c_int]),
    ("jl_last_error", C.c_char_p, []),
    ("jl_prefill", C.c_int, [C.POINTER(PrefillArgs), C.c_void_p]),
    ("jl_prefill_status", C.c_int, []),
    ("jl_decode_workspace_bytes", C.c_size_t, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    ("jl_decode_auto_splits", C.c_int32, [C.c_int32, C.c_int32, C.c_int64]),
    ("jl_decode", C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    ("jl_decode_static", C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    ("jl_decode_static_scratch_bytes", C.c_size_t, []),
    ("jl_merge", C.c_int, [C.POINTER(MergeArgs), C.c_void_p]),
    ("jl_rotate", C.c_int, [C.POINTER(RotateArgs), C.c_void_p]),
    ("jl_norm_rope", C.c_int, [C.POINTER(NormRopeArgs), C.c_void_p]),
    ("jl_rmsnorm", C.c_int, [C.POINTER(RmsNormArgs), C.c_void_p]),
    ("jl_peer_merge_buffer_bytes", C.c_size_t, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    ("jl_peer_merge", C.c_int, [C.POINTER(PeerMergeArgs), C.c_void_p]),
    ("jl_silu_mul", C.c_int, [C.POINTER(SiluMulArgs), C.c_void_p]),
    ("jl_step_advance", C.c_int, [C.POINTER(StepAdvanceArgs), C.c_void_p]),
    ("jl_decode_append", C.c_int, [C.POINTER(DecodeAppendArgs), C.c_void_p]),
]

_LIB = None


class NativeError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, fn: str, status: int, detail: str):
        self.status = status
        self.detail = detail
        super().__init__(f"{fn} failed: status {status} ({detail})")


def lib() -> C.CDLL:
    """The loaded shared library; raises (never falls back) if it has not been built."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_NAME} not found at {LIB_PATH}: the CUDA extension is required (no CPU or PyTorch "
                f"fallback exists). Build it with `python jet-long_b200/build.py`.")
        handle = C.CDLL(LIB_PATH)
        for name, restype, argtypes in EXPORTS:
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _LIB = handle
    return _LIB


def check(fn: str, status: int) -> None:
    if status != JL_OK:
        detail = lib().jl_last_error().decode() or lib().jl_status_string(status).decode()
        raise NativeError(fn, status, detail)
