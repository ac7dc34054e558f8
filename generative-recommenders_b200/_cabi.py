"""ctypes binding of libb200_hstu.so (declarations in include/b200_hstu.h).

The library is the product: when it is missing or cannot be loaded, importing an op raises -
there is no Python or CPU fallback behind these calls.
"""

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int32, c_int64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200_hstu.so")

F32, BF16, F16, E4M3 = 0, 1, 2, 3
IMPL_AUTO, IMPL_SIMT, IMPL_TCGEN05 = 0, 1, 2

EXPORTS = [
    "b200_hstu_attn_fwd",
    "b200_hstu_attn_bwd",
    "b200_hstu_attn_workspace_bytes",
    "b200_hstu_attn_fwd_static_scratch",
    "b200_hstu_attn_fwd_static_scratch_max_bytes",
    "b200_hstu_attn_status_async",
    "b200_hstu_selftest_bounded_wait",
    "b200_hstu_attn_fwd_fp8",
    "b200_hstu_quantize_e4m3_block",
    "b200_hstu_layer_norm_fwd",
    "b200_hstu_layer_norm_bwd",
    "b200_hstu_layer_norm_bwd_workspace_bytes",
    "b200_hstu_silu_fwd",
    "b200_hstu_silu_bwd",
    "b200_hstu_norm_mul_fwd",
    "b200_hstu_norm_mul_bwd",
    "b200_hstu_norm_mul_bwd_workspace_bytes",
    "b200_hstu_norm_mul_dropout_mask_bytes",
    "b200_hstu_ln_linear_silu_fwd",
    "b200_hstu_ln_linear_workspace_bytes",
    "b200_hstu_ln_linear_supported",
    "b200_hstu_concat_2d_jagged",
    "b200_hstu_split_2d_jagged",
    "b200_hstu_add_timestamp_positional_embeddings_fwd",
    "b200_hstu_add_timestamp_positional_embeddings_bwd",
    "b200_hstu_last_error",
    "b200_hstu_version",
    "b200_hstu_launch_count",
    "b200_hstu_host_kv_range",
    "b200_hstu_host_mask",
    "b200_hstu_host_bwd_q_tiles",
    "b200_hstu_host_interval_mask",
    "b200_hstu_profile_enable",
    "b200_hstu_profile_collect",
]


class AttnArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("out", c_void_p),
        ("dout", c_void_p), ("dq", c_void_p), ("dk", c_void_p), ("dv_", c_void_p),
        ("seq_offsets", c_void_p), ("num_targets", c_void_p),
        ("attn_scale", c_void_p), ("attn_scale_numel", c_int64),
        ("q_row_stride", c_int64), ("k_row_stride", c_int64), ("v_row_stride", c_int64), ("o_row_stride", c_int64),
        ("q_head_stride", c_int64), ("k_head_stride", c_int64), ("v_head_stride", c_int64), ("o_head_stride", c_int64),
        ("do_row_stride", c_int64), ("dq_row_stride", c_int64), ("dk_row_stride", c_int64), ("dv_row_stride", c_int64),
        ("do_head_stride", c_int64), ("dq_head_stride", c_int64), ("dk_head_stride", c_int64), ("dv_head_stride", c_int64),
        ("total_L", c_int64),
        ("B", c_int32), ("H", c_int32), ("dqk", c_int32), ("dv", c_int32),
        ("max_seq_len", c_int32),
        ("alpha", c_float),
        ("max_attn_len", c_int32), ("contextual_seq_len", c_int32), ("min_full_attn_seq_len", c_int32),
        ("dtype", c_int32), ("impl", c_int32),
        ("bias_by_distance", c_void_p), ("bias_numel", c_int32), ("plan_mode", c_int32),
        ("workspace", c_void_p), ("workspace_bytes", c_int64),
        ("delta_size", c_int32), ("dropout_ratio", c_float),
        ("d_bias_by_distance", c_void_p),
        ("dropout_seed", c_void_p),
    ]


class AttnFp8Args(Structure):
    _fields_ = [
        ("base", AttnArgs),
        ("q_scale", c_void_p), ("k_scale", c_void_p), ("v_scale", c_void_p),
        ("block_offsets", c_void_p),
    ]


class NormMulArgs(Structure):
    _fields_ = [
        ("attn", c_void_p), ("u", c_void_p), ("weight", c_void_p), ("bias", c_void_p),
        ("out", c_void_p),
        ("mean", c_void_p), ("rstd", c_void_p),
        ("dout", c_void_p),
        ("dattn", c_void_p), ("du", c_void_p), ("dweight", c_void_p), ("dbias", c_void_p),
        ("partial", c_void_p), ("partial_bytes", c_int64),
        ("attn_row_stride", c_int64), ("u_row_stride", c_int64), ("out_row_stride", c_int64),
        ("dout_row_stride", c_int64), ("dattn_row_stride", c_int64), ("du_row_stride", c_int64),
        ("rows", c_int64),
        ("H", c_int32), ("V", c_int32),
        ("concat_u", c_int32), ("concat_x", c_int32), ("act", c_int32), ("group_norm", c_int32),
        ("eps", c_float),
        ("dtype", c_int32),
        ("dropout_ratio", c_float), ("reserved0", c_int32),
        ("dropout_seed", c_void_p),
        ("dropout_mask", c_void_p),
    ]


class LnLinearArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("norm_weight", c_void_p), ("norm_bias", c_void_p), ("weight", c_void_p), ("bias", c_void_p),
        ("out", c_void_p), ("u", c_void_p),
        ("mean", c_void_p), ("rstd", c_void_p),
        ("workspace", c_void_p), ("workspace_bytes", c_int64),
        ("x_row_stride", c_int64), ("out_row_stride", c_int64), ("u_row_stride", c_int64),
        ("M", c_int64),
        ("D", c_int32), ("N", c_int32), ("silu_cols", c_int32),
        ("eps", c_float),
        ("dtype", c_int32), ("weights_prepared", c_int32),
        ("skip_pre_activation", c_int32), ("reserved0", c_int32),
    ]


class JaggedArgs(Structure):
    _fields_ = [
        ("left", c_void_p), ("right", c_void_p), ("combined", c_void_p),
        ("offsets_left", c_void_p), ("offsets_right", c_void_p),
        ("dense_len_left", c_int64), ("dense_len_right", c_int64),
        ("total_rows", c_int64), ("row_bytes", c_int64),
        ("B", c_int32), ("right_rows_first", c_int32),
    ]


class TsPosArgs(Structure):
    _fields_ = [
        ("seq_embeddings", c_void_p), ("pos_weight", c_void_p), ("ts_weight", c_void_p),
        ("out", c_void_p),
        ("d_out", c_void_p), ("d_seq_embeddings", c_void_p),
        ("d_pos_weight", c_void_p), ("d_ts_weight", c_void_p),
        ("seq_offsets", c_void_p), ("seq_lengths", c_void_p), ("num_targets", c_void_p), ("timestamps", c_void_p),
        ("total_rows", c_int64),
        ("B", c_int32), ("D", c_int32),
        ("max_contextual_seq_len", c_int32), ("max_pos_ind", c_int32), ("ts_rows", c_int32),
        ("ts_bucket_max", c_int32),
        ("interleave_targets", c_int32), ("time_bucket_fn", c_int32),
        ("alpha", c_float),
        ("dtype", c_int32), ("table_dtype", c_int32),
        ("reserved0", c_int32),
    ]


_lib = None


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "libb200_hstu.so is missing (%s). Build it with "
            "`python generative-recommenders_b200/build.py`; there is no fallback path." % LIB_PATH
        )
    L = ctypes.CDLL(LIB_PATH)
    L.b200_hstu_attn_fwd.argtypes = [POINTER(AttnArgs), c_void_p]
    L.b200_hstu_attn_fwd.restype = ctypes.c_int
    L.b200_hstu_attn_bwd.argtypes = [POINTER(AttnArgs), c_void_p]
    L.b200_hstu_attn_bwd.restype = ctypes.c_int
    L.b200_hstu_attn_fwd_static_scratch.argtypes = [POINTER(AttnArgs), c_void_p]
    L.b200_hstu_attn_fwd_static_scratch.restype = ctypes.c_int
    L.b200_hstu_attn_fwd_static_scratch_max_bytes.argtypes = []
    L.b200_hstu_attn_fwd_static_scratch_max_bytes.restype = c_int64
    L.b200_hstu_attn_status_async.argtypes = [POINTER(AttnArgs), ctypes.c_int, POINTER(c_int32), c_void_p]
    L.b200_hstu_attn_status_async.restype = ctypes.c_int
    L.b200_hstu_selftest_bounded_wait.argtypes = [c_void_p, c_void_p, c_void_p]
    L.b200_hstu_selftest_bounded_wait.restype = ctypes.c_int
    L.b200_hstu_attn_workspace_bytes.argtypes = [POINTER(AttnArgs), ctypes.c_int]
    L.b200_hstu_attn_workspace_bytes.restype = c_int64
    L.b200_hstu_attn_fwd_fp8.argtypes = [POINTER(AttnFp8Args), c_void_p]
    L.b200_hstu_attn_fwd_fp8.restype = ctypes.c_int
    L.b200_hstu_quantize_e4m3_block.argtypes = [
        c_void_p, c_int32, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
        c_int32, c_int32, c_int32, c_int64, c_int32, c_void_p,
    ]
    L.b200_hstu_quantize_e4m3_block.restype = ctypes.c_int
    L.b200_hstu_layer_norm_fwd.argtypes = [
        c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
        c_int64, c_int32, c_float, c_int32, c_void_p,
    ]
    L.b200_hstu_layer_norm_fwd.restype = ctypes.c_int
    L.b200_hstu_layer_norm_bwd.argtypes = [
        c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
        c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int32, c_int32, c_void_p,
    ]
    L.b200_hstu_layer_norm_bwd.restype = ctypes.c_int
    L.b200_hstu_layer_norm_bwd_workspace_bytes.argtypes = [c_int32]
    L.b200_hstu_layer_norm_bwd_workspace_bytes.restype = c_int64
    L.b200_hstu_silu_fwd.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int32, c_int32, c_void_p]
    L.b200_hstu_silu_fwd.restype = ctypes.c_int
    L.b200_hstu_silu_bwd.argtypes = [
        c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int32, c_int32, c_void_p,
    ]
    L.b200_hstu_silu_bwd.restype = ctypes.c_int
    L.b200_hstu_norm_mul_fwd.argtypes = [POINTER(NormMulArgs), c_void_p]
    L.b200_hstu_norm_mul_fwd.restype = ctypes.c_int
    L.b200_hstu_norm_mul_bwd.argtypes = [POINTER(NormMulArgs), c_void_p]
    L.b200_hstu_norm_mul_bwd.restype = ctypes.c_int
    L.b200_hstu_norm_mul_bwd_workspace_bytes.argtypes = [c_int32, c_int32, c_int32]
    L.b200_hstu_norm_mul_bwd_workspace_bytes.restype = c_int64
    L.b200_hstu_norm_mul_dropout_mask_bytes.argtypes = [POINTER(NormMulArgs)]
    L.b200_hstu_norm_mul_dropout_mask_bytes.restype = c_int64
    for name, struct in (("b200_hstu_concat_2d_jagged", JaggedArgs), ("b200_hstu_split_2d_jagged", JaggedArgs),
                         ("b200_hstu_add_timestamp_positional_embeddings_fwd", TsPosArgs),
                         ("b200_hstu_add_timestamp_positional_embeddings_bwd", TsPosArgs)):
        getattr(L, name).argtypes = [POINTER(struct), c_void_p]
        getattr(L, name).restype = ctypes.c_int
    L.b200_hstu_ln_linear_silu_fwd.argtypes = [POINTER(LnLinearArgs), c_void_p]
    L.b200_hstu_ln_linear_silu_fwd.restype = ctypes.c_int
    L.b200_hstu_ln_linear_workspace_bytes.argtypes = [c_int32, c_int32]
    L.b200_hstu_ln_linear_workspace_bytes.restype = c_int64
    L.b200_hstu_ln_linear_supported.argtypes = [c_int32] * 4
    L.b200_hstu_ln_linear_supported.restype = ctypes.c_int
    L.b200_hstu_last_error.argtypes = []
    L.b200_hstu_last_error.restype = c_char_p
    L.b200_hstu_version.restype = ctypes.c_int
    L.b200_hstu_launch_count.restype = c_int64
    L.b200_hstu_host_kv_range.argtypes = [c_int32] * 8 + [POINTER(c_int32)] * 3
    L.b200_hstu_host_kv_range.restype = None
    L.b200_hstu_host_bwd_q_tiles.argtypes = [c_int32] * 7 + [POINTER(c_int32)] * 3
    L.b200_hstu_host_bwd_q_tiles.restype = None
    L.b200_hstu_profile_enable.argtypes = [ctypes.c_int]
    L.b200_hstu_profile_enable.restype = None
    L.b200_hstu_profile_collect.argtypes = [ctypes.c_int, POINTER(c_float), ctypes.c_int]
    L.b200_hstu_profile_collect.restype = ctypes.c_int
    L.b200_hstu_host_interval_mask.argtypes = [c_int32] * 9
    L.b200_hstu_host_interval_mask.restype = ctypes.c_int
    L.b200_hstu_host_mask.argtypes = [c_int32] * 8
    L.b200_hstu_host_mask.restype = ctypes.c_int
    _lib = L
    return L


def check(status, what):
    """Turn a non-zero status into a RuntimeError (the reference raises RuntimeError from
    TORCH_CHECK, generative_recommenders/ops/cpp/hstu_attention/flash_common.cpp:420-594)."""
    if status != 0:
        msg = lib().b200_hstu_last_error().decode("utf-8", "replace")
        raise RuntimeError("%s failed (status %d): %s" % (what, status, msg))


def launch_count():
    return int(lib().b200_hstu_launch_count())


PROFILE_KINDS = {
    "plan": 0, "attn_fwd": 1, "attn_bwd_dkdv": 2, "attn_bwd_dq": 3, "attn_fwd_fp8": 4, "layer_norm_fwd": 5,
    "layer_norm_bwd": 6, "silu": 7, "norm_mul_fwd": 8, "norm_mul_bwd": 9, "quantize": 10, "attn_simt": 11,
    "jagged": 12, "ts_pos": 13, "ln_linear_prep": 14, "ln_linear": 15,
}


def profile_enable(on: bool) -> None:
    lib().b200_hstu_profile_enable(1 if on else 0)


def profile_collect(kind: str):
    """Durations (ms) of the launches of one kernel kind since profiling was enabled; call after
    a device synchronisation."""
    buf = (c_float * 512)()
    n = lib().b200_hstu_profile_collect(PROFILE_KINDS[kind], buf, 512)
    return [buf[i] for i in range(n)]
