"""FP8 (e4m3) inference forward of the jagged HSTU attention with per-block scales.

An extension of the reference API: the reference's CUDA op accepts per-(batch, head) descale
tensors (generative_recommenders/ops/cpp/hstu_attention/flash_common.cpp:680-711) but compiles FP8
out (generative_recommenders/ops/cpp/setup.py:365).  Here q, k, v are quantised with one fp32
scale per (128-token block counted from the start of each sequence, head); the output is bf16.
"""

from typing import Optional, Tuple

import torch

from . import _cabi
from .common import dtype_code, last_dim_contiguous, require_cuda, stream_ptr

BLOCK = 128


def block_offsets_for(seq_offsets: torch.Tensor) -> torch.Tensor:
    """``[B + 1]`` int32 offsets of every sequence's first scale row (no host synchronisation)."""
    lens = seq_offsets[1:] - seq_offsets[:-1]
    nblk = (lens + (BLOCK - 1)) // BLOCK
    return torch.cat([nblk.new_zeros(1), torch.cumsum(nblk, 0)]).to(torch.int32)


def quantize_e4m3_block(x: torch.Tensor, seq_offsets: torch.Tensor,
                        block_offsets: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``x [L, H, d]`` -> ``(x8 [L, H, d] float8_e4m3fn, scale [L // 128 + B, H] fp32, block_offsets)``.

    ``scale`` has room for the largest possible number of blocks; rows past
    ``block_offsets[-1]`` are unused."""
    require_cuda(x, seq_offsets)
    x = last_dim_contiguous(x)
    L, H, d = x.shape
    seq_offsets = seq_offsets.to(torch.int32).contiguous()
    B = seq_offsets.numel() - 1
    if block_offsets is None:
        block_offsets = block_offsets_for(seq_offsets)
    x8 = torch.empty((L, H, d), dtype=torch.float8_e4m3fn, device=x.device)
    scale = torch.ones((L // BLOCK + B, H), dtype=torch.float32, device=x.device)
    if L > 0:
        with torch.cuda.device(x.device):
            _cabi.check(
                _cabi.lib().b200_hstu_quantize_e4m3_block(
                    x.data_ptr(), dtype_code(x), x.stride(0), x.stride(1), x8.data_ptr(), scale.data_ptr(),
                    seq_offsets.data_ptr(), block_offsets.data_ptr(), B, H, d, L, 1 << 30, stream_ptr(x.device)),
                "b200_hstu_quantize_e4m3_block")
    return x8, scale, block_offsets


def hstu_mha_fp8(
    max_seq_len: int,
    alpha: float,
    q8: torch.Tensor,
    k8: torch.Tensor,
    v8: torch.Tensor,
    q_scale: torch.Tensor,
    k_scale: torch.Tensor,
    v_scale: torch.Tensor,
    block_offsets: torch.Tensor,
    seq_offsets: torch.Tensor,
    num_targets: Optional[torch.Tensor] = None,
    max_attn_len: int = 0,
    contextual_seq_len: int = 0,
    min_full_attn_seq_len: int = 0,
) -> torch.Tensor:
    """Forward only (inference); same mask semantics as :func:`hstu_mha`; returns bf16 ``[L, H, d]``."""
    require_cuda(q8, k8, v8, q_scale, k_scale, v_scale, block_offsets, seq_offsets, num_targets)
    for t in (q8, k8, v8):
        if t.dtype != torch.float8_e4m3fn or not t.is_contiguous():
            raise TypeError("q8 / k8 / v8 must be contiguous float8_e4m3fn tensors")
    L, H, d = q8.shape
    out = torch.empty((L, H, d), dtype=torch.bfloat16, device=q8.device)
    if L == 0:
        return out
    seq_offsets = seq_offsets.to(torch.int32).contiguous()
    nt = None if num_targets is None else num_targets.to(torch.int32).contiguous()
    fa = _cabi.AttnFp8Args()
    a = fa.base
    a.q, a.k, a.v, a.out = q8.data_ptr(), k8.data_ptr(), v8.data_ptr(), out.data_ptr()
    a.seq_offsets = seq_offsets.data_ptr()
    a.num_targets = None if nt is None else nt.data_ptr()
    a.q_row_stride = a.k_row_stride = a.v_row_stride = H * d
    a.q_head_stride = a.k_head_stride = a.v_head_stride = d
    a.o_row_stride, a.o_head_stride = out.stride(0), out.stride(1)
    a.total_L, a.B, a.H, a.dqk, a.dv = L, seq_offsets.numel() - 1, H, d, d
    a.max_seq_len, a.alpha = int(max_seq_len), float(alpha)
    a.max_attn_len, a.contextual_seq_len = int(max_attn_len), int(contextual_seq_len)
    a.min_full_attn_seq_len = int(min_full_attn_seq_len)
    a.dtype = _cabi.BF16
    a.impl = _cabi.IMPL_TCGEN05
    nbytes = _cabi.lib().b200_hstu_attn_workspace_bytes(a, 0)
    # the fp8 forward uses the same work list as the bf16 forward; size it from the same query
    # (q8 is not 2-byte data, so ask with the bf16 layout the list size depends on: B and total_L)
    ws = torch.empty(max(int(nbytes), 64 + 32 * (L // BLOCK + a.B + 1) + 256), dtype=torch.uint8, device=q8.device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    fa.q_scale, fa.k_scale, fa.v_scale = q_scale.data_ptr(), k_scale.data_ptr(), v_scale.data_ptr()
    fa.block_offsets = block_offsets.to(torch.int32).contiguous().data_ptr()
    with torch.cuda.device(q8.device):
        _cabi.check(_cabi.lib().b200_hstu_attn_fwd_fp8(fa, stream_ptr(q8.device)), "b200_hstu_attn_fwd_fp8")
    return out
