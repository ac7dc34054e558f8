"""The attention as registered PyTorch operators, ``torch.ops.b200_hstu.attn_fwd`` / ``attn_bwd``,
with fake (meta) implementations and an autograd formula, so that tracing front ends
(``torch.compile``, ``torch.export``, FX) see one opaque differentiable op instead of ctypes calls.

The reference registers its GPU kernels the same way and pins that the real and the fake
implementation of every op take the same arguments
(generative_recommenders/ops/triton/triton_hstu_attention.py:2813-2975,
generative_recommenders/ops/tests/fake_signature_test.py:49-162); scripted callers reach its
CUDA op through ``hstu_mha_cuda`` (generative_recommenders/ops/hstu_attention.py:50-98).
``hstu_mha_op`` below is the counterpart of that forwarder.  The eager ``hstu_mha`` keeps its own
autograd function (it lets the forward plan the backward's work lists); both run the same kernels.
"""

from typing import Optional, Tuple

import torch

from . import hstu_attention as _ha


@torch.library.custom_op("b200_hstu::attn_fwd", mutates_args=(), device_types="cuda")
def attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seq_offsets: torch.Tensor,
             num_targets: Optional[torch.Tensor], attn_scale: Optional[torch.Tensor],
             bias_by_distance: Optional[torch.Tensor], max_seq_len: int, alpha: float, max_attn_len: int,
             contextual_seq_len: int, min_full_attn_seq_len: int) -> torch.Tensor:
    return _ha.hstu_attention_fwd(max_seq_len, alpha, q, k, v, seq_offsets, num_targets, attn_scale, max_attn_len,
                                  contextual_seq_len, min_full_attn_seq_len, bias_by_distance)


def attn_fwd_fake(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seq_offsets: torch.Tensor,
                  num_targets: Optional[torch.Tensor], attn_scale: Optional[torch.Tensor],
                  bias_by_distance: Optional[torch.Tensor], max_seq_len: int, alpha: float, max_attn_len: int,
                  contextual_seq_len: int, min_full_attn_seq_len: int) -> torch.Tensor:
    return q.new_empty((q.shape[0], q.shape[1], v.shape[2]))


attn_fwd.register_fake(attn_fwd_fake)


@torch.library.custom_op("b200_hstu::attn_bwd", mutates_args=(), device_types="cuda")
def attn_bwd(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seq_offsets: torch.Tensor,
             num_targets: Optional[torch.Tensor], attn_scale: Optional[torch.Tensor],
             bias_by_distance: Optional[torch.Tensor], max_seq_len: int, alpha: float, max_attn_len: int,
             contextual_seq_len: int, min_full_attn_seq_len: int
             ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    dout = dout.contiguous()
    dq = torch.empty_like(q, memory_format=torch.contiguous_format)
    dk = torch.empty_like(k, memory_format=torch.contiguous_format)
    dv = torch.empty_like(v, memory_format=torch.contiguous_format)
    d_bias = torch.zeros_like(bias_by_distance) if bias_by_distance is not None else q.new_zeros((0,), dtype=torch.float32)
    _ha.hstu_attention_bwd(dout, max_seq_len, alpha, q, k, v, seq_offsets, num_targets, attn_scale, max_attn_len,
                           contextual_seq_len, min_full_attn_seq_len, dq, dk, dv, bias_by_distance,
                           d_bias=d_bias if bias_by_distance is not None else None)
    return dq, dk, dv, d_bias


def attn_bwd_fake(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seq_offsets: torch.Tensor,
                  num_targets: Optional[torch.Tensor], attn_scale: Optional[torch.Tensor],
                  bias_by_distance: Optional[torch.Tensor], max_seq_len: int, alpha: float, max_attn_len: int,
                  contextual_seq_len: int, min_full_attn_seq_len: int
                  ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    d_bias = torch.empty_like(bias_by_distance) if bias_by_distance is not None else q.new_empty((0,), dtype=torch.float32)
    return (torch.empty_like(q, memory_format=torch.contiguous_format),
            torch.empty_like(k, memory_format=torch.contiguous_format),
            torch.empty_like(v, memory_format=torch.contiguous_format), d_bias)


attn_bwd.register_fake(attn_bwd_fake)


def _setup_context(ctx, inputs, output):
    (q, k, v, seq_offsets, num_targets, attn_scale, bias, max_seq_len, alpha, max_attn_len, contextual_seq_len,
     min_full_attn_seq_len) = inputs
    ctx.save_for_backward(q, k, v, seq_offsets, num_targets, attn_scale, bias)
    ctx.params = (max_seq_len, alpha, max_attn_len, contextual_seq_len, min_full_attn_seq_len)


def _backward(ctx, dout):
    q, k, v, seq_offsets, num_targets, attn_scale, bias = ctx.saved_tensors
    dq, dk, dv, d_bias = attn_bwd(dout, q, k, v, seq_offsets, num_targets, attn_scale, bias, *ctx.params)
    return dq, dk, dv, None, None, None, (d_bias if bias is not None else None), None, None, None, None, None


attn_fwd.register_autograd(_backward, setup_context=_setup_context)


def hstu_mha_op(max_seq_len: int, alpha: float, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                seq_offsets: torch.Tensor, num_targets: Optional[torch.Tensor] = None, max_attn_len: int = 0,
                contextual_seq_len: int = 0, min_full_attn_seq_len: int = 0,
                attn_scale: Optional[torch.Tensor] = None,
                bias_by_distance: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``hstu_mha`` through the registered operator (for traced / compiled callers).  Offsets and
    targets must already be int32 tensors on the device; q, k, v have unit stride in the last
    dimension."""
    return torch.ops.b200_hstu.attn_fwd(q, k, v, seq_offsets, num_targets, attn_scale, bias_by_distance,
                                        int(max_seq_len), float(alpha), int(max_attn_len), int(contextual_seq_len),
                                        int(min_full_attn_seq_len))
