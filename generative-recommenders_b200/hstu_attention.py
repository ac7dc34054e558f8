"""``hstu_mha`` with the reference's calling convention, running the sm_100a kernels.

Mirrors generative_recommenders/ops/hstu_attention.py:101-207 (arguments, checks and return
value) and the autograd wrapper of its GPU backends
(generative_recommenders/ops/triton/triton_hstu_attention.py:2978-3092).
"""

import ctypes
import os
from typing import Optional

import torch

from . import _cabi
from .common import HammerKernel, _require_cuda_backend, dtype_code, last_dim_contiguous, require_cuda, stream_ptr

_IMPL = {"auto": _cabi.IMPL_AUTO, "simt": _cabi.IMPL_SIMT, "tcgen05": _cabi.IMPL_TCGEN05}
_forced_impl = "auto"


def set_attention_impl(name: str) -> None:
    """Force the kernel family ("auto", "simt", "tcgen05") - for tests and profiling."""
    global _forced_impl
    if name not in _IMPL:
        raise ValueError(name)
    _forced_impl = name


def _i32(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    # tests of the reference pass int64 offsets (hstu_attention_test.py:81-84); its CUDA op wants
    # int32 (flash_common.cpp:460-472).  The kernels read int32.
    if t is None:
        return None
    return t.to(torch.int32).contiguous()


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None or t.numel() == 0 else t.data_ptr()


def _fill_common(a, q, k, v, seq_offsets, num_targets, attn_scale, max_seq_len, alpha, max_attn_len,
                 contextual_seq_len, min_full_attn_seq_len, bias_by_distance, dropout_pr=0.0, dropout_seed=None):
    L, H, dqk = q.shape
    a.q, a.k, a.v = _ptr(q), _ptr(k), _ptr(v)
    a.seq_offsets = _ptr(seq_offsets)
    a.num_targets = _ptr(num_targets)
    if attn_scale is not None:
        a.attn_scale = attn_scale.data_ptr()
        a.attn_scale_numel = attn_scale.numel()
    a.q_row_stride, a.q_head_stride = q.stride(0), q.stride(1)
    a.k_row_stride, a.k_head_stride = k.stride(0), k.stride(1)
    a.v_row_stride, a.v_head_stride = v.stride(0), v.stride(1)
    a.total_L = k.shape[0]
    a.B = seq_offsets.numel() - 1
    a.H, a.dqk, a.dv = H, dqk, v.shape[2]
    a.max_seq_len = max_seq_len
    a.alpha = alpha
    a.max_attn_len = max_attn_len
    a.contextual_seq_len = contextual_seq_len
    a.min_full_attn_seq_len = min_full_attn_seq_len
    a.dtype = dtype_code(q)
    a.impl = _IMPL[_forced_impl]
    if bias_by_distance is not None:
        a.bias_by_distance = bias_by_distance.data_ptr()
        a.bias_numel = bias_by_distance.numel()
    if dropout_seed is not None and dropout_pr > 0.0:
        a.dropout_ratio = dropout_pr
        a.dropout_seed = dropout_seed.data_ptr()


_PLAN_OWN, _PLAN_FOR_BACKWARD, _PLAN_REUSE = 0, 1, 2

# B200_HSTU_CHECK_STATUS=1: after every tensor-core attention launch, wait for it and read the status
# words of its work lists back; a bounded wait that gave up inside the kernel (which then returned
# early, leaving its output incomplete) becomes a RuntimeError instead of passing silently.  A
# debugging aid: it synchronises the stream after every call.
_CHECK_STATUS = os.environ.get("B200_HSTU_CHECK_STATUS", "0") not in ("", "0")


def set_status_check(on: bool) -> None:
    global _CHECK_STATUS
    _CHECK_STATUS = bool(on)


def attention_status(a, which: int, device):
    """Status words ``[forward, backward dK/dV, backward dQ]`` of the launches that used the scratch
    in ``a`` (0 = ran to completion, otherwise the id of the wait that gave up); waits for the stream."""
    host = torch.zeros(3, dtype=torch.int32).pin_memory()
    with torch.cuda.device(device):
        _cabi.check(_cabi.lib().b200_hstu_attn_status_async(
            a, which, ctypes.cast(host.data_ptr(), ctypes.POINTER(ctypes.c_int32)), stream_ptr(device)),
            "b200_hstu_attn_status_async")
        torch.cuda.current_stream(device).synchronize()
    return host.tolist()


def _raise_on_status(a, which, device, what):
    st = attention_status(a, which, device)
    if any(st):
        raise RuntimeError("%s: a bounded wait inside the kernel gave up (status forward / dK,dV / dQ = %s); "
                           "the output is incomplete" % (what, st))


def _workspace(a, which: int, device) -> Optional[torch.Tensor]:
    """Scratch for a forward (0), a backward (1) or a forward that also plans the backward (2)."""
    n = _cabi.lib().b200_hstu_attn_workspace_bytes(a, which)
    if n <= 0:
        return None
    ws = torch.empty(n, dtype=torch.uint8, device=device)
    a.workspace = ws.data_ptr()
    a.workspace_bytes = n
    return ws


def hstu_attention_fwd(max_seq_len, alpha, q, k, v, seq_offsets, num_targets, attn_scale, max_attn_len,
                       contextual_seq_len, min_full_attn_seq_len, bias_by_distance=None, plan_for_backward=False,
                       dropout_pr=0.0, dropout_seed=None):
    """One forward launch; all tensors already validated / int32 / on the device.

    With ``plan_for_backward`` the planning kernel also builds the backward's work lists and the
    scratch tensor holding them is returned next to the output (``(out, scratch)``), to be passed
    to one ``hstu_attention_bwd`` call: one planning launch per training step instead of two."""
    L, H, _ = q.shape
    out = torch.empty((L, H, v.shape[2]), dtype=q.dtype, device=q.device)
    if L == 0:
        return (out, None) if plan_for_backward else out
    a = _cabi.AttnArgs()
    _fill_common(a, q, k, v, seq_offsets, num_targets, attn_scale, max_seq_len, alpha, max_attn_len,
                 contextual_seq_len, min_full_attn_seq_len, bias_by_distance, dropout_pr, dropout_seed)
    a.out = out.data_ptr()
    a.o_row_stride, a.o_head_stride = out.stride(0), out.stride(1)
    ws = _workspace(a, 2 if plan_for_backward else 0, q.device)  # kept alive until the launch is queued
    if plan_for_backward and ws is not None:
        a.plan_mode = _PLAN_FOR_BACKWARD
    with torch.cuda.device(q.device):
        _cabi.check(_cabi.lib().b200_hstu_attn_fwd(a, stream_ptr(q.device)), "b200_hstu_attn_fwd")
    if _CHECK_STATUS and ws is not None:
        _raise_on_status(a, 0, q.device, "b200_hstu_attn_fwd")
    return (out, ws) if plan_for_backward else out


def hstu_attention_bwd(dout, max_seq_len, alpha, q, k, v, seq_offsets, num_targets, attn_scale, max_attn_len,
                       contextual_seq_len, min_full_attn_seq_len, dq, dk, dv, bias_by_distance=None,
                       planned_scratch=None, d_bias=None, dropout_pr=0.0, dropout_seed=None) -> None:
    """Fills caller-allocated dq / dk / dv (the ownership rule of the reference's backward,
    triton_hstu_attention.py:3059-3079).  ``planned_scratch``: the scratch a forward with
    ``plan_for_backward`` returned for the same arguments; its lists serve one backward call.
    ``d_bias``: zero-filled fp32 tensor shaped like ``bias_by_distance``; the gradient of the
    bias is added into it."""
    if q.shape[0] == 0:
        return
    a = _cabi.AttnArgs()
    _fill_common(a, q, k, v, seq_offsets, num_targets, attn_scale, max_seq_len, alpha, max_attn_len,
                 contextual_seq_len, min_full_attn_seq_len, bias_by_distance, dropout_pr, dropout_seed)
    a.dout = dout.data_ptr()
    a.dq, a.dk, a.dv_ = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.do_row_stride, a.do_head_stride = dout.stride(0), dout.stride(1)
    a.dq_row_stride, a.dq_head_stride = dq.stride(0), dq.stride(1)
    a.dk_row_stride, a.dk_head_stride = dk.stride(0), dk.stride(1)
    a.dv_row_stride, a.dv_head_stride = dv.stride(0), dv.stride(1)
    if d_bias is not None and bias_by_distance is not None:
        a.d_bias_by_distance = d_bias.data_ptr()
    reuse = planned_scratch is not None and _cabi.lib().b200_hstu_attn_workspace_bytes(a, 1) > 0
    if reuse:
        a.plan_mode = _PLAN_REUSE
        a.workspace = planned_scratch.data_ptr()
        a.workspace_bytes = planned_scratch.numel()
    else:
        ws = _workspace(a, 1, q.device)  # noqa: F841
    with torch.cuda.device(q.device):
        _cabi.check(_cabi.lib().b200_hstu_attn_bwd(a, stream_ptr(q.device)), "b200_hstu_attn_bwd")
    if _CHECK_STATUS and a.workspace:
        _raise_on_status(a, 2 if reuse else 1, q.device, "b200_hstu_attn_bwd")


class _HstuMhaFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, seq_offsets, num_targets, attn_scale, bias_by_distance, max_seq_len, alpha,
                max_attn_len, contextual_seq_len, min_full_attn_seq_len, dropout_pr=0.0, dropout_seed=None):
        # when a gradient will be asked for, the forward's planning launch builds the backward's
        # work lists as well; the first backward call consumes them
        plan = any(ctx.needs_input_grad[:3]) or ctx.needs_input_grad[6]
        out = hstu_attention_fwd(max_seq_len, alpha, q, k, v, seq_offsets, num_targets, attn_scale, max_attn_len,
                                 contextual_seq_len, min_full_attn_seq_len, bias_by_distance, plan_for_backward=plan,
                                 dropout_pr=dropout_pr, dropout_seed=dropout_seed)
        ctx.planned_scratch = None
        if plan:
            out, ctx.planned_scratch = out
        ctx.save_for_backward(q, k, v, seq_offsets, num_targets, attn_scale, bias_by_distance, dropout_seed)
        ctx.params = (max_seq_len, alpha, max_attn_len, contextual_seq_len, min_full_attn_seq_len, dropout_pr)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, seq_offsets, num_targets, attn_scale, bias_by_distance, dropout_seed = ctx.saved_tensors
        max_seq_len, alpha, max_attn_len, contextual_seq_len, min_full_attn_seq_len, dropout_pr = ctx.params
        dout = last_dim_contiguous(dout)
        # heads side by side, rows not overlapping (a gradient that autograd expanded from a reduced
        # tensor - the backward of ``out.sum(0)`` - has row stride 0)
        if dout.stride(1) != dout.shape[2] or dout.stride(0) < dout.shape[1] * dout.shape[2]:
            dout = dout.contiguous()
        dq = torch.empty_like(q, memory_format=torch.contiguous_format)
        dk = torch.empty_like(k, memory_format=torch.contiguous_format)
        dv = torch.empty_like(v, memory_format=torch.contiguous_format)
        planned, ctx.planned_scratch = ctx.planned_scratch, None   # a second backward plans for itself
        d_bias = None
        if bias_by_distance is not None and ctx.needs_input_grad[6]:
            d_bias = torch.zeros_like(bias_by_distance)
        hstu_attention_bwd(dout, max_seq_len, alpha, q, k, v, seq_offsets, num_targets, attn_scale, max_attn_len,
                           contextual_seq_len, min_full_attn_seq_len, dq, dk, dv, bias_by_distance,
                           planned_scratch=planned, d_bias=d_bias, dropout_pr=dropout_pr, dropout_seed=dropout_seed)
        return dq, dk, dv, None, None, None, d_bias, None, None, None, None, None, None, None


def hstu_mha(
    max_seq_len: int,
    alpha: float,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    seq_offsets: torch.Tensor,
    causal: bool = True,
    dropout_pr: float = 0.0,
    training: bool = True,
    num_targets: Optional[torch.Tensor] = None,
    attn_scale: Optional[torch.Tensor] = None,
    max_attn_len: int = 0,
    contextual_seq_len: int = 0,
    min_full_attn_seq_len: int = 0,
    sort_by_length: bool = False,
    kernel: HammerKernel = HammerKernel.CUDA,
    enable_tma: bool = False,
    bias_by_distance: Optional[torch.Tensor] = None,
    dropout_seed: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Jagged HSTU attention; same arguments, checks and result as the reference's
    ``hstu_mha`` (generative_recommenders/ops/hstu_attention.py:101-207).

    ``dropout_pr`` (in training): dropout on the attention weights after scale and mask, as the
    reference's PyTorch path applies it (ops/pytorch/pt_hstu_attention.py:180-181).  The mask is
    generated inside the CUDA-core kernels from a counter-based generator keyed by ``dropout_seed``
    (an extension: a one-element int64 tensor on the device, drawn from torch's CUDA generator when
    not given) and regenerated by the backward; the tensor-core kernels do not take part (no layer
    of the reference passes a non-zero rate, ops/hstu_compute.py:327-328), so such a call runs at
    CUDA-core speed.

    ``sort_by_length`` and ``enable_tma`` are accepted and ignored: work is always scheduled
    longest-first and K/V always stream through TMA.  ``bias_by_distance`` is an extension
    (fp32 ``[n]``: a relative-position bias added to ``alpha * q.k`` before SiLU, indexed by
    ``|i - j|``, shared by all heads; differentiable - the research model trains the tables it is
    gathered from, generative_recommenders/research/modeling/sequential/hstu.py:65-143).
    """
    _require_cuda_backend(kernel)
    torch._assert(max_seq_len > 0, "max_seq_len must be larger than 0")
    torch._assert(q.dim() == 3, "q must be 3-D")
    torch._assert(k.shape == q.shape, "k must be the same shape as q")
    torch._assert(v.dim() == 3, "v must be 3-D")
    torch._assert(v.shape[0] == q.shape[0], "wrong v shape[0]")
    torch._assert(v.shape[1] == q.shape[1], "wrong v shape[1]")
    torch._assert(causal, "only support causal attention")
    drop = float(dropout_pr) if (training and dropout_pr > 0.0) else 0.0
    if drop > 1.0:
        raise ValueError("dropout probability has to be between 0 and 1")
    require_cuda(q, k, v, seq_offsets, num_targets, attn_scale, bias_by_distance)
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("q, k, v must share a dtype")
    q = last_dim_contiguous(q)
    k = last_dim_contiguous(k)
    v = last_dim_contiguous(v)
    seq_offsets = _i32(seq_offsets)
    num_targets = _i32(num_targets)
    if num_targets is not None and num_targets.numel() != seq_offsets.numel() - 1:
        raise RuntimeError("num_targets must have one entry per sequence")
    if attn_scale is not None:
        attn_scale = attn_scale.to(torch.float32).reshape(-1).contiguous()
        if attn_scale.numel() not in (1, q.shape[0]):
            raise RuntimeError("attn_scale must be a scalar or have one entry per token")
    if bias_by_distance is not None:
        bias_by_distance = bias_by_distance.to(torch.float32).reshape(-1).contiguous()
    if drop >= 1.0:      # everything dropped (torch's dropout returns zeros for p = 1)
        drop = 0.0
        zero_all = True
    else:
        zero_all = False
    if drop > 0.0:
        if dropout_seed is None:
            # from torch's CUDA generator: reproducible under torch.manual_seed
            dropout_seed = torch.randint(0, 2 ** 62, (1,), dtype=torch.int64, device=q.device)
        require_cuda(dropout_seed)
        if dropout_seed.dtype != torch.int64 or dropout_seed.numel() != 1:
            raise TypeError("dropout_seed must be a one-element int64 tensor")
    else:
        dropout_seed = None
    out = _HstuMhaFunction.apply(q, k, v, seq_offsets, num_targets, attn_scale, bias_by_distance, int(max_seq_len),
                                 float(alpha), int(max_attn_len), int(contextual_seq_len),
                                 int(min_full_attn_seq_len), drop, dropout_seed)
    return out * 0 if zero_all else out


def delta_hstu_mha(
    max_seq_len: int,
    alpha: float,
    delta_q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    seq_offsets: torch.Tensor,
    num_targets: Optional[torch.Tensor] = None,
    max_attn_len: int = 0,
    contextual_seq_len: int = 0,
    kernel: HammerKernel = HammerKernel.CUDA,
    enable_tma: bool = False,
) -> torch.Tensor:
    """Cached-inference attention: the last ``delta`` positions of every sequence attend to the
    sequence's full (cached) K / V.  Same arguments, checks and result as the reference's
    ``delta_hstu_mha`` (generative_recommenders/ops/hstu_attention.py:210-275): ``delta_q`` is
    ``[B * delta, H, d]``, ``k`` / ``v`` are jagged over ``seq_offsets``, the result is
    ``[B * delta, H, d_v]``.  Every sequence must be at least ``delta`` and at most ``max_seq_len``
    long (the reference's mask gather assumes the same).  No gradient: this is the inference path.
    """
    _require_cuda_backend(kernel)
    L, H, D = delta_q.shape if delta_q.dim() == 3 else (0, 0, 0)
    B = seq_offsets.size(0) - 1
    torch._assert(max_seq_len > 0, "max_seq_len must be larger than 0")
    torch._assert(delta_q.dim() == 3, "delta_q must be 3-D")
    torch._assert(B > 0 and L % B == 0, "delta_q must be padded")
    torch._assert(k.dim() == 3, "k must be 3-D")
    torch._assert(k.shape[1] == H, "wrong k shape[1]")
    torch._assert(k.shape[2] == D, "wrong k shape[2]")
    torch._assert(v.dim() == 3, "v must be 3-D")
    torch._assert(v.shape[1] == H, "wrong v shape[1]")
    require_cuda(delta_q, k, v, seq_offsets, num_targets)
    if k.dtype != delta_q.dtype or v.dtype != delta_q.dtype:
        raise TypeError("delta_q, k, v must share a dtype")
    delta = L // B
    out = torch.zeros((L, H, v.shape[2]), dtype=delta_q.dtype, device=delta_q.device)
    if L == 0 or k.shape[0] == 0:
        return out
    q = last_dim_contiguous(delta_q.detach())
    k = last_dim_contiguous(k.detach())
    v = last_dim_contiguous(v.detach())
    seq_offsets = _i32(seq_offsets)
    num_targets = _i32(num_targets)
    a = _cabi.AttnArgs()
    _fill_common(a, q, k, v, seq_offsets, num_targets, None, int(max_seq_len), float(alpha), int(max_attn_len),
                 int(contextual_seq_len), 0, None)
    a.delta_size = delta
    a.out = out.data_ptr()
    a.o_row_stride, a.o_head_stride = out.stride(0), out.stride(1)
    ws = _workspace(a, 0, q.device)  # noqa: F841  (kept alive until the launch is queued)
    with torch.cuda.device(q.device):
        _cabi.check(_cabi.lib().b200_hstu_attn_fwd(a, stream_ptr(q.device)), "b200_hstu_attn_fwd (delta)")
    return out
