"""The LayerNorm + linear stages around the attention, with the reference's signatures
(generative_recommenders/ops/hstu_compute.py:54-335)."""

import weakref
from typing import Optional, Tuple

import torch

from . import _cabi
from .common import HammerKernel, _require_cuda_backend, dtype_code, require_cuda, stream_ptr
from .hstu_attention import hstu_mha
from .layer_norm import layer_norm
from .mm import addmm

_ACT = {"none": 0, "sigmoid": 1, "silu": 2}


class _SiluColumnsFunction(torch.autograd.Function):
    """u = SiLU(x[:, :width]) written densely; x itself (the uvqk buffer) is left untouched."""

    @staticmethod
    def forward(ctx, x, width):
        rows = x.shape[0]
        u = torch.empty((rows, width), dtype=x.dtype, device=x.device)
        if rows > 0:
            with torch.cuda.device(x.device):
                _cabi.check(
                    _cabi.lib().b200_hstu_silu_fwd(x.data_ptr(), x.stride(0), u.data_ptr(), u.stride(0), rows, width,
                                                   dtype_code(x), stream_ptr(x.device)),
                    "b200_hstu_silu_fwd")
        ctx.save_for_backward(x)
        ctx.width = width
        return u

    @staticmethod
    def backward(ctx, du):
        (x,) = ctx.saved_tensors
        rows, width = x.shape[0], ctx.width
        if du.stride(-1) != 1:
            du = du.contiguous()
        dx = torch.zeros_like(x) if x.shape[1] != width else torch.empty_like(x)
        if rows > 0:
            with torch.cuda.device(x.device):
                _cabi.check(
                    _cabi.lib().b200_hstu_silu_bwd(du.data_ptr(), du.stride(0), x.data_ptr(), x.stride(0),
                                                   dx.data_ptr(), dx.stride(0), rows, width, dtype_code(x),
                                                   stream_ptr(x.device)),
                    "b200_hstu_silu_bwd")
        return dx, None


def _aligned16(t: torch.Tensor) -> torch.Tensor:
    """``t`` itself when its first element sits on a 16-byte boundary (what the tensor-core kernel's
    bulk loads need), else a fresh copy - a contiguous slice of a flat parameter buffer can start
    anywhere."""
    return t if t.data_ptr() % 16 == 0 else t.clone()


def _fused_uqvk_supported(x, uvqk_weight, hv) -> bool:
    if x.dtype not in (torch.bfloat16, torch.float16) or x.dim() != 2 or x.shape[0] == 0:
        return False
    if x.stride(-1) != 1 or x.stride(0) % 8 or x.stride(0) < x.shape[1] or x.data_ptr() % 16:
        return False
    D, N = uvqk_weight.shape
    return bool(_cabi.lib().b200_hstu_ln_linear_supported(D, N, hv, dtype_code(x)))


# Inference only: the workspace of the fused kernel holds what the preparation launches derive from
# the four parameter tensors (W' = diag(gamma) W and two column vectors).  While those tensors are
# alive and unmodified (same objects, same storage, same version counters) the workspace is kept
# and the preparation is skipped.  The version counter sees optimizer steps, load_state_dict and
# every other in-place operation on the parameter itself; it does NOT see a write through
# ``param.data`` (``param.data.copy_(new)``), which shares the storage but not the counter.  Code
# that refreshes weights that way calls ``clear_prepared_weights()`` afterwards, or switches the
# cache off with ``set_prepared_weights_cache(False)``.
_PREPARED = {}
_PREPARED_ON = True


def clear_prepared_weights() -> None:
    """Forget every cached preparation of the fused uvqk stage (see the comment above)."""
    _PREPARED.clear()


def set_prepared_weights_cache(on: bool) -> None:
    """Keep (default) or never keep the derived weights of the fused uvqk stage between
    inference calls."""
    global _PREPARED_ON
    _PREPARED_ON = bool(on)
    if not on:
        _PREPARED.clear()


def _prepared_workspace(nw, nb, w, b, nbytes, device, allow_cache):
    # Only module parameters are worth remembering, and only when all four tensors are the
    # parameters themselves: a cast copy made for one call never comes back, and its id / address /
    # version can recur on a later, different copy.
    if (not allow_cache or not _PREPARED_ON or torch.cuda.is_current_stream_capturing()
            or not all(isinstance(t, torch.nn.Parameter) for t in (w, nw, nb, b))):
        return torch.empty(nbytes, dtype=torch.uint8, device=device), False
    key = id(w)
    stream = torch.cuda.current_stream(device).cuda_stream
    sig = tuple((id(t), t.data_ptr(), t._version) for t in (w, nw, nb, b)) + (stream,)
    hit = _PREPARED.get(key)
    # the workspace was prepared on `stream`; a call on another stream is not ordered after that
    # preparation, so it prepares (and then owns) a new one
    if hit is not None and hit[0]() is w and hit[1] == sig and hit[2].numel() == nbytes:
        return hit[2], True
    ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
    if len(_PREPARED) > 256:
        _PREPARED.clear()
    _PREPARED[key] = (weakref.ref(w), sig, ws)
    return ws, False


def _fused_uqvk_launch(x, nw, nb, eps, w, b, hv, allow_cache=False):
    """One launch of the fused kernel: returns (uvqk [M, N], u [M, hv], mean [M], rstd [M])."""
    M, D = x.shape
    N = w.shape[1]
    uvqk = torch.empty((M, N), dtype=x.dtype, device=x.device)
    u = torch.empty((M, hv), dtype=x.dtype, device=x.device)
    mean = torch.empty(M, dtype=torch.float32, device=x.device)
    rstd = torch.empty(M, dtype=torch.float32, device=x.device)
    nbytes = _cabi.lib().b200_hstu_ln_linear_workspace_bytes(D, N)
    ws, prepared = _prepared_workspace(nw, nb, w, b, nbytes, x.device, allow_cache)
    a = _cabi.LnLinearArgs()
    a.weights_prepared = 1 if prepared else 0
    a.skip_pre_activation = 1 if allow_cache else 0   # no gradient wanted: nobody reads the pre-activation u
    a.x, a.norm_weight, a.norm_bias, a.weight, a.bias = (x.data_ptr(), nw.data_ptr(), nb.data_ptr(),
                                                          w.data_ptr(), b.data_ptr())
    a.out, a.u, a.mean, a.rstd = uvqk.data_ptr(), u.data_ptr(), mean.data_ptr(), rstd.data_ptr()
    a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
    a.x_row_stride, a.out_row_stride, a.u_row_stride = x.stride(0), uvqk.stride(0), u.stride(0)
    a.M, a.D, a.N, a.silu_cols = M, D, N, hv
    a.eps, a.dtype = eps, dtype_code(x)
    with torch.cuda.device(x.device):
        _cabi.check(_cabi.lib().b200_hstu_ln_linear_silu_fwd(a, stream_ptr(x.device)),
                    "b200_hstu_ln_linear_silu_fwd")
    return uvqk, u, mean, rstd


def _fused_uqvk_backward(x, nw, nb, w, uvqk, mean, rstd, eps, hv, du, d_uvqk):
    """Backward of the fused stage.  ``d_uvqk`` [M, N] already holds the gradients of the v, q, k
    columns; the u columns are filled here (``du * SiLU'``).  Recomputes ``LN(x)`` from the saved
    statistics (the reference's ``recompute_normed_x_in_backward``,
    generative_recommenders/ops/triton/triton_hstu_preprocess_and_attention.py:122-127, 185-203)
    and uses library GEMMs.  Returns (dx, d_norm_weight, d_norm_bias, d_weight, d_bias)."""
    M, D = x.shape
    lib = _cabi.lib()
    dt = dtype_code(x)
    st = stream_ptr(x.device)
    with torch.cuda.device(x.device):
        if du is not None:
            if du.stride(-1) != 1:
                du = du.contiguous()
            _cabi.check(lib.b200_hstu_silu_bwd(du.data_ptr(), du.stride(0), uvqk.data_ptr(), uvqk.stride(0),
                                               d_uvqk.data_ptr(), d_uvqk.stride(0), M, hv, dt, st),
                        "b200_hstu_silu_bwd")
        else:
            d_uvqk[:, :hv].zero_()
        normed = torch.empty_like(x)
        _cabi.check(lib.b200_hstu_layer_norm_fwd(x.data_ptr(), x.stride(0), nw.data_ptr(), nb.data_ptr(),
                                                 normed.data_ptr(), normed.stride(0), None, None, M, D, eps, dt, st),
                    "b200_hstu_layer_norm_fwd")
        dw = normed.t() @ d_uvqk
        # column sums on the tensor cores: cheaper than a strided reduction over [M, N]
        db = (torch.ones((1, M), dtype=x.dtype, device=x.device) @ d_uvqk).view(-1)
        dnormed = d_uvqk @ w.t()
        dx = torch.empty_like(x)
        dnw = torch.empty(D, dtype=x.dtype, device=x.device)
        dnb = torch.empty(D, dtype=x.dtype, device=x.device)
        nbytes = lib.b200_hstu_layer_norm_bwd_workspace_bytes(D)
        partial = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
        _cabi.check(lib.b200_hstu_layer_norm_bwd(dnormed.data_ptr(), dnormed.stride(0), x.data_ptr(), x.stride(0),
                                                 nw.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                                 dx.stride(0), dnw.data_ptr(), dnb.data_ptr(), partial.data_ptr(),
                                                 nbytes, M, D, dt, st),
                    "b200_hstu_layer_norm_bwd")
    return dx, dnw, dnb, dw, db


class _FusedUqvkFunction(torch.autograd.Function):
    """``uvqk = LN(x) W + b`` and ``u = SiLU(uvqk[:, :hv])`` from one tensor-core kernel
    (csrc/ln_linear_sm100.cu)."""

    @staticmethod
    def forward(ctx, x, norm_weight, norm_bias, eps, weight, bias, num_heads, attn_dim, hidden_dim, grad_mode=True):
        M = x.shape[0]
        hv, ha = hidden_dim * num_heads, attn_dim * num_heads
        nw = norm_weight.to(x.dtype).contiguous()
        nb = norm_bias.to(x.dtype).contiguous()
        w = _aligned16(weight.to(x.dtype).contiguous())
        b = bias.to(x.dtype).contiguous()
        no_grad = not (grad_mode and any(ctx.needs_input_grad))
        uvqk, u, mean, rstd = _fused_uqvk_launch(x, nw, nb, eps, w, b, hv, no_grad)
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(x, nw, nb, w, uvqk, mean, rstd)
        ctx.cfg = (eps, hv, ha, norm_weight.dtype, norm_bias.dtype, weight.dtype, bias.dtype)
        # q, k, v are views of the uvqk buffer, handed out as separate results so that the backward
        # receives their gradients one by one instead of three zero-padded [M, N] sums
        v = uvqk[:, hv:2 * hv].view(M, num_heads, hidden_dim)
        q = uvqk[:, 2 * hv:2 * hv + ha].view(M, num_heads, attn_dim)
        k = uvqk[:, 2 * hv + ha:].view(M, num_heads, attn_dim)
        return u, q, k, v

    @staticmethod
    def backward(ctx, du, dq, dk, dv):
        x, nw, nb, w, uvqk, mean, rstd = ctx.saved_tensors
        eps, hv, ha, nw_dtype, nb_dtype, w_dtype, b_dtype = ctx.cfg
        M, N = uvqk.shape
        d_uvqk = torch.empty((M, N), dtype=x.dtype, device=x.device)
        for lo, width, g in ((hv, hv, dv), (2 * hv, ha, dq), (2 * hv + ha, ha, dk)):
            if g is None:
                d_uvqk[:, lo:lo + width].zero_()
            else:
                d_uvqk[:, lo:lo + width].copy_(g.reshape(M, width))
        dx, dnw, dnb, dw, db = _fused_uqvk_backward(x, nw, nb, w, uvqk, mean, rstd, eps, hv, du, d_uvqk)
        return dx, dnw.to(nw_dtype), dnb.to(nb_dtype), None, dw.to(w_dtype), db.to(b_dtype), None, None, None, None


class _FusedPreprocessAttentionFunction(torch.autograd.Function):
    """The fused uvqk stage and the attention as one autograd node: the attention backward writes
    dq / dk / dv straight into the column blocks of ``d_uvqk``, which then feeds the stage's
    backward GEMMs - no gradient copies in between.  Returns (u, attn [M, H, dv], k, v)."""

    @staticmethod
    def forward(ctx, x, norm_weight, norm_bias, eps, weight, bias, num_heads, attn_dim, hidden_dim, seq_offsets,
                num_targets, bias_by_distance, max_seq_len, alpha, max_attn_len, contextual_seq_len, grad_mode=True,
                recompute_uvqk=False):
        from .hstu_attention import hstu_attention_fwd

        M = x.shape[0]
        hv, ha = hidden_dim * num_heads, attn_dim * num_heads
        nw = norm_weight.to(x.dtype).contiguous()
        nb = norm_bias.to(x.dtype).contiguous()
        w = _aligned16(weight.to(x.dtype).contiguous())
        b = bias.to(x.dtype).contiguous()
        no_grad = not (grad_mode and any(ctx.needs_input_grad))
        uvqk, u, mean, rstd = _fused_uqvk_launch(x, nw, nb, eps, w, b, hv, no_grad)
        v = uvqk[:, hv:2 * hv].view(M, num_heads, hidden_dim)
        q = uvqk[:, 2 * hv:2 * hv + ha].view(M, num_heads, attn_dim)
        k = uvqk[:, 2 * hv + ha:].view(M, num_heads, attn_dim)
        plan = not no_grad and (any(ctx.needs_input_grad[:6]) or ctx.needs_input_grad[11])
        ctx.set_materialize_grads(False)  # k / v usually get no gradient: do not add zeros for them
        out = hstu_attention_fwd(max_seq_len, alpha, q, k, v, seq_offsets, num_targets, None, max_attn_len,
                                 contextual_seq_len, 0, bias_by_distance, plan_for_backward=plan)
        ctx.planned_scratch = None
        if plan:
            out, ctx.planned_scratch = out
        # recompute_uvqk: the [M, 4 H d] projection - the largest activation of the layer - is not kept;
        # the backward runs the fused kernel once more (the reference's recompute_uvqk_in_backward,
        # generative_recommenders/ops/triton/triton_hstu_preprocess_and_attention.py:122-127, 185-203).
        # k and v go out as views of that buffer either way: it lives on only while the caller keeps them
        # (the layer does so for its KV cache, otherwise it drops them at once).
        keep = None if (recompute_uvqk and not no_grad) else uvqk
        ctx.save_for_backward(x, nw, nb, w, b, keep, mean, rstd, seq_offsets, num_targets, bias_by_distance)
        ctx.cfg = (eps, num_heads, attn_dim, hidden_dim, max_seq_len, alpha, max_attn_len, contextual_seq_len,
                   norm_weight.dtype, norm_bias.dtype, weight.dtype, bias.dtype)
        return u, out, k, v

    @staticmethod
    def backward(ctx, du, dattn, dk_ext, dv_ext):
        from .hstu_attention import hstu_attention_bwd

        x, nw, nb, w, b, uvqk, mean, rstd, seq_offsets, num_targets, bias_by_distance = ctx.saved_tensors
        (eps, H, A, V, max_seq_len, alpha, max_attn_len, contextual_seq_len,
         nw_dtype, nb_dtype, w_dtype, b_dtype) = ctx.cfg
        hv, ha = V * H, A * H
        if uvqk is None:   # not kept: one more launch of the fused kernel
            uvqk, _, mean, rstd = _fused_uqvk_launch(x, nw, nb, eps, w, b, hv, False)
        M, N = uvqk.shape
        d_uvqk = torch.empty((M, N), dtype=x.dtype, device=x.device)
        dv = d_uvqk[:, hv:2 * hv].view(M, H, V)
        dq = d_uvqk[:, 2 * hv:2 * hv + ha].view(M, H, A)
        dk = d_uvqk[:, 2 * hv + ha:].view(M, H, A)
        d_bias = None
        if dattn is None:
            d_uvqk[:, hv:].zero_()
        else:
            if (dattn.stride(-1) != 1 or dattn.stride(1) != dattn.shape[2]
                    or dattn.stride(0) < dattn.shape[1] * dattn.shape[2]):
                dattn = dattn.contiguous()
            v_ = uvqk[:, hv:2 * hv].view(M, H, V)
            q_ = uvqk[:, 2 * hv:2 * hv + ha].view(M, H, A)
            k_ = uvqk[:, 2 * hv + ha:].view(M, H, A)
            planned, ctx.planned_scratch = ctx.planned_scratch, None
            if bias_by_distance is not None and ctx.needs_input_grad[11]:
                d_bias = torch.zeros_like(bias_by_distance)
            hstu_attention_bwd(dattn, max_seq_len, alpha, q_, k_, v_, seq_offsets, num_targets, None, max_attn_len,
                               contextual_seq_len, 0, dq, dk, dv, bias_by_distance, planned_scratch=planned,
                               d_bias=d_bias)
        if dk_ext is not None:
            dk.add_(dk_ext)
        if dv_ext is not None:
            dv.add_(dv_ext)
        dx, dnw, dnb, dw, db = _fused_uqvk_backward(x, nw, nb, w, uvqk, mean, rstd, eps, hv, du, d_uvqk)
        return (dx, dnw.to(nw_dtype), dnb.to(nb_dtype), None, dw.to(w_dtype), db.to(b_dtype), None, None, None,
                None, None, d_bias, None, None, None, None, None, None)


_FUSED_UQVK = True


def set_fused_uqvk(on: bool) -> None:
    """Switch between the fused tensor-core uvqk stage (default, where the shapes allow it) and the
    three separate stages (LayerNorm kernel, library GEMM, SiLU kernel)."""
    global _FUSED_UQVK
    _FUSED_UQVK = bool(on)


def hstu_compute_uqvk(
    x: torch.Tensor,
    norm_weight: torch.Tensor,
    norm_bias: torch.Tensor,
    norm_eps: float,
    num_heads: int,
    attn_dim: int,
    hidden_dim: int,
    uvqk_weight: torch.Tensor,
    uvqk_bias: torch.Tensor,
    kernel: HammerKernel = HammerKernel.CUDA,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """LN -> addmm -> split [u | v | q | k] -> SiLU(u); returns (u, q, k, v) with q, k, v as
    ``[L, H, d]`` views of the uvqk buffer (generative_recommenders/ops/hstu_compute.py:54-104)."""
    _require_cuda_backend(kernel)
    require_cuda(x, norm_weight, norm_bias, uvqk_weight, uvqk_bias)
    hv, ha = hidden_dim * num_heads, attn_dim * num_heads
    if _FUSED_UQVK and _fused_uqvk_supported(x, uvqk_weight, hv):
        return _FusedUqvkFunction.apply(x, norm_weight, norm_bias, float(norm_eps), uvqk_weight, uvqk_bias,
                                        num_heads, attn_dim, hidden_dim, torch.is_grad_enabled())
    else:
        normed_x = layer_norm(x, weight=norm_weight, bias=norm_bias, eps=norm_eps, kernel=kernel)
        uvqk = addmm(uvqk_bias, normed_x, uvqk_weight, kernel)
        u = _SiluColumnsFunction.apply(uvqk[:, :hv], hv)
    v = uvqk[:, hv : 2 * hv].view(-1, num_heads, hidden_dim)
    q = uvqk[:, 2 * hv : 2 * hv + ha].view(-1, num_heads, attn_dim)
    k = uvqk[:, 2 * hv + ha :].view(-1, num_heads, attn_dim)
    return u, q, k, v


def _norm_mul_forward(attn, u, weight, bias, eps, num_heads, linear_dim, concat_u, concat_x, act, group_norm,
                      dropout_ratio, dropout_seed, want_mask=False):
    """One launch of the norm-mul kernel; returns ``(out, mean, rstd)`` (inputs already contiguous in
    their last dimension, weight / bias already of the activation dtype)."""
    rows = attn.shape[0]
    D = num_heads * linear_dim
    if group_norm:
        mult = 3 if (concat_u and concat_x) else 1
    else:
        mult = 1 + int(concat_u) + int(concat_x)
    out = torch.empty((rows, mult * D), dtype=attn.dtype, device=attn.device)
    groups = num_heads if group_norm else 1
    mean = torch.empty(rows * groups, dtype=torch.float32, device=attn.device)
    rstd = torch.empty(rows * groups, dtype=torch.float32, device=attn.device)
    a = _cabi.NormMulArgs()
    a.attn, a.u, a.weight, a.bias = attn.data_ptr(), u.data_ptr(), weight.data_ptr(), bias.data_ptr()
    a.out, a.mean, a.rstd = out.data_ptr(), mean.data_ptr(), rstd.data_ptr()
    a.attn_row_stride, a.u_row_stride, a.out_row_stride = attn.stride(0), u.stride(0), out.stride(0)
    a.rows, a.H, a.V = rows, num_heads, linear_dim
    a.concat_u, a.concat_x, a.act, a.group_norm = int(concat_u), int(concat_x), act, int(group_norm)
    a.eps, a.dtype = eps, dtype_code(attn)
    mask = None
    if dropout_seed is not None and dropout_ratio > 0.0:
        a.dropout_ratio, a.dropout_seed = dropout_ratio, dropout_seed.data_ptr()
        if want_mask and rows > 0:
            # one bit per output element, for a backward that reads the mask instead of running the
            # generator again (where the library can store it: 16-bit elements, whole aligned vectors)
            nbytes = _cabi.lib().b200_hstu_norm_mul_dropout_mask_bytes(a)
            if nbytes > 0:
                mask = torch.empty(nbytes, dtype=torch.uint8, device=attn.device)
                a.dropout_mask = mask.data_ptr()
    if rows > 0:
        with torch.cuda.device(attn.device):
            _cabi.check(_cabi.lib().b200_hstu_norm_mul_fwd(a, stream_ptr(attn.device)), "b200_hstu_norm_mul_fwd")
    if want_mask:
        return out, mean, rstd, mask
    return out, mean, rstd


def _norm_mul_backward(dout, attn, u, weight, bias, mean, rstd, eps, num_heads, linear_dim, concat_u, concat_x, act,
                       group_norm, dropout_ratio, dropout_seed, dropout_mask=None):
    """Backward of the norm-mul kernel; returns ``(dattn, du, dweight, dbias)``.  ``dropout_mask``: the
    bits the forward stored; without them the kernel regenerates the mask from the seed."""
    rows = attn.shape[0]
    if dout.stride(-1) != 1:
        dout = dout.contiguous()
    dattn = torch.empty((rows, num_heads * linear_dim), dtype=attn.dtype, device=attn.device)
    du = torch.empty_like(dattn)
    dw = torch.empty_like(weight)
    db = torch.empty_like(bias)
    nbytes = _cabi.lib().b200_hstu_norm_mul_bwd_workspace_bytes(num_heads, linear_dim, int(group_norm))
    partial = torch.empty(nbytes, dtype=torch.uint8, device=attn.device)
    a = _cabi.NormMulArgs()
    a.attn, a.u, a.weight, a.bias = attn.data_ptr(), u.data_ptr(), weight.data_ptr(), bias.data_ptr()
    a.mean, a.rstd = mean.data_ptr(), rstd.data_ptr()
    a.dout, a.dattn, a.du = dout.data_ptr(), dattn.data_ptr(), du.data_ptr()
    a.dweight, a.dbias = dw.data_ptr(), db.data_ptr()
    a.partial, a.partial_bytes = partial.data_ptr(), nbytes
    a.attn_row_stride, a.u_row_stride = attn.stride(0), u.stride(0)
    a.dout_row_stride, a.dattn_row_stride, a.du_row_stride = dout.stride(0), dattn.stride(0), du.stride(0)
    a.rows, a.H, a.V = rows, num_heads, linear_dim
    a.concat_u, a.concat_x, a.act, a.group_norm = int(concat_u), int(concat_x), act, int(group_norm)
    a.eps, a.dtype = eps, dtype_code(attn)
    if dropout_seed is not None and dropout_ratio > 0.0:   # the forward's mask: stored bits, or regenerated
        a.dropout_ratio, a.dropout_seed = dropout_ratio, dropout_seed.data_ptr()
        if dropout_mask is not None and dout.data_ptr() % 16 == 0 and dout.stride(0) % 8 == 0:
            a.dropout_mask = dropout_mask.data_ptr()
    with torch.cuda.device(attn.device):
        _cabi.check(_cabi.lib().b200_hstu_norm_mul_bwd(a, stream_ptr(attn.device)), "b200_hstu_norm_mul_bwd")
    return dattn, du, dw, db


# By default the backward of the norm-mul stage regenerates the dropout mask from the seed and nothing
# is stored.  Switched on, the forward also writes the mask as bits (6 % of the output's bytes) and the
# backward reads them: measured on B200 that forward is 8 % slower and that backward between 4 % and
# 28 % faster from run to run (both kernels are bound by instruction issue at the occupancy their
# registers allow and follow the SM clock), so it is off.  With recompute_y the mask is never stored.
_STORE_DROPOUT_MASK = False


def set_store_dropout_mask(on: bool) -> None:
    global _STORE_DROPOUT_MASK
    _STORE_DROPOUT_MASK = bool(on)


class _NormMulFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, attn, u, weight, bias, eps, num_heads, linear_dim, concat_u, concat_x, act, group_norm,
                dropout_ratio=0.0, dropout_seed=None):
        if attn.stride(-1) != 1:
            attn = attn.contiguous()
        if u.stride(-1) != 1:
            u = u.contiguous()
        weight = weight.to(attn.dtype).contiguous()
        bias = bias.to(attn.dtype).contiguous()
        keep_mask = _STORE_DROPOUT_MASK and any(ctx.needs_input_grad)   # (grad mode is off inside forward())
        out, mean, rstd, mask = _norm_mul_forward(attn, u, weight, bias, eps, num_heads, linear_dim, concat_u, concat_x,
                                                  act, group_norm, dropout_ratio, dropout_seed, want_mask=True) \
            if keep_mask else _norm_mul_forward(attn, u, weight, bias, eps, num_heads, linear_dim, concat_u, concat_x,
                                                act, group_norm, dropout_ratio, dropout_seed) + (None,)
        ctx.save_for_backward(attn, u, weight, bias, mean, rstd, dropout_seed, mask)
        ctx.cfg = (eps, num_heads, linear_dim, concat_u, concat_x, act, group_norm, dropout_ratio)
        return out

    @staticmethod
    def backward(ctx, dout):
        attn, u, weight, bias, mean, rstd, dropout_seed, mask = ctx.saved_tensors
        dattn, du, dw, db = _norm_mul_backward(dout, attn, u, weight, bias, mean, rstd, *ctx.cfg, dropout_seed, mask)
        return dattn, du, dw, db, None, None, None, None, None, None, None, None, None


class _OutputStageFunction(torch.autograd.Function):
    """The whole output stage, ``x + dropout(cat([u, attn, act(u) * Norm(attn)])) @ W``, as one autograd
    node that keeps its inputs and the row statistics only: the concatenated activation (three
    times as wide as ``attn``) is recomputed in the backward by one more launch of the norm-mul
    kernel - with the same dropout seed, hence the same mask - before the two backward GEMMs read it.
    This is the reference's ``recompute_y_in_backward``
    (generative_recommenders/ops/triton/triton_hstu_linear.py:1895-2040)."""

    @staticmethod
    def forward(ctx, attn, u, x, weight, bias, output_weight, eps, num_heads, linear_dim, concat_u, concat_x, act,
                group_norm, dropout_ratio, dropout_seed):
        if attn.stride(-1) != 1:
            attn = attn.contiguous()
        if u.stride(-1) != 1:
            u = u.contiguous()
        w = weight.to(attn.dtype).contiguous()
        b = bias.to(attn.dtype).contiguous()
        wo = output_weight.to(x.dtype)
        cfg = (eps, num_heads, linear_dim, concat_u, concat_x, act, group_norm, dropout_ratio)
        y, mean, rstd = _norm_mul_forward(attn, u, w, b, *cfg, dropout_seed)
        out = torch.addmm(x, y, wo)
        ctx.save_for_backward(attn, u, w, b, wo, mean, rstd, dropout_seed)
        ctx.cfg = cfg
        ctx.dtypes = (weight.dtype, bias.dtype, output_weight.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        attn, u, w, b, wo, mean, rstd, dropout_seed = ctx.saved_tensors
        y, _, _ = _norm_mul_forward(attn, u, w, b, *ctx.cfg, dropout_seed)
        if dout.stride(-1) != 1:
            dout = dout.contiguous()
        d_wo = y.t() @ dout
        del y
        dy = dout @ wo.t()
        dattn, du, dw, db = _norm_mul_backward(dy, attn, u, w, b, mean, rstd, *ctx.cfg, dropout_seed)
        wdt, bdt, odt = ctx.dtypes
        return (dattn, du, dout, dw.to(wdt), db.to(bdt), d_wo.to(odt), None, None, None, None, None, None, None, None,
                None)


def _draw_dropout_seed(device) -> torch.Tensor:
    # from torch's CUDA generator: reproducible under torch.manual_seed, and a fresh value on every
    # replay when the step is captured in a CUDA graph
    return torch.randint(0, 2 ** 62, (1,), dtype=torch.int64, device=device)


def hstu_norm_mul_dropout(
    attn: torch.Tensor,
    u: torch.Tensor,
    norm_weight: torch.Tensor,
    norm_bias: torch.Tensor,
    norm_eps: float,
    dropout_ratio: float,
    training: bool,
    concat_u: bool = False,
    concat_x: bool = False,
    mul_u_activation_type: str = "none",
    group_norm: bool = False,
    num_heads: int = 1,
    linear_dim: int = -1,
    dropout_seed: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """``dropout(cat([u, attn, act(u) * Norm(attn)]))`` - the input of the output linear
    (generative_recommenders/ops/pytorch/pt_hstu_linear.py:23-82).

    In training the dropout mask is generated inside the kernel (counter-based Philox keyed by
    ``dropout_seed``, a one-element int64 tensor on the device; drawn from torch's CUDA generator when
    not given) and regenerated by the backward, like the reference's GPU path
    (ops/triton/triton_hstu_linear.py:365-492); the mask bits are this library's own.  The
    group-norm variant applies ``torch.nn.functional.dropout`` afterwards."""
    if mul_u_activation_type not in _ACT:
        raise ValueError("mul_u_activation_type must be one of none / sigmoid / silu")
    if group_norm and concat_u != concat_x:
        # the reference's group-norm branch only concatenates when both flags are set (:52-54)
        concat_u = concat_x = False
    act = 0 if group_norm else _ACT[mul_u_activation_type]
    if linear_dim <= 0:
        linear_dim = attn.shape[1] // num_heads
    drop = training and dropout_ratio > 0.0
    fused_drop = drop and not group_norm and dropout_ratio < 1.0
    if fused_drop and dropout_seed is None:
        dropout_seed = _draw_dropout_seed(attn.device)
    y = _NormMulFunction.apply(attn, u, norm_weight, norm_bias, float(norm_eps), int(num_heads), int(linear_dim),
                               bool(concat_u), bool(concat_x), act, bool(group_norm),
                               float(dropout_ratio) if fused_drop else 0.0, dropout_seed if fused_drop else None)
    if drop and not fused_drop:
        y = torch.nn.functional.dropout(y, p=dropout_ratio, training=True)
    return y


def hstu_compute_output(
    attn: torch.Tensor,
    u: torch.Tensor,
    x: torch.Tensor,
    norm_weight: torch.Tensor,
    norm_bias: torch.Tensor,
    norm_eps: float,
    output_weight: torch.Tensor,
    num_heads: int,
    linear_dim: int,
    dropout_ratio: float,
    training: bool,
    concat_u: bool,
    concat_x: bool,
    mul_u_activation_type: str,
    group_norm: bool,
    recompute_y_in_backward: bool,
    kernel: HammerKernel = HammerKernel.CUDA,
) -> torch.Tensor:
    """``x + dropout(cat([u, attn, act(u) * Norm(attn)])) @ W_out``
    (generative_recommenders/ops/hstu_compute.py:107-214,
    generative_recommenders/ops/pytorch/pt_hstu_linear.py:85-120).
    With ``recompute_y_in_backward`` the stage is one autograd node that does not keep the
    concatenated activation (see ``_OutputStageFunction``)."""
    _require_cuda_backend(kernel)
    require_cuda(attn, u, x, norm_weight, norm_bias, output_weight)
    if recompute_y_in_backward and torch.is_grad_enabled() and mul_u_activation_type in _ACT and attn.shape[0] > 0:
        g_ = bool(group_norm)
        cu, cx = bool(concat_u), bool(concat_x)
        if g_ and cu != cx:
            cu = cx = False
        drop = training and dropout_ratio > 0.0
        if not (drop and g_):   # the group-norm variant draws its mask with torch's dropout: kept on the plain path
            seed = _draw_dropout_seed(attn.device) if (drop and dropout_ratio < 1.0) else None
            ld = linear_dim if linear_dim > 0 else attn.shape[1] // num_heads
            return _OutputStageFunction.apply(attn, u, x, norm_weight, norm_bias, output_weight, float(norm_eps),
                                              int(num_heads), int(ld), cu, cx, 0 if g_ else _ACT[mul_u_activation_type],
                                              g_, float(dropout_ratio) if seed is not None else 0.0, seed)
    y = hstu_norm_mul_dropout(attn, u, norm_weight, norm_bias, norm_eps, dropout_ratio, training, concat_u, concat_x,
                              mul_u_activation_type, group_norm, num_heads, linear_dim)
    return addmm(x, y, output_weight.to(x.dtype), kernel)


def hstu_preprocess_and_attention(
    x: torch.Tensor,
    norm_weight: torch.Tensor,
    norm_bias: torch.Tensor,
    norm_eps: float,
    num_heads: int,
    attn_dim: int,
    hidden_dim: int,
    uvqk_weight: torch.Tensor,
    uvqk_bias: torch.Tensor,
    max_seq_len: int,
    seq_offsets: torch.Tensor,
    attn_alpha: float,
    causal: bool,
    num_targets: Optional[torch.Tensor],
    max_attn_len: int,
    contextual_seq_len: int,
    recompute_uvqk_in_backward: bool,
    recompute_normed_x_in_backward: bool,
    sort_by_length: bool,
    prefill: bool = False,
    kernel: HammerKernel = HammerKernel.CUDA,
    enable_tma: Optional[bool] = None,
    bias_by_distance: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """uqvk stage followed by the attention; returns ``(u, attn_output [L, H*dv], k, v)``
    (generative_recommenders/ops/hstu_compute.py:217-335; like the reference's composite the
    attention runs with dropout off, :327-328)."""
    _require_cuda_backend(kernel)
    torch._assert(max_seq_len > 0, "max_seq_len must be larger than 0")
    torch._assert(x.dim() == 2, "x must be 2-D")
    torch._assert(x.shape[1] == uvqk_weight.shape[0], "x.shape[1] must equal uvqk_weight.shape[0]")
    torch._assert(
        uvqk_weight.shape[1] == 2 * num_heads * (hidden_dim + attn_dim),
        "uvqk_weight.shape[1] must equal 2 * num_heads * (hidden_dim + attn_dim)",
    )
    torch._assert(causal is True, "only causal attention is supported.")
    hv = hidden_dim * num_heads
    if (_FUSED_UQVK and x.is_cuda and _fused_uqvk_supported(x, uvqk_weight, hv)
            and attn_dim == hidden_dim and attn_dim in (64, 128)):
        # one autograd node for the stage and the attention (see _FusedPreprocessAttentionFunction)
        from .hstu_attention import _i32
        require_cuda(x, norm_weight, norm_bias, uvqk_weight, uvqk_bias, seq_offsets, num_targets, bias_by_distance)
        offs = _i32(seq_offsets)
        nt = _i32(num_targets)
        if nt is not None and nt.numel() != offs.numel() - 1:
            raise RuntimeError("num_targets must have one entry per sequence")
        rab = None if bias_by_distance is None else bias_by_distance.to(torch.float32).reshape(-1).contiguous()
        u, attn, k, v = _FusedPreprocessAttentionFunction.apply(
            x, norm_weight, norm_bias, float(norm_eps), uvqk_weight, uvqk_bias, num_heads, attn_dim, hidden_dim,
            offs, nt, rab, int(max_seq_len), float(attn_alpha), int(max_attn_len), int(contextual_seq_len),
            torch.is_grad_enabled(), bool(recompute_uvqk_in_backward))
        return u, attn.view(-1, hidden_dim * num_heads), k, v
    u, q, k, v = hstu_compute_uqvk(
        x=x, norm_weight=norm_weight, norm_bias=norm_bias, norm_eps=norm_eps, num_heads=num_heads,
        attn_dim=attn_dim, hidden_dim=hidden_dim, uvqk_weight=uvqk_weight, uvqk_bias=uvqk_bias, kernel=kernel,
    )
    attn_output = hstu_mha(
        max_seq_len=max_seq_len, alpha=attn_alpha, q=q, k=k, v=v, seq_offsets=seq_offsets, causal=causal,
        dropout_pr=0.0, training=False, num_targets=num_targets, max_attn_len=max_attn_len,
        contextual_seq_len=contextual_seq_len, sort_by_length=sort_by_length, kernel=kernel,
        bias_by_distance=bias_by_distance,
    ).view(-1, hidden_dim * num_heads)
    return u, attn_output, k, v
