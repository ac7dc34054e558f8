"""``concat_2D_jagged`` / ``split_2D_jagged`` with the reference's signatures
(generative_recommenders/ops/jagged_tensors.py:55-162), running one sm_100a row-mover kernel
(csrc/jagged.cu).  Each op is the other's backward.

As in the reference's kernels, sequences are taken whole: a side given by offsets contributes
``offsets[b + 1] - offsets[b]`` rows for sequence ``b`` (the PyTorch restatement in the reference
truncates at ``max_len_*``, generative_recommenders/ops/pytorch/pt_jagged_tensors.py:41-53, which
never triggers for consistent arguments).
"""

from typing import Optional, Tuple

import torch

from . import _cabi
from .common import HammerKernel, _require_cuda_backend, require_cuda, stream_ptr


def _offsets_arg(off: Optional[torch.Tensor], device) -> Optional[torch.Tensor]:
    if off is None:
        return None
    return off.to(device=device, dtype=torch.int64).contiguous()


def _args(left, right, combined, off_l, off_r, dense_l, dense_r, B, shift=0):
    a = _cabi.JaggedArgs()
    a.left, a.right, a.combined = left.data_ptr(), right.data_ptr(), combined.data_ptr()
    a.offsets_left = off_l.data_ptr() if off_l is not None else None
    a.offsets_right = off_r.data_ptr() if off_r is not None else None
    a.dense_len_left = int(dense_l)
    a.dense_len_right = int(dense_r)
    a.total_rows = combined.shape[0]
    a.row_bytes = combined.shape[1] * combined.element_size()
    a.B = B
    a.right_rows_first = int(shift)
    return a


def _run(split: bool, left, right, combined, off_l, off_r, dense_l, dense_r, B, shift=0) -> None:
    if combined.shape[0] == 0 or combined.shape[1] == 0:
        return
    a = _args(left, right, combined, off_l, off_r, dense_l, dense_r, B, shift)
    fn = _cabi.lib().b200_hstu_split_2d_jagged if split else _cabi.lib().b200_hstu_concat_2d_jagged
    with torch.cuda.device(combined.device):
        _cabi.check(fn(a, stream_ptr(combined.device)),
                    "b200_hstu_split_2d_jagged" if split else "b200_hstu_concat_2d_jagged")


class _Concat2DJagged(torch.autograd.Function):
    @staticmethod
    def forward(ctx, left, right, off_l, off_r, dense_l, dense_r, B, shift=0):
        left = left.contiguous()
        right = right.contiguous()
        out = torch.empty((left.shape[0] + right.shape[0], left.shape[1]), dtype=left.dtype, device=left.device)
        _run(False, left, right, out, off_l, off_r, dense_l, dense_r, B, shift)
        ctx.meta = (off_l, off_r, dense_l, dense_r, B, left.shape[0], right.shape[0], shift)
        return out

    @staticmethod
    def backward(ctx, d_out):
        off_l, off_r, dense_l, dense_r, B, n_l, n_r, shift = ctx.meta
        d_out = d_out.contiguous()
        d_left = torch.empty((n_l, d_out.shape[1]), dtype=d_out.dtype, device=d_out.device)
        d_right = torch.empty((n_r, d_out.shape[1]), dtype=d_out.dtype, device=d_out.device)
        _run(True, d_left, d_right, d_out, off_l, off_r, dense_l, dense_r, B, shift)
        return d_left, d_right, None, None, None, None, None, None


class _Split2DJagged(torch.autograd.Function):
    @staticmethod
    def forward(ctx, values, off_l, off_r, dense_l, dense_r, B, n_l, n_r, shift=0):
        values = values.contiguous()
        left = torch.empty((n_l, values.shape[1]), dtype=values.dtype, device=values.device)
        right = torch.empty((n_r, values.shape[1]), dtype=values.dtype, device=values.device)
        _run(True, left, right, values, off_l, off_r, dense_l, dense_r, B, shift)
        ctx.meta = (off_l, off_r, dense_l, dense_r, B, shift)
        return left, right

    @staticmethod
    def backward(ctx, d_left, d_right):
        off_l, off_r, dense_l, dense_r, B, shift = ctx.meta
        d_left = d_left.contiguous()
        d_right = d_right.contiguous()
        d_values = torch.empty((d_left.shape[0] + d_right.shape[0], d_left.shape[1]), dtype=d_left.dtype,
                               device=d_left.device)
        _run(False, d_left, d_right, d_values, off_l, off_r, dense_l, dense_r, B, shift)
        return d_values, None, None, None, None, None, None, None, None


def concat_2D_jagged(
    max_seq_len: int,
    values_left: torch.Tensor,
    values_right: torch.Tensor,
    max_len_left: Optional[int] = None,
    max_len_right: Optional[int] = None,
    offsets_left: Optional[torch.Tensor] = None,
    offsets_right: Optional[torch.Tensor] = None,
    kernel: HammerKernel = HammerKernel.CUDA,
) -> torch.Tensor:
    """Per sequence, the rows of ``values_left`` followed by the rows of ``values_right``.

    Same arguments and checks as generative_recommenders/ops/jagged_tensors.py:55-108; a side
    without offsets is dense with ``max_len_*`` rows per sequence."""
    _require_cuda_backend(kernel)
    require_cuda(values_left, values_right, offsets_left, offsets_right)
    torch._assert(values_left.dim() == 2, "values_left must be 2D")
    torch._assert(values_right.dim() == 2, "values_right must be 2D")
    torch._assert(
        values_right.shape[1] == values_left.shape[1],
        f"values_left shape[1] must be equal to values_right shape[1] {values_left.shape[1]} vs {values_right.shape[1]}",
    )
    torch._assert(values_left.dtype == values_right.dtype, "values_left and values_right must share a dtype")
    dev = values_left.device
    off_l = _offsets_arg(offsets_left, dev)
    off_r = _offsets_arg(offsets_right, dev)
    if off_l is None:
        assert max_len_left is not None and max_len_left > 0
        B = values_left.shape[0] // max_len_left
    else:
        B = off_l.numel() - 1
    if off_r is None:
        assert max_len_right is not None and max_len_right > 0
        torch._assert(values_right.shape[0] == B * max_len_right or off_l is None,
                      "values_right must hold max_len_right rows per sequence")
        if off_l is None:
            B = values_right.shape[0] // max_len_right
    else:
        torch._assert(off_r.numel() - 1 == B, "offsets_left and offsets_right must describe the same batch")
    return _Concat2DJagged.apply(values_left, values_right, off_l, off_r,
                                 max_len_left if off_l is None else 0,
                                 max_len_right if off_r is None else 0, B)


def split_2D_jagged(
    max_seq_len: int,
    values: torch.Tensor,
    total_len_left: Optional[int] = None,
    total_len_right: Optional[int] = None,
    max_len_left: Optional[int] = None,
    max_len_right: Optional[int] = None,
    offsets_left: Optional[torch.Tensor] = None,
    offsets_right: Optional[torch.Tensor] = None,
    kernel: HammerKernel = HammerKernel.CUDA,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """The inverse of :func:`concat_2D_jagged` (generative_recommenders/ops/jagged_tensors.py:111-162).

    ``total_len_left`` / ``total_len_right`` (rows of the two results) save a device
    synchronisation when a side is given by offsets; without them the last offset is read back."""
    _require_cuda_backend(kernel)
    require_cuda(values, offsets_left, offsets_right)
    torch._assert(values.dim() == 2, "values must be 2D")
    torch._assert(
        offsets_left is not None or offsets_right is not None,
        "offsets_left and offsets_right cannot be None at the same time",
    )
    if offsets_left is None:
        torch._assert(max_len_left is not None, "max_len_left must be provided when offsets_left is None")
    if offsets_right is None:
        torch._assert(max_len_right is not None, "max_len_right must be provided when offsets_right is None")
    if offsets_left is not None and offsets_right is not None:
        torch._assert(
            offsets_left.shape[0] == offsets_right.shape[0],
            "offsets_left shape[0] must be equal to offsets_right shape[0]",
        )
    dev = values.device
    off_l = _offsets_arg(offsets_left, dev)
    off_r = _offsets_arg(offsets_right, dev)
    B = (off_l if off_l is not None else off_r).numel() - 1
    total = values.shape[0]
    if off_l is None:
        n_l = B * int(max_len_left)
    elif total_len_left is not None:
        n_l = int(total_len_left)
    elif off_r is None:
        n_l = total - B * int(max_len_right)
    elif total_len_right is not None:
        n_l = total - int(total_len_right)
    else:
        n_l = int(off_l[-1].item())
    n_r = total - n_l
    return _Split2DJagged.apply(values, off_l, off_r,
                                max_len_left if off_l is None else 0,
                                max_len_right if off_r is None else 0, B, n_l, n_r)


def hstu_split_l2_embeddings(
    max_seq_len: int,
    x: torch.Tensor,
    prefix_offsets: torch.Tensor,
    l2_offsets: torch.Tensor,
    contextual_seq_len: int,
    kernel: HammerKernel = HammerKernel.CUDA,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(prefix_x, l2_x)``: every sequence of ``x`` is ``contextual_seq_len`` rows of the l2 part, then
    the prefix rows, then the rest of the l2 part
    (generative_recommenders/ops/jagged_tensors.py:165-192)."""
    _require_cuda_backend(kernel)
    require_cuda(x, prefix_offsets, l2_offsets)
    torch._assert(x.dim() == 2, "x must be 2D")
    off_l = _offsets_arg(prefix_offsets, x.device)
    off_r = _offsets_arg(l2_offsets, x.device)
    torch._assert(off_l.numel() == off_r.numel(), "prefix_offsets and l2_offsets must describe the same batch")
    n_l = int(off_l[-1].item())
    return _Split2DJagged.apply(x, off_l, off_r, 0, 0, off_l.numel() - 1, n_l, x.shape[0] - n_l,
                                int(contextual_seq_len))


def hstu_concat_l2_embeddings(
    max_prefix_len: int,
    prefix_x: torch.Tensor,
    prefix_offsets: torch.Tensor,
    max_l2_len: int,
    l2_x: torch.Tensor,
    l2_offsets: torch.Tensor,
    contextual_seq_len: int,
    kernel: HammerKernel = HammerKernel.CUDA,
) -> torch.Tensor:
    """The inverse of :func:`hstu_split_l2_embeddings`
    (generative_recommenders/ops/jagged_tensors.py:195-227)."""
    _require_cuda_backend(kernel)
    require_cuda(prefix_x, l2_x, prefix_offsets, l2_offsets)
    torch._assert(prefix_x.dim() == 2 and l2_x.dim() == 2, "prefix_x and l2_x must be 2D")
    torch._assert(prefix_x.shape[1] == l2_x.shape[1] and prefix_x.dtype == l2_x.dtype,
                  "prefix_x and l2_x must have the same width and dtype")
    off_l = _offsets_arg(prefix_offsets, prefix_x.device)
    off_r = _offsets_arg(l2_offsets, prefix_x.device)
    torch._assert(off_l.numel() == off_r.numel(), "prefix_offsets and l2_offsets must describe the same batch")
    return _Concat2DJagged.apply(prefix_x, l2_x, off_l, off_r, 0, 0, off_l.numel() - 1, int(contextual_seq_len))
