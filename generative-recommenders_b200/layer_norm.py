"""``layer_norm`` with the reference's signature (generative_recommenders/ops/layer_norm.py:50-94),
running the warp-per-row sm_100a kernels (fp32 statistics, result cast back to the input dtype as
generative_recommenders/ops/pytorch/pt_layer_norm.py:24-38 does)."""

import torch

from . import _cabi
from .common import HammerKernel, _require_cuda_backend, dtype_code, require_cuda, stream_ptr


def _rows2d(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    return x2


class _LayerNormFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        x2 = _rows2d(x)
        rows, D = x2.shape
        weight = weight.to(x.dtype).contiguous()
        bias = bias.to(x.dtype).contiguous()
        y = torch.empty((rows, D), dtype=x.dtype, device=x.device)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        if rows > 0:
            with torch.cuda.device(x.device):
                _cabi.check(
                    _cabi.lib().b200_hstu_layer_norm_fwd(
                        x2.data_ptr(), x2.stride(0), weight.data_ptr(), bias.data_ptr(), y.data_ptr(), y.stride(0),
                        mean.data_ptr(), rstd.data_ptr(), rows, D, eps, dtype_code(x), stream_ptr(x.device)),
                    "b200_hstu_layer_norm_fwd")
        ctx.save_for_backward(x2, weight, mean, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, mean, rstd = ctx.saved_tensors
        rows, D = x2.shape
        dy2 = _rows2d(dy)
        dx = torch.empty((rows, D), dtype=x2.dtype, device=x2.device)
        dw = torch.empty(D, dtype=x2.dtype, device=x2.device)
        db = torch.empty(D, dtype=x2.dtype, device=x2.device)
        nbytes = _cabi.lib().b200_hstu_layer_norm_bwd_workspace_bytes(D)
        partial = torch.empty(nbytes, dtype=torch.uint8, device=x2.device)
        with torch.cuda.device(x2.device):
            _cabi.check(
                _cabi.lib().b200_hstu_layer_norm_bwd(
                    dy2.data_ptr(), dy2.stride(0), x2.data_ptr(), x2.stride(0), weight.data_ptr(), mean.data_ptr(),
                    rstd.data_ptr(), dx.data_ptr(), dx.stride(0), dw.data_ptr(), db.data_ptr(), partial.data_ptr(),
                    nbytes, rows, D, dtype_code(x2), stream_ptr(x2.device)),
                "b200_hstu_layer_norm_bwd")
        return dx.view(ctx.shape), dw, db, None


def layer_norm(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor,
    eps: float = 1e-5,
    kernel: HammerKernel = HammerKernel.CUDA,
) -> torch.Tensor:
    _require_cuda_backend(kernel)
    require_cuda(x, weight, bias)
    dtype_code(x)
    return _LayerNormFunction.apply(x, weight, bias, float(eps))
