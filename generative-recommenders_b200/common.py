"""Types shared by the ops: the backend selector the reference threads through every call."""

from enum import Enum, unique

import torch

from . import _cabi


@unique
class HammerKernel(Enum):
    """Same members as generative_recommenders/common.py:112-119.

    This library implements exactly one backend, ``CUDA`` (hand-written sm_100a kernels).
    The reference leaves ``CUDA`` unhandled in ``hstu_mha`` (it falls through to the PyTorch
    branch, generative_recommenders/ops/hstu_attention.py:191-207); here it is the only value
    that runs, every other member raises so that nothing silently takes a slower path.
    """

    TRITON = "TRITON"
    TLX = "TLX"
    PYTORCH = "PYTORCH"
    CUDA = "CUDA"
    TRITON_CC = "TRITON_CC"
    CUTEDSL = "CUTEDSL"


def _require_cuda_backend(kernel) -> None:
    name = getattr(kernel, "name", kernel)
    if name != "CUDA":
        raise NotImplementedError(
            "generative-recommenders_b200 only implements HammerKernel.CUDA (got %r); "
            "other backends are not part of this library" % (kernel,)
        )


_DTYPES = {torch.float32: _cabi.F32, torch.bfloat16: _cabi.BF16, torch.float16: _cabi.F16}


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError("unsupported dtype %s (float32, bfloat16 and float16 are)" % t.dtype)


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("tensors must live on a CUDA device; this library has no CPU path")


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def last_dim_contiguous(t: torch.Tensor) -> torch.Tensor:
    """Same rule as the reference's switch_to_contiguous_if_needed
    (generative_recommenders/common.py:262-269): only a non-unit last stride forces a copy."""
    if t.dim() > 0 and t.stride(-1) != 1 and t.shape[-1] > 1:
        return t.contiguous()
    return t
