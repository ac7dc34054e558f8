"""``addmm`` with the reference's signature (generative_recommenders/ops/mm.py:29-44).

The two dense linears of the HSTU layer are plain library GEMMs: cuBLAS through ``torch.addmm``,
which is also what the reference itself selects on Blackwell
(generative_recommenders/ops/triton/triton_addmm.py:1829-1835)."""

import torch

from .common import HammerKernel, _require_cuda_backend


def addmm(input: torch.Tensor, mat1: torch.Tensor, mat2: torch.Tensor,
          kernel: HammerKernel = HammerKernel.CUDA) -> torch.Tensor:
    _require_cuda_backend(kernel)
    return torch.addmm(input, mat1, mat2)
