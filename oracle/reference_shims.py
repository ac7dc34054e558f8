"""Stand-ins for the two third-party packages the reference's PyTorch path needs.

TEST INFRASTRUCTURE ONLY, and only usable where a checkout of the reference is
present (it is not shipped with this repository).  ``tests/golden/make_golden.py``
uses it to run the *unmodified* reference and store its outputs as fixtures.

The reference pins ``fbgemm_gpu>=1.1.0`` and ``torchrec`` (requirements.txt:2), neither
vendored.  On this path they only move data:

* ``fbgemm::jagged_to_padded_dense(values, offsets, max_lengths, padding_value)`` -
  rows ``offsets[b]..offsets[b+1]`` of ``values`` go to ``out[b, :len]``, truncated at
  ``max_lengths[0]``, the rest filled with ``padding_value``
  (call sites: generative_recommenders/ops/pytorch/pt_hstu_attention.py:97,107,117,155);
* ``fbgemm::dense_to_jagged(dense, offsets, total_L)`` - the inverse gather
  (call site :183);
* ``fbgemm::asynchronous_complete_cumsum(lengths)`` - cumsum with a leading zero
  (call site generative_recommenders/common.py:454).

Parity of these three shims themselves is unpinned (the reference has no test for
them); they are exercised only through the reference's own attention code.
"""

import sys
import types
from typing import List, Optional, Tuple

import torch

_LIBS = []


def _jagged_to_padded_dense(values, offsets, max_lengths, padding_value=0.0):
    off = offsets[0].to(torch.int64)
    N = int(max_lengths[0])
    B = off.numel() - 1
    lens = (off[1:] - off[:-1]).clamp(max=N)
    pos = torch.arange(N, device=values.device).view(1, N)
    valid = pos < lens.view(B, 1)
    src = (off[:-1].view(B, 1) + pos).clamp(max=max(values.shape[0] - 1, 0))
    if values.shape[0] == 0:
        return values.new_full((B, N) + tuple(values.shape[1:]), padding_value)
    gathered = values[src.reshape(-1)].view(B, N, *values.shape[1:])
    mask = valid.view(B, N, *([1] * (values.dim() - 1)))
    return torch.where(mask, gathered, torch.full_like(gathered, padding_value))


def _dense_to_jagged(dense, x_offsets, total_L=None):
    off = x_offsets[0].to(torch.int64)
    B, N = dense.shape[0], dense.shape[1]
    lens = (off[1:] - off[:-1])
    pos = torch.arange(N, device=dense.device).view(1, N)
    valid = pos < lens.view(B, 1)
    out = dense[valid]
    if total_L is not None and out.shape[0] < int(total_L):  # rows beyond N come back as zeros
        full = dense.new_zeros((int(total_L),) + tuple(dense.shape[2:]))
        dst = (off[:-1].view(B, 1) + pos)[valid]
        full = full.index_put((dst,), out)
        out = full
    return out, [off]


def _complete_cumsum(x):
    return torch.cat([x.new_zeros(1), torch.cumsum(x, dim=0)])


def install() -> None:
    """Define the three fbgemm ops (if no real fbgemm_gpu is loaded) and a torchrec stub."""
    if not _LIBS:
        have = hasattr(torch.ops, "fbgemm") and hasattr(torch.ops.fbgemm, "jagged_to_padded_dense")
        try:
            if have:
                torch.ops.fbgemm.jagged_to_padded_dense  # noqa: B018
        except (AttributeError, RuntimeError):
            have = False
        if not have:
            lib = torch.library.Library("fbgemm", "DEF")
            lib.define(
                "jagged_to_padded_dense(Tensor values, Tensor[] offsets, SymInt[] max_lengths, "
                "float padding_value=0.0) -> Tensor"
            )
            lib.define(
                "dense_to_jagged(Tensor dense, Tensor[] x_offsets, SymInt? total_L=None) -> (Tensor, Tensor[])"
            )
            lib.define("asynchronous_complete_cumsum(Tensor t_in) -> Tensor")
            lib.impl("jagged_to_padded_dense", _jagged_to_padded_dense, "CompositeImplicitAutograd")
            lib.impl("dense_to_jagged", _dense_to_jagged, "CompositeImplicitAutograd")
            lib.impl("asynchronous_complete_cumsum", _complete_cumsum, "CompositeImplicitAutograd")
            _LIBS.append(lib)
    if "torchrec" not in sys.modules:
        # generative_recommenders/ops/pytorch/pt_jagged.py:23 imports this name; it is
        # only used by an op outside the restated path.
        tr = types.ModuleType("torchrec")
        trm = types.ModuleType("torchrec.modules")
        trs = types.ModuleType("torchrec.modules.sorted_index_select")

        def maybe_sorted_index_select(x, dim, index):  # pragma: no cover
            return torch.index_select(x, dim, index)

        trs.maybe_sorted_index_select = maybe_sorted_index_select
        tr.modules = trm
        trm.sorted_index_select = trs
        sys.modules["torchrec"] = tr
        sys.modules["torchrec.modules"] = trm
        sys.modules["torchrec.modules.sorted_index_select"] = trs


def import_reference(path: str):
    """Put the reference checkout at ``path`` on ``sys.path`` (after the shims)."""
    install()
    if path not in sys.path:
        sys.path.insert(0, path)
    import generative_recommenders  # noqa: F401

    return generative_recommenders
