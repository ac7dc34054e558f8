"""The forward entry point that brings its own scratch (for callers that cannot allocate device
memory) against the regular entry point, through the C ABI.

Collected last on purpose (file name): a run that stops at the first failure has then already
run every other test.  Works alone in a fresh process and after the rest of the suite: the
built-in scratch is rewritten by every call, so earlier users of the library leave nothing behind
that matters."""

import ctypes

import pytest
import torch

from generative_recommenders_b200 import _cabi
from generative_recommenders_b200 import workloads as W
from generative_recommenders_b200.hstu_attention import _fill_common
from oracle import hstu_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 1e-2  # the bf16 tolerance of the attention tests


def _args(q, k, v, out, offs, nt, N, alpha, bias=None):
    a = _cabi.AttnArgs()
    _fill_common(a, q, k, v, offs, nt, None, N, alpha, 0, 0, 0, bias)
    a.impl = _cabi.IMPL_AUTO
    a.out = out.data_ptr()
    a.o_row_stride, a.o_head_stride = out.stride(0), out.stride(1)
    return a


def _case(seed, lengths, targets):
    g = torch.Generator().manual_seed(seed)
    lengths = torch.tensor(lengths)
    offs = W._offsets(lengths)
    L, H, d = int(offs[-1]), 2, 128
    q = (torch.randn(L, H, d, generator=g) * 0.5).bfloat16().to(DEV)
    k = (torch.randn(L, H, d, generator=g) * 0.5).bfloat16().to(DEV)
    v = (torch.randn(L, H, d, generator=g) * 0.5).bfloat16().to(DEV)
    return q, k, v, offs.to(torch.int32).to(DEV), torch.tensor(targets, dtype=torch.int32).to(DEV)


def test_static_scratch_forward_matches_regular_forward_twice():
    lib = _cabi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.b200_hstu_attn_fwd_static_scratch_max_bytes() == 1 << 20
    # two different batches, back to back on one stream: the second call reuses the scratch that
    # still holds the first call's (longer) work list
    for seed, lengths, targets in [(1, [300, 77, 513, 128, 1], [9, 3, 20, 5, 0]), (2, [640, 200], [31, 2])]:
        q, k, v, offs, nt = _case(seed, lengths, targets)
        N, alpha = 700, 1.0 / 128
        # regular entry point, scratch from torch
        ref_out = torch.empty_like(v)
        a = _args(q, k, v, ref_out, offs, nt, N, alpha)
        n = lib.b200_hstu_attn_workspace_bytes(a, 0)
        ws = torch.empty(max(int(n), 1), dtype=torch.uint8, device=DEV)
        a.workspace, a.workspace_bytes = ws.data_ptr(), n
        _cabi.check(lib.b200_hstu_attn_fwd(a, stream), "b200_hstu_attn_fwd")
        # the entry point under test: no workspace passed at all
        out = torch.full_like(v, float("nan"))
        b = _args(q, k, v, out, offs, nt, N, alpha)
        _cabi.check(lib.b200_hstu_attn_fwd_static_scratch(b, stream), "b200_hstu_attn_fwd_static_scratch")
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all()
        assert O.rel_l2(out, ref_out) < TOL
        # and both agree with the oracle
        oracle = O.hstu_mha(N, alpha, q.float().cpu(), k.float().cpu(), v.float().cpu(), offs.cpu().long(),
                            num_targets=nt.cpu().long())
        assert O.rel_l2(out, oracle) < TOL


def test_static_scratch_forward_with_relative_bias():
    """With a relative bias the built-in array holds the signed-distance table in front of the work
    list.  A call with a bias, then one without, then one with another bias, back to back: every
    call rebuilds what it reads, so each must match the regular entry point bit for bit."""
    lib = _cabi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(5)
    N, alpha = 520, 1.0 / 128
    for seed, lengths, targets, with_bias in [(7, [300, 77, 513], [9, 3, 20], True), (8, [450, 129], [4, 0], False),
                                              (9, [64, 520], [1, 30], True)]:
        q, k, v, offs, nt = _case(seed, lengths, targets)
        bias = (torch.randn(N, generator=g) * 0.3).to(DEV) if with_bias else None
        ref_out = torch.empty_like(v)
        a = _args(q, k, v, ref_out, offs, nt, N, alpha, bias)
        n = lib.b200_hstu_attn_workspace_bytes(a, 0)
        ws = torch.empty(max(int(n), 1), dtype=torch.uint8, device=DEV)
        a.workspace, a.workspace_bytes = ws.data_ptr(), n
        _cabi.check(lib.b200_hstu_attn_fwd(a, stream), "b200_hstu_attn_fwd")
        out = torch.full_like(v, float("nan"))
        b = _args(q, k, v, out, offs, nt, N, alpha, bias)
        _cabi.check(lib.b200_hstu_attn_fwd_static_scratch(b, stream), "b200_hstu_attn_fwd_static_scratch")
        torch.cuda.synchronize()
        assert torch.equal(out, ref_out)
        rb = None
        if with_bias:
            i = torch.arange(N)
            rb = bias.cpu()[(i.view(N, 1) - i.view(1, N)).abs()]
        oracle = O.hstu_mha(N, alpha, q.float().cpu(), k.float().cpu(), v.float().cpu(), offs.cpu().long(),
                            num_targets=nt.cpu().long(), rel_bias=rb)
        assert O.rel_l2(out, oracle) < TOL


def test_static_scratch_rejects_batches_beyond_its_size():
    lib = _cabi.lib()
    q, k, v, offs, nt = _case(3, [64], [1])
    out = torch.empty_like(v)
    a = _args(q, k, v, out, offs, nt, 64, 0.1)
    a.total_L = 5_000_000  # would need a work list of ~1.25 MiB; rejected on the host, nothing is launched
    st = lib.b200_hstu_attn_fwd_static_scratch(a, torch.cuda.current_stream().cuda_stream)
    assert st == -3
    assert b"built-in buffer" in lib.b200_hstu_last_error()
    torch.cuda.synchronize()
