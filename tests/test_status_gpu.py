"""The bounded waits of the tensor-core kernels as seen from the host: the status words of a
launch's work lists read back through the C ABI, and the wait loop itself made to run out in the one
safe way - a one-warp kernel waiting one millisecond on a barrier nobody arrives at, which then
returns with the site recorded (nothing faults, traps or hangs; the context stays usable)."""

import ctypes

import pytest
import torch

import generative_recommenders_b200 as G
from generative_recommenders_b200 import _cabi, hstu_attention as HA
from generative_recommenders_b200 import workloads as W

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(seed=0):
    g = torch.Generator().manual_seed(seed)
    lengths = torch.tensor([300, 77, 513])
    offs = W._offsets(lengths)
    L = int(offs[-1])
    q, k, v, do = ((torch.randn(L, 2, 128, generator=g) * 0.5).bfloat16().to(DEV) for _ in range(4))
    return q, k, v, do, offs.to(DEV), torch.tensor([9, 3, 20]).to(DEV)


def test_expired_wait_returns_and_records_its_site():
    lib = _cabi.lib()
    status = torch.full((1,), -5, dtype=torch.int32, device=DEV)
    elapsed = torch.zeros(1, dtype=torch.int64, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    _cabi.check(lib.b200_hstu_selftest_bounded_wait(status.data_ptr(), elapsed.data_ptr(), stream), "selftest")
    torch.cuda.synchronize()
    assert int(status.item()) == 777                      # the site id the waiter passed
    assert 1_000_000 <= int(elapsed.item()) < 200_000_000  # gave up after the 1 ms limit, not much later
    # the context is intact: a regular launch right after it runs and reports completion
    q, k, v, do, offs, nt = _inputs()
    out = G.hstu_mha(600, 0.1, q, k, v, offs, num_targets=nt)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()


def test_status_words_of_regular_launches_are_zero():
    """Forward, forward that plans the backward, and backward (own lists and reused lists): every
    status word reads 0, through the explicit C-ABI call and through the ops' own check
    (B200_HSTU_CHECK_STATUS / set_status_check)."""
    q, k, v, do, offs, nt = _inputs(1)
    offs32, nt32 = offs.to(torch.int32), nt.to(torch.int32)
    args = (600, 1.0 / 128, q, k, v, offs32, nt32, None, 100, 2, 0)
    HA.set_status_check(True)
    try:
        out = HA.hstu_attention_fwd(*args)
        out2, scratch = HA.hstu_attention_fwd(*args, plan_for_backward=True)
        g = [torch.empty_like(t) for t in (q, k, v)]
        HA.hstu_attention_bwd(do, *args, *g)
        HA.hstu_attention_bwd(do, *args, *g, planned_scratch=scratch)
        qd, kd, vd = (t.clone().requires_grad_(True) for t in (q, k, v))
        G.hstu_mha(600, 1.0 / 128, qd, kd, vd, offs, num_targets=nt, max_attn_len=100, contextual_seq_len=2).backward(do)
    finally:
        HA.set_status_check(False)
    torch.cuda.synchronize()
    assert torch.equal(out, out2)
    # the explicit call on a workspace of this test's own
    a = _cabi.AttnArgs()
    HA._fill_common(a, q, k, v, offs32, nt32, None, 600, 1.0 / 128, 100, 2, 0, None)
    o = torch.empty_like(v)
    a.out = o.data_ptr()
    a.o_row_stride, a.o_head_stride = o.stride(0), o.stride(1)
    ws = HA._workspace(a, 0, q.device)
    with torch.cuda.device(q.device):
        _cabi.check(_cabi.lib().b200_hstu_attn_fwd(a, torch.cuda.current_stream().cuda_stream), "fwd")
    assert ws is not None
    assert HA.attention_status(a, 0, q.device) == [0, 0, 0]
    assert torch.equal(o, out)


def test_status_check_reports_a_recorded_site():
    """A status word that is not zero (written here by the test into the list header, where an
    expired wait would put it) turns into an error."""
    q, k, v, do, offs, nt = _inputs(2)
    offs32, nt32 = offs.to(torch.int32), nt.to(torch.int32)
    a = _cabi.AttnArgs()
    HA._fill_common(a, q, k, v, offs32, nt32, None, 600, 1.0 / 128, 0, 0, 0, None)
    o = torch.empty_like(v)
    a.out = o.data_ptr()
    a.o_row_stride, a.o_head_stride = o.stride(0), o.stride(1)
    ws = HA._workspace(a, 0, q.device)
    with torch.cuda.device(q.device):
        _cabi.check(_cabi.lib().b200_hstu_attn_fwd(a, torch.cuda.current_stream().cuda_stream), "fwd")
    torch.cuda.synchronize()
    ws.view(torch.int32)[1] = 301          # PlanHeader.status of the forward's list
    assert HA.attention_status(a, 0, q.device) == [301, 0, 0]
    with pytest.raises(RuntimeError, match="bounded wait"):
        HA._raise_on_status(a, 0, q.device, "test")
