"""The registered operators (torch.ops.b200_hstu.*) on the device: same bits as the eager op,
gradients through the registered autograd formula, PyTorch's own operator checks (schema, fake
implementation against the real one, autograd registration), and tracing without a graph break."""

import pytest
import torch

import generative_recommenders_b200 as G
from generative_recommenders_b200 import torch_ops
from generative_recommenders_b200 import workloads as W

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(bias):
    g = torch.Generator().manual_seed(4)
    lengths = torch.tensor([130, 300, 17, 257])
    offs = W._offsets(lengths).to(torch.int32).to(DEV)
    nt = torch.tensor([3, 20, 1, 9], dtype=torch.int32, device=DEV)
    L = int(lengths.sum())
    q, k, v, do = ((torch.randn(L, 2, 128, generator=g) * 0.6).bfloat16().to(DEV) for _ in range(4))
    b = (torch.randn(320, generator=g) * 0.3).to(DEV) if bias else None
    return q, k, v, do, offs, nt, b


@pytest.mark.parametrize("bias", [False, True])
def test_registered_op_matches_eager_op(bias):
    q, k, v, do, offs, nt, b = _case(bias)
    res = []
    for fn in ("eager", "op"):
        qd, kd, vd = (t.clone().requires_grad_(True) for t in (q, k, v))
        bd = None if b is None else b.clone().requires_grad_(True)
        if fn == "eager":
            out = G.hstu_mha(320, 0.09, qd, kd, vd, offs, num_targets=nt, max_attn_len=100, contextual_seq_len=2,
                             bias_by_distance=bd)
        else:
            out = torch_ops.hstu_mha_op(320, 0.09, qd, kd, vd, offs, nt, 100, 2, 0, None, bd)
        out.backward(do)
        res.append((out.detach(), qd.grad, kd.grad, vd.grad, None if bd is None else bd.grad))
    for a, c in zip(res[0][:4], res[1][:4]):
        assert torch.equal(a, c)
    if bias:   # summed with atomics: equal up to the order of the additions
        torch.testing.assert_close(res[0][4], res[1][4], rtol=1e-4, atol=1e-6)


def test_opcheck():
    q, k, v, do, offs, nt, b = _case(True)
    args = (q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True), offs, nt, None, b, 320, 0.09, 100, 2, 0)
    torch.library.opcheck(torch.ops.b200_hstu.attn_fwd.default, args,
                          test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))
    torch.library.opcheck(torch.ops.b200_hstu.attn_bwd.default, (do, q.detach(), k.detach(), v.detach(), offs, nt, None, b,
                                                                 320, 0.09, 100, 2, 0),
                          test_utils=("test_schema", "test_faketensor"))


def test_traces_without_a_graph_break():
    q, k, v, do, offs, nt, b = _case(False)

    def f(q_, k_, v_):
        return torch_ops.hstu_mha_op(320, 0.09, q_, k_, v_, offs, nt, 100, 2) * 2.0

    compiled = torch.compile(f, backend="eager", fullgraph=True)
    assert torch.equal(compiled(q, k, v), f(q, k, v))
