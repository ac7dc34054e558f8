"""Host-side plumbing of the drop-in boundary, no GPU needed: the registered operators' real and
fake implementations take the same arguments (what the reference pins for its own operators in
ops/tests/fake_signature_test.py:49-162) and produce the same shapes, and ``install()`` rebinds
the reference's entry points for ``HammerKernel.CUDA`` only."""

import inspect
import sys
import types
from enum import Enum

import torch

import generative_recommenders_b200 as G
from generative_recommenders_b200 import integration, torch_ops


def _params(fn):
    fn = getattr(fn, "_init_fn", fn)   # a CustomOpDef keeps the Python function it was made from
    return list(inspect.signature(fn).parameters)


def test_real_and_fake_implementations_have_the_same_signature():
    assert _params(torch_ops.attn_fwd) == _params(torch_ops.attn_fwd_fake)
    assert _params(torch_ops.attn_bwd) == _params(torch_ops.attn_bwd_fake)
    # and the schema the dispatcher holds names the same arguments in the same order
    fwd_schema = [a.name for a in torch.ops.b200_hstu.attn_fwd.default._schema.arguments]
    bwd_schema = [a.name for a in torch.ops.b200_hstu.attn_bwd.default._schema.arguments]
    assert fwd_schema == _params(torch_ops.attn_fwd_fake)
    assert bwd_schema == _params(torch_ops.attn_bwd_fake)


def test_fake_implementations_give_the_output_shapes():
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        q = torch.empty(100, 4, 128, dtype=torch.bfloat16, device="cuda")
        v = torch.empty(100, 4, 64, dtype=torch.bfloat16, device="cuda")
        offs = torch.empty(5, dtype=torch.int32, device="cuda")
        bias = torch.empty(77, dtype=torch.float32, device="cuda")
        out = torch.ops.b200_hstu.attn_fwd(q, q, v, offs, None, None, bias, 64, 0.1, 0, 0, 0)
        assert out.shape == (100, 4, 64) and out.dtype == torch.bfloat16
        dq, dk, dv, db = torch.ops.b200_hstu.attn_bwd(out, q, q, v, offs, None, None, bias, 64, 0.1, 0, 0, 0)
        assert dq.shape == q.shape and dk.shape == q.shape and dv.shape == v.shape and db.shape == bias.shape
        _, _, _, db0 = torch.ops.b200_hstu.attn_bwd(out, q, q, v, offs, None, None, None, 64, 0.1, 0, 0, 0)
        assert db0.numel() == 0


class _Kernel(Enum):   # stands for the reference's HammerKernel (generative_recommenders/common.py:112-119)
    TRITON = "TRITON"
    PYTORCH = "PYTORCH"
    CUDA = "CUDA"


def _fake_reference(monkeypatch):
    """A module tree shaped like the reference's, with recording stubs."""
    calls = []
    pkg = types.ModuleType("fake_gr")
    ops = types.ModuleType("fake_gr.ops")
    att = types.ModuleType("fake_gr.ops.hstu_attention")
    comp = types.ModuleType("fake_gr.ops.hstu_compute")
    mods = types.ModuleType("fake_gr.modules")
    stu = types.ModuleType("fake_gr.modules.stu")

    def hstu_mha(max_seq_len, alpha, q, k, v, seq_offsets, causal=True, dropout_pr=0.0, training=True,
                 num_targets=None, attn_scale=None, max_attn_len=0, contextual_seq_len=0, min_full_attn_seq_len=0,
                 sort_by_length=False, kernel=_Kernel.PYTORCH, enable_tma=False):
        calls.append(("theirs.hstu_mha", kernel))
        return "theirs"

    def hstu_compute_uqvk(x, norm_weight, norm_bias, norm_eps, num_heads, attn_dim, hidden_dim, uvqk_weight,
                          uvqk_bias, kernel=_Kernel.PYTORCH):
        calls.append(("theirs.uqvk", kernel))
        return "theirs"

    att.hstu_mha = hstu_mha
    comp.hstu_compute_uqvk = hstu_compute_uqvk
    stu.hstu_compute_uqvk = hstu_compute_uqvk   # ``from ...ops.hstu_compute import hstu_compute_uqvk``
    for m in (pkg, ops, att, comp, mods, stu):
        monkeypatch.setitem(sys.modules, m.__name__, m)
    return calls, att, comp, stu


def test_install_rebinds_for_the_cuda_backend_only(monkeypatch):
    calls, att, comp, stu = _fake_reference(monkeypatch)
    ours = []
    monkeypatch.setattr(G, "hstu_mha", lambda *a, **kw: ours.append(("ours.hstu_mha", kw.get("kernel"))) or "ours")
    monkeypatch.setattr(G, "hstu_compute_uqvk", lambda *a, **kw: ours.append(("ours.uqvk", a[-1] if a else None)) or "ours")
    original = att.hstu_mha
    try:
        n = integration.install("fake_gr")
        assert n == 3                                    # two entry points + the name stu.py imported
        assert att.hstu_mha is not original and stu.hstu_compute_uqvk is comp.hstu_compute_uqvk
        assert att.hstu_mha(8, 1.0, None, None, None, None, kernel=_Kernel.TRITON) == "theirs"
        assert att.hstu_mha(8, 1.0, None, None, None, None) == "theirs"          # the default backend stays theirs
        assert att.hstu_mha(8, 1.0, None, None, None, None, kernel=_Kernel.CUDA) == "ours"
        assert ours[-1] == ("ours.hstu_mha", G.HammerKernel.CUDA)                 # translated to this library's enum
        # positional kernel argument (10th of hstu_compute_uqvk)
        assert stu.hstu_compute_uqvk(0, 1, 2, 3, 4, 5, 6, 7, 8, _Kernel.CUDA) == "ours"
        assert ours[-1] == ("ours.uqvk", G.HammerKernel.CUDA)
        assert stu.hstu_compute_uqvk(0, 1, 2, 3, 4, 5, 6, 7, 8, _Kernel.PYTORCH) == "theirs"
        assert integration.install("fake_gr") == 3       # idempotent
    finally:
        integration.uninstall()
    assert att.hstu_mha is original and stu.hstu_compute_uqvk is comp.hstu_compute_uqvk
    assert [c[0] for c in calls] == ["theirs.hstu_mha", "theirs.hstu_mha", "theirs.uqvk"]
