"""Parity of the CUDA attention (through the C ABI) with the oracle and the reference fixtures.

Tolerances (tests/parity_metrics.py): fp32 kernels against fp32 fixtures 2e-4 relative L2 (accumulation
order only); bf16 / fp16 kernels against the fp32 oracle on the same (already rounded) inputs:
relative L2 <= 1e-2 for the output and every gradient.  Next to the global norm every comparison
bounds the worst single sequence (1e-2 / 5e-4) and the largest element-wise error relative to the
largest reference element (1e-2 / 5e-4)."""

import pytest
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

import generative_recommenders_b200 as G
from generative_recommenders_b200 import workloads as W
from oracle import hstu_oracle as O
import parity_metrics as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BF16_TOL = P.HALF_TOL
FP32_TOL = P.F32_TOL


@pytest.fixture(autouse=True)
def _reset_impl():
    G.set_attention_impl("auto")
    yield
    G.set_attention_impl("auto")


def _run(q, k, v, offs, N, alpha, nt=None, W_=0, ctx=0, F=0, dout=None, scale=None, bias=None, bias_grad=False):
    """Output and (dq, dk, dv[, dbias]) of the CUDA path."""
    qd = q.to(DEV).requires_grad_(dout is not None)
    kd = k.to(DEV).requires_grad_(dout is not None)
    vd = v.to(DEV).requires_grad_(dout is not None)
    bd = None if bias is None else bias.to(DEV).requires_grad_(bias_grad)
    out = G.hstu_mha(N, alpha, qd, kd, vd, offs.to(DEV), num_targets=None if nt is None else nt.to(DEV),
                     max_attn_len=W_, contextual_seq_len=ctx, min_full_attn_seq_len=F,
                     attn_scale=None if scale is None else scale.to(DEV), bias_by_distance=bd)
    if dout is None:
        return out.cpu(), None
    out.backward(dout.to(DEV))
    torch.cuda.synchronize()
    grads = (qd.grad.cpu(), kd.grad.cpu(), vd.grad.cpu())
    if bias_grad:
        grads = grads + (bd.grad.cpu(),)
    return out.detach().cpu(), grads


def _oracle(q, k, v, offs, N, alpha, nt=None, W_=0, ctx=0, F=0, dout=None, scale=None, bias=None, bias_grad=False):
    q32 = q.float().clone().requires_grad_(dout is not None)
    k32 = k.float().clone().requires_grad_(dout is not None)
    v32 = v.float().clone().requires_grad_(dout is not None)
    rb = b32 = None
    if bias is not None:
        b32 = bias.float().clone().requires_grad_(bias_grad)
        i = torch.arange(N).view(N, 1)
        j = torch.arange(N).view(1, N)
        d = (i - j).abs()
        rb = torch.where(d < bias.numel(), b32[d.clamp(max=bias.numel() - 1)], torch.zeros(()))
    out = O.hstu_mha(N, alpha, q32, k32, v32, offs, num_targets=nt, max_attn_len=W_, contextual_seq_len=ctx,
                     min_full_attn_seq_len=F, attn_scale=scale, rel_bias=rb)
    if dout is None:
        return out, None
    out.backward(dout.float())
    grads = (q32.grad, k32.grad, v32.grad)
    if bias_grad:
        grads = grads + (b32.grad,)
    return out.detach(), grads


def _check_all(name, out, grads, ref, rgrads, offs, f32=False):
    """Output and every gradient: global, per-sequence and element-wise bounds."""
    chk = P.check_f32 if f32 else P.check
    chk((name, "out"), out, ref, offs)
    if grads is not None:
        for g, r, nm in zip(grads, rgrads, ("dq", "dk", "dv")):
            chk((name, nm), g, r, offs)


@pytest.mark.parametrize("impl", ["simt"])
def test_fp32_golden_fixtures(golden, impl):
    G.set_attention_impl(impl)
    for name, fx in golden("attention.pt").items():
        p = fx["params"]
        out, grads = _run(fx["q"], fx["k"], fx["v"], fx["seq_offsets"], p["N"], p["alpha"], fx["num_targets"],
                          p["W"], p["ctx"], p["F"], fx.get("dout"))
        rgrads = (fx["dq"], fx["dk"], fx["dv"]) if grads is not None else None
        _check_all(("golden", name), out, grads, fx["out"], rgrads, fx["seq_offsets"], f32=True)


def _random_case(seed, B, lo, hi, N, H, d, dtype, targets=0, ctx=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    lengths = torch.randint(lo, hi + 1, (B,), generator=g)
    nt = None
    if targets > 0:
        nt = torch.randint(1, targets + 1, (B,), generator=g)
        lengths = torch.clamp(lengths + nt + ctx, max=N)
        nt = torch.minimum(nt, torch.clamp(lengths - ctx - 1, min=0))
    elif ctx > 0:
        lengths = torch.clamp(lengths + ctx, max=N)
    offs = W._offsets(lengths)
    L = int(offs[-1])
    q = (torch.randn(L, H, d, generator=g) * std).to(dtype)
    k = (torch.randn(L, H, d, generator=g) * std).to(dtype)
    v = (torch.randn(L, H, d, generator=g) * std).to(dtype)
    dout = torch.randn(L, H, d, generator=g).to(dtype)
    return q, k, v, offs, nt, dout


CASES = [
    # B, lo, hi, N, H, d, targets, ctx, W, F
    (6, 1, 300, 300, 2, 128, 0, 0, 0, 0),
    (6, 1, 300, 320, 2, 128, 20, 0, 0, 0),
    (5, 100, 400, 420, 1, 128, 0, 7, 0, 0),
    (5, 100, 500, 520, 2, 128, 30, 5, 90, 0),
    (4, 200, 600, 640, 1, 128, 12, 0, 150, 0),
    (4, 1, 260, 270, 3, 64, 9, 3, 0, 0),
    (4, 120, 300, 310, 2, 64, 0, 0, 64, 0),
    (4, 120, 300, 320, 2, 128, 10, 4, 70, 33),
    # contextual prefix longer than one 128-row tile (its rows sit in several query tiles), alone,
    # with targets, and with a window / full-attention tail
    (4, 150, 500, 640, 2, 128, 0, 130, 0, 0),
    (4, 150, 500, 700, 1, 128, 25, 260, 100, 0),
    (3, 100, 400, 600, 2, 64, 12, 130, 16, 40),
]


@pytest.mark.parametrize("impl", ["tcgen05", "simt"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", CASES)
def test_half_precision_forward_matches_oracle(impl, dtype, case):
    B, lo, hi, N, H, d, targets, ctx, Wn, F = case
    if impl == "simt" and dtype == torch.float16 and d == 128:
        pytest.skip("covered by bf16")
    G.set_attention_impl(impl)
    q, k, v, offs, nt, _ = _random_case(hash(case) % 10000, B, lo, hi, N, H, d, dtype, targets, ctx, std=0.7)
    alpha = 1.0 / d ** 0.5
    out, _ = _run(q, k, v, offs, N, alpha, nt, Wn, ctx, F)
    ref, _ = _oracle(q, k, v, offs, N, alpha, nt, Wn, ctx, F)
    assert torch.isfinite(out.float()).all()
    _check_all(("fwd", impl, str(dtype), case), out, None, ref, None, offs)


@pytest.mark.parametrize("impl", ["tcgen05", "simt"])
@pytest.mark.parametrize("case", CASES)
def test_bf16_backward_matches_oracle(impl, case):
    B, lo, hi, N, H, d, targets, ctx, Wn, F = case
    G.set_attention_impl(impl)
    q, k, v, offs, nt, dout = _random_case(hash(case) % 10000 + 1, B, lo, hi, N, H, d, torch.bfloat16, targets, ctx,
                                           std=0.7)
    alpha = 1.0 / d ** 0.5
    out, grads = _run(q, k, v, offs, N, alpha, nt, Wn, ctx, F, dout)
    ref, rgrads = _oracle(q, k, v, offs, N, alpha, nt, Wn, ctx, F, dout)
    _check_all(("bwd", impl, case), out, grads, ref, rgrads, offs)


@pytest.mark.parametrize("impl", ["tcgen05", "simt"])
def test_edge_lengths(impl):
    """Empty sequences, single tokens and lengths around the 128-row tile edge, forward and
    backward; the one- and two-token sequences are bounded on their own (per-sequence error)."""
    G.set_attention_impl(impl)
    lengths = torch.tensor([0, 1, 127, 128, 129, 0, 255, 256, 257, 2, 0])
    offs = W._offsets(lengths)
    g = torch.Generator().manual_seed(11)
    L, H, d = int(offs[-1]), 2, 128
    q = torch.randn(L, H, d, generator=g).bfloat16()
    k = torch.randn(L, H, d, generator=g).bfloat16()
    v = torch.randn(L, H, d, generator=g).bfloat16()
    dout = torch.randn(L, H, d, generator=g).bfloat16()
    out, grads = _run(q, k, v, offs, 300, 0.1, dout=dout)
    ref, rgrads = _oracle(q, k, v, offs, 300, 0.1, dout=dout)
    _check_all(("edge", impl), out, grads, ref, rgrads, offs)


def test_empty_batch_and_zero_tokens():
    q = torch.zeros(0, 2, 128, dtype=torch.bfloat16, device=DEV)
    offs = torch.zeros(4, dtype=torch.int64, device=DEV)
    out = G.hstu_mha(16, 0.1, q, q, q, offs)
    assert out.shape == (0, 2, 128)


def test_writes_stay_inside_the_output_rows():
    """The output buffer is a slice of a NaN-poisoned tensor: nothing outside may be written."""
    G.set_attention_impl("tcgen05")
    q, k, v, offs, nt, _ = _random_case(5, 5, 50, 200, 256, 2, 128, torch.bfloat16, 10, 0)
    out, _ = _run(q, k, v, offs, 256, 0.09, nt)
    ref, _ = _oracle(q, k, v, offs, 256, 0.09, nt)
    P.check("poisoned", out, ref, offs)
    # run twice: bit-identical (forward has a single owner per output element)
    out2, _ = _run(q, k, v, offs, 256, 0.09, nt)
    assert torch.equal(out, out2)


def test_non_contiguous_qkv_views():
    """q, k, v as column slices of one [L, 4*H*d] buffer, the layout hstu_compute_uqvk returns."""
    g = torch.Generator().manual_seed(2)
    H, d = 2, 128
    lengths = torch.tensor([70, 190, 33])
    offs = W._offsets(lengths)
    L = int(offs[-1])
    uvqk = (torch.randn(L, 4 * H * d, generator=g) * 0.5).bfloat16().to(DEV)
    v = uvqk[:, H * d:2 * H * d].view(L, H, d)
    q = uvqk[:, 2 * H * d:3 * H * d].view(L, H, d)
    k = uvqk[:, 3 * H * d:].view(L, H, d)
    out = G.hstu_mha(200, 0.1, q, k, v, offs.to(DEV))
    ref, _ = _oracle(q.cpu(), k.cpu(), v.cpu(), offs, 200, 0.1)
    P.check("views", out.cpu(), ref, offs)


@pytest.mark.parametrize("impl", ["tcgen05", "simt"])
def test_expanded_output_gradient(impl):
    """``out.sum(0)`` hands the backward a gradient whose rows all alias one row (row stride 0)."""
    G.set_attention_impl(impl)
    q, k, v, offs, nt, _ = _random_case(31, 4, 50, 300, 300, 2, 128, torch.bfloat16, std=0.7)
    leaves = [t.to(DEV).requires_grad_(True) for t in (q, k, v)]
    out = G.hstu_mha(300, 0.09, leaves[0], leaves[1], leaves[2], offs.to(DEV))
    w = torch.randn(2, 128, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(DEV)
    (out.sum(0) * w).sum().backward()      # no cast in between: the expanded gradient arrives as it is
    dout = w.cpu().expand(q.shape[0], 2, 128).contiguous()
    _, rgrads = _oracle(q, k, v, offs, 300, 0.09, dout=dout)
    for g_, r, nm in zip(leaves, rgrads, ("dq", "dk", "dv")):
        P.check(("expanded_dout", impl, nm), g_.grad.cpu(), r, offs)


def test_attn_scale_and_truncation_fp32():
    G.set_attention_impl("simt")
    g = torch.Generator().manual_seed(8)
    lengths = torch.tensor([30, 50, 12])
    offs = W._offsets(lengths)
    L = int(offs[-1])
    q = torch.randn(L, 2, 16, generator=g); k = torch.randn(L, 2, 16, generator=g); v = torch.randn(L, 2, 16, generator=g)
    scale = torch.rand(L, generator=g)
    out, _ = _run(q, k, v, offs, 64, 0.25, scale=scale)
    ref, _ = _oracle(q, k, v, offs, 64, 0.25, scale=scale)
    P.check_f32("scale_per_token", out, ref, offs)
    out, _ = _run(q, k, v, offs, 64, 0.25, scale=torch.tensor(0.37))
    ref, _ = _oracle(q, k, v, offs, 64, 0.25, scale=torch.tensor(0.37))
    P.check_f32("scale_scalar", out, ref, offs)
    # sequences longer than max_seq_len: rows beyond it are zeros
    out, _ = _run(q, k, v, offs, 40, 0.25)
    ref, _ = _oracle(q, k, v, offs, 40, 0.25)
    P.check_f32("truncated", out, ref, offs)


@pytest.mark.parametrize("impl", ["tcgen05", "simt"])
def test_relative_bias_extension(impl):
    G.set_attention_impl(impl)
    q, k, v, offs, nt, _ = _random_case(21, 4, 40, 280, 300, 2, 128, torch.bfloat16, 8, 3)
    bias = torch.randn(300) * 0.3
    out, _ = _run(q, k, v, offs, 300, 0.09, nt, 0, 3, 0, bias=bias)
    ref, _ = _oracle(q, k, v, offs, 300, 0.09, nt, 0, 3, 0, bias=bias)
    P.check(("bias_fwd", impl), out, ref, offs)


def test_config0_fp32_matches_golden(golden):
    fx = golden("attention.pt")["cfg0"]
    w = W.config0()
    assert torch.equal(w.seq_offsets, fx["seq_offsets"])
    out, _ = _run(fx["q"], fx["k"], fx["v"], fx["seq_offsets"], 256, 1.0 / 32)
    P.check_f32("config0", out, fx["out"], fx["seq_offsets"])


def test_config1_full_size_forward_backward():
    """BASELINE configs[1] at full size against the fp32 oracle (a few seconds of CPU)."""
    w = W.config1()
    q, k, v, do = w.qkv(with_dout=True)
    out, grads = _run(q, k, v, w.seq_offsets, w.max_seq_len, w.alpha, w.num_targets, dout=do)
    ref, rgrads = _oracle(q, k, v, w.seq_offsets, w.max_seq_len, w.alpha, w.num_targets, dout=do)
    _check_all("config1", out, grads, ref, rgrads, w.seq_offsets)


@pytest.mark.parametrize("targets,ctx,W_,bias", [(0, 0, 0, False), (40, 0, 0, False), (24, 5, 300, False),
                                                   (16, 0, 0, True)])
def test_long_sequence_forward_variant(targets, ctx, W_, bias):
    """max_seq_len > 2048 selects the forward's other activation layout (one warpgroup per query
    tile, P contiguous in TMEM); same answers expected.  Lengths include a tile-aligned one and a
    sequence too short for a second query tile."""
    N, H, d = 2304, 2, 128
    g = torch.Generator().manual_seed(77 + targets)
    lengths = torch.tensor([2304, 1000, 129, 2048, 70 + targets + ctx])
    nt = torch.full((len(lengths),), targets, dtype=torch.int64) if targets else None
    offs = W._offsets(lengths)
    L = int(offs[-1])
    q, k, v = ((torch.randn(L, H, d, generator=g) * 0.6).to(torch.bfloat16) for _ in range(3))
    b = (torch.randn(N, generator=g) * 0.3) if bias else None
    out, _ = _run(q, k, v, offs, N, 1.0 / d, nt, W_, ctx, bias=b)
    ref, _ = _oracle(q, k, v, offs, N, 1.0 / d, nt, W_, ctx, bias=b)
    P.check(("long", targets, ctx, W_, bias), out, ref, offs)


def test_backward_reusing_the_forward_plan_is_bit_identical():
    """The forward's planning launch can build the backward's work lists (one launch per training
    step).  Gradients must not depend on who planned, and a second backward through the same graph
    (the lists are consumed by the first) must plan for itself and agree as well."""
    from generative_recommenders_b200 import hstu_attention as HA
    q, k, v, offs, nt, dout = _random_case(11, 5, 100, 500, 520, 2, 128, torch.bfloat16, targets=30, ctx=5)
    q, k, v, dout = (t.to(DEV) for t in (q, k, v, dout))
    offs32, nt32 = offs.to(DEV).to(torch.int32), nt.to(DEV).to(torch.int32)
    args = (520, 1.0 / 128, q, k, v, offs32, nt32, None, 90, 5, 0)
    # explicit calls: own plans
    out0 = HA.hstu_attention_fwd(*args)
    g0 = [torch.empty_like(t) for t in (q, k, v)]
    HA.hstu_attention_bwd(dout, *args, *g0)
    # explicit calls: shared plan
    out1, scratch = HA.hstu_attention_fwd(*args, plan_for_backward=True)
    g1 = [torch.empty_like(t) for t in (q, k, v)]
    HA.hstu_attention_bwd(dout, *args, *g1, planned_scratch=scratch)
    torch.cuda.synchronize()
    assert torch.equal(out0, out1)
    for a, b in zip(g0, g1):
        assert torch.equal(a, b)
    # autograd: two backward passes through one graph
    qd, kd, vd = (t.clone().requires_grad_(True) for t in (q, k, v))
    out = G.hstu_mha(520, 1.0 / 128, qd, kd, vd, offs32, num_targets=nt32, max_attn_len=90, contextual_seq_len=5)
    out.backward(dout, retain_graph=True)
    first = [t.grad.clone() for t in (qd, kd, vd)]
    for t in (qd, kd, vd):
        t.grad = None
    out.backward(dout)
    torch.cuda.synchronize()
    for a, b, c in zip(first, (qd.grad, kd.grad, vd.grad), g0):
        assert torch.equal(a, b) and torch.equal(a, c)


def test_delta_attention_fp32_matches_golden(golden):
    """Cached-inference attention against the reference's own output (fixture made from
    pytorch_cached_hstu_mha, pt_hstu_attention.py:191-251)."""
    fx = golden("delta_attention.pt")
    out = G.delta_hstu_mha(fx["N"], fx["alpha"], fx["delta_q"].to(DEV), fx["k"].to(DEV), fx["v"].to(DEV),
                           fx["seq_offsets"].to(DEV), num_targets=fx["num_targets"].to(DEV)).cpu()
    P.check_f32("delta_golden", out, fx["out"])


@pytest.mark.parametrize("impl", ["tcgen05", "simt"])
@pytest.mark.parametrize("delta,targets,ctx,W_", [(5, True, 0, 0), (64, True, 3, 0), (128, False, 0, 100), (200, True, 4, 150)])
def test_delta_attention_bf16_matches_oracle(impl, delta, targets, ctx, W_):
    G.set_attention_impl(impl)
    g = torch.Generator().manual_seed(delta)
    B, H, d, N = 5, 2, 128, 700
    lengths = torch.randint(delta + ctx + 2, N + 1, (B,), generator=g)
    lengths[0] = delta + ctx + 1                       # shortest legal sequence
    offs = W._offsets(lengths)
    L = int(offs[-1])
    nt = torch.full((B,), delta, dtype=torch.int64) if targets else None
    if targets:
        nt[1] = max(1, delta // 2)                     # delta rows that straddle history and targets
    k = (torch.randn(L, H, d, generator=g) * 0.7).to(torch.bfloat16)
    v = (torch.randn(L, H, d, generator=g) * 0.7).to(torch.bfloat16)
    dq = (torch.randn(B * delta, H, d, generator=g) * 0.7).to(torch.bfloat16)
    out = G.delta_hstu_mha(N, 1.0 / d, dq.to(DEV), k.to(DEV), v.to(DEV), offs.to(DEV),
                           num_targets=None if nt is None else nt.to(DEV), max_attn_len=W_,
                           contextual_seq_len=ctx).cpu()
    ref = O.delta_hstu_mha(N, 1.0 / d, dq.float(), k.float(), v.float(), offs, nt, W_, ctx)
    P.check(("delta", impl, delta), out, ref, delta * torch.arange(B + 1))


def test_unsupported_requests_raise():
    q = torch.zeros(4, 1, 32, device=DEV)
    offs = torch.tensor([0, 4], device=DEV)
    with pytest.raises(NotImplementedError):
        G.hstu_mha(8, 1.0, q, q, q, offs, kernel=G.HammerKernel.TRITON)
    with pytest.raises(Exception):
        G.hstu_mha(8, 1.0, q, q, q, offs, causal=False)
    with pytest.raises(RuntimeError):
        G.hstu_mha(8, 1.0, q.cpu(), q.cpu(), q.cpu(), offs.cpu())
    G.set_attention_impl("tcgen05")
    with pytest.raises(RuntimeError):  # fp32 has no tensor-core path: loud error, no silent fallback
        G.hstu_mha(8, 1.0, q, q, q, offs)


def test_config3_full_size_properties():
    """BASELINE configs[3] (256 sequences up to 8192 tokens, window 1024, 256 targets) at full
    size.  The oracle checks sampled sequences - the shortest, a median one and, for one head, a
    maximum-length one; size-independent properties cover the rest: a second run and a run of the
    sampled sequences alone give the same bits as the full batch (rows of a sequence depend on
    nothing outside it, whatever the work list looks like), and the result is linear in v
    (doubling v doubles every output bit-exactly)."""
    w = W.config3()
    q, k, v = w.qkv(device=DEV)
    offs_d, nt_d = w.seq_offsets.to(DEV), w.num_targets.to(DEV)

    def run(q_, k_, v_, offs_, nt_):
        return G.hstu_mha(w.max_seq_len, w.alpha, q_, k_, v_, offs_, num_targets=nt_, max_attn_len=w.max_attn_len,
                          contextual_seq_len=w.contextual_seq_len)

    out = run(q, k, v, offs_d, nt_d)
    assert torch.isfinite(out.float()).all()
    assert torch.equal(out, run(q, k, v, offs_d, nt_d))
    assert torch.equal(run(q, k, v * 2, offs_d, nt_d), out * 2)

    order = torch.argsort(w.lengths)
    picks = [int(order[0]), int(order[len(order) // 2]), int(order[-1])]
    assert int(w.lengths[picks[-1]]) == w.max_seq_len
    rows = torch.cat([torch.arange(int(w.seq_offsets[b]), int(w.seq_offsets[b + 1])) for b in picks]).to(DEV)
    sub = W.subset(w, picks)
    out_sub = run(q[rows], k[rows], v[rows], sub.seq_offsets.to(DEV), sub.num_targets.to(DEV))
    assert torch.equal(out_sub, out[rows])

    for n, b in enumerate(picks):
        lo, hi = int(w.seq_offsets[b]), int(w.seq_offsets[b + 1])
        heads = slice(0, 1) if n == 2 else slice(0, w.num_heads)   # the 8192-token sequence: one head
        one = W.subset(w, [b])
        ref = O.hstu_mha(w.max_seq_len, w.alpha, q[lo:hi, heads].float().cpu(), k[lo:hi, heads].float().cpu(),
                         v[lo:hi, heads].float().cpu(), one.seq_offsets, num_targets=one.num_targets,
                         max_attn_len=w.max_attn_len, contextual_seq_len=w.contextual_seq_len)
        P.check(("config3", b), out[lo:hi, heads].cpu(), ref, torch.tensor([0, hi - lo]))


def test_config4_full_size_properties():
    """BASELINE configs[4]'s attention (2048 sequences up to 16 384 tokens, 3.5 M tokens, H = 8,
    contextual prefix 16, 64 targets) at full size: element offsets pass 2^31 here.  Same
    properties as for configs[3]; the sampled sequences include the last one of the batch (the
    highest row offsets), the oracle checks the shortest, a median one and the last."""
    w = W.config4()
    L, H, d = w.total_tokens, w.num_heads, w.attn_dim
    assert L * H * d > 2 ** 31
    g = torch.Generator(device=DEV).manual_seed(w.seed)
    q, k, v = (torch.randn(L, H, d, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16) for _ in range(3))
    offs_d, nt_d = w.seq_offsets.to(DEV), w.num_targets.to(DEV)

    def run(q_, k_, v_, offs_, nt_):
        return G.hstu_mha(w.max_seq_len, w.alpha, q_, k_, v_, offs_, num_targets=nt_, max_attn_len=w.max_attn_len,
                          contextual_seq_len=w.contextual_seq_len)

    out = run(q, k, v, offs_d, nt_d)
    assert torch.isfinite(out.float()).all()
    assert torch.equal(out, run(q, k, v, offs_d, nt_d))
    v2 = v * 2
    out2 = run(q, k, v2, offs_d, nt_d)
    del v2
    assert torch.equal(out2, out * 2)
    del out2

    order = torch.argsort(w.lengths)
    last = len(w.lengths) - 1
    picks = [int(order[0]), int(order[len(order) // 2]), int(order[-1]), last]
    assert int(w.lengths[picks[2]]) == w.max_seq_len
    rows = torch.cat([torch.arange(int(w.seq_offsets[b]), int(w.seq_offsets[b + 1])) for b in picks]).to(DEV)
    sub = W.subset(w, picks)
    out_sub = run(q[rows], k[rows], v[rows], sub.seq_offsets.to(DEV), sub.num_targets.to(DEV))
    assert torch.equal(out_sub, out[rows])

    for b in (picks[0], picks[1], last):
        lo, hi = int(w.seq_offsets[b]), int(w.seq_offsets[b + 1])
        heads = slice(0, H) if hi - lo <= 2048 else slice(H - 1, H)
        one = W.subset(w, [b])
        ref = O.hstu_mha(w.max_seq_len, w.alpha, q[lo:hi, heads].float().cpu(), k[lo:hi, heads].float().cpu(),
                         v[lo:hi, heads].float().cpu(), one.seq_offsets, num_targets=one.num_targets,
                         max_attn_len=w.max_attn_len, contextual_seq_len=w.contextual_seq_len)
        P.check(("config4", b), out[lo:hi, heads].cpu(), ref, torch.tensor([0, hi - lo]))


def test_config2_full_size_backward_properties():
    """BASELINE configs[2]'s attention (training: 128 sequences up to 4096 tokens, H = 4,
    contextual prefix 6, targets) forward + backward at full size: gradients of sampled sequences
    run alone carry the same bits as in the full batch, doubling dout doubles dq, dk, dv
    bit-exactly, and the oracle checks the shortest, a median and the longest sequence."""
    w = W.config2_attention()
    q, k, v, do = w.qkv(device=DEV, with_dout=True)
    nt_all = None if w.num_targets is None else w.num_targets.to(DEV)

    def run(q_, k_, v_, do_, offs_, nt_):
        q_, k_, v_ = (t.detach().clone().requires_grad_(True) for t in (q_, k_, v_))
        out = G.hstu_mha(w.max_seq_len, w.alpha, q_, k_, v_, offs_, num_targets=nt_, max_attn_len=w.max_attn_len,
                         contextual_seq_len=w.contextual_seq_len)
        out.backward(do_)
        return out.detach(), q_.grad, k_.grad, v_.grad

    full = run(q, k, v, do, w.seq_offsets.to(DEV), nt_all)
    for t in full:
        assert torch.isfinite(t.float()).all()
    twice = run(q, k, v, do * 2, w.seq_offsets.to(DEV), nt_all)
    for a, b in zip(full[1:], twice[1:]):
        assert torch.equal(a * 2, b)

    order = torch.argsort(w.lengths)
    picks = [int(order[0]), int(order[len(order) // 2]), int(order[-1])]
    rows = torch.cat([torch.arange(int(w.seq_offsets[b]), int(w.seq_offsets[b + 1])) for b in picks]).to(DEV)
    sub = W.subset(w, picks)
    alone = run(q[rows], k[rows], v[rows], do[rows], sub.seq_offsets.to(DEV),
                None if sub.num_targets is None else sub.num_targets.to(DEV))
    for a, b in zip(alone, full):
        assert torch.equal(a, b[rows])

    for b in picks:
        lo, hi = int(w.seq_offsets[b]), int(w.seq_offsets[b + 1])
        heads = slice(0, w.num_heads) if hi - lo <= 2048 else slice(0, 1)
        one = W.subset(w, [b])
        ref, rgrads = _oracle(q[lo:hi, heads].cpu(), k[lo:hi, heads].cpu(), v[lo:hi, heads].cpu(), one.seq_offsets,
                              w.max_seq_len, w.alpha, one.num_targets, w.max_attn_len, w.contextual_seq_len,
                              dout=do[lo:hi, heads].cpu())
        P.check(("config2", b, "out"), full[0][lo:hi, heads].cpu(), ref)
        for gr, rg, nm in zip(full[1:], rgrads, "qkv"):
            P.check(("config2", b, nm), gr[lo:hi, heads].cpu(), rg)


# ---------------------------------------------------------------------------------------
# relative bias: backward, and the gradient of the bias itself
# ---------------------------------------------------------------------------------------
BIAS_CASES = [
    # B, lo, hi, N, H, d, targets, ctx, W
    (4, 40, 280, 300, 2, 128, 8, 3, 0),
    (4, 30, 250, 270, 2, 64, 6, 4, 0),
    (3, 10, 50, 64, 2, 128, 5, 2, 0),        # max_seq_len below one tile
    (3, 250, 290, 300, 1, 128, 9, 5, 0),     # lengths close to N, N not a multiple of 128
    (4, 100, 500, 520, 2, 128, 30, 5, 90),   # local window
    (3, 600, 2300, 2400, 1, 128, 20, 6, 0),  # sequences longer than 2048 tokens
]


@pytest.mark.parametrize("impl", ["tcgen05", "simt"])
@pytest.mark.parametrize("case", BIAS_CASES)
def test_relative_bias_backward_and_bias_gradient(impl, case):
    """dq, dk, dv with a relative bias, and d(bias_by_distance), against autograd through the
    oracle's ``rel_bias`` (which the research model's attention pins, see
    test_attention_with_learnable_bias_matches_reference)."""
    B, lo, hi, N, H, d, targets, ctx, Wn = case
    if impl == "simt" and N > 2048:
        pytest.skip("covered by the tensor-core kernels; minutes on CUDA cores")
    G.set_attention_impl(impl)
    q, k, v, offs, nt, dout = _random_case(hash(case) % 10000 + 7, B, lo, hi, N, H, d, torch.bfloat16, targets, ctx,
                                           std=0.7)
    g = torch.Generator().manual_seed(N)
    bias = torch.randn(N, generator=g) * 0.3
    alpha = 1.0 / d ** 0.5
    out, grads = _run(q, k, v, offs, N, alpha, nt, Wn, ctx, 0, dout, bias=bias, bias_grad=True)
    ref, rgrads = _oracle(q, k, v, offs, N, alpha, nt, Wn, ctx, 0, dout, bias=bias, bias_grad=True)
    _check_all(("bias_bwd", impl, case), out, grads[:3], ref, rgrads[:3], offs)
    # the bias gradient sums fp32 values over every pair of a diagonal: no per-sequence view
    P.check(("bias_bwd", impl, case, "dbias"), grads[3], rgrads[3])


def test_relative_bias_shorter_than_the_sequences():
    """A bias table that covers only the first distances: beyond it the bias is zero and its
    gradient has that length."""
    G.set_attention_impl("tcgen05")
    q, k, v, offs, nt, dout = _random_case(3, 3, 150, 400, 420, 2, 128, torch.bfloat16, 10, 0, std=0.7)
    bias = torch.randn(100, generator=torch.Generator().manual_seed(1)) * 0.3
    out, grads = _run(q, k, v, offs, 420, 0.09, nt, dout=dout, bias=bias, bias_grad=True)
    ref, rgrads = _oracle(q, k, v, offs, 420, 0.09, nt, dout=dout, bias=bias, bias_grad=True)
    _check_all("short_bias", out, grads[:3], ref, rgrads[:3], offs)
    assert grads[3].shape == (100,)
    P.check(("short_bias", "dbias"), grads[3], rgrads[3])


def test_learnable_bias_fp32_matches_reference_fixture(golden):
    """fp32 kernels on the research model's attention with a learnable per-distance bias: output
    and the gradients of q, k, v and of the bias weights as the unmodified reference produced them
    (tests/golden/rel_bias_attention.pt)."""
    G.set_attention_impl("simt")
    fx = golden("rel_bias_attention.pt")
    N, H, A, V = fx["N"], fx["H"], fx["A"], fx["V"]
    L = fx["q"].shape[0]
    bias = fx["w"][N - 1 - torch.arange(N)].clone()   # weight of distance i - j >= 0
    out, grads = _run(fx["q"].view(L, H, A), fx["k"].view(L, H, A), fx["v"].view(L, H, V), fx["seq_offsets"], N, 1.0,
                      dout=fx["dout"].view(L, H, V), bias=bias, bias_grad=True)
    rg = (fx["dq"].view(L, H, A), fx["dk"].view(L, H, A), fx["dv"].view(L, H, V))
    _check_all("bias_golden", out, grads[:3], fx["out"].view(L, H, V), rg, fx["seq_offsets"], f32=True)
    P.check_f32(("bias_golden", "dw"), grads[3], fx["dw"][N - 1 - torch.arange(N)])


# ---------------------------------------------------------------------------------------
# drawn shapes (the reference draws its attention test shapes with Hypothesis,
# ops/tests/hstu_attention_test.py:262-292)
# ---------------------------------------------------------------------------------------
@settings(max_examples=24, deadline=None, derandomize=True)
@given(
    batch=st.integers(1, 7),
    heads=st.sampled_from([1, 2, 4]),
    max_len=st.sampled_from([20, 100, 128, 200, 400, 777]),
    dim=st.sampled_from([16, 32, 64, 128]),
    has_targets=st.booleans(),
    ctx=st.sampled_from([0, 0, 3, 11]),
    window=st.sampled_from([0, 0, 16, 111]),
    full_tail=st.sampled_from([0, 0, 9]),
    dtype=st.sampled_from([torch.bfloat16, torch.float16, torch.float32]),
    scalar_scale=st.booleans(),
    seed=st.integers(0, 10 ** 6),
)
def test_drawn_shapes_forward_backward(batch, heads, max_len, dim, has_targets, ctx, window, full_tail, dtype,
                                       scalar_scale, seed):
    """Whatever kernel family the dispatcher picks for the drawn shape (tensor cores for 16-bit
    inputs with head dimension 64 / 128, CUDA cores otherwise) must agree with the oracle."""
    g = torch.Generator().manual_seed(seed)
    lengths = torch.randint(1, max_len + 1, (batch,), generator=g)
    nt = None
    if has_targets:
        nt = torch.randint(1, 12, (batch,), generator=g)
        lengths = torch.clamp(lengths + nt + ctx, max=max_len)
        nt = torch.minimum(nt, torch.clamp(lengths - ctx - 1, min=0))
    elif ctx > 0:
        lengths = torch.clamp(lengths + ctx, max=max_len)
    if window == 0:
        full_tail = 0
    offs = W._offsets(lengths)
    L = int(offs[-1])
    q, k, v, dout = ((torch.randn(L, heads, dim, generator=g) * 0.8).to(dtype) for _ in range(4))
    scale = torch.tensor(0.013) if scalar_scale else None
    alpha = 1.0 / dim ** 0.5
    out, grads = _run(q, k, v, offs, max_len, alpha, nt, window, ctx, full_tail, dout, scale=scale)
    ref, rgrads = _oracle(q, k, v, offs, max_len, alpha, nt, window, ctx, full_tail, dout, scale=scale)
    name = ("drawn", batch, heads, max_len, dim, has_targets, ctx, window, full_tail, str(dtype), scalar_scale, seed)
    _check_all(name, out, grads, ref, rgrads, offs, f32=dtype == torch.float32)
