"""The fused uvqk stage (LayerNorm -> linear -> split -> SiLU as one tcgen05 kernel) against the
oracle's fp32 evaluation and against the three separate stages."""

import importlib

import pytest
import torch

from oracle import hstu_oracle as O
import parity_metrics as P

pytestmark = pytest.mark.gpu

G = importlib.import_module("generative-recommenders_b200")
HC = importlib.import_module("generative-recommenders_b200.hstu_compute")
DEV = "cuda"


def _inputs(M, D, H, A, V, dtype, seed, shift=0.0):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(M, D, generator=g) * 1.5 + shift).to(dtype)
    nw = (1.0 + 0.2 * torch.randn(D, generator=g)).to(dtype)
    nb = (0.1 * torch.randn(D, generator=g)).to(dtype)
    N = (2 * V + 2 * A) * H
    W = (torch.randn(D, N, generator=g) / D ** 0.5).to(dtype)
    b = (0.1 * torch.randn(N, generator=g)).to(dtype)
    return x, nw, nb, W, b


@pytest.mark.parametrize("M,D,H,A,V", [(1, 64, 2, 32, 32), (127, 64, 2, 32, 32), (128, 128, 2, 64, 64),
                                       (300, 256, 4, 64, 64), (1000, 512, 4, 128, 128), (333, 512, 2, 128, 96),
                                       (4500, 256, 4, 128, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fused_uqvk_matches_oracle(M, D, H, A, V, dtype):
    x, nw, nb, W, b = _inputs(M, D, H, A, V, dtype, seed=M + D)
    ref = O.hstu_compute_uqvk(x.float(), nw.float(), nb.float(), 1e-6, H, A, V, W.float(), b.float())
    HC.set_fused_uqvk(True)
    assert HC._fused_uqvk_supported(x.to(DEV), W.to(DEV), V * H)
    n0 = G._cabi.launch_count()
    got = G.hstu_compute_uqvk(x.to(DEV), nw.to(DEV), nb.to(DEV), 1e-6, H, A, V, W.to(DEV), b.to(DEV))
    assert G._cabi.launch_count() - n0 == 3  # two preparation launches + fused kernel
    for name, a, r in zip("uqkv", got, ref):
        assert a.shape == r.shape
        assert O.rel_l2(a.float().cpu(), r) < 1e-2, name
    HC.set_fused_uqvk(False)
    sep = G.hstu_compute_uqvk(x.to(DEV), nw.to(DEV), nb.to(DEV), 1e-6, H, A, V, W.to(DEV), b.to(DEV))
    HC.set_fused_uqvk(True)
    for name, a, r_, r in zip("uqkv", got, sep, ref):
        # the fused kernel multiplies the exact rows of x: it is at least as close to fp32 as the
        # separate stages, which round LN(x) to 16 bits first
        assert O.rel_l2(a.float().cpu(), r) <= 1.2 * O.rel_l2(r_.float().cpu(), r) + 1e-4, name


def test_fused_uqvk_parameters_sliced_from_a_flat_buffer():
    """All four parameters as contiguous slices of one flat buffer that start off the 16-byte grid
    (flattened-parameter training setups hand such views to the ops): same results as with
    separately allocated parameters, forward and backward."""
    M, D, H, A, V = 300, 256, 2, 64, 64
    x, nw, nb, W, b = (t.to(DEV) for t in _inputs(M, D, H, A, V, torch.bfloat16, seed=21))
    flat = torch.zeros(3 + nw.numel() + 1 + nb.numel() + 3 + W.numel() + 5 + b.numel(), dtype=torch.bfloat16, device=DEV)
    views, at = [], 3
    for t, gap in ((nw, 1), (nb, 3), (W, 5), (b, 0)):
        v = flat[at:at + t.numel()].view(t.shape)
        v.copy_(t)
        views.append(v.requires_grad_(True))
        at += t.numel() + gap
    assert views[2].data_ptr() % 16 != 0 and views[2].is_contiguous()
    plain = [t.clone().requires_grad_(True) for t in (nw, nb, W, b)]
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    got = G.hstu_compute_uqvk(xa, views[0], views[1], 1e-6, H, A, V, views[2], views[3])
    want = G.hstu_compute_uqvk(xb, plain[0], plain[1], 1e-6, H, A, V, plain[2], plain[3])
    g = torch.Generator().manual_seed(5)
    douts = [torch.randn(o.shape, generator=g).bfloat16().to(DEV) for o in want]
    torch.autograd.backward(list(got), douts)
    torch.autograd.backward(list(want), douts)
    for a_, b_ in zip(got, want):
        assert torch.equal(a_, b_)
    assert torch.equal(xa.grad, xb.grad)
    for a_, b_ in zip(views, plain):
        assert torch.equal(a_.grad, b_.grad)


def test_fused_uqvk_large_mean_rows():
    """Rows with |mean| >> std: the statistics use shifted sums, the epilogue subtracts mean * c1."""
    x, nw, nb, W, b = _inputs(500, 256, 2, 64, 64, torch.bfloat16, seed=9, shift=40.0)
    ref = O.hstu_compute_uqvk(x.float(), nw.float(), nb.float(), 1e-6, 2, 64, 64, W.float(), b.float())
    ref16 = O.hstu_compute_uqvk(x, nw, nb, 1e-6, 2, 64, 64, W, b)   # the reference's arithmetic in bf16
    got = G.hstu_compute_uqvk(x.to(DEV), nw.to(DEV), nb.to(DEV), 1e-6, 2, 64, 64, W.to(DEV), b.to(DEV))
    for name, a, r, r16 in zip("uqkv", got, ref, ref16):
        P.check_vs_bf16_reference(("large_mean", name), a.float().cpu(), r, r16.float())


def test_fused_uqvk_gradients_match_separate_stages():
    M, D, H, A, V = 700, 256, 2, 64, 64
    x, nw, nb, W, b = _inputs(M, D, H, A, V, torch.bfloat16, seed=4)
    g = torch.Generator().manual_seed(1)
    grads = [torch.randn(M, V * H, generator=g), torch.randn(M, H, A, generator=g), torch.randn(M, H, A, generator=g),
             torch.randn(M, H, V, generator=g)]
    res = {}
    for fused in (True, False):
        HC.set_fused_uqvk(fused)
        leaves = [t.to(DEV).requires_grad_(True) for t in (x, nw, nb, W, b)]
        outs = G.hstu_compute_uqvk(leaves[0], leaves[1], leaves[2], 1e-6, H, A, V, leaves[3], leaves[4])
        torch.autograd.backward(list(outs), [t.to(DEV).to(torch.bfloat16) for t in grads])
        res[fused] = [t.grad.float().cpu() for t in leaves]
    HC.set_fused_uqvk(True)
    # fp32 reference through the oracle, and the reference's own arithmetic in bf16
    leaves = [t.float().requires_grad_(True) for t in (x, nw, nb, W, b)]
    outs = O.hstu_compute_uqvk(leaves[0], leaves[1], leaves[2], 1e-6, H, A, V, leaves[3], leaves[4])
    torch.autograd.backward(list(outs), [t.to(torch.bfloat16).float() for t in grads])
    leaves16 = [t.clone().requires_grad_(True) for t in (x, nw, nb, W, b)]
    outs16 = O.hstu_compute_uqvk(leaves16[0], leaves16[1], leaves16[2], 1e-6, H, A, V, leaves16[3], leaves16[4])
    torch.autograd.backward(list(outs16), [t.to(torch.bfloat16) for t in grads])
    for name, a, s_, r, r16 in zip(("dx", "dnw", "dnb", "dW", "db"), res[True], res[False], leaves, leaves16):
        P.check_vs_bf16_reference(("uqvk_grad", "fused", name), a, r.grad, r16.grad.float())
        P.check_vs_bf16_reference(("uqvk_grad", "separate", name), s_, r.grad, r16.grad.float())


def test_fused_uqvk_unsupported_shapes_take_the_separate_stages():
    x, nw, nb, W, b = _inputs(50, 32, 2, 16, 16, torch.bfloat16, seed=2)   # D = 32
    assert not HC._fused_uqvk_supported(x.to(DEV), W.to(DEV), 32)
    ref = O.hstu_compute_uqvk(x.float(), nw.float(), nb.float(), 1e-6, 2, 16, 16, W.float(), b.float())
    got = G.hstu_compute_uqvk(x.to(DEV), nw.to(DEV), nb.to(DEV), 1e-6, 2, 16, 16, W.to(DEV), b.to(DEV))
    for a, r in zip(got, ref):
        assert O.rel_l2(a.float().cpu(), r) < 1e-2
    a = G._cabi.LnLinearArgs()
    a.D, a.N, a.M, a.dtype = 32, 128, 4, G._cabi.BF16
    assert G._cabi.lib().b200_hstu_ln_linear_silu_fwd(a, None) == -2


@pytest.mark.parametrize("ctx,W_", [(0, 0), (4, 50)])
def test_fused_layer_gradients_match_oracle(ctx, W_):
    """A bf16 STU layer through the single autograd node (fused uvqk stage + attention, whose
    backward writes dq / dk / dv into the stage's gradient buffer): output, input gradient and all
    parameter gradients against fp32 autograd through the oracle, and against the separate stages."""
    torch.manual_seed(5)
    torch.backends.cuda.matmul.allow_tf32 = False
    D, H, d = 256, 2, 128
    cfg = G.STULayerConfig(embedding_dim=D, num_heads=H, hidden_dim=d, attention_dim=d, output_dropout_ratio=0.0,
                           contextual_seq_len=ctx, max_attn_len=W_)
    layer = G.STULayer(cfg).to(DEV).to(torch.bfloat16)
    with torch.no_grad():
        for p_ in layer.parameters():
            if p_.dim() == 1:
                p_.add_(0.1 * torch.randn_like(p_))
    lengths = torch.tensor([130, 300, 17, 257, 64])
    nt = torch.tensor([3, 20, 1, 9, 5])
    offs = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(lengths, 0)])
    g = torch.Generator().manual_seed(2)
    x = torch.randn(int(offs[-1]), D, generator=g).bfloat16()
    dy = torch.randn(int(offs[-1]), D, generator=g).bfloat16()
    res = {}
    for fused in (True, False):
        HC.set_fused_uqvk(fused)
        layer.zero_grad()
        xin = x.to(DEV).requires_grad_(True)
        n0 = G._cabi.launch_count()
        y = layer(xin, lengths.to(DEV), offs.to(DEV), 320, nt.to(DEV))
        y.backward(dy.to(DEV))
        res[fused] = (y.detach().float().cpu(), xin.grad.float().cpu(),
                      {n: p_.grad.float().cpu() for n, p_ in layer.named_parameters()}, G._cabi.launch_count() - n0)
    HC.set_fused_uqvk(True)
    params = {n[1:]: p_.detach().float().cpu().requires_grad_(True) for n, p_ in layer.named_parameters()}
    xr = x.float().requires_grad_(True)
    ref = O.stu_layer(xr, offs, 320, nt, params, H, d, d, max_attn_len=W_, contextual_seq_len=ctx)
    ref.backward(dy.float())
    # the reference's own arithmetic in bf16: the oracle on 16-bit tensors
    params16 = {n[1:]: p_.detach().cpu().clone().requires_grad_(True) for n, p_ in layer.named_parameters()}
    x16 = x.clone().requires_grad_(True)
    ref16 = O.stu_layer(x16, offs, 320, nt, params16, H, d, d, max_attn_len=W_, contextual_seq_len=ctx)
    ref16.backward(dy)
    for fused in (True, False):
        y, dx, grads, _ = res[fused]
        tag = ("layer", ctx, W_, "fused" if fused else "separate")
        P.check_vs_bf16_reference(tag + ("y",), y, ref.detach(), ref16.detach().float())
        P.check_vs_bf16_reference(tag + ("dx",), dx, xr.grad, x16.grad.float())
        for n, gr in grads.items():
            P.check_vs_bf16_reference(tag + (n,), gr, params[n[1:]].grad, params16[n[1:]].grad.float())


def test_prepared_weights_are_reused_only_while_unchanged():
    """Inference with module parameters: the preparation launches are skipped while the parameter
    tensors are the same unmodified objects, and come back after an in-place update or when a
    gradient is wanted."""
    x, nw, nb, W, b = (t.to(DEV) for t in _inputs(300, 256, 2, 64, 64, torch.bfloat16, seed=3))
    nw, nb, W, b = (torch.nn.Parameter(t, requires_grad=False) for t in (nw, nb, W, b))
    call = lambda: G.hstu_compute_uqvk(x, nw, nb, 1e-6, 2, 64, 64, W, b)  # noqa: E731
    first = call()
    n0 = G._cabi.launch_count()
    again = call()
    assert G._cabi.launch_count() - n0 == 1  # the fused kernel alone
    for a_, b_ in zip(first, again):
        assert torch.equal(a_, b_)
    with torch.no_grad():
        W.mul_(2.0)
    n0 = G._cabi.launch_count()
    changed = call()
    assert G._cabi.launch_count() - n0 == 3
    assert not torch.equal(changed[1], first[1])
    ref = O.hstu_compute_uqvk(x.float().cpu(), nw.float().cpu(), nb.float().cpu(), 1e-6, 2, 64, 64,
                              W.detach().float().cpu(), b.float().cpu())
    for a_, r_ in zip(changed, ref):
        assert O.rel_l2(a_.float().cpu(), r_) < 1e-2
    W.requires_grad_(True)   # training: always prepared afresh
    call()
    n0 = G._cabi.launch_count()
    call()
    assert G._cabi.launch_count() - n0 == 3
    # plain tensors (e.g. a cast made for one call) are never remembered
    n0 = G._cabi.launch_count()
    G.hstu_compute_uqvk(x, nw.data, nb.data, 1e-6, 2, 64, 64, W.detach().clone(), b.data)
    G.hstu_compute_uqvk(x, nw.data, nb.data, 1e-6, 2, 64, 64, W.detach().clone(), b.data)
    assert G._cabi.launch_count() - n0 == 6
    # a write through .data leaves the version counter alone: the documented remedy is an explicit
    # clear (or the cache switched off), after which the new weights are in use
    W.requires_grad_(False)
    before = call()
    W.data.mul_(0.5)
    HC.clear_prepared_weights()
    after = call()
    assert not torch.equal(before[1], after[1])
    ref = O.hstu_compute_uqvk(x.float().cpu(), nw.float().cpu(), nb.float().cpu(), 1e-6, 2, 64, 64,
                              W.detach().float().cpu(), b.float().cpu())
    assert O.rel_l2(after[1].float().cpu(), ref[1]) < 1e-2
    HC.set_prepared_weights_cache(False)
    n0 = G._cabi.launch_count()
    call()
    call()
    assert G._cabi.launch_count() - n0 == 6
    HC.set_prepared_weights_cache(True)


def test_fused_uqvk_full_size_matches_separate_stages():
    """configs[1]'s token count, D = 512, N = 2048: the fused kernel against the separate stages
    (element-wise within 16-bit rounding of two different evaluation orders) and u == SiLU(uvqk)."""
    from generative_recommenders_b200 import workloads as W
    M = int(W.config1().total_tokens)
    x, nw, nb, Wt, b = (t.to(DEV) for t in _inputs(M, 512, 4, 128, 128, torch.bfloat16, seed=77))
    with torch.no_grad():
        HC.set_fused_uqvk(True)
        fu = G.hstu_compute_uqvk(x, nw, nb, 1e-6, 4, 128, 128, Wt, b)
        HC.set_fused_uqvk(False)
        se = G.hstu_compute_uqvk(x, nw, nb, 1e-6, 4, 128, 128, Wt, b)
        HC.set_fused_uqvk(True)
    for name, a_, s_ in zip("uqkv", fu, se):
        assert a_.shape == s_.shape
        assert O.rel_l2(a_.float(), s_.float()) < 6e-3, name
        assert (a_.float() - s_.float()).abs().max() < 0.25, name
    assert not torch.isnan(fu[0]).any()
