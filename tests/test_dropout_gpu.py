"""Dropout of the output stage, generated inside the norm-mul kernels: the mask replayed from its
seed by the oracle's Philox, forward and backward, and the public ops with dropout on."""

import pytest
import torch

import generative_recommenders_b200 as G
from oracle import hstu_oracle as O
import parity_metrics as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("dtype,H,V,concat", [
    (torch.bfloat16, 4, 128, (True, True)),     # the layer's own configuration: [u | attn | y], 1536 columns
    (torch.bfloat16, 2, 64, (False, False)),
    (torch.float16, 2, 96, (True, False)),
    (torch.float32, 2, 64, (True, True)),       # 4 elements per 16-byte vector: half a generator call each
    (torch.bfloat16, 2, 34, (True, True)),      # H*V = 68: rows not made of whole vectors (element-wise path)
])
def test_dropout_mask_replay_forward_backward(dtype, H, V, concat):
    g = torch.Generator().manual_seed(11)
    rows, D, p = 333, H * V, 0.3
    attn = torch.randn(rows, D, generator=g).to(dtype)
    u = torch.randn(rows, D, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(D, generator=g)).to(dtype)
    b = (0.1 * torch.randn(D, generator=g)).to(dtype)
    mult = 1 + int(concat[0]) + int(concat[1])
    dy = torch.randn(rows, mult * D, generator=g).to(dtype)
    seed = torch.tensor([0x1234_5678_9ABC_DEF], dtype=torch.int64, device=DEV)
    ld = [t.to(DEV).requires_grad_(True) for t in (attn, u, w, b)]
    y = G.hstu_norm_mul_dropout(ld[0], ld[1], ld[2], ld[3], 1e-6, p, True, concat[0], concat[1], "none", False, H, V,
                                dropout_seed=seed)
    y.backward(dy.to(DEV))
    keep, scale = O.dropout_keep_mask(int(seed.item()), rows, mult * D, p)
    assert abs(float(keep.float().mean()) - (1 - p)) < 0.01
    lr = [t.float().requires_grad_(True) for t in (attn, u, w, b)]
    yr = O.norm_mul_dropout(lr[0], lr[1], lr[2], lr[3], 1e-6, concat[0], concat[1], "none", False, H, V)
    yr = yr * keep * scale
    yr.backward(dy.float())
    # the zeros are where the replayed mask puts them (a kept element is zero with probability ~0)
    assert torch.equal(y.detach().cpu() == 0, ~keep | (yr.detach() == 0))
    tol = dict(tol=2e-4, max_tol=5e-4) if dtype == torch.float32 else {}
    P.check(("dropout", str(dtype), H, V, concat, "y"), y, yr.detach(), **tol)
    for a, r, nm in zip(ld, lr, ("dattn", "du", "dw", "db")):
        P.check(("dropout", str(dtype), H, V, concat, nm), a.grad, r.grad, **tol)
    # the same seed gives the same bits, another seed another mask
    y2 = G.hstu_norm_mul_dropout(ld[0], ld[1], ld[2], ld[3], 1e-6, p, True, concat[0], concat[1], "none", False, H, V,
                                 dropout_seed=seed)
    y3 = G.hstu_norm_mul_dropout(ld[0], ld[1], ld[2], ld[3], 1e-6, p, True, concat[0], concat[1], "none", False, H, V,
                                 dropout_seed=seed + 1)
    assert torch.equal(y, y2) and not torch.equal(y, y3)


def test_compute_output_with_dropout():
    """``hstu_compute_output`` in training mode: one launch produces the dropped-out concat (no
    separate dropout pass), the keep fraction is 1 - p, results are reproducible under
    ``torch.manual_seed`` and differ from call to call, and eval mode is untouched."""
    g = torch.Generator().manual_seed(2)
    rows, H, V, D, p = 2000, 4, 128, 512, 0.3
    attn, u = (torch.randn(rows, H * V, generator=g).bfloat16().to(DEV) for _ in range(2))
    x = torch.randn(rows, D, generator=g).bfloat16().to(DEV)
    nw, nb = torch.ones(H * V, device=DEV).bfloat16(), torch.zeros(H * V, device=DEV).bfloat16()
    Wo = (torch.randn(3 * H * V, D, generator=g) / 40).bfloat16().to(DEV)

    def run(training):
        return G.hstu_compute_output(attn, u, x, nw, nb, 1e-6, Wo, H, V, p, training, True, True, "none", False, False)

    torch.manual_seed(5)
    a1 = run(True)
    a2 = run(True)
    torch.manual_seed(5)
    b1 = run(True)
    assert torch.equal(a1, b1) and not torch.equal(a1, a2)
    ref = O.hstu_compute_output(attn.float().cpu(), u.float().cpu(), x.float().cpu(), nw.float().cpu(), nb.float().cpu(),
                                1e-6, Wo.float().cpu(), H, V, True, True)
    P.check("compute_output_eval", run(False), ref)
    n0 = G._cabi.launch_count()
    y = G.hstu_norm_mul_dropout(attn, u, nw, nb, 1e-6, p, True, True, True, "none", False, H, V)
    assert G._cabi.launch_count() - n0 == 1
    frac = float((y != 0).float().mean())
    assert abs(frac - (1 - p)) < 5e-3, frac
    # E[dropout(y)] = y: the mean over many elements stays put
    y0 = G.hstu_norm_mul_dropout(attn, u, nw, nb, 1e-6, 0.0, False, True, True, "none", False, H, V)
    assert abs(float(y.float().abs().mean()) / float(y0.float().abs().mean()) - 1.0) < 2e-2


def test_group_norm_variant_keeps_torch_dropout():
    g = torch.Generator().manual_seed(3)
    rows, H, V = 400, 4, 32
    attn, u = (torch.randn(rows, H * V, generator=g).bfloat16().to(DEV) for _ in range(2))
    w, b = torch.ones(H, device=DEV).bfloat16(), torch.zeros(H, device=DEV).bfloat16()
    y = G.hstu_norm_mul_dropout(attn, u, w, b, 1e-6, 0.5, True, True, True, "none", True, H, V)
    frac = float((y != 0).float().mean())
    assert 0.45 < frac < 0.55


@pytest.mark.parametrize("dtype,H,V,concat", [
    (torch.bfloat16, 4, 128, (True, True)),
    (torch.float16, 2, 96, (True, False)),
    (torch.bfloat16, 2, 64, (False, False)),
    (torch.bfloat16, 2, 34, (True, True)),      # rows not made of whole vectors: no mask is stored
    (torch.float32, 2, 64, (True, True)),       # 32-bit elements: no mask is stored
])
def test_stored_mask_and_regenerated_mask_give_the_same_backward(dtype, H, V, concat):
    """The forward keeps its dropout mask as bits for the backward where it can; a backward that
    regenerates the mask from the seed instead produces the same gradients bit for bit."""
    import importlib
    HC = G.hstu_compute
    assert HC is importlib.import_module("generative-recommenders_b200.hstu_compute")   # one module under both names
    g = torch.Generator().manual_seed(3)
    rows, D, p = 517, H * V, 0.25
    attn = torch.randn(rows, D, generator=g).to(dtype)
    u = torch.randn(rows, D, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(D, generator=g)).to(dtype)
    b = (0.1 * torch.randn(D, generator=g)).to(dtype)
    mult = 1 + int(concat[0]) + int(concat[1])
    dy = torch.randn(rows, mult * D, generator=g).to(dtype).to(DEV)
    seed = torch.tensor([987654321], dtype=torch.int64, device=DEV)
    results = []
    can_store = dtype != torch.float32 and D % 8 == 0
    for store in (True, False):
        HC.set_store_dropout_mask(store)
        ld = [t.to(DEV).requires_grad_(True) for t in (attn, u, w, b)]
        n0 = G._cabi.launch_count()
        y = G.hstu_norm_mul_dropout(ld[0], ld[1], ld[2], ld[3], 1e-6, p, True, concat[0], concat[1], "silu", False, H, V,
                                    dropout_seed=seed)
        saved = y.grad_fn.saved_tensors
        assert (saved[-1] is not None) == (store and can_store)      # the mask bits, where they can be kept
        if saved[-1] is not None:
            assert saved[-1].numel() == rows * mult * D // 8
            kept = torch.count_nonzero(y.detach().reshape(-1) != 0)
            bits = sum(int(torch.count_nonzero(saved[-1] & (1 << i))) for i in range(8))
            assert abs(bits - int(kept)) <= 8            # a kept element that is exactly zero is as good as never
        y.backward(dy)
        results.append([y.detach()] + [t.grad for t in ld])
        assert G._cabi.launch_count() - n0 == 3      # forward, backward, reduction of the weight gradients
    HC.set_store_dropout_mask(False)
    for a_, b_ in zip(*results):
        assert torch.equal(a_, b_)


# ---------------------------------------------------------------------------------------------
# dropout on the attention weights (CUDA-core kernels)
# ---------------------------------------------------------------------------------------------
def _attention_inputs(dtype, seed=4, N=200, H=2, d=32, with_targets=True):
    from generative_recommenders_b200 import workloads as W
    g = torch.Generator().manual_seed(seed)
    lengths = torch.tensor([200, 37, 1, 150, 96])
    nt = torch.tensor([3, 2, 0, 9, 1]) if with_targets else None
    offs = W._offsets(lengths)
    L = int(offs[-1])
    q, k, v, dout = ((torch.randn(L, H, d, generator=g) * 0.8).to(dtype) for _ in range(4))
    return N, lengths, nt, offs, q, k, v, dout


@pytest.mark.parametrize("dtype,ctx,window,p", [
    (torch.float32, 0, 0, 0.3),
    (torch.float32, 3, 40, 0.5),
    (torch.bfloat16, 0, 0, 0.1),
    (torch.bfloat16, 2, 64, 0.3),
    (torch.float16, 0, 33, 0.25),
])
def test_attention_dropout_mask_replay(dtype, ctx, window, p):
    """``hstu_mha(dropout_pr=p, training=True)``: the mask - element ``(row * H + h) * max_seq_len + j``
    of the counter-based generator - is replayed by the oracle, which applies it where the reference
    does (after scale and mask); output and all three gradients agree, the same seed gives the same
    bits and another seed another mask."""
    N, lengths, nt, offs, q, k, v, dout = _attention_inputs(dtype)
    H, d = q.shape[1], q.shape[2]
    L = q.shape[0]
    alpha = 1.0 / d ** 0.5
    seed = torch.tensor([0x0BAD_5EED_1234], dtype=torch.int64, device=DEV)
    ld = [t.to(DEV).requires_grad_(True) for t in (q, k, v)]
    n0 = G._cabi.launch_count()
    out = G.hstu_mha(N, alpha, ld[0], ld[1], ld[2], offs.to(DEV), dropout_pr=p, training=True, num_targets=nt.to(DEV),
                     max_attn_len=window, contextual_seq_len=ctx, dropout_seed=seed)
    out.backward(dout.to(DEV))
    assert G._cabi.launch_count() - n0 == 3          # forward, dQ, dK / dV: CUDA-core kernels, no planning launch
    keep, scale = O.dropout_keep_mask(int(seed.item()), L * H, N, p)
    keep = keep.view(L, H, N)
    eff = 1.0 - 1.0 / scale                         # the ratio the 16-bit threshold realises
    assert abs(eff - p) < 1e-4
    lr = [t.float().requires_grad_(True) for t in (q, k, v)]
    ref = O.hstu_mha(N, alpha, lr[0], lr[1], lr[2], offs, dropout_pr=eff, num_targets=nt, max_attn_len=window,
                     contextual_seq_len=ctx, dropout_keep=keep)
    ref.backward(dout.float())
    plain = O.hstu_mha(N, alpha, q.float(), k.float(), v.float(), offs, num_targets=nt, max_attn_len=window,
                       contextual_seq_len=ctx)
    assert float((ref.detach() - plain).norm() / plain.norm()) > 0.1      # the mask matters
    name = ("attention dropout", str(dtype), ctx, window, p)
    chk = P.check_f32 if dtype == torch.float32 else P.check
    chk(name + ("out",), out, ref.detach(), offs)
    for a, r, nm in zip(ld, lr, ("dq", "dk", "dv")):
        chk(name + (nm,), a.grad, r.grad, offs)
    with torch.no_grad():
        again = G.hstu_mha(N, alpha, ld[0], ld[1], ld[2], offs.to(DEV), dropout_pr=p, training=True,
                           num_targets=nt.to(DEV), max_attn_len=window, contextual_seq_len=ctx, dropout_seed=seed)
        other = G.hstu_mha(N, alpha, ld[0], ld[1], ld[2], offs.to(DEV), dropout_pr=p, training=True,
                           num_targets=nt.to(DEV), max_attn_len=window, contextual_seq_len=ctx, dropout_seed=seed + 1)
    assert torch.equal(again, out.detach()) and not torch.equal(other, out.detach())


def test_attention_dropout_modes():
    """Eval mode ignores the rate; without a seed one is drawn from torch's generator (reproducible
    under ``torch.manual_seed``); p = 1 returns zeros like ``F.dropout``; the tensor-core kernels
    refuse instead of silently dropping nothing; the bias gradient sees the mask."""
    N, lengths, nt, offs, q, k, v, dout = _attention_inputs(torch.bfloat16, H=2, d=64, with_targets=False)
    alpha = 0.125
    qd, kd, vd, od = q.to(DEV), k.to(DEV), v.to(DEV), offs.to(DEV)
    base = G.hstu_mha(N, alpha, qd, kd, vd, od)
    assert torch.equal(G.hstu_mha(N, alpha, qd, kd, vd, od, dropout_pr=0.4, training=False), base)
    torch.manual_seed(5)
    a = G.hstu_mha(N, alpha, qd, kd, vd, od, dropout_pr=0.4, training=True)
    b = G.hstu_mha(N, alpha, qd, kd, vd, od, dropout_pr=0.4, training=True)
    torch.manual_seed(5)
    c = G.hstu_mha(N, alpha, qd, kd, vd, od, dropout_pr=0.4, training=True)
    assert torch.equal(a, c) and not torch.equal(a, b) and not torch.equal(a, base)
    assert float(G.hstu_mha(N, alpha, qd, kd, vd, od, dropout_pr=1.0, training=True).abs().max()) == 0.0
    with pytest.raises(ValueError):
        G.hstu_mha(N, alpha, qd, kd, vd, od, dropout_pr=1.5, training=True)
    G.set_attention_impl("tcgen05")
    try:
        with pytest.raises(RuntimeError, match="CUDA-core"):
            G.hstu_mha(N, alpha, qd, kd, vd, od, dropout_pr=0.4, training=True)
    finally:
        G.set_attention_impl("auto")
    # relative bias with dropout: the table's gradient against the oracle's
    L, H = q.shape[0], q.shape[1]
    g = torch.Generator().manual_seed(9)
    bias = torch.randn(N, generator=g) * 0.3
    seed = torch.tensor([77], dtype=torch.int64, device=DEV)
    leaves = [t.to(DEV).requires_grad_(True) for t in (q, k, v)]
    bd = bias.to(DEV).requires_grad_(True)
    out = G.hstu_mha(N, alpha, leaves[0], leaves[1], leaves[2], od, dropout_pr=0.25, training=True,
                     bias_by_distance=bd, dropout_seed=seed)
    out.backward(dout.to(DEV))
    keep, scale = O.dropout_keep_mask(77, L * H, N, 0.25)
    lr = [t.float().requires_grad_(True) for t in (q, k, v)]
    br = bias.clone().requires_grad_(True)
    i, j = torch.arange(N).view(-1, 1), torch.arange(N).view(1, -1)
    ref = O.hstu_mha(N, alpha, lr[0], lr[1], lr[2], offs, dropout_pr=1.0 - 1.0 / scale, rel_bias=br[(i - j).abs()],
                     dropout_keep=keep.view(L, H, N))
    ref.backward(dout.float())
    P.check(("attention dropout", "bias", "out"), out, ref.detach(), offs)
    assert O.rel_l2(bd.grad, br.grad) < 2.5e-2
