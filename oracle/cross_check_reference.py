"""Random cross-check of the restatement in ``hstu_oracle.py`` against the unmodified reference.

    python oracle/cross_check_reference.py --reference /path/to/generative-recommenders [--cases 3000] [--seed 0]

TEST INFRASTRUCTURE ONLY.  The golden fixtures pin the oracle on a fixed set of inputs; this script
draws as many more as asked for - attention forward and backward (every mask feature, dropout on the
weights with the reference's own mask, targets that
reach beyond the history, sequences longer than ``max_seq_len``, empty sequences, scalar and
per-token scales), cached attention, the uvqk stage, all variants of the output stage, jagged
concat / split in every layout, the timestamp + position embeddings and whole STU layers (output
and every gradient) - runs the
reference's own PyTorch functions on them (CPU, fp32, through ``reference_shims.py``) and compares.
The oracle uses the same torch primitives in the same order, so the two agree to rounding (1e-5 is
the bound; measured 1e-6 or exactly 0).  Exit status 0 = all cases agree.

It needs a checkout of the reference, which does not travel with this repository:
``tests/test_oracle_golden.py`` runs it only where one lies next to the repository (or
``HSTU_REFERENCE`` names one).
"""

import argparse
import os
import random
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

from oracle import hstu_oracle as O  # noqa: E402
from oracle import reference_shims  # noqa: E402


def _offsets(lengths):
    return torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(lengths, 0)])


def _max_diff(a, b):
    return float((a.detach() - b.detach()).abs().max()) if a.numel() else 0.0


def _scaled_diff(a, b):
    # a parameter gradient sums over every token: its size, not 1, is the scale fp32 rounding refers to
    return _max_diff(a, b) / max(1.0, float(b.detach().abs().max())) if a.numel() else 0.0


def attention_case(rng, ref):
    g = torch.Generator().manual_seed(rng.randrange(10 ** 9))
    N = rng.choice([8, 24, 40, 64])
    B = rng.randint(1, 5)
    ctx = rng.choice([0, 0, 1, 3, 9, 70])
    W = rng.choice([0, 0, 1, 5, 20, 100])
    F = rng.choice([0, 0, 1, 4, 30]) if W else 0
    over = 20 if rng.random() < 0.3 else 0
    lengths = torch.randint(0, N + 1 + over, (B,), generator=g)
    nt = None
    if rng.random() < 0.6:
        nt = torch.randint(0, 12, (B,), generator=g)
        if rng.random() < 0.7:
            nt = torch.minimum(nt, lengths)
    offs = _offsets(lengths)
    L = int(offs[-1])
    if L == 0:
        return None
    H, A, V = rng.choice([1, 2]), rng.choice([4, 16]), rng.choice([4, 16])
    q, k = (torch.randn(L, H, A, generator=g, requires_grad=True) for _ in range(2))
    v = torch.randn(L, H, V, generator=g, requires_grad=True)
    dout = torch.randn(L, H, V, generator=g)
    pick = rng.random()
    sc = torch.tensor(0.37) if pick < 0.2 else (torch.rand(L, generator=g) if pick < 0.4 else None)
    # dropout on the weights: the reference draws its mask with F.dropout on the padded [B, H, N, N]
    # weights - its only use of the generator - so the same seed and shape reproduce the mask here
    drop = rng.choice([0.0, 0.0, 0.0, 0.1, 0.5])
    keep = None
    if drop > 0:
        seed = rng.randrange(10 ** 9)
        torch.manual_seed(seed)
        dense = torch.nn.functional.dropout(torch.ones(B, H, N, N), drop, True) != 0
        keep = torch.zeros(L, H, N, dtype=torch.bool)
        for b in range(B):
            n = min(int(lengths[b]), N)
            keep[int(offs[b]):int(offs[b]) + n] = dense[b, :, :n].transpose(0, 1)
        torch.manual_seed(seed)
    want = ref.pytorch_hstu_mha(N, 0.25, q, k, v, offs, True, drop, drop > 0, nt, sc, W, ctx, F)
    want.backward(dout)
    wg = [t.grad.clone() for t in (q, k, v)]
    for t in (q, k, v):
        t.grad = None
    got = O.hstu_mha(N, 0.25, q, k, v, offs, num_targets=nt, attn_scale=sc, max_attn_len=W, contextual_seq_len=ctx,
                     min_full_attn_seq_len=F, dropout_pr=drop, dropout_keep=keep)
    got.backward(dout)
    e = max([_max_diff(got, want)] + [_max_diff(t.grad, w_) for t, w_ in zip((q, k, v), wg)])
    return e, ("attention", N, lengths.tolist(), None if nt is None else nt.tolist(), ctx, W, F, drop)


def cached_case(rng, ref):
    g = torch.Generator().manual_seed(rng.randrange(10 ** 9))
    N, B, delta = rng.choice([24, 40, 64]), rng.randint(1, 4), rng.choice([1, 3, 8])
    ctx, W = rng.choice([0, 0, 2, 5]), rng.choice([0, 0, 4, 20])
    lengths = torch.randint(delta + ctx + 1, N + 1, (B,), generator=g)
    nt = None
    if rng.random() < 0.6:
        nt = torch.minimum(torch.randint(0, delta + 3, (B,), generator=g), lengths - ctx - 1)
    offs = _offsets(lengths)
    L = int(offs[-1])
    dq = torch.randn(B * delta, 2, 8, generator=g)
    k = torch.randn(L, 2, 8, generator=g)
    v = torch.randn(L, 2, 4, generator=g)
    want = ref.pytorch_cached_hstu_mha(N, 0.3, dq, k, v, offs, nt, W, ctx)
    got = O.delta_hstu_mha(N, 0.3, dq, k, v, offs, nt, W, ctx)
    return _max_diff(got, want), ("cached", N, delta, ctx, W, lengths.tolist(), None if nt is None else nt.tolist())


def output_case(rng, lin):
    g = torch.Generator().manual_seed(rng.randrange(10 ** 9))
    rows, H, V, D = rng.randint(1, 30), rng.choice([1, 2, 3]), rng.choice([4, 8]), rng.choice([6, 16])
    cu, cx = rng.choice([(True, True), (False, False), (True, False), (False, True)])
    act = rng.choice(["none", "silu", "sigmoid"])
    gn = rng.random() < 0.3
    mult = 1 if (gn and cu != cx) else 1 + int(cu) + int(cx)
    attn, u = (torch.randn(rows, H * V, generator=g, requires_grad=True) for _ in range(2))
    x = torch.randn(rows, D, generator=g, requires_grad=True)
    nw, nb = (torch.randn(H if gn else H * V, generator=g, requires_grad=True) for _ in range(2))
    Wo = torch.randn(mult * H * V, D, generator=g, requires_grad=True)
    dout = torch.randn(rows, D, generator=g)
    leaves = (attn, u, x, nw, nb, Wo)
    want = lin.pytorch_hstu_compute_output(attn, u, x, nw, nb, Wo, 1e-6, 0.0, False, concat_u=cu, concat_x=cx,
                                           mul_u_activation_type=act, group_norm=gn, num_heads=H, linear_dim=V)
    want.backward(dout)
    wg = [t.grad.clone() for t in leaves]
    for t in leaves:
        t.grad = None
    got = O.hstu_compute_output(attn, u, x, nw, nb, 1e-6, Wo, H, V, cu, cx, act, gn)
    got.backward(dout)
    e = max([_max_diff(got, want)] + [_max_diff(t.grad, w_) for t, w_ in zip(leaves, wg)])
    return e, ("output", rows, H, V, D, cu, cx, act, gn)


def uqvk_case(rng, ops, kernel):
    g = torch.Generator().manual_seed(rng.randrange(10 ** 9))
    rows, H, A, V, D = rng.randint(1, 30), rng.choice([1, 2]), rng.choice([4, 8]), rng.choice([4, 12]), rng.choice([6, 16])
    x = torch.randn(rows, D, generator=g)
    nw, nb = torch.randn(D, generator=g), torch.randn(D, generator=g)
    Wt = torch.randn(D, 2 * H * (A + V), generator=g)
    b = torch.randn(2 * H * (A + V), generator=g)
    want = ops.hstu_compute_uqvk(x, nw, nb, 1e-6, H, A, V, Wt, b, kernel)
    got = O.hstu_compute_uqvk(x, nw, nb, 1e-6, H, A, V, Wt, b)
    return max(_max_diff(a.reshape(-1), w_.reshape(-1)) for a, w_ in zip(got, want)), ("uqvk", rows, H, A, V, D)


def jagged_case(rng, jag):
    g = torch.Generator().manual_seed(rng.randrange(10 ** 9))
    B, D = rng.randint(1, 8), rng.choice([1, 5, 16])
    kind = rng.choice(["jagged_jagged", "dense_right", "dense_left", "l2"])
    if kind == "l2":
        ctx = rng.choice([0, 2, 3])
        lp = torch.randint(0, 9, (B,), generator=g)
        l2 = torch.randint(ctx, ctx + 7, (B,), generator=g)
        po, lo = _offsets(lp), _offsets(l2)
        prefix_x = torch.randn(int(po[-1]), D, generator=g)
        l2_x = torch.randn(int(lo[-1]), D, generator=g)
        want = jag.pytorch_hstu_concat_l2_embeddings(max_prefix_len=9, prefix_x=prefix_x, prefix_offsets=po,
                                                     max_l2_len=ctx + 7, l2_x=l2_x, l2_offsets=lo,
                                                     contextual_seq_len=ctx)
        wp, wl = jag.pytorch_hstu_split_l2_embeddings(max_seq_len=9 + ctx + 7, x=want, prefix_offsets=po,
                                                      l2_offsets=lo, contextual_seq_len=ctx)
        got = O.hstu_concat_l2_embeddings(prefix_x, po, l2_x, lo, ctx)
        gp, gl = O.hstu_split_l2_embeddings(want, po, lo, ctx)
        ok = torch.equal(got, want) and torch.equal(gp, wp) and torch.equal(gl, wl)
        return (0.0 if ok else 1.0), ("jagged", kind, ctx, lp.tolist(), l2.tolist())
    max_l, max_r = 9, 7
    ll = torch.randint(0, max_l + 1, (B,), generator=g)
    lr = torch.randint(0, max_r + 1, (B,), generator=g)
    if kind == "dense_right":
        max_r = rng.randint(1, 5)
        lr = torch.full((B,), max_r)
    if kind == "dense_left":
        max_l = rng.randint(1, 5)
        ll = torch.full((B,), max_l)
    ol, orr = _offsets(ll), _offsets(lr)
    left = torch.randn(int(ol[-1]), D, generator=g)
    right = torch.randn(int(orr[-1]), D, generator=g)
    kw = dict(max_len_left=max_l, max_len_right=max_r, offsets_left=None if kind == "dense_left" else ol,
              offsets_right=None if kind == "dense_right" else orr)
    want = jag.pytorch_concat_2D_jagged(values_left=left, values_right=right, **kw)
    wl, wr = jag.pytorch_split_2D_jagged(max_seq_len=max_l + max_r, values=want, **kw)
    got = O.concat_2D_jagged(left, right, **kw)
    gl, gr_ = O.split_2D_jagged(want, **kw)
    ok = torch.equal(got, want) and torch.equal(gl, wl) and torch.equal(gr_, wr)
    return (0.0 if ok else 1.0), ("jagged", kind, ll.tolist(), lr.tolist())


def position_case(rng, pos, kernel):
    g = torch.Generator().manual_seed(rng.randrange(10 ** 9))
    B, D, N = rng.randint(1, 6), rng.choice([8, 32]), 40
    ctx = rng.choice([0, 2, 3])
    fn = rng.choice(["sqrt", "log"])
    targets = rng.random() < 0.7
    interleave = targets and rng.random() < 0.3
    nt = torch.randint(1, 4, (B,), generator=g)
    lengths = torch.randint(2, 20, (B,), generator=g) + nt * (2 if interleave else 1) + ctx
    if not targets:
        # without num_targets the reference indexes the position table with negative numbers past the
        # end of a sequence: only full-length sequences run there
        lengths = torch.full((B,), N)
    offsets = _offsets(lengths)
    total = int(offsets[-1])
    x = torch.randn(total, D, generator=g)
    gaps = (torch.rand(total, generator=g) * 12).exp().long()
    ts = torch.cat([torch.cumsum(gaps[int(offsets[b]):int(offsets[b + 1])], 0) + 1_700_000_000 for b in range(B)])
    pos_w = torch.randn(N + ctx + 1, D, generator=g) * 0.3
    ts_w = torch.randn(D + 17, D, generator=g) * 0.3
    want = pos.add_timestamp_positional_embeddings(
        alpha=D ** 0.5, max_seq_len=N, max_contextual_seq_len=ctx, position_embeddings_weight=pos_w,
        timestamp_embeddings_weight=ts_w, seq_offsets=offsets, seq_lengths=lengths, seq_embeddings=x, timestamps=ts,
        num_targets=nt if targets else None, interleave_targets=interleave, time_bucket_fn=fn, kernel=kernel)
    got = O.add_timestamp_positional_embeddings(D ** 0.5, ctx, pos_w, ts_w, offsets, lengths, x, ts,
                                                nt if targets else None, interleave, fn)
    return _max_diff(got, want), ("position", fn, ctx, targets, interleave, lengths.tolist())


def layer_case(rng, stu, kernel):
    """One STULayer of the reference (eval mode, PyTorch kernels) against ``stu_layer``: output, input
    gradient and every parameter gradient."""
    seed = rng.randrange(10 ** 9)
    torch.manual_seed(seed)
    g = torch.Generator().manual_seed(seed)
    D, H, A = rng.choice([8, 32]), rng.choice([1, 2]), rng.choice([4, 16])
    ctx, W, ta = rng.choice([0, 0, 3]), rng.choice([0, 0, 9]), rng.random() < 0.7
    cfg = stu.STULayerConfig(embedding_dim=D, num_heads=H, hidden_dim=A, attention_dim=A, output_dropout_ratio=0.0,
                             causal=True, target_aware=ta, max_attn_len=W, attn_alpha=None, use_group_norm=False,
                             recompute_normed_x=False, recompute_uvqk=False, recompute_y=False, sort_by_length=False,
                             contextual_seq_len=ctx)
    layer = stu.STULayer(cfg, is_inference=False)
    layer.recursive_setattr("_hammer_kernel", kernel)
    layer.eval()
    for p_ in layer.parameters():
        if p_.dim() == 1:
            p_.data.add_(torch.randn(p_.shape, generator=g) * 0.1)
    B, N = rng.randint(1, 4), 48
    nt = torch.randint(1, 6, (B,), generator=g)
    lengths = torch.randint(1, 30, (B,), generator=g) + nt + ctx
    offs = _offsets(lengths)
    x = torch.randn(int(offs[-1]), D, generator=g, requires_grad=True)
    dy = torch.randn(int(offs[-1]), D, generator=g)
    want = layer(x=x, x_lengths=lengths, x_offsets=offs, max_seq_len=N, num_targets=nt)
    want.backward(dy)
    wdx = x.grad.clone()
    x.grad = None
    params = {n[1:]: p_.detach().clone().requires_grad_(True) for n, p_ in layer.named_parameters()}
    got = O.stu_layer(x, offs, N, nt if ta else None, params, H, A, A, max_attn_len=W, contextual_seq_len=ctx)
    got.backward(dy)
    e = max([_max_diff(got, want), _max_diff(x.grad, wdx)] +
            [_scaled_diff(params[n[1:]].grad, p_.grad) for n, p_ in layer.named_parameters()])
    return e, ("layer", D, H, A, ctx, W, ta, lengths.tolist(), nt.tolist())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--cases", type=int, default=3000)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()
    reference_shims.import_reference(args.reference)
    from generative_recommenders.common import HammerKernel
    from generative_recommenders.ops import hstu_compute as ref_ops
    from generative_recommenders.ops.pytorch import pt_hstu_attention as ref_attn
    from generative_recommenders.ops.pytorch import pt_hstu_linear as ref_lin
    from generative_recommenders.ops.pytorch import pt_jagged_tensors as ref_jag
    from generative_recommenders.ops import position as ref_pos
    from generative_recommenders.modules import stu as ref_stu

    torch.set_num_threads(4)
    rng = random.Random(args.seed)
    kinds = [lambda: attention_case(rng, ref_attn)] * 3 + [lambda: cached_case(rng, ref_attn),
                                                           lambda: output_case(rng, ref_lin),
                                                           lambda: uqvk_case(rng, ref_ops, HammerKernel.PYTORCH),
                                                           lambda: jagged_case(rng, ref_jag),
                                                           lambda: layer_case(rng, ref_stu, HammerKernel.PYTORCH),
                                                           lambda: position_case(rng, ref_pos, HammerKernel.PYTORCH)]
    worst, bad, done = {}, 0, 0
    for _ in range(args.cases):
        r = rng.choice(kinds)()
        if r is None:
            continue
        e, what = r
        done += 1
        worst[what[0]] = max(worst.get(what[0], 0.0), e)
        if not e <= (1e-4 if what[0] == "layer" else 1e-5):
            bad += 1
            print("MISMATCH", e, what)
    print("cases %d, mismatches %d, largest difference per kind: %s" % (done, bad, worst))
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
