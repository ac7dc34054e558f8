"""Generate the golden fixtures in this directory by running the UNMODIFIED reference.

Usage (needs a checkout of meta-recsys/generative-recommenders; not shipped here):

    python tests/golden/make_golden.py --reference /path/to/generative-recommenders

The reference ships no golden vectors for the HSTU attention path, so the fixtures
written here - outputs of its own PyTorch implementation
(generative_recommenders/ops/pytorch/*, generative_recommenders/modules/stu.py) on
seeded inputs - are what pins the CPU restatement in ``oracle/hstu_oracle.py`` and,
through it, the CUDA kernels.  Inputs are stored next to the outputs so the fixtures
do not depend on a random-number generator.
"""

import argparse
import itertools
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import reference_shims  # noqa: E402


def _lengths(g, B, lo, hi):
    return torch.randint(lo, hi + 1, (B,), generator=g)


def _offsets(lengths):
    return torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(lengths, 0)])


def attention_cases():
    """(name, dict of scalar params) for the attention fixtures."""
    cases = []
    # the CPU-runnable benchmark configuration: B=16, L~U[1,256], N=256, H=2, d=32, causal only
    cases.append(("cfg0", dict(seed=20260, B=16, lo=1, hi=256, N=256, H=2, A=32, V=32, std=1.0,
                               targets=0, ctx=0, W=0, F=0, alpha=1.0 / 32, grads=False)))
    base = dict(B=5, lo=1, hi=80, N=80, H=2, A=16, V=16, std=1.0, alpha=0.25, grads=True)
    variants = [
        ("causal", dict(targets=0, ctx=0, W=0, F=0)),
        ("targets", dict(targets=9, ctx=0, W=0, F=0)),
        ("ctx", dict(targets=0, ctx=5, W=0, F=0)),
        ("window", dict(targets=0, ctx=0, W=11, F=0)),
        ("targets_ctx", dict(targets=9, ctx=5, W=0, F=0)),
        ("targets_window", dict(targets=9, ctx=0, W=11, F=0)),
        ("ctx_window", dict(targets=0, ctx=5, W=11, F=0)),
        ("all", dict(targets=9, ctx=5, W=11, F=0)),
        ("all_fullattn", dict(targets=9, ctx=5, W=11, F=7)),
        ("window_fullattn", dict(targets=0, ctx=0, W=6, F=13)),
    ]
    for i, (nm, v) in enumerate(variants):
        d = dict(base)
        d.update(v)
        d["seed"] = 777 + i
        cases.append((nm, d))
    # different qk / v head dims, one head, lengths above one 128-row tile
    cases.append(("two_tiles", dict(seed=900, B=3, lo=100, hi=300, N=300, H=1, A=32, V=16, std=0.5,
                                    targets=17, ctx=3, W=150, F=0, alpha=0.2, grads=True)))
    # truncation: sequences longer than max_seq_len
    cases.append(("truncate", dict(seed=901, B=4, lo=20, hi=60, N=40, H=2, A=16, V=16, std=1.0,
                                   targets=0, ctx=0, W=0, F=0, alpha=0.25, grads=False)))
    # truncation together with what depends on the sequence length: the reference takes max_ids from
    # the untruncated lengths (pt_hstu_attention.py:44), so targets, the contextual prefix and the
    # full-attention tail of a truncated sequence refer to positions beyond max_seq_len
    trunc = dict(B=6, lo=20, hi=60, N=40, H=2, A=16, V=16, std=1.0, alpha=0.25, grads=True)
    for i, (nm, v) in enumerate([
        ("truncate_targets", dict(targets=7, ctx=0, W=0, F=0)),
        ("truncate_all", dict(targets=7, ctx=3, W=9, F=5)),
        ("truncate_window_full", dict(targets=0, ctx=0, W=6, F=9)),
        ("truncate_ctx_window", dict(targets=0, ctx=4, W=8, F=0)),
    ]):
        d = dict(trunc)
        d.update(v)
        d["seed"] = 902 + i
        cases.append((nm, d))
    return cases


def make_attention(ref_ops, name, p):
    g = torch.Generator().manual_seed(p["seed"])
    lengths = _lengths(g, p["B"], p["lo"], p["hi"])
    num_targets = None
    if p["targets"] > 0:
        num_targets = torch.randint(1, p["targets"] + 1, (p["B"],), generator=g)
        # history + contextual must stay non-empty: lengths are history + ctx + targets
        lengths = lengths + num_targets + p["ctx"]
        lengths = torch.clamp(lengths, max=p["N"]) if not name.startswith("truncate") else lengths
        num_targets = torch.minimum(num_targets, torch.clamp(lengths - p["ctx"] - 1, min=0))
    elif p["ctx"] > 0:
        lengths = lengths + p["ctx"]
        lengths = torch.clamp(lengths, max=p["N"]) if not name.startswith("truncate") else lengths
    offsets = _offsets(lengths)
    L = int(offsets[-1])
    q = (torch.randn(L, p["H"], p["A"], generator=g) * p["std"]).requires_grad_(True)
    k = (torch.randn(L, p["H"], p["A"], generator=g) * p["std"]).requires_grad_(True)
    v = (torch.randn(L, p["H"], p["V"], generator=g) * p["std"]).requires_grad_(True)
    dout = torch.randn(L, p["H"], p["V"], generator=g)
    out = ref_ops.pytorch_hstu_mha(
        max_seq_len=p["N"], alpha=p["alpha"], q=q, k=k, v=v, seq_offsets=offsets, causal=True,
        dropout_pr=0.0, training=False, num_targets=num_targets, max_attn_len=p["W"],
        contextual_seq_len=p["ctx"], min_full_attn_seq_len=p["F"],
    )
    fx = dict(params=p, seq_offsets=offsets, num_targets=num_targets,
              q=q.detach(), k=k.detach(), v=v.detach(), out=out.detach())
    if p["grads"]:
        out.backward(dout)
        fx.update(dout=dout, dq=q.grad, dk=k.grad, dv=v.grad)
    return fx


def make_masks(ref_ops):
    """Reference masks for a grid of (L, targets, ctx, W, F), stored as uint8 [L, L]."""
    out = []
    N = 24
    # lengths 29 and 41 exceed N: the sequence is truncated to N rows while max_ids keeps the full length
    for L, t, c, W, Fm in itertools.product([1, 2, 7, 13, 24, 29, 41], [None, 0, 1, 4], [0, 1, 3], [0, 1, 5],
                                            [0, 2, 6]):
        if W == 0 and Fm > 0:
            continue
        tt = 0 if t is None else t
        if L - tt - c < 0:
            continue
        m = ref_ops._get_valid_attn_mask(
            device=torch.device("cpu"), causal=True, N=N,
            seq_lengths=torch.tensor([L]),
            num_targets=None if t is None else torch.tensor([t]),
            max_attn_len=W, contextual_seq_len=c, min_full_attn_seq_len=Fm,
        )
        Lt = min(L, N)
        out.append(dict(L=L, t=t, c=c, W=W, F=Fm, mask=m.expand(1, N, N)[0, :Lt, :Lt].to(torch.uint8).clone()))
    return out


def make_stages(gr):
    from generative_recommenders.ops.pytorch.pt_hstu_linear import pytorch_hstu_compute_output
    from generative_recommenders.ops.pytorch.pt_layer_norm import pytorch_layer_norm
    from generative_recommenders.ops.hstu_compute import hstu_compute_uqvk
    from generative_recommenders.common import HammerKernel

    g = torch.Generator().manual_seed(4242)
    fx = {}
    # layer norm
    x = torch.randn(37, 48, generator=g) * 2 + 0.5
    w = torch.randn(48, generator=g)
    b = torch.randn(48, generator=g)
    xr = x.clone().requires_grad_(True); wr = w.clone().requires_grad_(True); br = b.clone().requires_grad_(True)
    y = pytorch_layer_norm(xr, [48], wr, br, 1e-5)
    dy = torch.randn(37, 48, generator=g)
    y.backward(dy)
    fx["layer_norm"] = dict(x=x, w=w, b=b, eps=1e-5, y=y.detach(), dy=dy, dx=xr.grad, dw=wr.grad, db=br.grad)
    # uqvk
    H, A, V, D, L = 2, 16, 24, 40, 29
    x = torch.randn(L, D, generator=g)
    nw = torch.randn(D, generator=g); nb = torch.randn(D, generator=g)
    W = torch.randn(D, 2 * H * (A + V), generator=g) * 0.2
    bias = torch.randn(2 * H * (A + V), generator=g) * 0.1
    leaves = [t.clone().requires_grad_(True) for t in (x, nw, nb, W, bias)]
    u, q, k, v = hstu_compute_uqvk(leaves[0], leaves[1], leaves[2], 1e-6, H, A, V, leaves[3], leaves[4],
                                   kernel=HammerKernel.PYTORCH)
    du = torch.randn(u.shape, generator=g); dq = torch.randn(q.shape, generator=g)
    dk = torch.randn(k.shape, generator=g); dv = torch.randn(v.shape, generator=g)
    torch.autograd.backward([u, q, k, v], [du, dq, dk, dv])
    fx["uqvk"] = dict(H=H, A=A, V=V, x=x, nw=nw, nb=nb, W=W, bias=bias, eps=1e-6,
                      u=u.detach(), q=q.detach().clone(), k=k.detach().clone(), v=v.detach().clone(),
                      du=du, dq=dq, dk=dk, dv=dv, grads=[t.grad for t in leaves])
    # compute_output, all layout variants
    H, V, D, L = 2, 24, 40, 31
    outs = []
    for concat_u, concat_x, act, gn in itertools.product([False, True], [False, True], ["none", "sigmoid", "silu"], [False, True]):
        if gn and (concat_u != concat_x):
            continue  # the reference's group-norm branch only concatenates when both are set
        mult = 1 + int(concat_u) + int(concat_x)
        attn = torch.randn(L, H * V, generator=g)
        u = torch.randn(L, H * V, generator=g)
        x = torch.randn(L, D, generator=g)
        nw = torch.randn(H if gn else H * V, generator=g); nb = torch.randn(H if gn else H * V, generator=g)
        Wo = torch.randn(mult * H * V, D, generator=g) * 0.2
        leaves = [t.clone().requires_grad_(True) for t in (attn, u, x, nw, nb, Wo)]
        o = pytorch_hstu_compute_output(
            attn=leaves[0], u=leaves[1], x=leaves[2], norm_weight=leaves[3], norm_bias=leaves[4],
            output_weight=leaves[5], eps=1e-6, dropout_ratio=0.0, training=False, concat_u=concat_u,
            concat_x=concat_x, mul_u_activation_type=act, group_norm=gn, num_heads=H, linear_dim=V)
        do = torch.randn(o.shape, generator=g)
        o.backward(do)
        outs.append(dict(concat_u=concat_u, concat_x=concat_x, act=act, group_norm=gn, H=H, V=V,
                         attn=attn, u=u, x=x, nw=nw, nb=nb, Wo=Wo, eps=1e-6, out=o.detach(), dout=do,
                         grads=[t.grad for t in leaves]))
    fx["compute_output"] = outs
    return fx


def make_layer(gr):
    from generative_recommenders.modules.stu import STULayer, STULayerConfig, STUStack
    from generative_recommenders.common import HammerKernel

    torch.manual_seed(31337)
    g = torch.Generator().manual_seed(31337)
    cfgs = []
    for (ctx, W, ta) in [(0, 0, True), (3, 9, True), (0, 0, False)]:
        cfg = STULayerConfig(embedding_dim=32, num_heads=2, hidden_dim=16, attention_dim=16,
                             output_dropout_ratio=0.0, causal=True, target_aware=ta, max_attn_len=W,
                             attn_alpha=None, use_group_norm=False, recompute_normed_x=False,
                             recompute_uvqk=False, recompute_y=False, sort_by_length=False,
                             contextual_seq_len=ctx)
        stack = STUStack([STULayer(cfg, is_inference=False), STULayer(cfg, is_inference=False)], is_inference=False)
        stack.recursive_setattr("_hammer_kernel", HammerKernel.PYTORCH)
        stack.eval()
        for p_ in stack.parameters():  # non-trivial norm weights / biases
            if p_.dim() == 1:
                p_.data.add_(torch.randn(p_.shape, generator=g) * 0.1)
        B, N = 4, 48
        num_targets = torch.randint(1, 6, (B,), generator=g)
        lengths = torch.randint(1, 30, (B,), generator=g) + num_targets + ctx
        offsets = _offsets(lengths)
        x = torch.randn(int(offsets[-1]), 32, generator=g).requires_grad_(True)
        y = stack(x=x, x_lengths=lengths, x_offsets=offsets, max_seq_len=N, num_targets=num_targets)
        dy = torch.randn(y.shape, generator=g)
        y.backward(dy)
        cfgs.append(dict(ctx=ctx, W=W, target_aware=ta, H=2, A=16, V=16, D=32, N=N,
                         state={k_: v_.detach().clone() for k_, v_ in stack.state_dict().items()},
                         param_grads={k_: v_.grad.clone() for k_, v_ in stack.named_parameters()},
                         lengths=lengths, seq_offsets=offsets, num_targets=num_targets,
                         x=x.detach(), y=y.detach(), dy=dy, dx=x.grad))
    return cfgs


def make_delta(ref_ops):
    g = torch.Generator().manual_seed(99)
    B, N, H, A, V, delta = 4, 64, 2, 16, 16, 5
    num_targets = torch.full((B,), delta, dtype=torch.int64)
    lengths = torch.randint(3, 40, (B,), generator=g) + delta + 2
    offsets = _offsets(lengths)
    L = int(offsets[-1])
    k = torch.randn(L, H, A, generator=g); v = torch.randn(L, H, V, generator=g)
    dq = torch.randn(B * delta, H, A, generator=g)
    out = ref_ops.pytorch_cached_hstu_mha(max_seq_len=N, alpha=0.25, delta_q=dq, k=k, v=v, seq_offsets=offsets,
                                          num_targets=num_targets, max_attn_len=0, contextual_seq_len=2)
    return dict(N=N, alpha=0.25, delta_q=dq, k=k, v=v, seq_offsets=offsets, num_targets=num_targets,
                ctx=2, out=out)


def make_bias():
    """Bucket function + Toeplitz construction of the research relative bias."""
    from generative_recommenders.research.modeling.sequential.hstu import (
        RelativeBucketedTimeAndPositionBasedBias,
    )
    torch.manual_seed(5)
    N = 40
    mod = RelativeBucketedTimeAndPositionBasedBias(
        max_seq_len=N, num_buckets=128,
        bucketization_fn=lambda x: (torch.log(torch.abs(x).clamp(min=1)) / 0.301).long())
    # timestamps = positions: ts(next item) - ts(item) is then a pure position distance
    ts = torch.arange(N).view(1, N) * 7
    with torch.no_grad():
        mod._pos_w.zero_()
        rab = mod(ts)
    return dict(N=N, ts_w=mod._ts_w.detach().clone(), timestamps=ts, rab=rab[0].clone())


def make_bias_attention():
    """The research model's attention with a learnable relative position bias
    (research/modeling/sequential/hstu.py: ``RelativePositionalBias`` :65-83,
    ``_hstu_attention_maybe_from_cache`` :150-229): output, and the gradients of q, k, v and of
    the bias weights ``_w`` (one weight per signed distance).  The mask is plain causal."""
    from generative_recommenders.research.modeling.sequential.hstu import (
        RelativePositionalBias,
        _hstu_attention_maybe_from_cache,
    )
    g = torch.Generator().manual_seed(31)
    torch.manual_seed(31)
    N, H, A, V = 48, 2, 16, 16
    lengths = torch.tensor([48, 7, 30, 1, 19])
    offsets = _offsets(lengths)
    L = int(offsets[-1])
    q = torch.randn(L, H * A, generator=g).requires_grad_(True)
    k = torch.randn(L, H * A, generator=g).requires_grad_(True)
    v = torch.randn(L, H * V, generator=g).requires_grad_(True)
    dout = torch.randn(L, H * V, generator=g)
    mod = RelativePositionalBias(max_seq_len=N)
    with torch.no_grad():
        mod._w.mul_(20.0)   # std 0.4: large enough to matter next to q.k
    causal = torch.tril(torch.ones(N, N))
    ts = torch.zeros(len(lengths), N, dtype=torch.int64)
    out, _, _ = _hstu_attention_maybe_from_cache(
        num_heads=H, attention_dim=A, linear_dim=V, q=q, k=k, v=v, cached_q=None, cached_k=None,
        delta_x_offsets=None, x_offsets=offsets, all_timestamps=ts, invalid_attn_mask=causal,
        rel_attn_bias=mod)
    out.backward(dout)
    with torch.no_grad():
        rab = mod(ts)[0].clone()
    return dict(N=N, H=H, A=A, V=V, seq_offsets=offsets, q=q.detach().clone(), k=k.detach().clone(),
                v=v.detach().clone(), dout=dout, w=mod._w.detach().clone(), rab=rab, out=out.detach().clone(),
                dq=q.grad.clone(), dk=k.grad.clone(), dv=v.grad.clone(), dw=mod._w.grad.clone())


def make_jagged(gr):
    """concat_2D_jagged / split_2D_jagged and add_timestamp_positional_embeddings of the reference's
    PyTorch implementations."""
    from generative_recommenders.ops.pytorch.pt_jagged_tensors import (
        pytorch_concat_2D_jagged,
        pytorch_split_2D_jagged,
    )
    from generative_recommenders.ops.position import add_timestamp_positional_embeddings
    from generative_recommenders.common import HammerKernel

    g = torch.Generator().manual_seed(4242)
    fx = dict(concat=[], split=[], ts_pos=[])
    B, D = 6, 24
    for kind in ("jagged_jagged", "dense_right", "dense_left", "with_empty"):
        ll = torch.randint(0 if kind == "with_empty" else 1, 9, (B,), generator=g)
        lr = torch.randint(0 if kind == "with_empty" else 1, 7, (B,), generator=g)
        max_l, max_r = 9, 7
        if kind == "dense_right":
            lr = torch.full((B,), 4); max_r = 4
        if kind == "dense_left":
            ll = torch.full((B,), 3); max_l = 3
        ol, orr = _offsets(ll), _offsets(lr)
        left = torch.randn(int(ol[-1]), D, generator=g)
        right = torch.randn(int(orr[-1]), D, generator=g)
        kw = dict(max_len_left=max_l, max_len_right=max_r,
                  offsets_left=None if kind == "dense_left" else ol,
                  offsets_right=None if kind == "dense_right" else orr)
        out = pytorch_concat_2D_jagged(values_left=left, values_right=right, **kw)
        fx["concat"].append(dict(kind=kind, left=left, right=right, out=out, **kw))
        sl, sr = pytorch_split_2D_jagged(max_seq_len=max_l + max_r, values=out, **kw)
        fx["split"].append(dict(kind=kind, values=out, left=sl, right=sr, **kw))
    from generative_recommenders.ops.pytorch.pt_jagged_tensors import (
        pytorch_hstu_concat_l2_embeddings,
        pytorch_hstu_split_l2_embeddings,
    )
    fx["l2"] = []
    for ctx in (0, 3):
        B, D = 6, 16
        lp = torch.randint(0, 9, (B,), generator=g)
        l2 = torch.randint(ctx, ctx + 7, (B,), generator=g)
        po, lo = _offsets(lp), _offsets(l2)
        prefix_x = torch.randn(int(po[-1]), D, generator=g)
        l2_x = torch.randn(int(lo[-1]), D, generator=g)
        x = pytorch_hstu_concat_l2_embeddings(max_prefix_len=9, prefix_x=prefix_x, prefix_offsets=po,
                                              max_l2_len=ctx + 7, l2_x=l2_x, l2_offsets=lo, contextual_seq_len=ctx)
        sp, sl = pytorch_hstu_split_l2_embeddings(max_seq_len=9 + ctx + 7, x=x, prefix_offsets=po, l2_offsets=lo,
                                                  contextual_seq_len=ctx)
        fx["l2"].append(dict(ctx=ctx, prefix_x=prefix_x, l2_x=l2_x, prefix_offsets=po, l2_offsets=lo, x=x,
                             split_prefix=sp, split_l2=sl))
    for i, (targets, interleave, fn, ctx, dtype) in enumerate([
            (False, False, "sqrt", 0, torch.float32), (True, False, "sqrt", 0, torch.float32),
            (True, True, "sqrt", 0, torch.float32), (True, False, "log", 3, torch.float32),
            (False, False, "log", 2, torch.float32), (True, False, "sqrt", 3, torch.bfloat16)]):
        B, D, N = 5, 32, 40
        nt = torch.randint(1, 4, (B,), generator=g)
        lengths = torch.randint(2, 20, (B,), generator=g) + nt * (2 if interleave else 1) + ctx
        if not targets:
            # without num_targets the reference indexes the position table with seq_length - column for
            # every padded column, which is negative past the end of a sequence: only full-length
            # sequences run there
            lengths = torch.full((B,), N)
        offsets = _offsets(lengths)
        total = int(offsets[-1])
        x = torch.randn(total, D, generator=g).to(dtype)
        # increasing timestamps per sequence, gaps from seconds to weeks
        gaps = (torch.rand(total, generator=g) * 12).exp().long()
        ts = torch.cat([torch.cumsum(gaps[int(offsets[b]):int(offsets[b + 1])], 0) + 1_700_000_000 for b in range(B)])
        pos_w = torch.randn(N + ctx + 1, D, generator=g) * 0.3
        ts_w = torch.randn(D + 17, D, generator=g) * 0.3  # the reference clamps buckets to size(1) - 1
        out = add_timestamp_positional_embeddings(
            alpha=D ** 0.5, max_seq_len=N, max_contextual_seq_len=ctx, position_embeddings_weight=pos_w,
            timestamp_embeddings_weight=ts_w, seq_offsets=offsets, seq_lengths=lengths, seq_embeddings=x,
            timestamps=ts, num_targets=nt if targets else None, interleave_targets=interleave,
            time_bucket_fn=fn, kernel=HammerKernel.PYTORCH)
        fx["ts_pos"].append(dict(alpha=D ** 0.5, N=N, ctx=ctx, pos_w=pos_w, ts_w=ts_w, seq_offsets=offsets,
                                 seq_lengths=lengths, x=x, timestamps=ts, num_targets=nt if targets else None,
                                 interleave=interleave, fn=fn, out=out))
    return fx


def make_cached_layer(gr):
    """STUStack.forward with kv_caching_lengths followed by cached_forward on the last delta rows
    (the flow of the reference's own test, modules/tests/stu_test.py:324-453), PyTorch kernels."""
    from generative_recommenders.modules.stu import STULayer, STULayerConfig, STUStack
    from generative_recommenders.common import HammerKernel
    from generative_recommenders.ops.pytorch.pt_jagged_tensors import pytorch_split_2D_jagged

    torch.manual_seed(777)
    g = torch.Generator().manual_seed(777)
    out = []
    for ctx in (0, 3):
        cfg = STULayerConfig(embedding_dim=32, num_heads=2, hidden_dim=16, attention_dim=16,
                             output_dropout_ratio=0.0, causal=True, target_aware=True, max_attn_len=None,
                             attn_alpha=None, use_group_norm=False, recompute_normed_x=False,
                             recompute_uvqk=False, recompute_y=False, sort_by_length=False,
                             contextual_seq_len=ctx)
        stack = STUStack([STULayer(cfg, is_inference=True), STULayer(cfg, is_inference=True)], is_inference=True)
        stack.recursive_setattr("_hammer_kernel", HammerKernel.PYTORCH)
        stack.eval()
        for p_ in stack.parameters():
            if p_.dim() == 1:
                p_.data.add_(torch.randn(p_.shape, generator=g) * 0.1)
        B, delta = 4, 5
        num_targets = torch.randint(delta, 2 * delta + 1, (B,), generator=g)
        lengths = torch.randint(4, 30, (B,), generator=g) + num_targets + ctx
        N = 30 + 2 * delta + ctx
        offsets = _offsets(lengths)
        x = torch.randn(int(offsets[-1]), 32, generator=g)
        with torch.inference_mode():
            ref_y = stack(x=x, x_lengths=lengths, x_offsets=offsets, max_seq_len=N, num_targets=num_targets)
            prime_lengths = lengths - delta
            prime_offsets = _offsets(prime_lengths)
            _, ref_delta_y = pytorch_split_2D_jagged(max_seq_len=N, values=ref_y, max_len_left=None,
                                                     max_len_right=delta, offsets_left=prime_offsets,
                                                     offsets_right=None)
            prime_x, delta_x = pytorch_split_2D_jagged(max_seq_len=N, values=x, max_len_left=None,
                                                       max_len_right=delta, offsets_left=prime_offsets,
                                                       offsets_right=None)
            stack(x=prime_x, x_lengths=prime_lengths, x_offsets=prime_offsets, max_seq_len=N,
                  num_targets=num_targets - delta, max_kv_caching_len=N - delta,
                  kv_caching_lengths=lengths - delta)
            delta_y = stack.cached_forward(delta_x=delta_x, num_targets=num_targets)
        out.append(dict(ctx=ctx, H=2, A=16, V=16, D=32, N=N, delta=delta,
                        state={k_: v_.detach().clone() for k_, v_ in stack.state_dict().items()},
                        lengths=lengths, seq_offsets=offsets, num_targets=num_targets, x=x,
                        full_y=ref_y.clone(), full_delta_y=ref_delta_y.clone(), cached_delta_y=delta_y.clone()))
    return out


def make_attention_dropout(ref_ops):
    """``pytorch_hstu_mha(dropout_pr > 0, training=True)``: the reference draws its mask with ``F.dropout``
    on the padded ``[B, H, N, N]`` weights - its only use of the generator - so the same seed and shape
    give the mask, which is stored next to the outputs as ``keep`` ``[L, H, N]`` (query row, head, key
    position) for an implementation that takes the mask from outside."""
    cases = []
    for i, (drop, ctx, W, with_targets) in enumerate([(0.1, 0, 0, False), (0.5, 2, 9, True), (0.3, 0, 0, True)]):
        g = torch.Generator().manual_seed(700 + i)
        B, N, H, A, V = 3, 40, 2, 8, 8
        lengths = torch.randint(4, N + 1, (B,), generator=g)
        nt = torch.randint(1, 4, (B,), generator=g) if with_targets else None
        offsets = _offsets(lengths)
        L = int(offsets[-1])
        q, k = (torch.randn(L, H, A, generator=g, requires_grad=True) for _ in range(2))
        v = torch.randn(L, H, V, generator=g, requires_grad=True)
        dout = torch.randn(L, H, V, generator=g)
        seed = 4100 + i
        torch.manual_seed(seed)
        dense = torch.nn.functional.dropout(torch.ones(B, H, N, N), drop, True) != 0
        keep = torch.zeros(L, H, N, dtype=torch.bool)
        for b in range(B):
            n = int(lengths[b])
            keep[int(offsets[b]):int(offsets[b]) + n] = dense[b, :, :n].transpose(0, 1)
        torch.manual_seed(seed)
        out = ref_ops.pytorch_hstu_mha(N, 0.3, q, k, v, offsets, True, drop, True, nt, None, W, ctx, 0)
        out.backward(dout)
        cases.append(dict(N=N, alpha=0.3, q=q.detach(), k=k.detach(), v=v.detach(), seq_offsets=offsets, num_targets=nt,
                          max_attn_len=W, ctx=ctx, dropout_pr=drop, keep=keep, dout=dout, out=out.detach(),
                          dq=q.grad.clone(), dk=k.grad.clone(), dv=v.grad.clone()))
    return cases


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--only", default="", help="comma-separated fixture names to (re)generate; default all")
    args = ap.parse_args()
    only = set(filter(None, args.only.split(",")))
    gr = reference_shims.import_reference(args.reference)
    from generative_recommenders.ops.pytorch import pt_hstu_attention as ref_ops

    torch.set_num_threads(4)

    def want(name):
        return not only or name in only

    if want("attention"):
        attn = {}
        for name, p in attention_cases():
            attn[name] = make_attention(ref_ops, name, p)
            print("attention", name, tuple(attn[name]["q"].shape))
        torch.save(attn, os.path.join(HERE, "attention.pt"))
    for name, fn in (("masks", lambda: make_masks(ref_ops)), ("stages", lambda: make_stages(gr)),
                     ("stu_layer", lambda: make_layer(gr)), ("delta_attention", lambda: make_delta(ref_ops)),
                     ("rel_bias", make_bias), ("rel_bias_attention", make_bias_attention),
                     ("jagged", lambda: make_jagged(gr)),
                     ("stu_cached", lambda: make_cached_layer(gr)),
                     ("attention_dropout", lambda: make_attention_dropout(ref_ops))):
        if want(name):
            torch.save(fn(), os.path.join(HERE, name + ".pt"))
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".pt"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
