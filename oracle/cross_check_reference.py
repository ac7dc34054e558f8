"""Random cross-check of the restatement in ``hstu_oracle.py`` against the unmodified reference.

    python oracle/cross_check_reference.py --reference /path/to/generative-recommenders [--cases 3000] [--seed 0]

TEST INFRASTRUCTURE ONLY.  The golden fixtures pin the oracle on a fixed set of inputs; this script
draws as many more as asked for - attention forward and backward (every mask feature, targets that
reach beyond the history, sequences longer than ``max_seq_len``, empty sequences, scalar and
per-token scales), cached attention, the uvqk stage and all variants of the output stage - runs the
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
    want = ref.pytorch_hstu_mha(N, 0.25, q, k, v, offs, True, 0.0, False, nt, sc, W, ctx, F)
    want.backward(dout)
    wg = [t.grad.clone() for t in (q, k, v)]
    for t in (q, k, v):
        t.grad = None
    got = O.hstu_mha(N, 0.25, q, k, v, offs, num_targets=nt, attn_scale=sc, max_attn_len=W, contextual_seq_len=ctx,
                     min_full_attn_seq_len=F)
    got.backward(dout)
    e = max([_max_diff(got, want)] + [_max_diff(t.grad, w_) for t, w_ in zip((q, k, v), wg)])
    return e, ("attention", N, lengths.tolist(), None if nt is None else nt.tolist(), ctx, W, F)


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

    torch.set_num_threads(4)
    rng = random.Random(args.seed)
    kinds = [lambda: attention_case(rng, ref_attn)] * 3 + [lambda: cached_case(rng, ref_attn),
                                                           lambda: output_case(rng, ref_lin),
                                                           lambda: uqvk_case(rng, ref_ops, HammerKernel.PYTORCH)]
    worst, bad, done = {}, 0, 0
    for _ in range(args.cases):
        r = rng.choice(kinds)()
        if r is None:
            continue
        e, what = r
        done += 1
        worst[what[0]] = max(worst.get(what[0], 0.0), e)
        if not e <= 1e-5:
            bad += 1
            print("MISMATCH", e, what)
    print("cases %d, mismatches %d, largest difference per kind: %s" % (done, bad, worst))
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
