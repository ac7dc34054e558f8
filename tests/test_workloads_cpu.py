import torch

from generative_recommenders_b200 import workloads as W
from oracle import hstu_oracle as O


def test_config_shapes():
    c0 = W.config0()
    assert c0.lengths.numel() == 16 and c0.dtype == torch.float32 and int(c0.lengths.max()) <= 256
    c1 = W.config1()
    assert c1.lengths.numel() == 64 and 128 <= int(c1.lengths.min()) and int(c1.lengths.max()) <= 1024
    assert 30000 < c1.total_tokens < 45000
    c3 = W.config3(32)
    assert int(c3.lengths.min()) >= 64 + 256 and int(c3.lengths.max()) <= 8192
    c4 = W.config4(64)
    assert int(c4.lengths.max()) <= 16384


def test_exact_pair_count_matches_mask():
    g = torch.Generator().manual_seed(3)
    for ctx, Wn, tg in [(0, 0, 0), (3, 0, 5), (0, 7, 4), (4, 9, 6), (2, 30, 0)]:
        lengths = torch.randint(12, 60, (6,), generator=g)
        nt = torch.randint(0, tg + 1, (6,), generator=g) if tg else None
        w = W.AttentionWorkload("t", 64, 1.0, 1, 8, 8, lengths, W._offsets(lengths), nt, Wn, ctx)
        want = 0
        for i, L in enumerate(lengths.tolist()):
            want += int(O.valid_attn_mask(L, 0 if nt is None else int(nt[i]), nt is not None, Wn, ctx).sum())
        assert w.exact_pairs() == want, (ctx, Wn, tg)
