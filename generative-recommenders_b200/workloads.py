"""Seeded synthetic inputs with the shapes, lengths and value distributions of the benchmark
configurations (they stand in for the reference benchmark's generator,
generative_recommenders/ops/benchmarks/hstu_attention_bench.py:217-271).  Everything is drawn on
the CPU from ``torch.Generator().manual_seed(20260 + index)`` / numpy's PCG64 with the same seed
and moved to the target device afterwards, so every box sees the same numbers."""

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch


@dataclass
class AttentionWorkload:
    name: str
    max_seq_len: int
    alpha: float
    num_heads: int
    attn_dim: int
    hidden_dim: int
    lengths: torch.Tensor            # [B] int64
    seq_offsets: torch.Tensor        # [B + 1] int64
    num_targets: Optional[torch.Tensor]
    max_attn_len: int = 0
    contextual_seq_len: int = 0
    dtype: torch.dtype = torch.bfloat16
    value_std: float = 1.0
    seed: int = 0

    @property
    def total_tokens(self) -> int:
        return int(self.seq_offsets[-1])

    def qkv(self, device="cpu", with_dout=False):
        g = torch.Generator().manual_seed(self.seed + 1000)
        L, H = self.total_tokens, self.num_heads
        q = (torch.randn(L, H, self.attn_dim, generator=g) * self.value_std).to(self.dtype).to(device)
        k = (torch.randn(L, H, self.attn_dim, generator=g) * self.value_std).to(self.dtype).to(device)
        v = (torch.randn(L, H, self.hidden_dim, generator=g) * self.value_std).to(self.dtype).to(device)
        if with_dout:
            do = torch.randn(L, H, self.hidden_dim, generator=g).to(self.dtype).to(device)
            return q, k, v, do
        return q, k, v

    def causal_flops_fwd(self) -> float:
        """4 * H * d * sum(L_i^2) / 2 - the nominal causal count."""
        l = self.lengths.to(torch.float64)
        return float(4.0 * self.num_heads * self.attn_dim * (l * l).sum() / 2.0)

    def exact_pairs(self) -> int:
        """Number of unmasked (query, key) pairs, from the closed form of the mask."""
        tot = 0
        c, W = self.contextual_seq_len, self.max_attn_len
        nts = [0] * len(self.lengths) if self.num_targets is None else self.num_targets.tolist()
        for L, t in zip(self.lengths.tolist(), nts):
            L = min(L, self.max_seq_len)
            u = L - t
            # history rows i in [c, u): see min(i - c, W or inf) history cols + self + ctx cols if visible
            n = 0
            if u > c:
                i = np.arange(c, u, dtype=np.int64)
                hist = i - c
                if W > 0:
                    hist = np.minimum(hist, W)
                    ctx = np.where(i - c + 1 <= W, c, 0)
                else:
                    ctx = np.full_like(i, c)
                n += int((hist + 1 + ctx).sum())
            # contextual rows: all of [0, u)
            n += min(c, L) * max(u, 0) if u >= c else 0
            # target rows: history cols within the window from u, ctx if visible, self
            if t > 0:
                hist = u - c
                ctxv = c
                if W > 0:
                    hist = min(hist, W)
                    ctxv = c if u - c + 1 <= W else 0
                n += t * (hist + ctxv + 1)
            tot += n
        return tot


def _offsets(lengths: torch.Tensor) -> torch.Tensor:
    return torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(lengths.to(torch.int64), 0)])


def config0() -> AttentionWorkload:
    """fp32, B=16, L ~ U{1..256}, N=256, H=2, d=32, q,k,v ~ N(0,1), alpha=1/32, causal only."""
    seed = 20260
    g = torch.Generator().manual_seed(seed)
    lengths = torch.randint(1, 257, (16,), generator=g)
    return AttentionWorkload("config0", 256, 1.0 / 32, 2, 32, 32, lengths, _offsets(lengths), None,
                             dtype=torch.float32, value_std=1.0, seed=seed)


def config1(scale_batch: int = 64) -> AttentionWorkload:
    """bf16, B=64, L ~ U{128..1024}, N=1024, H=4, d=128, q,k,v ~ N(0,1)*0.5, alpha=1/128,
    num_targets ~ U{1..32}."""
    seed = 20261
    g = torch.Generator().manual_seed(seed)
    lengths = torch.randint(128, 1025, (scale_batch,), generator=g)
    nt = torch.randint(1, 33, (scale_batch,), generator=g)
    return AttentionWorkload("config1", 1024, 1.0 / 128, 4, 128, 128, lengths, _offsets(lengths), nt,
                             dtype=torch.bfloat16, value_std=0.5, seed=seed)


def config2_lengths(batch: int = 128):
    """Power-law lengths L = clip(floor(16 * (1-u)^(-1/1.2)), 16, 4096), contextual 6,
    num_targets ~ U{1..64} clamped to L - contextual - 1."""
    seed = 20262
    g = torch.Generator().manual_seed(seed)
    u = torch.rand(batch, generator=g, dtype=torch.float64)
    lengths = torch.clamp(torch.floor(16.0 * (1.0 - u) ** (-1.0 / 1.2)), 16, 4096).to(torch.int64)
    nt = torch.randint(1, 65, (batch,), generator=g)
    nt = torch.minimum(nt, lengths - 6 - 1)
    return lengths, nt, seed


def config2_attention(batch: int = 128) -> AttentionWorkload:
    lengths, nt, seed = config2_lengths(batch)
    return AttentionWorkload("config2", 4096, 1.0 / 128 ** 0.5, 4, 128, 128, lengths, _offsets(lengths), nt,
                             contextual_seq_len=6, dtype=torch.bfloat16, value_std=1.0, seed=seed)


def config3(batch: int = 256) -> AttentionWorkload:
    """Inference: history = clip(zipf(1.1), 64, 8192-256), L = history + 256 targets, N=8192,
    H=4, d=128, q,k,v ~ N(0,1), alpha=1/128, max_attn_len=1024."""
    seed = 20263
    rng = np.random.Generator(np.random.PCG64(seed))
    hist = np.clip(rng.zipf(1.1, size=batch), 64, 8192 - 256).astype(np.int64)
    lengths = torch.from_numpy(hist + 256)
    nt = torch.full((batch,), 256, dtype=torch.int64)
    return AttentionWorkload("config3", 8192, 1.0 / 128, 4, 128, 128, lengths, _offsets(lengths), nt,
                             max_attn_len=1024, dtype=torch.bfloat16, value_std=1.0, seed=seed)


def config4(batch: int = 2048) -> AttentionWorkload:
    """Ranking-style inference: L = clip(round(exp(N(7,1))), 32, 16384), N=16384, H=8, d=128,
    num_targets=64, contextual 16."""
    seed = 20264
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(batch, generator=g, dtype=torch.float64)
    lengths = torch.clamp(torch.round(torch.exp(7.0 + z)), 32, 16384).to(torch.int64)
    # targets and the contextual prefix have to fit in the sequence
    lengths = torch.clamp(lengths, min=64 + 16 + 1)
    nt = torch.full((batch,), 64, dtype=torch.int64)
    return AttentionWorkload("config4", 16384, 1.0 / 128 ** 0.5, 8, 128, 128, lengths, _offsets(lengths), nt,
                             contextual_seq_len=16, dtype=torch.bfloat16, value_std=1.0, seed=seed)


def subset(w: AttentionWorkload, idx) -> AttentionWorkload:
    """The workload restricted to the sequences ``idx`` (same per-sequence lengths / targets)."""
    idx = torch.as_tensor(idx, dtype=torch.int64)
    lengths = w.lengths[idx]
    nt = None if w.num_targets is None else w.num_targets[idx]
    return AttentionWorkload(w.name + "_subset", w.max_seq_len, w.alpha, w.num_heads, w.attn_dim, w.hidden_dim,
                             lengths, _offsets(lengths), nt, w.max_attn_len, w.contextual_seq_len, w.dtype,
                             w.value_std, w.seed)
