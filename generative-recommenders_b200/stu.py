"""The HSTU layer as a module, composed from this package's ops.

Mirrors ``STULayer`` / ``STUStack`` of the reference
(generative_recommenders/modules/stu.py:65-81, 176-356, 427-456): same configuration fields, same
parameter names, shapes and initialisation, so a reference checkpoint loads with
``load_state_dict``.  The KV-cache path of the reference layer (``update_kv_cache``,
``construct_full_kv``, ``cached_forward``; stu.py:84-173, 253-296, 358-424) is here too: a forward
with ``kv_caching_lengths`` keeps the first ``kv_caching_lengths[b]`` rows of K and V of every
sequence (a jagged split), ``cached_forward`` appends the new rows' K and V (a jagged concat) and
runs ``delta_hstu_mha`` for the new rows only.

One extension: ``rel_bias_table`` (``num_buckets + 1`` learnable entries, indexed by
``clamp(floor(ln(max(|i - j|, 1)) / 0.301), 0, num_buckets)`` of the position distance) adds the
research model's bucketised relative bias (generative_recommenders/research/modeling/sequential/
hstu.py:86-143, 610-613 with the time bias off) to the attention scores.  The table is trained like
the reference's: the attention backward returns the gradient per distance, autograd scatters it
to the buckets.
"""

from dataclasses import dataclass
from typing import List, Optional

import torch

from .common import HammerKernel
from .hstu_attention import delta_hstu_mha
from .hstu_compute import hstu_compute_output, hstu_compute_uqvk, hstu_preprocess_and_attention
from .jagged_tensors import concat_2D_jagged, split_2D_jagged


@dataclass
class STULayerConfig:
    embedding_dim: int
    num_heads: int
    hidden_dim: int
    attention_dim: int
    output_dropout_ratio: float = 0.3
    causal: bool = True
    target_aware: bool = True
    max_attn_len: Optional[int] = None
    attn_alpha: Optional[float] = None
    use_group_norm: bool = False
    recompute_normed_x: bool = True
    recompute_uvqk: bool = True
    recompute_y: bool = True
    sort_by_length: bool = True
    contextual_seq_len: int = 0
    rel_bias_buckets: int = 0  # extension: > 0 adds a bucketised relative position bias


_BUCKETS = {}  # (n, buckets, device) -> bucket index of every distance: the same for all layers and steps


class _BucketGather(torch.autograd.Function):
    """``table[bucket]`` in fp32 whose backward is one ``index_add_`` (a single kernel of atomic
    adds) instead of the sort-based scatter autograd uses for a general index."""

    @staticmethod
    def forward(ctx, table, bucket):
        ctx.save_for_backward(bucket)
        ctx.shape, ctx.dtype = table.shape, table.dtype
        return table.detach().to(torch.float32)[bucket].contiguous()

    @staticmethod
    def backward(ctx, g):
        (bucket,) = ctx.saved_tensors
        d = torch.zeros(ctx.shape, dtype=torch.float32, device=g.device)
        d.index_add_(0, bucket, g.to(torch.float32))
        return d.to(ctx.dtype), None


def position_bias_by_distance(table: torch.Tensor, n: int) -> torch.Tensor:
    """``bias[dist] = table[bucket(dist)]`` for ``dist`` in ``[0, n)`` (fp32); differentiable with
    respect to ``table``."""
    nb = table.numel() - 1
    key = (n, nb, table.device)
    bucket = _BUCKETS.get(key)
    if bucket is None:
        d = torch.arange(n, device=table.device, dtype=torch.float32).clamp(min=1.0)
        bucket = torch.clamp((torch.log(d) / 0.301).long(), min=0, max=nb)
        if len(_BUCKETS) > 64:
            _BUCKETS.clear()
        _BUCKETS[key] = bucket
    return _BucketGather.apply(table, bucket)


class STULayer(torch.nn.Module):
    def __init__(self, config: STULayerConfig, is_inference: bool = False) -> None:
        super().__init__()
        self._is_inference = is_inference
        self._hammer_kernel = HammerKernel.CUDA
        self._num_heads = config.num_heads
        self._embedding_dim = config.embedding_dim
        self._hidden_dim = config.hidden_dim
        self._attention_dim = config.attention_dim
        self._output_dropout_ratio = config.output_dropout_ratio
        self._target_aware = config.target_aware
        self._causal = config.causal
        self._max_attn_len = config.max_attn_len or 0
        self._attn_alpha = config.attn_alpha or 1.0 / (self._attention_dim ** 0.5)
        self._use_group_norm = config.use_group_norm
        self._sort_by_length = config.sort_by_length
        self._contextual_seq_len = config.contextual_seq_len
        self._recompute_normed_x = config.recompute_normed_x
        self._recompute_uvqk = config.recompute_uvqk
        self._recompute_y = config.recompute_y
        H, dv, dqk, D = self._num_heads, self._hidden_dim, self._attention_dim, self._embedding_dim
        self._uvqk_weight = torch.nn.Parameter(torch.empty((D, (dv * 2 + dqk * 2) * H)))
        torch.nn.init.xavier_uniform_(self._uvqk_weight)
        self._uvqk_beta = torch.nn.Parameter(torch.zeros((dv * 2 + dqk * 2) * H))
        self._input_norm_weight = torch.nn.Parameter(torch.ones((D,)))
        self._input_norm_bias = torch.nn.Parameter(torch.zeros((D,)))
        self._output_weight = torch.nn.Parameter(torch.empty((dv * H * 3, D)))
        torch.nn.init.xavier_uniform_(self._output_weight)
        norm_shape = dv * H if not self._use_group_norm else H
        self._output_norm_weight = torch.nn.Parameter(torch.ones((norm_shape,)))
        self._output_norm_bias = torch.nn.Parameter(torch.zeros((norm_shape,)))
        if config.rel_bias_buckets > 0:
            self._rel_bias_table = torch.nn.Parameter(
                torch.empty(config.rel_bias_buckets + 1).normal_(mean=0, std=0.02))
        else:
            self._rel_bias_table = None
        self.reset_kv_cache()

    def reset_kv_cache(self) -> None:
        self.k_cache: Optional[torch.Tensor] = None
        self.v_cache: Optional[torch.Tensor] = None
        self.kv_caching_offsets: Optional[torch.Tensor] = None
        self.max_kv_caching_len: int = 0

    def update_kv_cache(
        self,
        max_seq_len: int,
        seq_offsets: torch.Tensor,
        k: Optional[torch.Tensor],
        v: Optional[torch.Tensor],
        max_kv_caching_len: int,
        kv_caching_lengths: Optional[torch.Tensor],
    ) -> None:
        """Keep the first ``kv_caching_lengths[b]`` rows of K and V of every sequence (reference
        ``_update_kv_cache``, stu.py:84-134); without ``kv_caching_lengths`` the cache stays."""
        if kv_caching_lengths is None:
            return
        lengths = kv_caching_lengths.to(torch.int64)
        offsets = torch.zeros(lengths.numel() + 1, dtype=torch.int64, device=lengths.device)
        torch.cumsum(lengths, 0, out=offsets[1:])
        delta_offsets = seq_offsets.to(torch.int64) - offsets
        self.k_cache, _ = split_2D_jagged(max_seq_len=max_seq_len, values=k.flatten(1, 2), offsets_left=offsets,
                                          offsets_right=delta_offsets, kernel=self._hammer_kernel)
        self.v_cache, _ = split_2D_jagged(max_seq_len=max_seq_len, values=v.flatten(1, 2), offsets_left=offsets,
                                          offsets_right=delta_offsets, kernel=self._hammer_kernel)
        if max_kv_caching_len == 0:
            max_kv_caching_len = int(lengths.max().item())
        self.max_kv_caching_len = max_kv_caching_len
        self.kv_caching_offsets = offsets

    def construct_full_kv(self, delta_k: torch.Tensor, delta_v: torch.Tensor):
        """Cached K / V of every sequence followed by its ``delta_size`` new rows (reference
        ``_construct_full_kv``, stu.py:137-173); returns ``(k, v, max_seq_len, seq_offsets)``."""
        if self.k_cache is None or self.v_cache is None or self.kv_caching_offsets is None:
            raise RuntimeError("cached_forward needs a KV cache: run forward() with kv_caching_lengths first")
        L = delta_k.shape[0]
        B = self.kv_caching_offsets.numel() - 1
        delta_size = L // B
        full = []
        for cache, delta in ((self.k_cache, delta_k), (self.v_cache, delta_v)):
            full.append(concat_2D_jagged(max_seq_len=self.max_kv_caching_len + delta_size, values_left=cache,
                                         values_right=delta, max_len_left=self.max_kv_caching_len,
                                         max_len_right=delta_size, offsets_left=self.kv_caching_offsets,
                                         offsets_right=None, kernel=self._hammer_kernel))
        offsets = self.kv_caching_offsets + delta_size * torch.arange(B + 1, device=delta_k.device)
        return full[0], full[1], self.max_kv_caching_len + delta_size, offsets

    def cached_forward(
        self,
        delta_x: torch.Tensor,
        num_targets: torch.Tensor,
        max_kv_caching_len: int = 0,
        kv_caching_lengths: Optional[torch.Tensor] = None,
    ) -> torch.Tensor:
        """The layer on the last ``delta_size`` rows of every sequence against the cached K / V
        (reference stu.py:358-424); ``delta_x`` is ``[B * delta_size, D]``."""
        if self._rel_bias_table is not None:
            raise NotImplementedError("cached_forward with a relative bias table")
        with torch.autograd.profiler.record_function("## stu_compute_uqvk ##"):
            delta_u, delta_q, delta_k, delta_v = hstu_compute_uqvk(
                x=delta_x,
                norm_weight=self._input_norm_weight.to(delta_x.dtype),
                norm_bias=self._input_norm_bias.to(delta_x.dtype),
                norm_eps=1e-6,
                num_heads=self._num_heads,
                attn_dim=self._attention_dim,
                hidden_dim=self._hidden_dim,
                uvqk_weight=self._uvqk_weight.to(delta_x.dtype),
                uvqk_bias=self._uvqk_beta.to(delta_x.dtype),
                kernel=self._hammer_kernel,
            )
        k, v, max_seq_len, seq_offsets = self.construct_full_kv(
            delta_k=delta_k.flatten(1, 2), delta_v=delta_v.flatten(1, 2))
        k = k.view(-1, self._num_heads, self._attention_dim)
        v = v.view(-1, self._num_heads, self._hidden_dim)
        self.update_kv_cache(max_seq_len=max_seq_len, seq_offsets=seq_offsets, k=k, v=v,
                             max_kv_caching_len=max_kv_caching_len, kv_caching_lengths=kv_caching_lengths)
        with torch.autograd.profiler.record_function("## delta_hstu_mha ##"):
            delta_attn_output = delta_hstu_mha(
                max_seq_len=max_seq_len,
                alpha=self._attn_alpha,
                delta_q=delta_q,
                k=k,
                v=v,
                seq_offsets=seq_offsets,
                num_targets=num_targets if self._target_aware else None,
                max_attn_len=self._max_attn_len,
                contextual_seq_len=self._contextual_seq_len,
                kernel=self._hammer_kernel,
            ).view(-1, self._hidden_dim * self._num_heads)
        with torch.autograd.profiler.record_function("## stu_compute_output ##"):
            return hstu_compute_output(
                attn=delta_attn_output,
                u=delta_u,
                x=delta_x,
                norm_weight=self._output_norm_weight.to(delta_x.dtype),
                norm_bias=self._output_norm_bias.to(delta_x.dtype),
                norm_eps=1e-6,
                dropout_ratio=self._output_dropout_ratio,
                output_weight=self._output_weight.to(delta_x.dtype),
                group_norm=self._use_group_norm,
                num_heads=self._num_heads,
                linear_dim=self._hidden_dim,
                concat_u=True,
                concat_x=True,
                mul_u_activation_type="none",
                training=self.training,
                kernel=self._hammer_kernel,
                recompute_y_in_backward=False,
            )

    def forward(
        self,
        x: torch.Tensor,
        x_lengths: torch.Tensor,
        x_offsets: torch.Tensor,
        max_seq_len: int,
        num_targets: Optional[torch.Tensor],
        max_kv_caching_len: int = 0,
        kv_caching_lengths: Optional[torch.Tensor] = None,
    ) -> torch.Tensor:
        bias = None
        if self._rel_bias_table is not None:
            bias = position_bias_by_distance(self._rel_bias_table, max_seq_len)
        with torch.autograd.profiler.record_function("## stu_preprocess_and_attention ##"):
            u, attn_output, k, v = hstu_preprocess_and_attention(
                x=x,
                norm_weight=self._input_norm_weight.to(x.dtype),
                norm_bias=self._input_norm_bias.to(x.dtype),
                norm_eps=1e-6,
                num_heads=self._num_heads,
                attn_dim=self._attention_dim,
                hidden_dim=self._hidden_dim,
                uvqk_weight=self._uvqk_weight.to(x.dtype),
                uvqk_bias=self._uvqk_beta.to(x.dtype),
                max_seq_len=max_seq_len,
                seq_offsets=x_offsets,
                attn_alpha=self._attn_alpha,
                causal=self._causal,
                num_targets=num_targets if self._target_aware else None,
                max_attn_len=self._max_attn_len,
                contextual_seq_len=self._contextual_seq_len,
                recompute_uvqk_in_backward=self._recompute_uvqk,
                recompute_normed_x_in_backward=self._recompute_normed_x,
                sort_by_length=self._sort_by_length,
                kernel=self._hammer_kernel,
                bias_by_distance=bias,
            )
        self.update_kv_cache(max_seq_len=max_seq_len, seq_offsets=x_offsets, k=k, v=v,
                             max_kv_caching_len=max_kv_caching_len, kv_caching_lengths=kv_caching_lengths)
        with torch.autograd.profiler.record_function("## stu_compute_output ##"):
            return hstu_compute_output(
                attn=attn_output,
                u=u,
                x=x,
                norm_weight=self._output_norm_weight.to(x.dtype),
                norm_bias=self._output_norm_bias.to(x.dtype),
                norm_eps=1e-6,
                dropout_ratio=self._output_dropout_ratio,
                output_weight=self._output_weight.to(x.dtype),
                group_norm=self._use_group_norm,
                num_heads=self._num_heads,
                linear_dim=self._hidden_dim,
                concat_u=True,
                concat_x=True,
                mul_u_activation_type="none",
                training=self.training,
                kernel=self._hammer_kernel,
                recompute_y_in_backward=self._recompute_y,
            )


class STUStack(torch.nn.Module):
    def __init__(self, stu_list: List[STULayer], is_inference: bool = False) -> None:
        super().__init__()
        self._is_inference = is_inference
        self._stu_layers = torch.nn.ModuleList(modules=stu_list)

    def forward(
        self,
        x: torch.Tensor,
        x_lengths: torch.Tensor,
        x_offsets: torch.Tensor,
        max_seq_len: int,
        num_targets: Optional[torch.Tensor],
        max_kv_caching_len: int = 0,
        kv_caching_lengths: Optional[torch.Tensor] = None,
    ) -> torch.Tensor:
        for layer in self._stu_layers:
            x = layer(x=x, x_lengths=x_lengths, x_offsets=x_offsets, max_seq_len=max_seq_len,
                      num_targets=num_targets, max_kv_caching_len=max_kv_caching_len,
                      kv_caching_lengths=kv_caching_lengths)
        return x

    def cached_forward(
        self,
        delta_x: torch.Tensor,
        num_targets: torch.Tensor,
        max_kv_caching_len: int = 0,
        kv_caching_lengths: Optional[torch.Tensor] = None,
    ) -> torch.Tensor:
        for layer in self._stu_layers:
            delta_x = layer.cached_forward(delta_x=delta_x, num_targets=num_targets,
                                           max_kv_caching_len=max_kv_caching_len,
                                           kv_caching_lengths=kv_caching_lengths)
        return delta_x
