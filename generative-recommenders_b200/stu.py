"""The HSTU layer as a module, composed from this package's ops.

Mirrors ``STULayer`` / ``STUStack`` of the reference
(generative_recommenders/modules/stu.py:65-81, 176-356, 427-456): same configuration fields, same
parameter names, shapes and initialisation, so a reference checkpoint loads with
``load_state_dict``.  The KV-cache path of the reference layer (``cached_forward``,
``update_kv_cache``) is not part of this module.

One extension: ``rel_bias_table`` (``num_buckets + 1`` learnable entries, indexed by
``clamp(floor(ln(max(|i - j|, 1)) / 0.301), 0, num_buckets)`` of the position distance) adds the
research model's bucketised relative bias (generative_recommenders/research/modeling/sequential/
hstu.py:86-143, 610-613 with the time bias off) to the attention scores.  The attention kernels
produce no gradient for the table.
"""

from dataclasses import dataclass
from typing import List, Optional

import torch

from .common import HammerKernel
from .hstu_compute import hstu_compute_output, hstu_preprocess_and_attention


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


def position_bias_by_distance(table: torch.Tensor, n: int) -> torch.Tensor:
    """``bias[dist] = table[bucket(dist)]`` for ``dist`` in ``[0, n)`` (fp32)."""
    nb = table.numel() - 1
    d = torch.arange(n, device=table.device, dtype=torch.float32).clamp(min=1.0)
    bucket = torch.clamp((torch.log(d) / 0.301).long(), min=0, max=nb)
    return table.to(torch.float32)[bucket].contiguous()


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
        if kv_caching_lengths is not None:
            raise NotImplementedError("KV caching is not part of this module")
        bias = None
        if self._rel_bias_table is not None:
            bias = position_bias_by_distance(self._rel_bias_table.detach(), max_seq_len)
        with torch.autograd.profiler.record_function("## stu_preprocess_and_attention ##"):
            u, attn_output, _, _ = hstu_preprocess_and_attention(
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
                recompute_uvqk_in_backward=False,
                recompute_normed_x_in_backward=False,
                sort_by_length=self._sort_by_length,
                kernel=self._hammer_kernel,
                bias_by_distance=bias,
            )
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
                recompute_y_in_backward=False,
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
