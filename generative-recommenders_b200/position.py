"""``add_timestamp_positional_embeddings`` with the reference's signature
(generative_recommenders/ops/position.py:40-118): the step before layer 0 of the HSTU stack,

    out[t] = alpha * seq_embeddings[t] + (ts_weight[bucket(t)] + pos_weight[index(t)])

as one sm_100a kernel per direction (csrc/jagged.cu).  ``index`` and ``bucket`` follow
generative_recommenders/ops/pytorch/pt_position.py:40-160, including its clamp of the bucket to
``timestamp_embeddings_weight.size(1) - 1``.
"""

from typing import Optional

import torch

from . import _cabi
from .common import HammerKernel, _require_cuda_backend, dtype_code, require_cuda, stream_ptr


def _fill(a, seq_offsets, seq_lengths, num_targets, timestamps, total, D, pos_w, ts_w, max_contextual_seq_len,
          interleave_targets, time_bucket_fn, alpha, dtype, table_dtype):
    a.seq_offsets = seq_offsets.data_ptr()
    a.seq_lengths = seq_lengths.data_ptr()
    a.num_targets = num_targets.data_ptr() if num_targets is not None else None
    a.timestamps = timestamps.data_ptr()
    a.total_rows = total
    a.B = seq_lengths.numel()
    a.D = D
    a.max_contextual_seq_len = max_contextual_seq_len
    a.max_pos_ind = pos_w.shape[0]
    a.ts_rows = ts_w.shape[0]
    a.ts_bucket_max = ts_w.shape[1] - 1
    a.interleave_targets = 1 if interleave_targets else 0
    a.time_bucket_fn = 1 if time_bucket_fn == "log" else 0
    a.alpha = alpha
    a.dtype = dtype
    a.table_dtype = table_dtype


class _AddTimestampPositionalEmbeddings(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pos_w, ts_w, seq_offsets, seq_lengths, num_targets, timestamps, alpha,
                max_contextual_seq_len, interleave_targets, time_bucket_fn):
        x = x.contiguous()
        table_dtype = torch.float32 if pos_w.dtype == torch.float32 and ts_w.dtype == torch.float32 else x.dtype
        pw = pos_w.detach().to(table_dtype).contiguous()
        tw = ts_w.detach().to(table_dtype).contiguous()
        out = torch.empty_like(x)
        a = _cabi.TsPosArgs()
        _fill(a, seq_offsets, seq_lengths, num_targets, timestamps, x.shape[0], x.shape[1], pw, tw,
              max_contextual_seq_len, interleave_targets, time_bucket_fn, alpha, dtype_code(x),
              _cabi.F32 if table_dtype == torch.float32 else dtype_code(x))
        a.seq_embeddings, a.pos_weight, a.ts_weight, a.out = x.data_ptr(), pw.data_ptr(), tw.data_ptr(), out.data_ptr()
        if x.shape[0] > 0:
            with torch.cuda.device(x.device):
                _cabi.check(_cabi.lib().b200_hstu_add_timestamp_positional_embeddings_fwd(a, stream_ptr(x.device)),
                            "b200_hstu_add_timestamp_positional_embeddings_fwd")
        ctx.save_for_backward(seq_offsets, seq_lengths, num_targets, timestamps)
        ctx.meta = (alpha, max_contextual_seq_len, interleave_targets, time_bucket_fn, pos_w.shape, ts_w.shape,
                    pos_w.dtype, ts_w.dtype)
        return out

    @staticmethod
    def backward(ctx, d_out):
        seq_offsets, seq_lengths, num_targets, timestamps = ctx.saved_tensors
        alpha, ctx_len, interleave, fn, pos_shape, ts_shape, pos_dtype, ts_dtype = ctx.meta
        d_out = d_out.contiguous()
        dx = torch.empty_like(d_out)
        d_pos = torch.zeros(pos_shape, dtype=torch.float32, device=d_out.device)
        d_ts = torch.zeros(ts_shape, dtype=torch.float32, device=d_out.device)
        a = _cabi.TsPosArgs()
        _fill(a, seq_offsets, seq_lengths, num_targets, timestamps, d_out.shape[0], d_out.shape[1], d_pos, d_ts,
              ctx_len, interleave, fn, alpha, dtype_code(d_out), _cabi.F32)
        a.d_out, a.d_seq_embeddings = d_out.data_ptr(), dx.data_ptr()
        a.d_pos_weight, a.d_ts_weight = d_pos.data_ptr(), d_ts.data_ptr()
        if d_out.shape[0] > 0:
            with torch.cuda.device(d_out.device):
                _cabi.check(_cabi.lib().b200_hstu_add_timestamp_positional_embeddings_bwd(a, stream_ptr(d_out.device)),
                            "b200_hstu_add_timestamp_positional_embeddings_bwd")
        return (dx, d_pos.to(pos_dtype), d_ts.to(ts_dtype), None, None, None, None, None, None, None, None)


def add_timestamp_positional_embeddings(
    alpha: float,
    max_seq_len: int,
    max_contextual_seq_len: int,
    position_embeddings_weight: torch.Tensor,
    timestamp_embeddings_weight: torch.Tensor,
    seq_offsets: torch.Tensor,
    seq_lengths: torch.Tensor,
    seq_embeddings: torch.Tensor,
    timestamps: torch.Tensor,
    num_targets: Optional[torch.Tensor],
    interleave_targets: bool,
    time_bucket_fn: str = "sqrt",
    kernel: HammerKernel = HammerKernel.CUDA,
) -> torch.Tensor:
    _require_cuda_backend(kernel)
    assert time_bucket_fn in ["sqrt", "log"]
    require_cuda(seq_embeddings, position_embeddings_weight, timestamp_embeddings_weight, seq_offsets, seq_lengths,
                 timestamps, num_targets)
    torch._assert(seq_embeddings.dim() == 2, "seq_embeddings must be [total, D]")
    torch._assert(timestamps.numel() == seq_embeddings.shape[0], "one timestamp per row of seq_embeddings")
    torch._assert(position_embeddings_weight.shape[1] == seq_embeddings.shape[1]
                  and timestamp_embeddings_weight.shape[1] == seq_embeddings.shape[1],
                  "embedding tables must have seq_embeddings' width")
    dev = seq_embeddings.device
    i64 = lambda t: None if t is None else t.to(device=dev, dtype=torch.int64).contiguous()  # noqa: E731
    return _AddTimestampPositionalEmbeddings.apply(
        seq_embeddings, position_embeddings_weight, timestamp_embeddings_weight, i64(seq_offsets), i64(seq_lengths),
        i64(num_targets), i64(timestamps.reshape(-1)), float(alpha), int(max_contextual_seq_len),
        bool(interleave_targets), time_bucket_fn)
