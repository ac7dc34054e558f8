"""CPU restatement of the reference's PyTorch implementation of the HSTU hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module; it is
the checker used by ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline /
reference legs of ``bench.py``.

Parity status: PINNED.  Every function here is checked against outputs of the
unmodified reference (generative_recommenders/ops/pytorch/*, run in the build
container through ``oracle/reference_shims.py``) stored as fixtures under
``tests/golden/`` by ``tests/golden/make_golden.py``.  The reference itself ships no
golden vectors for this path, so those generated fixtures are the pin.

The restatement differs from the reference in one deliberate way: instead of padding
the jagged batch to ``[B, H, N, N]`` it walks the sequences one by one (the padded
rows/columns are multiplied by a zero mask in the reference and dropped by
``dense_to_jagged``, so they never reach the output).  This keeps memory at
``H * L_i^2`` and lets the oracle run the larger configurations.
"""

from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------
# mask
# --------------------------------------------------------------------------------------
def valid_attn_mask(
    L: int,
    num_targets: int = 0,
    has_targets: bool = False,
    max_attn_len: int = 0,
    contextual_seq_len: int = 0,
    min_full_attn_seq_len: int = 0,
    device: Optional[torch.device] = None,
    seq_len: Optional[int] = None,
) -> torch.Tensor:
    """Boolean ``[L, L]`` mask of one sequence of length ``L``.

    Follows generative_recommenders/ops/pytorch/pt_hstu_attention.py:33-84
    (``_get_valid_attn_mask`` with ``causal=True``), restricted to the ``[L, L]``
    corner that survives ``dense_to_jagged`` (pt_hstu_attention.py:183-187).

    ``seq_len`` is the length the reference derives ``max_ids`` from: the difference of
    the sequence's offsets (pt_hstu_attention.py:44,170-172), which for a sequence longer
    than ``max_seq_len`` is larger than the ``L`` rows that ``jagged_to_padded_dense``
    keeps.  Defaults to ``L``.
    """
    ids = torch.arange(L, device=device, dtype=torch.int64)
    max_id = L if seq_len is None else seq_len
    if contextual_seq_len > 0:  # :45-48
        ids = torch.clamp(ids - contextual_seq_len + 1, min=0)
        max_id = max_id - contextual_seq_len + 1
    if has_targets:  # :49-54
        max_id = max_id - num_targets
        ids = torch.clamp(ids, max=max_id)
    row = ids.view(L, 1)
    col = ids.view(1, L)
    dist = row - col  # :61
    valid = torch.eye(L, dtype=torch.bool, device=device)  # :62
    valid = valid | (dist > 0)  # :65
    if max_attn_len > 0:  # :66-79
        if min_full_attn_seq_len > 0:
            valid = valid & ((dist <= max_attn_len) | (row >= max_id - min_full_attn_seq_len))
        else:
            valid = valid & (dist <= max_attn_len)
    if contextual_seq_len > 0:  # :80-83
        valid = valid | ((row == 0) & (col < max_id))
    return valid


def valid_attn_mask_positions(
    L: int,
    num_targets: int = 0,
    max_attn_len: int = 0,
    contextual_seq_len: int = 0,
    min_full_attn_seq_len: int = 0,
) -> torch.Tensor:
    """The same mask written on raw positions instead of clamped ids.

    This is the form the CUDA tile scheduler reasons with (interval of visible
    history columns per row + contextual prefix + self).  It is only defined on the
    regular domain ``L - num_targets >= contextual_seq_len + 1``; tests check it
    equals :func:`valid_attn_mask` there.
    """
    t, c, W, Fm = num_targets, contextual_seq_len, max_attn_len, min_full_attn_seq_len
    u = L - t
    assert u >= c + 1
    i = torch.arange(L).view(L, 1)
    j = torch.arange(L).view(1, L)
    is_ctx_row = i < c
    is_tgt_row = i >= u
    eff = torch.minimum(i, torch.tensor(u))  # row position clamped to first target
    if W == 0:
        full = torch.ones_like(i, dtype=torch.bool)
    else:
        full = (Fm > 0) & ((i >= u - Fm) | is_tgt_row)
    hi = torch.where(is_tgt_row, torch.tensor(u), i + 1)
    lo = torch.where(full, torch.tensor(0), torch.clamp(eff - W, min=c))
    ctx_ok = full | (eff - c + 1 <= W)
    valid = (j >= lo) & (j < hi) & (j >= c)
    valid = valid | ((j < c) & (j < hi) & ctx_ok)
    valid = valid | (is_ctx_row & (j < u))
    valid = valid | (i == j)
    return valid


# --------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------
def hstu_mha(
    max_seq_len: int,
    alpha: float,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    seq_offsets: torch.Tensor,
    causal: bool = True,
    dropout_pr: float = 0.0,
    training: bool = True,
    num_targets: Optional[torch.Tensor] = None,
    attn_scale: Optional[torch.Tensor] = None,
    max_attn_len: int = 0,
    contextual_seq_len: int = 0,
    min_full_attn_seq_len: int = 0,
    rel_bias: Optional[torch.Tensor] = None,
    compute_dtype: Optional[torch.dtype] = None,
    dropout_keep: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Jagged HSTU attention, ``out[i] = sum_j mask(i,j) * SiLU(alpha q_i.k_j) * s * v_j``.

    Follows ``pytorch_hstu_mha`` (pt_hstu_attention.py:130-187): scores ``* alpha``
    (:151), ``silu(.) / max_seq_len`` (:167) or ``silu(.) * attn_scale`` (:152-165),
    multiplied by the mask (:179), times V (:182).  ``rel_bias`` (``[N, N]`` or
    ``[B, N, N]``) is the extension used by the research layer, added to the scores
    before SiLU and broadcast over heads as in
    generative_recommenders/research/modeling/sequential/hstu.py:203-211; note that
    layer uses no ``alpha`` factor (pass ``alpha=1``).

    ``compute_dtype`` upcasts q/k/v first (use ``torch.float32`` to get the fp32
    answer for bf16 inputs); the result is returned in that dtype.

    Dropout on the weights (``F.dropout(qk_attn, p, training)`` after the mask, :180-181): the
    reference draws its mask from torch's generator, so a comparison needs the mask from outside -
    ``dropout_keep``, boolean ``[L_total, H, max_seq_len]`` (query row, head, key position);
    kept weights are scaled by ``1 / (1 - dropout_pr)`` like ``F.dropout`` does (to compare with
    the kernels, whose mask drops a weight with probability ``round(p * 65536) / 65536``, pass
    that ratio).
    """
    assert causal, "only causal attention exists in the reference (hstu_attention.py:128)"
    assert (dropout_pr == 0.0) == (dropout_keep is None), "dropout needs its keep mask, and only dropout does"
    if compute_dtype is not None:
        q, k, v = q.to(compute_dtype), k.to(compute_dtype), v.to(compute_dtype)
    L_total, H, _ = q.shape
    offs = seq_offsets.to(torch.int64).cpu().tolist()
    B = len(offs) - 1
    nt = None if num_targets is None else num_targets.to(torch.int64).cpu().tolist()
    outs: List[torch.Tensor] = []
    for b in range(B):
        s, e = offs[b], offs[b + 1]
        L = min(e - s, max_seq_len)  # jagged_to_padded_dense truncates at N
        qb = q[s : s + L].transpose(0, 1)  # [H, L, A]
        kb = k[s : s + L].transpose(0, 1)
        vb = v[s : s + L].transpose(0, 1)
        qk = torch.einsum("hxa,hya->hxy", qb, kb) * alpha
        if rel_bias is not None:
            rb = rel_bias if rel_bias.dim() == 2 else rel_bias[b]
            qk = qk + rb[:L, :L].to(qk.dtype).unsqueeze(0)
        if attn_scale is not None:
            if attn_scale.ndim > 0:
                sc = attn_scale[s : s + L].to(qk.dtype).view(1, L, 1)
            else:
                sc = attn_scale.to(qk.dtype)
            p = F.silu(qk) * sc
        else:
            p = F.silu(qk) / max_seq_len
        mask = valid_attn_mask(
            L,
            num_targets=0 if nt is None else nt[b],
            has_targets=nt is not None,
            max_attn_len=max_attn_len,
            contextual_seq_len=contextual_seq_len,
            min_full_attn_seq_len=min_full_attn_seq_len,
            device=q.device,
            seq_len=e - s,
        )
        p = p * mask.unsqueeze(0)
        if dropout_keep is not None:
            keep = dropout_keep[s : s + L, :, :L].transpose(0, 1).to(p.device)  # [H, L, L]
            p = p * keep.to(p.dtype) / (1.0 - dropout_pr)
        ob = torch.einsum("hxy,hyv->hxv", p, vb).transpose(0, 1)  # [L, H, V]
        if L < e - s:  # rows beyond max_seq_len come back as zeros from dense_to_jagged
            ob = torch.cat([ob, ob.new_zeros(e - s - L, H, ob.shape[2])], dim=0)
        outs.append(ob)
    if not outs:
        return q.new_zeros(0, H, v.shape[2])
    return torch.cat(outs, dim=0)


def delta_hstu_mha(
    max_seq_len: int,
    alpha: float,
    delta_q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    seq_offsets: torch.Tensor,
    num_targets: Optional[torch.Tensor] = None,
    max_attn_len: int = 0,
    contextual_seq_len: int = 0,
) -> torch.Tensor:
    """Attention of the last ``delta`` rows of each sequence against the full K/V.

    Follows ``pytorch_cached_hstu_mha`` (pt_hstu_attention.py:191-251): ``delta_q`` is
    ``[B * delta, H, A]``, the queries are the last ``delta`` positions of each
    sequence and use the corresponding rows of the full mask (:231-246).
    """
    Ld, H, _ = delta_q.shape
    offs = seq_offsets.to(torch.int64).cpu().tolist()
    B = len(offs) - 1
    delta = Ld // B
    nt = None if num_targets is None else num_targets.to(torch.int64).cpu().tolist()
    outs = []
    for b in range(B):
        s, e = offs[b], offs[b + 1]
        L = e - s
        qb = delta_q[b * delta : (b + 1) * delta].transpose(0, 1)
        kb = k[s:e].transpose(0, 1)
        vb = v[s:e].transpose(0, 1)
        qk = torch.einsum("hxa,hya->hxy", qb, kb) * alpha
        p = F.silu(qk) / max_seq_len
        mask = valid_attn_mask(
            L,
            num_targets=0 if nt is None else nt[b],
            has_targets=nt is not None,
            max_attn_len=max_attn_len,
            contextual_seq_len=contextual_seq_len,
            device=delta_q.device,
        )[L - delta : L]
        p = p * mask.unsqueeze(0)
        outs.append(torch.einsum("hxy,hyv->hxv", p, vb).transpose(0, 1))
    return torch.cat(outs, dim=0)


# --------------------------------------------------------------------------------------
# LayerNorm + linear stages
# --------------------------------------------------------------------------------------
def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    """fp32 LayerNorm cast back to the input dtype
    (generative_recommenders/ops/pytorch/pt_layer_norm.py:24-38)."""
    return F.layer_norm(
        x.to(torch.float32), (x.shape[-1],), weight.to(torch.float32), bias.to(torch.float32), eps
    ).to(x.dtype)


def hstu_compute_uqvk(
    x: torch.Tensor,
    norm_weight: torch.Tensor,
    norm_bias: torch.Tensor,
    norm_eps: float,
    num_heads: int,
    attn_dim: int,
    hidden_dim: int,
    uvqk_weight: torch.Tensor,
    uvqk_bias: torch.Tensor,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """LN -> addmm -> split [u|v|q|k] -> SiLU(u)
    (generative_recommenders/ops/hstu_compute.py:54-104; return order u,q,k,v :104)."""
    normed = layer_norm(x, norm_weight, norm_bias, norm_eps)
    uvqk = torch.addmm(uvqk_bias, normed, uvqk_weight)
    u, v, q, k = torch.split(
        uvqk,
        [hidden_dim * num_heads, hidden_dim * num_heads, attn_dim * num_heads, attn_dim * num_heads],
        dim=1,
    )
    u = F.silu(u)
    return (
        u,
        q.view(-1, num_heads, attn_dim),
        k.view(-1, num_heads, attn_dim),
        v.view(-1, num_heads, hidden_dim),
    )


def norm_mul_dropout(
    x: torch.Tensor,
    u: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor,
    eps: float,
    concat_u: bool = False,
    concat_x: bool = False,
    mul_u_activation_type: str = "none",
    group_norm: bool = False,
    num_heads: int = 1,
    linear_dim: int = -1,
) -> torch.Tensor:
    """``y = act(u) * LN(x)`` with the optional ``[u, x, y]`` concat, dropout off
    (generative_recommenders/ops/pytorch/pt_hstu_linear.py:23-82; the middle block of
    the concat is the raw, un-normalised ``x`` :71-72)."""
    dtype = x.dtype
    x = x.to(torch.float32)
    u = u.to(torch.float32)
    if group_norm:
        y = u * F.group_norm(
            x.view(-1, num_heads, linear_dim),
            num_groups=num_heads,
            weight=weight.to(torch.float32),
            bias=bias.to(torch.float32),
            eps=eps,
        ).view(-1, num_heads * linear_dim)
        if concat_u and concat_x:
            y = torch.cat([u, x, y], dim=1)
    else:
        mul_u = u
        if mul_u_activation_type == "sigmoid":
            mul_u = torch.sigmoid(u)
        elif mul_u_activation_type == "silu":
            mul_u = F.silu(u)
        y = mul_u * F.layer_norm(
            x, (x.shape[-1],), weight.to(torch.float32), bias.to(torch.float32), eps
        )
        if concat_u:
            y = torch.cat([u, x, y], dim=1) if concat_x else torch.cat([u, y], dim=1)
        elif concat_x:
            y = torch.cat([x, y], dim=1)
    return y.to(dtype)


def hstu_compute_output(
    attn: torch.Tensor,
    u: torch.Tensor,
    x: torch.Tensor,
    norm_weight: torch.Tensor,
    norm_bias: torch.Tensor,
    norm_eps: float,
    output_weight: torch.Tensor,
    num_heads: int = 1,
    linear_dim: int = -1,
    concat_u: bool = False,
    concat_x: bool = False,
    mul_u_activation_type: str = "none",
    group_norm: bool = False,
) -> torch.Tensor:
    """``x + norm_mul(attn, u) @ W_out`` (pt_hstu_linear.py:85-120)."""
    y = norm_mul_dropout(
        attn, u, norm_weight, norm_bias, norm_eps, concat_u, concat_x,
        mul_u_activation_type, group_norm, num_heads, linear_dim,
    )
    return torch.addmm(x, y, output_weight.to(x.dtype)).to(x.dtype)


def stu_layer(
    x: torch.Tensor,
    seq_offsets: torch.Tensor,
    max_seq_len: int,
    num_targets: Optional[torch.Tensor],
    params: dict,
    num_heads: int,
    attn_dim: int,
    hidden_dim: int,
    attn_alpha: Optional[float] = None,
    max_attn_len: int = 0,
    contextual_seq_len: int = 0,
    rel_bias: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """One HSTU layer as ``STULayer.forward`` composes it
    (generative_recommenders/modules/stu.py:293-356): uqvk stage -> attention ->
    output stage with ``concat_u=concat_x=True``, ``mul_u_activation_type="none"``,
    eps 1e-6 (:344-352), ``attn_alpha = 1/sqrt(attention_dim)`` by default (:199).
    Dropout is off (eval mode)."""
    alpha = attn_alpha if attn_alpha is not None else 1.0 / (attn_dim ** 0.5)
    dt = x.dtype
    u, q, k, v = hstu_compute_uqvk(
        x, params["input_norm_weight"].to(dt), params["input_norm_bias"].to(dt), 1e-6,
        num_heads, attn_dim, hidden_dim, params["uvqk_weight"].to(dt), params["uvqk_beta"].to(dt),
    )
    attn = hstu_mha(
        max_seq_len, alpha, q, k, v, seq_offsets, num_targets=num_targets,
        max_attn_len=max_attn_len, contextual_seq_len=contextual_seq_len, rel_bias=rel_bias,
    ).reshape(-1, hidden_dim * num_heads)
    return hstu_compute_output(
        attn, u, x, params["output_norm_weight"].to(dt), params["output_norm_bias"].to(dt), 1e-6,
        params["output_weight"].to(dt), num_heads, hidden_dim, concat_u=True, concat_x=True,
    )


# --------------------------------------------------------------------------------------
# jagged glue around the layer
# --------------------------------------------------------------------------------------
def _side_offsets(offsets: Optional[torch.Tensor], dense_len: Optional[int], B: int) -> torch.Tensor:
    if offsets is not None:
        return offsets.to(torch.int64)
    return int(dense_len) * torch.arange(B + 1, dtype=torch.int64)


def concat_2D_jagged(
    values_left: torch.Tensor,
    values_right: torch.Tensor,
    max_len_left: Optional[int] = None,
    max_len_right: Optional[int] = None,
    offsets_left: Optional[torch.Tensor] = None,
    offsets_right: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Per sequence: rows of the left tensor, then rows of the right tensor
    (generative_recommenders/ops/pytorch/pt_jagged_tensors.py:32-113; a side without offsets has
    ``max_len_*`` rows per sequence, :70-87).  Walks the sequences instead of padding."""
    if offsets_left is not None:
        B = offsets_left.numel() - 1
    elif offsets_right is not None:
        B = offsets_right.numel() - 1
    else:
        B = values_left.shape[0] // int(max_len_left)
    ol = _side_offsets(offsets_left, max_len_left, B)
    orr = _side_offsets(offsets_right, max_len_right, B)
    rows = []
    for b in range(B):
        rows.append(values_left[int(ol[b]):int(ol[b + 1])])
        rows.append(values_right[int(orr[b]):int(orr[b + 1])])
    return torch.cat(rows, 0) if rows else values_left.new_zeros((0, values_left.shape[1]))


def split_2D_jagged(
    values: torch.Tensor,
    max_len_left: Optional[int] = None,
    max_len_right: Optional[int] = None,
    offsets_left: Optional[torch.Tensor] = None,
    offsets_right: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Inverse of :func:`concat_2D_jagged`
    (generative_recommenders/ops/pytorch/pt_jagged_tensors.py:116-160)."""
    B = (offsets_left if offsets_left is not None else offsets_right).numel() - 1
    ol = _side_offsets(offsets_left, max_len_left, B)
    orr = _side_offsets(offsets_right, max_len_right, B)
    left, right = [], []
    for b in range(B):
        s = int(ol[b] + orr[b])
        nl = int(ol[b + 1] - ol[b])
        nr = int(orr[b + 1] - orr[b])
        left.append(values[s:s + nl])
        right.append(values[s + nl:s + nl + nr])
    return torch.cat(left, 0), torch.cat(right, 0)


def hstu_split_l2_embeddings(
    x: torch.Tensor, prefix_offsets: torch.Tensor, l2_offsets: torch.Tensor, contextual_seq_len: int
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per sequence ``x = [l2[:c] | prefix | l2[c:]]`` -> ``(prefix, l2)``
    (generative_recommenders/ops/pytorch/pt_jagged_tensors.py:163-199)."""
    c = contextual_seq_len
    B = prefix_offsets.numel() - 1
    pre, l2 = [], []
    for b in range(B):
        s = int(prefix_offsets[b] + l2_offsets[b])
        npre = int(prefix_offsets[b + 1] - prefix_offsets[b])
        nl2 = int(l2_offsets[b + 1] - l2_offsets[b])
        l2.append(x[s:s + c])
        pre.append(x[s + c:s + c + npre])
        l2.append(x[s + c + npre:s + npre + nl2])
    return torch.cat(pre, 0), torch.cat(l2, 0)


def hstu_concat_l2_embeddings(
    prefix_x: torch.Tensor, prefix_offsets: torch.Tensor, l2_x: torch.Tensor, l2_offsets: torch.Tensor,
    contextual_seq_len: int,
) -> torch.Tensor:
    """Inverse of :func:`hstu_split_l2_embeddings`
    (generative_recommenders/ops/pytorch/pt_jagged_tensors.py:202-243)."""
    c = contextual_seq_len
    B = prefix_offsets.numel() - 1
    rows = []
    for b in range(B):
        p0, p1 = int(prefix_offsets[b]), int(prefix_offsets[b + 1])
        l0, l1 = int(l2_offsets[b]), int(l2_offsets[b + 1])
        rows += [l2_x[l0:l0 + c], prefix_x[p0:p1], l2_x[l0 + c:l1]]
    return torch.cat(rows, 0)


def add_timestamp_positional_embeddings(
    alpha: float,
    max_contextual_seq_len: int,
    pos_weight: torch.Tensor,
    ts_weight: torch.Tensor,
    seq_offsets: torch.Tensor,
    seq_lengths: torch.Tensor,
    seq_embeddings: torch.Tensor,
    timestamps: torch.Tensor,
    num_targets: Optional[torch.Tensor],
    interleave_targets: bool,
    time_bucket_fn: str = "sqrt",
) -> torch.Tensor:
    """``alpha * x + (ts_weight[bucket] + pos_weight[index]).to(x.dtype)`` token by token
    (generative_recommenders/ops/position.py:71 for the scaling;
    ops/pytorch/pt_position.py:40-73 for the position index, :96-125 for the time bucket, which the
    reference clamps to ``ts_weight.size(1) - 1``, :98)."""
    max_pos_ind = pos_weight.shape[0]
    num_time_buckets = ts_weight.shape[1] - 1
    x = seq_embeddings * alpha
    out = torch.empty_like(x)
    B = seq_lengths.numel()
    for b in range(B):
        start = int(seq_offsets[b])
        n = int(seq_lengths[b])
        rows = int(seq_offsets[b + 1]) - start
        if rows == 0:
            continue
        p = torch.arange(rows, dtype=torch.int64)
        if num_targets is not None:
            high = n - int(num_targets[b]) * (2 if interleave_targets else 1)
            idx = high - torch.clamp(p, max=high)
        else:
            idx = n - p
        idx = torch.clamp(idx + max_contextual_seq_len, max=max_pos_ind - 1)
        if max_contextual_seq_len > 0:
            head = p < max_contextual_seq_len
            idx = torch.where(head, p, idx)
        ts = timestamps[start:start + rows]
        query_time = ts[max(n - 1, 0)]
        dt = (query_time - ts).clamp(min=1e-6) / 60.0
        dt = torch.log(dt) if time_bucket_fn == "log" else torch.sqrt(dt)
        bucket = torch.clamp(dt.clamp(min=0).int(), min=0, max=num_time_buckets).to(torch.int64)
        emb = ts_weight[bucket] + pos_weight[idx]
        out[start:start + rows] = x[start:start + rows] + emb.to(x.dtype)
    return out


# --------------------------------------------------------------------------------------
# relative position bias (research layer)
# --------------------------------------------------------------------------------------
def bucketized_position_bias(table: torch.Tensor, N: int) -> torch.Tensor:
    """``[N, N]`` bias ``table[clamp(floor(ln(max(|i-j|,1)) / 0.301), 0, nb)]``.

    The bucket function is the one the research model passes to its relative bias
    (generative_recommenders/research/modeling/sequential/hstu.py:610-613), applied to
    the position distance instead of a timestamp difference (time bias off); the
    bias is added to the scores before SiLU and shared by all heads (:203-211).
    """
    nb = table.numel() - 1
    i = torch.arange(N).view(N, 1)
    j = torch.arange(N).view(1, N)
    d = (i - j).abs().clamp(min=1).to(torch.float32)
    bucket = torch.clamp((torch.log(d) / 0.301).long(), min=0, max=nb)
    return table.to(torch.float32)[bucket]


# --------------------------------------------------------------------------------------
# FP8 block quantisation (no reference arithmetic exists; this states the format)
# --------------------------------------------------------------------------------------
def quantize_e4m3_block(x: torch.Tensor, seq_offsets: torch.Tensor, block: int = 128):
    """Per-(sequence-local ``block``-token block, head) absmax/448 scales.

    Blocks are counted from each sequence's first token so that a block never spans
    two sequences.  Returns ``(x_q [L,H,D] float8_e4m3fn, scales [n_blocks_total, H]
    fp32, block_offsets [B+1] int64)`` where sequence ``b`` owns scale rows
    ``block_offsets[b] .. block_offsets[b+1]``.
    """
    offs = seq_offsets.to(torch.int64).cpu().tolist()
    B = len(offs) - 1
    xq = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    scales = []
    boffs = [0]
    for b in range(B):
        s, e = offs[b], offs[b + 1]
        nb = (e - s + block - 1) // block
        boffs.append(boffs[-1] + nb)
        for t in range(nb):
            r0, r1 = s + t * block, min(s + (t + 1) * block, e)
            blk = x[r0:r1].to(torch.float32)
            amax = blk.abs().amax(dim=(0, 2))  # [H]
            sc = torch.clamp(amax, min=1e-12) / 448.0
            xq[r0:r1] = (blk / sc.view(1, -1, 1)).to(torch.float8_e4m3fn)
            scales.append(sc)
    H = x.shape[1]
    sc_t = torch.stack(scales) if scales else x.new_zeros(0, H, dtype=torch.float32)
    return xq, sc_t, torch.tensor(boffs, dtype=torch.int64)


def dequantize_e4m3_block(xq, scales, block_offsets, seq_offsets, block: int = 128) -> torch.Tensor:
    offs = seq_offsets.to(torch.int64).cpu().tolist()
    boffs = block_offsets.to(torch.int64).cpu().tolist()
    out = xq.to(torch.float32)
    for b in range(len(offs) - 1):
        s, e = offs[b], offs[b + 1]
        for t in range(boffs[b + 1] - boffs[b]):
            r0, r1 = s + t * block, min(s + (t + 1) * block, e)
            out[r0:r1] *= scales[boffs[b] + t].view(1, -1, 1)
    return out


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    """``||a-b|| / ||b||`` in fp64 (0 when both are empty or zero)."""
    a = a.detach().to(torch.float64).cpu()
    b = b.detach().to(torch.float64).cpu()
    den = b.norm().item()
    num = (a - b).norm().item()
    return num / den if den > 0 else num


def per_sequence_rel_l2(a: torch.Tensor, b: torch.Tensor, seq_offsets: torch.Tensor) -> float:
    """Largest ``rel_l2`` over the sequences of a jagged tensor (rows ``seq_offsets[s] ..
    seq_offsets[s+1]``), so that a short sequence cannot hide behind the norm of the long ones.  A
    sequence whose reference rows are all zero contributes its absolute error."""
    a = a.detach().to(torch.float64).cpu()
    b = b.detach().to(torch.float64).cpu()
    offs = seq_offsets.to(torch.int64).cpu().tolist()
    worst = 0.0
    for s, e in zip(offs[:-1], offs[1:]):
        if e <= s:
            continue
        den = b[s:e].norm().item()
        num = (a[s:e] - b[s:e]).norm().item()
        worst = max(worst, num / den if den > 0 else num)
    return worst


def max_abs_ratio(a: torch.Tensor, b: torch.Tensor) -> float:
    """``max|a - b| / max|b|``: the largest element-wise error in units of the largest reference
    element (0 for empty tensors)."""
    if b.numel() == 0:
        return 0.0
    a = a.detach().to(torch.float64).cpu()
    b = b.detach().to(torch.float64).cpu()
    den = b.abs().max().item()
    num = (a - b).abs().max().item()
    return num / den if den > 0 else num


# --------------------------------------------------------------------------------------
# dropout mask of the output stage (no reference arithmetic exists for the mask bits: the
# reference draws them from torch's or Triton's generator; this states the format the CUDA
# kernels use, so that a test can replay a mask)
# --------------------------------------------------------------------------------------
def philox4x32_10(key: int, counters):
    """Philox4x32 with 10 rounds (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3",
    SC'11) for 64-bit ``key`` and an array of 64-bit ``counters`` (the upper two counter words
    are zero); returns a ``[n, 4]`` uint32 array."""
    import numpy as np

    c = np.asarray(counters, dtype=np.uint64)
    m32 = np.uint64(0xFFFFFFFF)
    c0, c1 = c & m32, c >> np.uint64(32)
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    k0, k1 = np.uint64(key & 0xFFFFFFFF), np.uint64((key >> 32) & 0xFFFFFFFF)
    for _ in range(10):
        p0 = np.uint64(0xD2511F53) * c0
        p1 = np.uint64(0xCD9E8D57) * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & m32
        hi1, lo1 = p1 >> np.uint64(32), p1 & m32
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & m32, lo1, (hi0 ^ c3 ^ k1) & m32, lo0
        k0 = (k0 + np.uint64(0x9E3779B9)) & m32
        k1 = (k1 + np.uint64(0xBB67AE85)) & m32
    return np.stack([c0, c1, c2, c3], axis=-1).astype(np.uint32)


def dropout_keep_mask(seed: int, rows: int, width: int, dropout_ratio: float) -> torch.Tensor:
    """Boolean ``[rows, width]`` keep-mask of the output stage's dropout and the scale of the kept
    elements: element ``idx = row * width + col`` is dropped when the ``(idx % 8)``-th 16-bit piece
    of ``Philox4x32-10(key=seed, counter=idx // 8)`` is below ``round(dropout_ratio * 65536)``."""
    import numpy as np

    thr = min(int(dropout_ratio * 65536.0 + 0.5), 65535)
    n = rows * width
    groups = (n + 7) // 8
    words = philox4x32_10(seed, np.arange(groups, dtype=np.uint64))          # [groups, 4]
    pieces = np.stack([words & 0xFFFF, words >> 16], axis=-1).reshape(groups, 8)  # piece j: word j // 2, half j % 2
    keep = (pieces.reshape(-1)[:n] >= thr).reshape(rows, width)
    return torch.from_numpy(keep), 65536.0 / (65536 - thr)
