"""The jagged glue kernels (concat / split, timestamp + position embeddings) and the KV-cache path
of the STU module against the reference's outputs (tests/golden/jagged.pt, stu_cached.pt) and the
oracle."""

import importlib

import pytest
import torch

from oracle import hstu_oracle as O
import parity_metrics as PM

pytestmark = pytest.mark.gpu

G = importlib.import_module("generative-recommenders_b200")
J = importlib.import_module("generative-recommenders_b200.jagged_tensors")
P = importlib.import_module("generative-recommenders_b200.position")
DEV = "cuda"


def _dev(t):
    return None if t is None else t.to(DEV)


def test_concat_split_golden(golden):
    fx = golden("jagged.pt")
    for c in fx["concat"]:
        out = J.concat_2D_jagged(16, _dev(c["left"]), _dev(c["right"]), c["max_len_left"], c["max_len_right"],
                                 _dev(c["offsets_left"]), _dev(c["offsets_right"]))
        assert torch.equal(out.cpu(), c["out"]), c["kind"]
    for c in fx["split"]:
        left, right = J.split_2D_jagged(16, _dev(c["values"]), None, None, c["max_len_left"], c["max_len_right"],
                                        _dev(c["offsets_left"]), _dev(c["offsets_right"]))
        assert torch.equal(left.cpu(), c["left"]) and torch.equal(right.cpu(), c["right"]), c["kind"]


@pytest.mark.parametrize("dtype,width", [(torch.float32, 512), (torch.bfloat16, 512), (torch.bfloat16, 24),
                                         (torch.float16, 3), (torch.bfloat16, 1)])
def test_concat_split_random_roundtrip_and_grads(dtype, width):
    """Bit-exact against the oracle for every vector width of the row mover; split(concat) is the
    identity; each op's backward is the other."""
    g = torch.Generator().manual_seed(width)
    B = 37
    ll = torch.randint(0, 200, (B,), generator=g)
    lr = torch.randint(0, 50, (B,), generator=g)
    ol = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(ll, 0)])
    orr = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(lr, 0)])
    left = torch.randn(int(ol[-1]), width, generator=g).to(dtype)
    right = torch.randn(int(orr[-1]), width, generator=g).to(dtype)
    ref = O.concat_2D_jagged(left, right, None, None, ol, orr)
    lg = left.to(DEV).requires_grad_(True)
    rg = right.to(DEV).requires_grad_(True)
    out = J.concat_2D_jagged(250, lg, rg, 200, 50, ol.to(DEV), orr.to(DEV))
    assert torch.equal(out.cpu(), ref)
    sl, sr = J.split_2D_jagged(250, out, None, None, None, None, ol.to(DEV), orr.to(DEV))
    assert torch.equal(sl, lg) and torch.equal(sr, rg)
    d = torch.randn(out.shape, generator=g).to(dtype)
    out.backward(d.to(DEV))
    dl, dr = O.split_2D_jagged(d, None, None, ol, orr)
    assert torch.equal(lg.grad.cpu(), dl) and torch.equal(rg.grad.cpu(), dr)
    v = out.detach().clone().requires_grad_(True)
    a, b = J.split_2D_jagged(250, v, int(ol[-1]), int(orr[-1]), None, None, ol.to(DEV), orr.to(DEV))
    da, db = torch.randn_like(a), torch.randn_like(b)
    torch.autograd.backward([a, b], [da, db])
    assert torch.equal(v.grad.cpu(), O.concat_2D_jagged(da.cpu(), db.cpu(), None, None, ol, orr))


def test_concat_split_empty_and_dense():
    ol = torch.tensor([0, 0, 0], device=DEV)
    e = torch.empty(0, 8, device=DEV)
    right = torch.randn(6, 8, device=DEV)
    out = J.concat_2D_jagged(3, e, right, 0, 3, ol, None)
    assert torch.equal(out, right)
    a, b = J.split_2D_jagged(3, out, None, None, None, 3, ol, None)
    assert a.shape == (0, 8) and torch.equal(b, right)
    with pytest.raises(Exception):
        J.split_2D_jagged(3, out, None, None, None, None, None, None)
    with pytest.raises(NotImplementedError):
        J.concat_2D_jagged(3, e, right, 0, 3, ol, None, kernel=G.HammerKernel.TRITON)


def test_timestamp_positional_embeddings_golden(golden):
    for c in golden("jagged.pt")["ts_pos"]:
        out = P.add_timestamp_positional_embeddings(
            c["alpha"], c["N"], c["ctx"], _dev(c["pos_w"]), _dev(c["ts_w"]), _dev(c["seq_offsets"]),
            _dev(c["seq_lengths"]), _dev(c["x"]), _dev(c["timestamps"]), _dev(c["num_targets"]), c["interleave"],
            c["fn"])
        if c["fn"] == "sqrt":
            # sqrt and the division are correctly rounded on both sides: same buckets, same roundings
            assert torch.equal(out.cpu(), c["out"]), (c["fn"], c["ctx"], c["interleave"])
        else:
            torch.testing.assert_close(out.cpu(), c["out"], rtol=0, atol=0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("fn", ["sqrt", "log"])
def test_timestamp_positional_embeddings_ragged_and_grads(dtype, fn):
    """Ragged batch (also without num_targets, which the reference's PyTorch path cannot run)
    against the oracle, and the three gradients against autograd through the oracle."""
    g = torch.Generator().manual_seed(11)
    B, D, N, ctx = 33, 64, 300, 2
    for targets in (True, False):
        nt = torch.randint(0, 5, (B,), generator=g)
        lengths = torch.randint(1, 280, (B,), generator=g) + nt + ctx
        offsets = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(lengths, 0)])
        total = int(offsets[-1])
        x = torch.randn(total, D, generator=g).to(dtype)
        gaps = (torch.rand(total, generator=g) * 13).exp().long()
        ts = torch.cat([torch.cumsum(gaps[int(offsets[b]):int(offsets[b + 1])], 0) for b in range(B)])
        pos_w = (torch.randn(N + ctx + 1, D, generator=g) * 0.3).requires_grad_(True)
        ts_w = (torch.randn(2048, D, generator=g) * 0.3).requires_grad_(True)
        xr = x.clone().requires_grad_(True)
        ref = O.add_timestamp_positional_embeddings(8.0, ctx, pos_w, ts_w, offsets, lengths, xr, ts,
                                                    nt if targets else None, False, fn)
        xg = x.to(DEV).requires_grad_(True)
        pg = pos_w.detach().to(DEV).requires_grad_(True)
        tg = ts_w.detach().to(DEV).requires_grad_(True)
        out = P.add_timestamp_positional_embeddings(8.0, N, ctx, pg, tg, offsets.to(DEV), lengths.to(DEV), xg,
                                                    ts.to(DEV), nt.to(DEV) if targets else None, False, fn)
        assert torch.equal(out.cpu(), ref.detach())
        d = torch.randn(out.shape, generator=g).to(dtype)
        ref.backward(d)
        out.backward(d.to(DEV))
        assert torch.equal(xg.grad.cpu(), xr.grad)
        # fp32 sums in a different order
        torch.testing.assert_close(pg.grad.cpu(), pos_w.grad, rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(tg.grad.cpu(), ts_w.grad, rtol=1e-4, atol=2e-3)


def test_cached_forward_golden(golden):
    """forward() with kv_caching_lengths, then cached_forward() on the last delta rows: the
    reference's cached output, and the full forward's last rows."""
    torch.backends.cuda.matmul.allow_tf32 = False
    for c in golden("stu_cached.pt"):
        cfg = G.STULayerConfig(embedding_dim=c["D"], num_heads=c["H"], hidden_dim=c["V"], attention_dim=c["A"],
                               output_dropout_ratio=0.0, target_aware=True, max_attn_len=None,
                               contextual_seq_len=c["ctx"])
        stack = G.STUStack([G.STULayer(cfg, is_inference=True), G.STULayer(cfg, is_inference=True)]).to(DEV).eval()
        stack.load_state_dict(c["state"], strict=True)
        x, lengths, offs, nt = (c[k].to(DEV) for k in ("x", "lengths", "seq_offsets", "num_targets"))
        delta, N = c["delta"], c["N"]
        with torch.inference_mode():
            full = stack(x, lengths, offs, N, nt)
            assert O.rel_l2(full, c["full_y"]) < 1e-4
            prime_lengths = lengths - delta
            prime_offsets = torch.cat([offs.new_zeros(1), torch.cumsum(prime_lengths, 0)])
            prime_x, delta_x = J.split_2D_jagged(N, x, None, None, None, delta, prime_offsets, None)
            stack(prime_x, prime_lengths, prime_offsets, N, nt - delta, max_kv_caching_len=N - delta,
                  kv_caching_lengths=lengths - delta)
            for layer in stack._stu_layers:
                assert layer.k_cache.shape[0] == int(prime_offsets[-1])
            delta_y = stack.cached_forward(delta_x, nt)
            _, full_tail = J.split_2D_jagged(N, full, None, None, None, delta, prime_offsets, None)
        assert O.rel_l2(delta_y, c["cached_delta_y"]) < 1e-4
        assert O.rel_l2(delta_y, full_tail) < 1e-4


def test_cached_forward_bf16_matches_full_forward():
    """The reference's own check (modules/tests/stu_test.py:324-453) at bf16 on a larger batch."""
    torch.manual_seed(3)
    D, H, A, V, delta, ctx = 256, 4, 128, 128, 20, 0
    cfg = G.STULayerConfig(embedding_dim=D, num_heads=H, hidden_dim=V, attention_dim=A, output_dropout_ratio=0.0,
                           target_aware=True, contextual_seq_len=ctx)
    stack = G.STUStack([G.STULayer(cfg, True) for _ in range(2)]).to(DEV).to(torch.bfloat16).eval()
    B = 8
    nt = torch.randint(delta, 2 * delta + 1, (B,), device=DEV)
    lengths = torch.randint(100, 400, (B,), device=DEV) + nt
    N = 400 + 2 * delta
    offs = torch.cat([lengths.new_zeros(1), torch.cumsum(lengths, 0)])
    x = torch.randn(int(offs[-1]), D, device=DEV, dtype=torch.bfloat16)
    with torch.inference_mode():
        full = stack(x, lengths, offs, N, nt)
        prime_lengths = lengths - delta
        prime_offsets = torch.cat([offs.new_zeros(1), torch.cumsum(prime_lengths, 0)])
        prime_x, delta_x = J.split_2D_jagged(N, x, None, None, None, delta, prime_offsets, None)
        stack(prime_x, prime_lengths, prime_offsets, N, nt - delta, max_kv_caching_len=N - delta,
              kv_caching_lengths=prime_lengths)
        delta_y = stack.cached_forward(delta_x, nt)
        _, full_tail = J.split_2D_jagged(N, full, None, None, None, delta, prime_offsets, None)
    # both routes against the fp32 oracle of the full forward (and against the oracle in bf16, the
    # reference's own arithmetic at this precision: two stacked 16-bit layers)
    def oracle_tail(dtype):
        h = x.detach().cpu().to(dtype)
        for layer in stack._stu_layers:
            prm = {n[1:]: p_.detach().cpu().to(dtype) for n, p_ in layer.named_parameters()}
            h = O.stu_layer(h, offs.cpu(), N, nt.cpu(), prm, H, A, V, contextual_seq_len=ctx)
        return O.split_2D_jagged(h, None, delta, prime_offsets.cpu(), None)[1].float()
    ref32, ref16 = oracle_tail(torch.float32), oracle_tail(torch.bfloat16)
    PM.check_vs_bf16_reference("cached_bf16_full_route", full_tail, ref32, ref16)
    PM.check_vs_bf16_reference("cached_bf16_delta_route", delta_y, ref32, ref16)


def test_full_size_round_trips():
    """Size-independent properties at the benchmark's size (1.4 M rows of 1 KB): split(concat) is the
    identity, concat(split) is the identity, and the embedding op is affine in its input."""
    from generative_recommenders_b200 import workloads as W
    w = W.config4(400)
    lengths = w.lengths.to(DEV)
    B = lengths.numel()
    offs = torch.cat([lengths.new_zeros(1), torch.cumsum(lengths, 0)])
    prime = torch.cat([lengths.new_zeros(1), torch.cumsum(lengths - 20, 0)])
    rows = int(offs[-1])
    g = torch.Generator(device=DEV).manual_seed(1)
    x = torch.randn(rows, 512, device=DEV, generator=g).to(torch.bfloat16)
    left, right = J.split_2D_jagged(0, x, None, None, None, 20, prime, None)
    assert left.shape[0] == rows - 20 * B and right.shape[0] == 20 * B
    back = J.concat_2D_jagged(0, left, right, None, 20, prime, None)
    assert torch.equal(back, x)
    # last 20 rows of every sequence, checked directly for a few sequences
    for b in (0, B // 2, B - 1):
        assert torch.equal(right[20 * b:20 * b + 20], x[int(offs[b + 1]) - 20:int(offs[b + 1])])
    del left, right, back
    pos_w = torch.randn(16385, 512, device=DEV, generator=g) * 0.1
    ts_w = torch.randn(2049, 512, device=DEV, generator=g) * 0.1
    stamps = torch.cumsum((torch.rand(rows, device=DEV, generator=g) * 10).exp().long(), 0)
    nt = w.num_targets.to(DEV)
    f = lambda a, alpha: P.add_timestamp_positional_embeddings(  # noqa: E731
        alpha, 16384, 0, pos_w, ts_w, offs, lengths, a, stamps, nt, False, "sqrt")
    xf = x.float()
    e0 = f(torch.zeros_like(xf), 1.0)          # the embedding term alone
    y = f(xf, 2.0)
    assert torch.allclose(y, 2.0 * xf + e0, rtol=1e-6, atol=1e-6)
    # every row of the embedding term is a sum of one row of each table: spot-check the last token
    # of every sequence (time bucket 0, position index = number of targets -> clamped formula)
    last = offs[1:] - 1
    high = lengths - nt
    idx = high - torch.minimum(lengths - 1, high)
    assert torch.allclose(e0[last], ts_w[0].unsqueeze(0) + pos_w[idx], rtol=1e-6, atol=1e-6)


def test_l2_embedding_split_concat_golden_and_grads(golden):
    for c in golden("jagged.pt")["l2"]:
        po, lo = c["prefix_offsets"].to(DEV), c["l2_offsets"].to(DEV)
        px = c["prefix_x"].to(DEV).requires_grad_(True)
        lx = c["l2_x"].to(DEV).requires_grad_(True)
        x = J.hstu_concat_l2_embeddings(9, px, po, c["ctx"] + 7, lx, lo, c["ctx"])
        assert torch.equal(x.detach().cpu(), c["x"]), c["ctx"]
        p, l = J.hstu_split_l2_embeddings(16 + c["ctx"], x.detach(), po, lo, c["ctx"])
        assert torch.equal(p.cpu(), c["split_prefix"]) and torch.equal(l.cpu(), c["split_l2"])
        d = torch.randn_like(x)
        x.backward(d)
        dp, dl = O.hstu_split_l2_embeddings(d.cpu(), c["prefix_offsets"], c["l2_offsets"], c["ctx"])
        assert torch.equal(px.grad.cpu(), dp) and torch.equal(lx.grad.cpu(), dl)


def test_positional_encoder_module_matches_oracle():
    """The module in front of layer 0 (reference modules/positional_encoder.py): parameters as the
    reference names them, output and gradients against the oracle."""
    torch.manual_seed(4)
    D, N, ctx = 64, 200, 3
    enc = G.HSTUPositionalEncoder(num_position_buckets=N + ctx + 1, num_time_buckets=2048, embedding_dim=D,
                                  contextual_seq_len=ctx).to(DEV)
    assert set(dict(enc.named_parameters())) == {"_position_embeddings_weight", "_timestamp_embeddings_weight"}
    g = torch.Generator().manual_seed(8)
    nt = torch.randint(0, 4, (9,), generator=g)
    lengths = torch.randint(1, 150, (9,), generator=g) + nt + ctx
    offs = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(lengths, 0)])
    total = int(offs[-1])
    x = torch.randn(total, D, generator=g)
    ts = torch.cat([torch.cumsum((torch.rand(int(n), generator=g) * 11).exp().long(), 0) for n in lengths])
    xg = x.to(DEV).requires_grad_(True)
    y = enc(N, lengths.to(DEV), offs.to(DEV), ts.to(DEV), xg, nt.to(DEV))
    pw = enc._position_embeddings_weight.detach().cpu().requires_grad_(True)
    tw = enc._timestamp_embeddings_weight.detach().cpu().requires_grad_(True)
    xr = x.clone().requires_grad_(True)
    ref = O.add_timestamp_positional_embeddings(D ** 0.5, ctx, pw, tw, offs, lengths, xr, ts, nt, False, "sqrt")
    assert torch.equal(y.detach().cpu(), ref.detach())
    d = torch.randn(total, D, generator=g)
    y.backward(d.to(DEV))
    ref.backward(d)
    assert torch.equal(xg.grad.cpu(), xr.grad)
    torch.testing.assert_close(enc._position_embeddings_weight.grad.cpu(), pw.grad, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(enc._timestamp_embeddings_weight.grad.cpu(), tw.grad, rtol=1e-4, atol=2e-3)
