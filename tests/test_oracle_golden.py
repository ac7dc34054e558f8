"""The CPU restatement (oracle/hstu_oracle.py) against outputs of the unmodified reference
stored under tests/golden/ (see tests/golden/make_golden.py)."""

import itertools

import pytest
import torch

from oracle import hstu_oracle as O


def test_masks_match_reference(golden):
    cases = golden("masks.pt")
    assert len(cases) > 300
    for c in cases:
        rows = c["mask"].shape[0]    # min(L, 24): sequences longer than the padded length are truncated
        m = O.valid_attn_mask(rows, num_targets=c["t"] or 0, has_targets=c["t"] is not None,
                              max_attn_len=c["W"], contextual_seq_len=c["c"], min_full_attn_seq_len=c["F"],
                              seq_len=c["L"])
        assert torch.equal(m.to(torch.uint8), c["mask"]), c


def test_position_mask_equals_id_mask():
    # the tile scheduler's position-space form == the reference's id form on the regular domain
    n = 0
    for L, t, c, W, Fm in itertools.product(range(1, 20), [0, 1, 3, 7], [0, 1, 4], [0, 1, 3, 8], [0, 2, 5]):
        if L - t < c + 1 or (W == 0 and Fm > 0):
            continue
        a = O.valid_attn_mask(L, t, True, W, c, Fm)
        b = O.valid_attn_mask_positions(L, t, W, c, Fm)
        assert torch.equal(a, b), (L, t, c, W, Fm)
        n += 1
    assert n > 1000


def _attn(fx):
    p = fx["params"]
    q = fx["q"].clone().requires_grad_(True)
    k = fx["k"].clone().requires_grad_(True)
    v = fx["v"].clone().requires_grad_(True)
    out = O.hstu_mha(p["N"], p["alpha"], q, k, v, fx["seq_offsets"], num_targets=fx["num_targets"],
                     max_attn_len=p["W"], contextual_seq_len=p["ctx"], min_full_attn_seq_len=p["F"])
    return q, k, v, out


def test_attention_matches_reference(golden):
    fxs = golden("attention.pt")
    for name, fx in fxs.items():
        q, k, v, out = _attn(fx)
        torch.testing.assert_close(out, fx["out"], rtol=1e-5, atol=1e-6, msg=name)
        if "dq" in fx:
            out.backward(fx["dout"])
            torch.testing.assert_close(q.grad, fx["dq"], rtol=1e-5, atol=1e-6, msg=name)
            torch.testing.assert_close(k.grad, fx["dk"], rtol=1e-5, atol=1e-6, msg=name)
            torch.testing.assert_close(v.grad, fx["dv"], rtol=1e-5, atol=1e-6, msg=name)


def test_attention_dropout_matches_reference(golden):
    """Dropout on the weights: with the mask the reference itself drew (kept in the fixture), the
    oracle reproduces the reference's output and gradients - the mask goes on after scale and
    validity mask, kept weights are scaled by 1 / (1 - p)."""
    cases = golden("attention_dropout.pt")
    assert len(cases) == 3
    for c in cases:
        q, k, v = (c[n].clone().requires_grad_(True) for n in ("q", "k", "v"))
        out = O.hstu_mha(c["N"], c["alpha"], q, k, v, c["seq_offsets"], dropout_pr=c["dropout_pr"],
                         num_targets=c["num_targets"], max_attn_len=c["max_attn_len"], contextual_seq_len=c["ctx"],
                         dropout_keep=c["keep"])
        out.backward(c["dout"])
        torch.testing.assert_close(out, c["out"], rtol=1e-5, atol=1e-6)
        for a, n in ((q, "dq"), (k, "dk"), (v, "dv")):
            torch.testing.assert_close(a.grad, c[n], rtol=1e-5, atol=1e-6)
        plain = O.hstu_mha(c["N"], c["alpha"], c["q"], c["k"], c["v"], c["seq_offsets"], num_targets=c["num_targets"],
                           max_attn_len=c["max_attn_len"], contextual_seq_len=c["ctx"])
        assert float((plain - c["out"]).abs().max()) > 1e-3      # the mask matters


def test_delta_attention_matches_reference(golden):
    fx = golden("delta_attention.pt")
    out = O.delta_hstu_mha(fx["N"], fx["alpha"], fx["delta_q"], fx["k"], fx["v"], fx["seq_offsets"],
                           num_targets=fx["num_targets"], contextual_seq_len=fx["ctx"])
    torch.testing.assert_close(out, fx["out"], rtol=1e-5, atol=1e-6)


def test_stages_match_reference(golden):
    fx = golden("stages.pt")
    ln = fx["layer_norm"]
    torch.testing.assert_close(O.layer_norm(ln["x"], ln["w"], ln["b"], ln["eps"]), ln["y"])
    uq = fx["uqvk"]
    leaves = [uq[n].clone().requires_grad_(True) for n in ("x", "nw", "nb", "W", "bias")]
    u, q, k, v = O.hstu_compute_uqvk(leaves[0], leaves[1], leaves[2], uq["eps"], uq["H"], uq["A"], uq["V"],
                                    leaves[3], leaves[4])
    for a, b in zip((u, q, k, v), (uq["u"], uq["q"], uq["k"], uq["v"])):
        torch.testing.assert_close(a, b)
    torch.autograd.backward([u, q, k, v], [uq["du"], uq["dq"], uq["dk"], uq["dv"]])
    for a, b in zip(leaves, uq["grads"]):
        torch.testing.assert_close(a.grad, b, rtol=1e-4, atol=1e-5)
    assert len(fx["compute_output"]) >= 18
    for c in fx["compute_output"]:
        leaves = [c[n].clone().requires_grad_(True) for n in ("attn", "u", "x", "nw", "nb", "Wo")]
        o = O.hstu_compute_output(leaves[0], leaves[1], leaves[2], leaves[3], leaves[4], c["eps"], leaves[5],
                                  c["H"], c["V"], c["concat_u"], c["concat_x"], c["act"], c["group_norm"])
        torch.testing.assert_close(o, c["out"], rtol=1e-5, atol=1e-5)
        o.backward(c["dout"])
        for a, b in zip(leaves, c["grads"]):
            torch.testing.assert_close(a.grad, b, rtol=1e-4, atol=1e-5)


def test_stu_layer_matches_reference(golden):
    for c in golden("stu_layer.pt"):
        x = c["x"].clone().requires_grad_(True)
        h = x
        for layer in range(2):
            pre = "_stu_layers.%d._" % layer
            params = {n: c["state"][pre + n] for n in ("input_norm_weight", "input_norm_bias", "uvqk_weight",
                                                        "uvqk_beta", "output_norm_weight", "output_norm_bias",
                                                        "output_weight")}
            h = O.stu_layer(h, c["seq_offsets"], c["N"], c["num_targets"] if c["target_aware"] else None,
                            params, c["H"], c["A"], c["V"], max_attn_len=c["W"], contextual_seq_len=c["ctx"])
        torch.testing.assert_close(h, c["y"], rtol=1e-4, atol=1e-5)
        h.backward(c["dy"])
        torch.testing.assert_close(x.grad, c["dx"], rtol=1e-4, atol=1e-5)


def test_position_bias_matches_reference(golden):
    fx = golden("rel_bias.pt")
    N = fx["N"]
    # the research module evaluates bucket(ts[i+1] - ts[j]); with ts = 7 * position this is
    # bucket(7 * (i + 1 - j)) except in the last row, which repeats the last timestamp
    ts = fx["timestamps"][0]
    ext = torch.cat([ts, ts[N - 1:N]])
    d = (ext[1:].view(N, 1) - ext[:-1].view(1, N)).abs().clamp(min=1).float()
    bucket = torch.clamp((torch.log(d) / 0.301).long(), 0, 128)
    torch.testing.assert_close(fx["ts_w"][bucket], fx["rab"])
    # and the oracle's position-distance form uses the same bucket function
    b = O.bucketized_position_bias(fx["ts_w"], N)
    i, j = 9, 2
    assert b[i, j] == fx["ts_w"][int(torch.log(torch.tensor(7.0)) / 0.301)]


def _bias_attention_inputs(fx):
    """q, k, v as [L, H, d] leaves and the per-distance bias the fixture's weights stand for:
    the research module puts w[N - 1 - (i - j)] at (i, j) of its [N, N] bias for i >= j."""
    N, H, A, V = fx["N"], fx["H"], fx["A"], fx["V"]
    L = fx["q"].shape[0]
    q = fx["q"].view(L, H, A).clone().requires_grad_(True)
    k = fx["k"].view(L, H, A).clone().requires_grad_(True)
    v = fx["v"].view(L, H, V).clone().requires_grad_(True)
    bias = fx["w"][N - 1 - torch.arange(N)].clone().requires_grad_(True)
    return q, k, v, bias


def test_attention_with_learnable_bias_matches_reference(golden):
    """The oracle's ``rel_bias`` path - output and the gradients of q, k, v and of the bias itself -
    against the research model's attention with a ``RelativePositionalBias`` (fixture
    rel_bias_attention.pt)."""
    fx = golden("rel_bias_attention.pt")
    N = fx["N"]
    q, k, v, bias = _bias_attention_inputs(fx)
    i = torch.arange(N)
    rb = bias[(i.view(N, 1) - i.view(1, N)).abs()]
    torch.testing.assert_close(torch.tril(rb), torch.tril(fx["rab"]))
    out = O.hstu_mha(N, 1.0, q, k, v, fx["seq_offsets"], rel_bias=rb)
    L = q.shape[0]
    torch.testing.assert_close(out.reshape(L, -1), fx["out"], rtol=1e-5, atol=1e-6)
    out.backward(fx["dout"].view_as(out))
    torch.testing.assert_close(q.grad.reshape(L, -1), fx["dq"], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(k.grad.reshape(L, -1), fx["dk"], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(v.grad.reshape(L, -1), fx["dv"], rtol=1e-5, atol=1e-6)
    # weights of negative distances (j > i) never reach a causal score
    torch.testing.assert_close(bias.grad, fx["dw"][N - 1 - torch.arange(N)], rtol=1e-4, atol=1e-6)
    assert fx["dw"][N:].abs().max() == 0


def test_philox_known_answer_and_mask_fraction():
    """Philox4x32-10 against the published known-answer vector (counter 0, key 0 ->
    6627e8d5 e169c58d bc57ac4c 9b00dbd8, Random123's kat_vectors), and the dropout mask built on it."""
    assert [int(x) for x in O.philox4x32_10(0, [0])[0]] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    keep, scale = O.dropout_keep_mask(99, 500, 1536, 0.3)
    assert keep.shape == (500, 1536)
    assert abs(float(keep.float().mean()) - 0.7) < 3e-3
    assert abs(scale - 1 / 0.7) < 1e-4
    keep2, _ = O.dropout_keep_mask(100, 500, 1536, 0.3)
    assert not torch.equal(keep, keep2)


def test_fp8_block_quant_roundtrip():
    g = torch.Generator().manual_seed(0)
    off = torch.tensor([0, 5, 5, 300, 431])
    x = torch.randn(431, 2, 16, generator=g)
    xq, sc, boffs = O.quantize_e4m3_block(x, off)
    assert boffs.tolist() == [0, 1, 1, 4, 6] and sc.shape == (6, 2)
    xd = O.dequantize_e4m3_block(xq, sc, boffs, off)
    assert O.rel_l2(xd, x) < 0.04


def test_jagged_concat_split_match_reference(golden):
    fx = golden("jagged.pt")
    assert len(fx["concat"]) == 4 and len(fx["split"]) == 4
    for c in fx["concat"]:
        out = O.concat_2D_jagged(c["left"], c["right"], c["max_len_left"], c["max_len_right"], c["offsets_left"],
                                 c["offsets_right"])
        assert torch.equal(out, c["out"]), c["kind"]
    for c in fx["split"]:
        left, right = O.split_2D_jagged(c["values"], c["max_len_left"], c["max_len_right"], c["offsets_left"],
                                        c["offsets_right"])
        assert torch.equal(left, c["left"]) and torch.equal(right, c["right"]), c["kind"]


def test_timestamp_positional_embeddings_match_reference(golden):
    cases = golden("jagged.pt")["ts_pos"]
    assert len(cases) == 6
    for c in cases:
        out = O.add_timestamp_positional_embeddings(
            c["alpha"], c["ctx"], c["pos_w"], c["ts_w"], c["seq_offsets"], c["seq_lengths"], c["x"],
            c["timestamps"], c["num_targets"], c["interleave"], c["fn"])
        assert torch.equal(out, c["out"]), (c["fn"], c["ctx"], c["interleave"])


def test_cached_layer_fixture_is_consistent(golden):
    """The reference's cached forward reproduces the last rows of its full forward, and the oracle's
    full forward reproduces both."""
    for c in golden("stu_cached.pt"):
        torch.testing.assert_close(c["cached_delta_y"], c["full_delta_y"], rtol=1e-4, atol=1e-5)
        h = c["x"]
        for layer in range(2):
            pre = "_stu_layers.%d._" % layer
            params = {n: c["state"][pre + n] for n in ("input_norm_weight", "input_norm_bias", "uvqk_weight",
                                                        "uvqk_beta", "output_norm_weight", "output_norm_bias",
                                                        "output_weight")}
            h = O.stu_layer(h, c["seq_offsets"], c["N"], c["num_targets"], params, c["H"], c["A"], c["V"],
                            contextual_seq_len=c["ctx"])
        torch.testing.assert_close(h, c["full_y"], rtol=1e-4, atol=1e-5)
        prime = c["seq_offsets"][1:] - c["seq_offsets"][:-1] - c["delta"]
        off = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(prime, 0)])
        _, tail = O.split_2D_jagged(h, None, c["delta"], off, None)
        torch.testing.assert_close(tail, c["cached_delta_y"], rtol=1e-4, atol=1e-5)


def test_l2_embedding_split_concat_match_reference(golden):
    cases = golden("jagged.pt")["l2"]
    assert len(cases) == 2
    for c in cases:
        x = O.hstu_concat_l2_embeddings(c["prefix_x"], c["prefix_offsets"], c["l2_x"], c["l2_offsets"], c["ctx"])
        assert torch.equal(x, c["x"]), c["ctx"]
        p, l = O.hstu_split_l2_embeddings(c["x"], c["prefix_offsets"], c["l2_offsets"], c["ctx"])
        assert torch.equal(p, c["split_prefix"]) and torch.equal(l, c["split_l2"])
        assert torch.equal(p, c["prefix_x"]) and torch.equal(l, c["l2_x"])


def _reference_checkout():
    """A checkout of the reference next to this repository (or named by HSTU_REFERENCE), if any."""
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for cand in (os.environ.get("HSTU_REFERENCE"), os.path.join(os.path.dirname(root), "reference")):
        if cand and os.path.exists(os.path.join(cand, "generative_recommenders", "ops", "pytorch", "pt_hstu_attention.py")):
            return cand
    return None


@pytest.mark.skipif(_reference_checkout() is None, reason="no checkout of the reference on this machine")
def test_oracle_agrees_with_the_reference_on_random_inputs():
    """Beyond the fixtures: 1500 seeded random cases of attention (forward and backward), cached
    attention, the uvqk stage and the output stage, the unmodified reference against the oracle
    (oracle/cross_check_reference.py, in a process of its own so that the reference package does
    not stay imported here)."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "oracle", "cross_check_reference.py"),
                        "--reference", _reference_checkout(), "--cases", "1500"], capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "mismatches 0" in r.stdout
