"""Parity of the LayerNorm / SiLU-gating / norm-mul stages and of the composed HSTU layer."""

import itertools

import pytest
import torch

import generative_recommenders_b200 as G
from oracle import hstu_oracle as O
import parity_metrics as PM

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_layer_norm_golden(golden):
    ln = golden("stages.pt")["layer_norm"]
    x = ln["x"].to(DEV).requires_grad_(True)
    w = ln["w"].to(DEV).requires_grad_(True)
    b = ln["b"].to(DEV).requires_grad_(True)
    y = G.layer_norm(x, w, b, ln["eps"])
    y.backward(ln["dy"].to(DEV))
    assert O.rel_l2(y, ln["y"]) < 1e-5
    assert O.rel_l2(x.grad, ln["dx"]) < 1e-4
    assert O.rel_l2(w.grad, ln["dw"]) < 1e-4
    assert O.rel_l2(b.grad, ln["db"]) < 1e-4


@pytest.mark.parametrize("dtype,D,rows", [(torch.bfloat16, 512, 1000), (torch.bfloat16, 1024, 333),
                                          (torch.float32, 100, 77), (torch.float16, 2048, 64),
                                          (torch.bfloat16, 136, 50), (torch.float32, 1024, 9)])
def test_layer_norm_shapes(dtype, D, rows):
    g = torch.Generator().manual_seed(D + rows)
    x = (torch.randn(rows, D, generator=g) * 1.5 + 0.3).to(dtype)
    w = torch.randn(D, generator=g).to(dtype)
    b = torch.randn(D, generator=g).to(dtype)
    dy = torch.randn(rows, D, generator=g).to(dtype)
    xd, wd, bd = (t.to(DEV).requires_grad_(True) for t in (x, w, b))
    y = G.layer_norm(xd, wd, bd, 1e-6)
    y.backward(dy.to(DEV))
    xr, wr, br = (t.float().requires_grad_(True) for t in (x, w, b))
    yr = torch.nn.functional.layer_norm(xr, (D,), wr, br, 1e-6)
    yr.backward(dy.float())
    tol = 1e-2 if dtype != torch.float32 else 1e-4
    assert O.rel_l2(y, yr) < tol
    assert O.rel_l2(xd.grad, xr.grad) < tol
    assert O.rel_l2(wd.grad, wr.grad) < tol
    assert O.rel_l2(bd.grad, br.grad) < tol


def test_uqvk_golden(golden):
    uq = golden("stages.pt")["uqvk"]
    leaves = [uq[n].to(DEV).requires_grad_(True) for n in ("x", "nw", "nb", "W", "bias")]
    torch.backends.cuda.matmul.allow_tf32 = False
    u, q, k, v = G.hstu_compute_uqvk(leaves[0], leaves[1], leaves[2], uq["eps"], uq["H"], uq["A"], uq["V"],
                                     leaves[3], leaves[4])
    for a, b in zip((u, q, k, v), (uq["u"], uq["q"], uq["k"], uq["v"])):
        assert O.rel_l2(a, b) < 1e-4
    torch.autograd.backward([u, q, k, v], [uq[n].to(DEV) for n in ("du", "dq", "dk", "dv")])
    for a, b in zip(leaves, uq["grads"]):
        assert O.rel_l2(a.grad, b) < 1e-3


def test_compute_output_golden(golden):
    torch.backends.cuda.matmul.allow_tf32 = False
    cases = golden("stages.pt")["compute_output"]
    for c in cases:
        leaves = [c[n].to(DEV).requires_grad_(True) for n in ("attn", "u", "x", "nw", "nb", "Wo")]
        o = G.hstu_compute_output(leaves[0], leaves[1], leaves[2], leaves[3], leaves[4], c["eps"], leaves[5],
                                  c["H"], c["V"], 0.0, False, c["concat_u"], c["concat_x"], c["act"],
                                  c["group_norm"], False)
        key = (c["concat_u"], c["concat_x"], c["act"], c["group_norm"])
        assert O.rel_l2(o, c["out"]) < 1e-4, key
        o.backward(c["dout"].to(DEV))
        for a, b, nm in zip(leaves, c["grads"], ("attn", "u", "x", "nw", "nb", "Wo")):
            assert O.rel_l2(a.grad, b) < 1e-3, (key, nm)


@pytest.mark.parametrize("concat,act", list(itertools.product([(True, True), (False, False), (True, False)],
                                                               ["none", "silu"])))
def test_norm_mul_bf16(concat, act):
    g = torch.Generator().manual_seed(5)
    rows, H, V = 700, 4, 128
    attn = torch.randn(rows, H * V, generator=g).bfloat16()
    u = torch.randn(rows, H * V, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(H * V, generator=g)).bfloat16()
    b = (0.1 * torch.randn(H * V, generator=g)).bfloat16()
    mult = 1 + int(concat[0]) + int(concat[1])
    dy = torch.randn(rows, mult * H * V, generator=g).bfloat16()
    ld = [t.to(DEV).requires_grad_(True) for t in (attn, u, w, b)]
    y = G.hstu_norm_mul_dropout(ld[0], ld[1], ld[2], ld[3], 1e-6, 0.0, False, concat[0], concat[1], act, False, H, V)
    y.backward(dy.to(DEV))
    lr = [t.float().requires_grad_(True) for t in (attn, u, w, b)]
    yr = O.norm_mul_dropout(lr[0], lr[1], lr[2], lr[3], 1e-6, concat[0], concat[1], act, False, H, V)
    yr.backward(dy.float())
    assert O.rel_l2(y, yr) < 1e-2
    for a, r in zip(ld, lr):
        assert O.rel_l2(a.grad, r.grad) < 1e-2


def test_stu_layer_golden_fp32(golden):
    """Two stacked HSTU layers (uqvk stage -> attention -> output stage) against the reference's
    STUStack outputs and gradients."""
    torch.backends.cuda.matmul.allow_tf32 = False
    for c in golden("stu_layer.pt"):
        x = c["x"].to(DEV).requires_grad_(True)
        offs = c["seq_offsets"].to(DEV)
        nt = c["num_targets"].to(DEV) if c["target_aware"] else None
        h = x
        params = []
        for layer in range(2):
            pre = "_stu_layers.%d._" % layer
            P = {n: c["state"][pre + n].to(DEV).requires_grad_(True) for n in
                 ("input_norm_weight", "input_norm_bias", "uvqk_weight", "uvqk_beta", "output_norm_weight",
                  "output_norm_bias", "output_weight")}
            params.append(P)
            u, attn, _, _ = G.hstu_preprocess_and_attention(
                h, P["input_norm_weight"], P["input_norm_bias"], 1e-6, c["H"], c["A"], c["V"], P["uvqk_weight"],
                P["uvqk_beta"], c["N"], offs, 1.0 / c["A"] ** 0.5, True, nt, c["W"], c["ctx"], False, False, False)
            h = G.hstu_compute_output(attn, u, h, P["output_norm_weight"], P["output_norm_bias"], 1e-6,
                                      P["output_weight"], c["H"], c["V"], 0.0, False, True, True, "none", False, False)
        assert O.rel_l2(h, c["y"]) < 1e-4
        h.backward(c["dy"].to(DEV))
        assert O.rel_l2(x.grad, c["dx"]) < 1e-3
        for layer in range(2):
            for n, t in params[layer].items():
                ref = c["param_grads"]["_stu_layers.%d._%s" % (layer, n)]
                assert O.rel_l2(t.grad, ref) < 2e-3, (layer, n)


def test_stu_module_loads_reference_state_and_matches(golden):
    """STUStack module: loads the reference STUStack state_dict and reproduces its output and
    input gradient."""
    torch.backends.cuda.matmul.allow_tf32 = False
    for c in golden("stu_layer.pt"):
        cfg = G.STULayerConfig(embedding_dim=c["D"], num_heads=c["H"], hidden_dim=c["V"], attention_dim=c["A"],
                               output_dropout_ratio=0.0, target_aware=c["target_aware"], max_attn_len=c["W"],
                               contextual_seq_len=c["ctx"])
        stack = G.STUStack([G.STULayer(cfg), G.STULayer(cfg)]).to(DEV).eval()
        missing = stack.load_state_dict(c["state"], strict=True)
        assert not missing.missing_keys and not missing.unexpected_keys
        x = c["x"].to(DEV).requires_grad_(True)
        y = stack(x, c["lengths"].to(DEV), c["seq_offsets"].to(DEV), c["N"], c["num_targets"].to(DEV))
        assert O.rel_l2(y, c["y"]) < 1e-4
        y.backward(c["dy"].to(DEV))
        assert O.rel_l2(x.grad, c["dx"]) < 1e-3
        for name, prm in stack.named_parameters():
            assert O.rel_l2(prm.grad, c["param_grads"][name]) < 2e-3, name


def test_bf16_stack_with_relative_bias_runs_and_matches_oracle():
    """configs[2]-like layer: bf16, contextual prefix, targets, bucketised relative bias."""
    from generative_recommenders_b200 import workloads as W
    from generative_recommenders_b200.stu import position_bias_by_distance
    torch.manual_seed(0)
    cfg = G.STULayerConfig(embedding_dim=256, num_heads=2, hidden_dim=128, attention_dim=128,
                           output_dropout_ratio=0.0, contextual_seq_len=6, rel_bias_buckets=128)
    layer = G.STULayer(cfg).to(DEV).eval()
    lengths = torch.tensor([40, 300, 17, 200])
    nt = torch.tensor([3, 20, 1, 9])
    offs = W._offsets(lengths)
    x = torch.randn(int(offs[-1]), 256).bfloat16()
    y = layer(x.to(DEV), lengths.to(DEV), offs.to(DEV), 512, nt.to(DEV))
    params = {n[1:]: p.detach().float().cpu() for n, p in layer.named_parameters()}
    bias = position_bias_by_distance(params["rel_bias_table"], 512)
    i = torch.arange(512).view(-1, 1); j = torch.arange(512).view(1, -1)
    rb = bias[(i - j).abs()]
    ref = O.stu_layer(x.float(), offs, 512, nt, params, 2, 128, 128, contextual_seq_len=6, rel_bias=rb)
    params16 = {n: p.bfloat16() for n, p in params.items()}
    ref16 = O.stu_layer(x, offs, 512, nt, params16, 2, 128, 128, contextual_seq_len=6, rel_bias=rb)
    PM.check_vs_bf16_reference("bf16_layer_with_bias", y, ref, ref16.float())
