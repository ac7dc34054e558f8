"""FP8 (e4m3, per-128-token-block scales) forward against the fp32 oracle.

Two comparisons: against the oracle run on the de-quantised tensors (what the kernel should
compute: bf16-level agreement), and against the oracle on the unquantised tensors (the acceptance
bound rel-L2 <= 5e-2)."""

import pytest
import torch

import generative_recommenders_b200 as G
from generative_recommenders_b200 import workloads as W
from oracle import hstu_oracle as O
import parity_metrics as PM

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_block_quantiser_matches_oracle():
    g = torch.Generator().manual_seed(0)
    lengths = torch.tensor([5, 0, 300, 131, 128])
    offs = W._offsets(lengths)
    x = torch.randn(int(offs[-1]), 2, 128, generator=g).bfloat16()
    x8, sc, bo = G.quantize_e4m3_block(x.to(DEV), offs.to(DEV))
    r8, rsc, rbo = O.quantize_e4m3_block(x.float(), offs)
    assert bo.cpu().tolist() == rbo.tolist()
    n = int(rbo[-1])
    torch.testing.assert_close(sc[:n].cpu(), rsc, rtol=1e-6, atol=0)
    assert torch.equal(x8.cpu().view(torch.uint8), r8.view(torch.uint8))


@pytest.mark.parametrize("case", [
    # lengths, targets, window, ctx
    ([128], None, 0, 0),
    ([384], None, 0, 0),
    ([100, 300, 1, 257], None, 0, 0),
    ([400, 700, 330], [256, 256, 256], 300, 0),
    ([200, 500, 129], [7, 30, 2], 90, 3),
])
def test_fp8_forward(case):
    lengths, nt, Wn, ctx = case
    g = torch.Generator().manual_seed(sum(lengths))
    lengths = torch.tensor(lengths)
    offs = W._offsets(lengths)
    L, H, d, N = int(offs[-1]), 2, 128, 1024
    q = torch.randn(L, H, d, generator=g); k = torch.randn(L, H, d, generator=g); v = torch.randn(L, H, d, generator=g)
    ntt = None if nt is None else torch.tensor(nt)
    offs_d = offs.to(DEV)
    q8, qs, bo = G.quantize_e4m3_block(q.to(DEV), offs_d)
    k8, ks, _ = G.quantize_e4m3_block(k.to(DEV), offs_d)
    v8, vs, _ = G.quantize_e4m3_block(v.to(DEV), offs_d)
    out = G.hstu_mha_fp8(N, 1.0 / 128, q8, k8, v8, qs, ks, vs, bo, offs_d,
                         num_targets=None if ntt is None else ntt.to(DEV), max_attn_len=Wn, contextual_seq_len=ctx)
    torch.cuda.synchronize()
    nblk = int(bo[-1])
    deq = [O.dequantize_e4m3_block(t8.cpu(), s[:nblk].cpu(), bo.cpu().long(), offs)
           for t8, s in ((q8, qs), (k8, ks), (v8, vs))]
    ref_q = O.hstu_mha(N, 1.0 / 128, deq[0], deq[1], deq[2], offs, num_targets=ntt, max_attn_len=Wn,
                       contextual_seq_len=ctx)
    ref = O.hstu_mha(N, 1.0 / 128, q, k, v, offs, num_targets=ntt, max_attn_len=Wn, contextual_seq_len=ctx)
    e_kernel = O.rel_l2(out, ref_q)
    e_total = O.rel_l2(out, ref)
    PM._note(("fp8", tuple(lengths.tolist())), {"kernel_vs_dequantised": e_kernel, "vs_unquantised": e_total})
    assert torch.isfinite(out.float()).all()
    assert e_kernel < 1e-2, e_kernel   # arithmetic of the kernel itself: bf16-level
    assert e_total < 5e-2, e_total     # acceptance bound for fp8 against the unquantised fp32 result


@pytest.mark.parametrize("dist", ["student_t4", "outliers"])
def test_fp8_forward_heavy_tailed_inputs(dist):
    """Inputs with heavier tails than N(0, 1): Student-t with four degrees of freedom, and normal
    values with one element in 200 multiplied by 12.  A block's scale is then set by its largest
    element; e4m3 keeps a relative precision of 2^-4 over 4.5 decades below it, so the error against
    the unquantised result stays where the quantisation of q, k, v itself puts it."""
    g = torch.Generator().manual_seed(17)
    lengths = torch.tensor([300, 700, 129, 64])
    offs = W._offsets(lengths)
    L, H, d, N = int(offs[-1]), 2, 128, 1024

    def draw():
        x = torch.randn(L, H, d, generator=g)
        if dist == "student_t4":
            chi = torch.randn(L, H, d, 4, generator=g).pow(2).sum(-1)
            return x / torch.sqrt(chi / 4.0)
        spike = torch.rand(L, H, d, generator=g) < 0.005
        return torch.where(spike, x * 12.0, x)

    q, k, v = draw(), draw(), draw()
    ntt = torch.tensor([20, 40, 5, 3])
    offs_d = offs.to(DEV)
    q8, qs, bo = G.quantize_e4m3_block(q.to(DEV), offs_d)
    k8, ks, _ = G.quantize_e4m3_block(k.to(DEV), offs_d)
    v8, vs, _ = G.quantize_e4m3_block(v.to(DEV), offs_d)
    out = G.hstu_mha_fp8(N, 1.0 / 128, q8, k8, v8, qs, ks, vs, bo, offs_d, num_targets=ntt.to(DEV))
    torch.cuda.synchronize()
    nblk = int(bo[-1])
    deq = [O.dequantize_e4m3_block(t8.cpu(), s[:nblk].cpu(), bo.cpu().long(), offs)
           for t8, s in ((q8, qs), (k8, ks), (v8, vs))]
    ref_q = O.hstu_mha(N, 1.0 / 128, deq[0], deq[1], deq[2], offs, num_targets=ntt)
    ref = O.hstu_mha(N, 1.0 / 128, q, k, v, offs, num_targets=ntt)
    e_kernel, e_total, e_quant = O.rel_l2(out, ref_q), O.rel_l2(out, ref), O.rel_l2(ref_q, ref)
    PM._note(("fp8", dist), {"kernel_vs_dequantised": e_kernel, "vs_unquantised": e_total,
                             "quantisation_alone": e_quant})
    assert torch.isfinite(out.float()).all()
    assert e_kernel < 1e-2, e_kernel
    assert e_total < 5e-2, (e_total, e_quant)


def test_fp8_config3_full_size():
    """BASELINE configs[3] at full size through the FP8 forward: within the FP8 bound of the bf16
    kernel's result on the same inputs (itself checked against the oracle at this size), the same
    bits on a second run, and linear in the V scales (doubling them doubles the output exactly)."""
    w = W.config3()
    q, k, v = w.qkv(device=DEV)
    offs_d, nt_d = w.seq_offsets.to(DEV), w.num_targets.to(DEV)
    ref = G.hstu_mha(w.max_seq_len, w.alpha, q, k, v, offs_d, num_targets=nt_d, max_attn_len=w.max_attn_len,
                     contextual_seq_len=w.contextual_seq_len)
    q8, qs, bo = G.quantize_e4m3_block(q, offs_d)
    k8, ks, _ = G.quantize_e4m3_block(k, offs_d)
    v8, vs, _ = G.quantize_e4m3_block(v, offs_d)

    def run(vs_):
        return G.hstu_mha_fp8(w.max_seq_len, w.alpha, q8, k8, v8, qs, ks, vs_, bo, offs_d, num_targets=nt_d,
                              max_attn_len=w.max_attn_len, contextual_seq_len=w.contextual_seq_len)

    out = run(vs)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    assert torch.equal(out, run(vs))
    assert torch.equal(run(vs * 2), out * 2)
    err = float((out.float() - ref.float()).norm() / ref.float().norm())
    assert err < 5e-2, err
