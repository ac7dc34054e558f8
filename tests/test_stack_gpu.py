"""The composed HSTU stack against the composite oracle: configs[2] (8 layers, D = 512, learned
relative bias, contextual prefix, targets) forward + backward with every parameter gradient, the
reference's target-invariance property, and the 16-bit layer against both the fp32 oracle and the
reference's own arithmetic in bf16.

Tolerance of the 16-bit comparisons: relative L2 <= 1e-2 against the fp32 oracle, or - for a chain
of 16-bit stages, where the reference itself rounds between the stages - no further from the fp32
oracle than 1.25 x the distance of the oracle run in bf16 (tests/parity_metrics.py)."""

import pytest
import torch
from torch.utils.checkpoint import checkpoint

import generative_recommenders_b200 as G
from generative_recommenders_b200 import workloads as W
from oracle import hstu_oracle as O
import parity_metrics as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def oracle_stack(x, offs, N, nt, layer_params, H, d, ctx, W_=0, bias_buckets=0, use_checkpoint=True):
    """``STUStack.forward`` of the reference (generative_recommenders/modules/stu.py:427-456) as a
    chain of the oracle's ``stu_layer``; with ``bias_buckets`` the research model's bucketised
    relative bias is added to the scores of every layer from that layer's ``rel_bias_table``."""
    h = x
    bucket = None
    if bias_buckets > 0:
        # bucket of every (i, j): the bucket function of O.bucketized_position_bias, evaluated once
        # for all layers; indexing each layer's table with it keeps the table in the graph
        # (only the corner the longest sequence of the batch reaches)
        n = min(N, int((offs[1:] - offs[:-1]).max()))
        i = torch.arange(n).view(n, 1)
        dist = (i - i.view(1, n)).abs().clamp(min=1).to(torch.float32)
        bucket = torch.clamp((torch.log(dist) / 0.301).long(), min=0, max=bias_buckets).to(x.device)
    for prm in layer_params:
        def one(h_, *flat, _names=tuple(prm.keys())):
            p_ = dict(zip(_names, flat))
            rb = None if bucket is None else p_["rel_bias_table"].to(torch.float32)[bucket]
            return O.stu_layer(h_, offs, N, nt, p_, H, d, d, max_attn_len=W_, contextual_seq_len=ctx, rel_bias=rb)
        if use_checkpoint:
            h = checkpoint(one, h, *prm.values(), use_reentrant=False)
        else:
            h = one(h, *prm.values())
    return h


def _layer_params(stack, dtype, device, grad=True):
    out = []
    for layer in stack._stu_layers:
        out.append({n[1:]: p_.detach().to(device).to(dtype).requires_grad_(grad) for n, p_ in layer.named_parameters()})
    return out


def _perturb_vectors(stack, seed):
    """LayerNorm weights / biases and the projection bias away from their 1 / 0 initial values, so
    that their gradients and their place in the formulas matter."""
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for p_ in stack.parameters():
            if p_.dim() == 1:
                p_.add_((0.1 * torch.randn(p_.shape, generator=g)).to(p_.device).to(p_.dtype))


def _config2_reduced_batch():
    """Twelve sequences of configs[2]'s seeded 128-sequence draw: its shortest, its three longest
    (966 tokens at most: the power law rarely reaches the 4096-token clip) and eight in between."""
    lengths_all, nt_all, _ = W.config2_lengths(128)
    order = torch.argsort(lengths_all)
    pick = [int(order[i]) for i in (0, 10, 30, 50, 70, 90, 105, 115, 122, 125, 126, 127)]
    return lengths_all[pick], nt_all[pick]


# The gradient of a bias table is a sum over all (query, key) pairs of all heads and sequences, with
# heavy cancellation (sum of |terms| / |sum of terms| is 13 on the 2000-token case measured for
# this test), so it amplifies the ~3e-3 rounding noise of the 16-bit attention output that reaches
# it through the output LayerNorm's backward: for fixed inputs the kernel's bias gradient is within
# 2e-4 of the oracle (test_relative_bias_backward_and_bias_gradient), inside a 16-bit stack it is
# 0.9e-2 .. 2.7e-2 away, the oracle run in bf16 0.7e-2 .. 1.3e-2.  Two 16-bit evaluation orders of
# such a sum differ by more than the 1.25 allowed elsewhere; the fp32 run of the same case pins the
# logic tightly.
TABLE_SLACK = 2.5


def _run_stack_case(name, layers, lengths, nt, use_checkpoint, dtype=torch.bfloat16):
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    D, H, d, N, ctx, nb = 512, 4, 128, 4096, 6, 128
    offs = W._offsets(lengths)
    L = int(offs[-1])
    cfg = G.STULayerConfig(embedding_dim=D, num_heads=H, hidden_dim=d, attention_dim=d, output_dropout_ratio=0.0,
                           contextual_seq_len=ctx, rel_bias_buckets=nb)
    torch.manual_seed(20262)
    stack = G.STUStack([G.STULayer(cfg) for _ in range(layers)]).to(DEV).to(dtype)
    _perturb_vectors(stack, 1)
    with torch.no_grad():
        for layer in stack._stu_layers:
            layer._rel_bias_table.mul_(10.0)   # std 0.2: a bias that matters next to q.k / sqrt(d)
    g = torch.Generator().manual_seed(7)
    x = torch.randn(L, D, generator=g).to(dtype)
    dy = torch.randn(L, D, generator=g).to(dtype)

    xin = x.to(DEV).requires_grad_(True)
    n0 = G._cabi.launch_count()
    y = stack(xin, lengths.to(DEV), offs.to(DEV), N, nt.to(DEV))
    y.backward(dy.to(DEV))
    torch.cuda.synchronize()
    assert G._cabi.launch_count() > n0

    # fp32 oracle on the CPU, on the same (bf16-rounded) parameters and inputs
    p32 = _layer_params(stack, torch.float32, "cpu")
    x32 = x.float().requires_grad_(True)
    ref = oracle_stack(x32, offs, N, nt, p32, H, d, ctx, bias_buckets=nb, use_checkpoint=use_checkpoint)
    ref.backward(dy.float())
    if dtype == torch.float32:
        # fp32 kernels (CUDA-core attention, LayerNorm / SiLU kernels, fp32 library GEMMs): the
        # composite logic at accumulation-order tolerance
        tol = dict(tol=2e-3, seq_tol=2e-3, max_tol=2e-3)
        P.check((name, "fp32", "y"), y, ref.detach(), offs, **tol)
        P.check((name, "fp32", "dx"), xin.grad, x32.grad, offs, **tol)
        for li, layer in enumerate(stack._stu_layers):
            for n, p_ in layer.named_parameters():
                P.check((name, "fp32", li, n), p_.grad, p32[li][n[1:]].grad, None, **tol)
        return
    # the reference's own arithmetic in bf16: the same oracle code on 16-bit tensors, run on the
    # device (bf16 matrix products are slow on host cores without bf16 units)
    p16 = _layer_params(stack, torch.bfloat16, DEV)
    x16 = x.to(DEV).requires_grad_(True)
    ref16 = oracle_stack(x16, offs, N, nt, p16, H, d, ctx, bias_buckets=nb, use_checkpoint=False)
    ref16.backward(dy.to(DEV))

    P.check_vs_bf16_reference((name, "y"), y, ref.detach(), ref16.detach())
    P.check_vs_bf16_reference((name, "dx"), xin.grad, x32.grad, x16.grad)
    for li, layer in enumerate(stack._stu_layers):
        for n, p_ in layer.named_parameters():
            assert p_.grad is not None, (li, n)
            P.check_vs_bf16_reference((name, li, n), p_.grad, p32[li][n[1:]].grad, p16[li][n[1:]].grad,
                                      slack=TABLE_SLACK if n == "_rel_bias_table" else 1.25)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_config2_stack_forward_backward_all_parameter_gradients(dtype):
    """configs[2] at full depth and width (8 layers, D = 512, H = 4, d = 128, 128-bucket learned
    relative bias, contextual prefix 6, targets, max_seq_len 4096), bf16, on a reduced batch of its
    seeded sequences: y, dx and the gradient of every parameter of every layer - the bias tables
    included - against autograd through the composite oracle.  The fp32 run of the same stack (the
    CUDA-core attention kernels) checks the composition at 2e-3."""
    lengths, nt = _config2_reduced_batch()
    _run_stack_case("config2_stack", 8, lengths, nt, use_checkpoint=False, dtype=dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_config2_layers_with_a_4096_token_sequence(dtype):
    """The same layer configuration on a sequence at the length distribution's upper clip (4096
    tokens = max_seq_len: 32 tiles, the long-sequence kernel variants) next to a mid-sized and a
    minimal one; two layers keep the CPU oracle at some ten seconds."""
    _run_stack_case("config2_4096", 2, torch.tensor([4096, 300, 16]), torch.tensor([64, 20, 9]),
                    use_checkpoint=False, dtype=dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_target_invariance(dtype):
    """Targets attend to the history and to themselves and nobody attends to them, so exchanging
    two targets of a sequence at the input exchanges their rows at the output, and likewise for
    the input gradient when the upstream gradient is exchanged too (the property the reference
    checks in modules/tests/stu_test.py:180-321)."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.manual_seed(3)
    D, H, d = 64, 2, 64
    cfg = G.STULayerConfig(embedding_dim=D, num_heads=H, hidden_dim=d, attention_dim=d, output_dropout_ratio=0.0,
                           target_aware=True)
    stack = G.STUStack([G.STULayer(cfg), G.STULayer(cfg)]).to(DEV).to(dtype)
    g = torch.Generator().manual_seed(5)
    B = 8
    nt = torch.randint(2, 10, (B,), generator=g)
    lengths = torch.randint(2, 200, (B,), generator=g) + nt
    offs = W._offsets(lengths)
    L, N = int(offs[-1]), int(lengths.max())
    a = lengths - 1 - torch.remainder(torch.randint(0, 20, (B,), generator=g), nt)
    b = lengths - 1 - torch.remainder(torch.randint(0, 20, (B,), generator=g), nt)
    perm = torch.arange(L)
    for s in range(B):
        ia, ib = int(offs[s] + a[s]), int(offs[s] + b[s])
        perm[ia], perm[ib] = ib, ia
    x = torch.randn(L, D, generator=g).to(dtype)
    dy = torch.randn(L, D, generator=g).to(dtype)

    def run(x_, dy_):
        xin = x_.to(DEV).requires_grad_(True)
        y = stack(xin, lengths.to(DEV), offs.to(DEV), N, nt.to(DEV))
        y.backward(dy_.to(DEV))
        return y.detach().cpu(), xin.grad.cpu()

    y0, dx0 = run(x, dy)
    y1, dx1 = run(x[perm], dy[perm])
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(y1[perm], y0, **tol)
    torch.testing.assert_close(dx1[perm], dx0, **tol)


def test_recompute_flags_change_memory_not_results():
    """``recompute_uvqk`` / ``recompute_y`` (the reference's STULayerConfig fields, modules/stu.py:77-79)
    drop the two widest activations of a layer - the [L, 4 H d] projection and the [L, 3 H d] input
    of the output linear - and rebuild them in the backward with the same kernels: every result
    carries the same bits, dropout included (the mask is regenerated from the same seed), and the
    memory held between forward and backward shrinks."""
    torch.backends.cuda.matmul.allow_tf32 = False
    D, H, d = 512, 4, 128
    g = torch.Generator().manual_seed(9)
    lengths = torch.randint(200, 900, (12,), generator=g)
    nt = torch.randint(1, 30, (12,), generator=g)
    offs = W._offsets(lengths)
    L = int(offs[-1])
    x = torch.randn(L, D, generator=g).bfloat16().to(DEV)
    dy = torch.randn(L, D, generator=g).bfloat16().to(DEV)
    res, held = {}, {}
    for rec in (False, True):
        cfg = G.STULayerConfig(embedding_dim=D, num_heads=H, hidden_dim=d, attention_dim=d, output_dropout_ratio=0.3,
                               contextual_seq_len=3, recompute_normed_x=rec, recompute_uvqk=rec, recompute_y=rec)
        torch.manual_seed(1)
        stack = G.STUStack([G.STULayer(cfg) for _ in range(2)]).to(DEV).to(torch.bfloat16)
        stack.train(True)
        xin = x.clone().requires_grad_(True)
        torch.manual_seed(77)        # the dropout seeds come from torch's generator
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        base = torch.cuda.memory_allocated()
        y = stack(xin, lengths.to(DEV), offs.to(DEV), 1024, nt.to(DEV))
        torch.cuda.synchronize()
        held[rec] = torch.cuda.memory_allocated() - base
        y.backward(dy)
        torch.cuda.synchronize()
        res[rec] = [y.detach(), xin.grad] + [p_.grad for p_ in stack.parameters()]
    for a, b in zip(res[False], res[True]):
        assert torch.equal(a, b)
    assert float((res[True][0] == res[False][0]).float().mean()) == 1.0
    # per layer the projection (2048 columns) and the concat (1536) go, of ~7 D columns kept otherwise
    assert held[True] < 0.7 * held[False], held
