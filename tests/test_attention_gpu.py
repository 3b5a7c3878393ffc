"""Batched tcgen05 GEMM (4-D TMA maps) and the attention built on it, against fp32 PyTorch."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("Bo,Bi,M,N,K", [(1, 3, 128, 256, 64), (2, 4, 200, 72, 96), (1, 16, 512, 512, 64),
                                         (3, 1, 77, 130, 40), (2, 8, 256, 64, 256)])
def test_batched_gemm_contiguous(Bo, Bi, M, N, K):
    from ferrum_b200.ops import gemm

    torch.manual_seed(0)
    a = torch.randn(Bo, Bi, M, K, device="cuda").bfloat16()
    b = torch.randn(Bo, Bi, N, K, device="cuda").bfloat16()
    ref = torch.matmul(a.float(), b.float().transpose(-1, -2)) * 0.5
    out = gemm.gemm_bf16_batched(a, b, alpha=0.5)
    assert out.shape == (Bo, Bi, M, N) and _rel(out, ref) < 6e-3
    out32 = gemm.gemm_bf16_batched(a, b, out_dtype=torch.float32, alpha=0.5)
    assert _rel(out32, ref) < 1e-5
    acc = torch.ones_like(out32)
    gemm.gemm_bf16_batched(a, b, out=acc, alpha=0.5, accumulate=True)
    assert _rel(acc, ref + 1) < 1e-5


def test_batched_gemm_strided_head_views():
    from ferrum_b200.ops import gemm

    torch.manual_seed(1)
    B, S, H, D = 2, 192, 4, 64
    q = torch.randn(B, S, H * D, device="cuda").bfloat16()
    k = torch.randn(B, S, H * D, device="cuda").bfloat16()
    v = torch.randn(B, S, H * D, device="cuda").bfloat16()
    qh, kh, vh = (t.view(B, S, H, D).permute(0, 2, 1, 3) for t in (q, k, v))  # no copies
    assert gemm.batched_operand_ok(qh) and gemm.batched_operand_ok(vh.transpose(-1, -2))
    s = gemm.gemm_bf16_batched(qh, kh, out_dtype=torch.float32, alpha=0.125)
    assert _rel(s, torch.matmul(qh.float(), kh.float().transpose(-1, -2)) * 0.125) < 1e-5
    p = torch.softmax(s, -1).bfloat16()
    # P @ V: V^T as the [N, K] operand is an MN-major view; output written in [B, S, H, D] order
    out = torch.empty(B, S, H, D, device="cuda", dtype=torch.bfloat16).permute(0, 2, 1, 3)
    gemm.gemm_bf16_batched(p, vh.transpose(-1, -2), out=out)
    assert _rel(out, torch.matmul(p.float(), vh.float())) < 6e-3
    # both operands MN-major (the dV = P^T dO product)
    do = torch.randn(B, H, S, D, device="cuda").bfloat16()
    dv = gemm.gemm_bf16_batched(p.transpose(-1, -2), do.transpose(-1, -2), out_dtype=torch.float32)
    assert _rel(dv, torch.matmul(p.float().transpose(-1, -2), do.float())) < 1e-5


def test_matmul_batched_autocast_uses_tensor_cores_and_differentiates():
    import ferrum_b200 as fb
    from ferrum_b200 import _lib
    from ferrum_b200.ops import functional as F

    torch.manual_seed(2)
    a = torch.randn(6, 96, 64, device="cuda", requires_grad=True)
    b = torch.randn(6, 64, 80, device="cuda", requires_grad=True)
    before = _lib.launch_count()
    with fb.autocast():
        y = F.matmul(a, b)
    y.float().square().mean().backward()
    assert _lib.launch_count() > before
    ar, br = a.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    yr = torch.matmul(ar, br)
    yr.square().mean().backward()
    assert _rel(y, yr) < 1e-2 and _rel(a.grad, ar.grad) < 2e-2 and _rel(b.grad, br.grad) < 2e-2


@pytest.mark.parametrize("masked", [False, True])
def test_multi_head_attention_matches_fp32_reference(masked):
    import ferrum_b200 as fb
    from ferrum_b200.nn import MultiHeadAttention

    torch.manual_seed(3)
    B, S, E, H = 2, 128, 256, 4
    mha = MultiHeadAttention(E, H, device=fb.Device.Cuda(0))
    x = torch.randn(B, S, E, device="cuda", requires_grad=True)
    mask = torch.tril(torch.ones(S, S, device="cuda", dtype=torch.bool)) if masked else None

    def reference(xr):
        Wq, Wk, Wv, Wo = (m.weight.detach().float() for m in (mha.q_proj, mha.k_proj, mha.v_proj, mha.out_proj))
        bq, bk, bv, bo = (m.bias.detach().float() for m in (mha.q_proj, mha.k_proj, mha.v_proj, mha.out_proj))
        sp = lambda t: t.view(B, S, H, E // H).transpose(1, 2)
        q, k, v = sp(xr @ Wq.t() + bq), sp(xr @ Wk.t() + bk), sp(xr @ Wv.t() + bv)
        s = q @ k.transpose(-1, -2) / math.sqrt(E // H)
        if mask is not None:
            s = s.masked_fill(~mask, -1e9)
        return (torch.softmax(s, -1) @ v).transpose(1, 2).reshape(B, S, E) @ Wo.t() + bo

    # fp32 path (SIMT batched kernel)
    y32 = mha.forward_attn(x, x, x, mask)
    xr = x.detach().clone().requires_grad_(True)
    yr = reference(xr)
    assert _rel(y32, yr) < 1e-4
    y32.square().mean().backward()
    yr.square().mean().backward()
    assert _rel(x.grad, xr.grad) < 1e-3
    # bf16 tensor-core path
    x.grad = None
    with fb.autocast():
        y16 = mha.forward_attn(x, x, x, mask)
    assert _rel(y16, yr) < 3e-2
    y16.float().square().mean().backward()
    assert _rel(x.grad, xr.grad) < 6e-2


def test_transformer_encoder_layer_trains_under_autocast():
    import ferrum_b200 as fb
    from ferrum_b200 import nn, optim

    torch.manual_seed(4)
    dev = fb.Device.Cuda(0)
    layer = nn.TransformerEncoderLayer(128, 4, 256, device=dev)
    head = nn.Linear(128, 5, device=dev)
    opt = optim.Adam(list(layer.parameters()) + list(head.parameters()), optim.AdamConfig(lr=1e-3))
    x = torch.randn(8, 32, 128, device="cuda")
    y = torch.randint(0, 5, (8,), device="cuda")
    losses = []
    for _ in range(30):
        opt.zero_grad()
        with fb.autocast():
            h = layer(x)
            logits = head(h.float().mean(1))
            loss = nn.cross_entropy(logits, y)
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert losses[-1] < 0.5 * losses[0]


@pytest.mark.parametrize("B,H,Sq,Skv,D", [(2, 3, 128, 128, 64), (1, 2, 256, 384, 64), (2, 2, 200, 200, 64),
                                          (1, 4, 64, 1000, 64), (1, 16, 1024, 1024, 64), (2, 3, 128, 128, 128),
                                          (1, 2, 200, 333, 128), (1, 8, 1024, 1024, 128)])
def test_flash_attention_forward_matches_softmax_attention(B, H, Sq, Skv, D):
    """Blockwise tcgen05 attention (online softmax, scores never materialised) against fp32 softmax(QK^T)V, with
    head-interleaved [B, S, H, D] storage, ragged sequence lengths, several key tiles and both head dimensions."""
    from ferrum_b200.ops import functional as F
    from ferrum_b200.utils.runtime import check_status

    torch.manual_seed(B * 7 + Sq + Skv)
    q = (torch.randn(B, Sq, H, D, device="cuda") * 0.8).bfloat16().permute(0, 2, 1, 3)
    k = (torch.randn(B, Skv, H, D, device="cuda") * 0.8).bfloat16().permute(0, 2, 1, 3)
    v = torch.randn(B, Skv, H, D, device="cuda").bfloat16().permute(0, 2, 1, 3)
    assert F.flash_attention_ok(q, k, v)
    scale = D ** -0.5
    out, lse = F.flash_attention(q, k, v, scale, return_lse=True)
    check_status()
    s = (q.float() @ k.float().transpose(-1, -2)) * scale
    ref = torch.softmax(s, -1) @ v.float()
    assert out.shape == ref.shape
    err = (out.float() - ref).abs().max().item()
    assert err < 2e-2, err  # bf16 probabilities and bf16 output
    assert torch.allclose(lse, torch.logsumexp(s, -1), atol=2e-3, rtol=1e-4)
    assert out.permute(0, 2, 1, 3).is_contiguous()  # stored [B, Sq, H, D]


def test_attention_module_uses_the_blockwise_kernel_without_gradients():
    import ferrum_b200 as fb
    from ferrum_b200 import _lib, nn

    torch.manual_seed(5)
    mha = nn.MultiHeadAttention(256, 4, device=fb.Device.Cuda(0))  # head dimension 64
    x = torch.randn(2, 192, 256, device="cuda")
    with fb.autocast():
        y_train = mha(x)              # differentiable path: batched GEMMs + softmax kernel
        with fb.no_grad():
            y_eval = mha(x)           # blockwise kernel
    assert y_eval.shape == y_train.shape
    assert (y_eval.float() - y_train.float()).abs().max().item() < 6e-2  # two bf16 roundings of values near 2


def test_memory_efficient_attention_gradients_match_the_materialising_path():
    """memory_efficient=True: blockwise forward + recomputing backward gives the same gradients as the path that
    keeps the probabilities."""
    import copy

    import ferrum_b200 as fb
    from ferrum_b200 import nn

    torch.manual_seed(6)
    ref = nn.MultiHeadAttention(128, 2, device=fb.Device.Cuda(0))
    eff = copy.deepcopy(ref)
    eff.memory_efficient = True
    x = torch.randn(2, 160, 128, device="cuda")
    outs, grads = [], []
    for m in (ref, eff):
        xi = x.clone().requires_grad_(True)
        with fb.autocast():
            y = m(xi)
        (y.float() * torch.linspace(-1, 1, y.numel(), device="cuda").reshape(y.shape)).sum().backward()
        outs.append(y.float().detach())
        grads.append([xi.grad] + [p.grad for p in m.torch_parameters()])
    assert _rel(outs[1], outs[0]) < 2e-2
    for a, b in zip(grads[1], grads[0]):
        assert _rel(a, b) < 3e-2, _rel(a, b)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("B,H,Sq,Skv", [(1, 2, 256, 256), (2, 2, 200, 300), (1, 3, 128, 640), (1, 1, 384, 384)])
def test_flash_attention_causal(B, H, Sq, Skv, D):
    """Causal (bottom-right aligned) masking inside the blockwise kernel: key tiles past the diagonal are skipped,
    the diagonal tiles masked per row, also when the offset Skv - Sq is not a multiple of the tile."""
    from ferrum_b200.ops import functional as F
    from ferrum_b200.utils.runtime import check_status

    torch.manual_seed(Sq + Skv)
    q = torch.randn(B, H, Sq, D, device="cuda").bfloat16()
    k = torch.randn(B, H, Skv, D, device="cuda").bfloat16()
    v = torch.randn(B, H, Skv, D, device="cuda").bfloat16()
    out = F.flash_attention(q, k, v, D ** -0.5, causal=True)
    check_status()
    s = (q.float() @ k.float().transpose(-1, -2)) * D ** -0.5
    i = torch.arange(Sq, device="cuda")[:, None]
    j = torch.arange(Skv, device="cuda")[None, :]
    s = s.masked_fill(j > i + (Skv - Sq), float("-inf"))
    ref = torch.softmax(s, -1) @ v.float()
    assert (out.float() - ref).abs().max().item() < 3e-2


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("B,H,Sq,Skv,causal", [(1, 2, 128, 128, False), (2, 3, 256, 384, False), (1, 2, 200, 200, True),
                                               (2, 2, 130, 333, False), (1, 4, 384, 512, True), (1, 1, 77, 77, True)])
def test_blockwise_attention_backward_matches_fp32_reference(B, H, Sq, Skv, causal, D):
    """dQ, dK, dV of the blockwise tcgen05 kernels (probabilities recomputed tile by tile from the saved row
    log-sum-exp) against PyTorch autograd in fp32 on the same bf16 operands: ragged sequence lengths, more keys than
    queries, causal masks with the diagonal inside a tile, head-interleaved (strided) operand views."""
    from ferrum_b200.ops import functional as F
    from ferrum_b200.utils.runtime import check_status

    torch.manual_seed(B * 100 + Sq + Skv)
    # operands as MultiHeadAttention produces them: [B, S, H * D] projections viewed as [B, H, S, D]
    q, k, v = (torch.randn(B, S, H * D, device="cuda").bfloat16().view(B, S, H, D).permute(0, 2, 1, 3)
               .requires_grad_(True) for S in (Sq, Skv, Skv))
    scale = 1.0 / math.sqrt(D)
    out = F.attention_blockwise(q, k, v, scale, causal=causal)
    go = torch.randn(B, H, Sq, D, device="cuda").bfloat16()
    gq, gk, gv = torch.autograd.grad(out, (q, k, v), go)
    check_status()
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    s = torch.matmul(qr, kr.transpose(-1, -2)) * scale
    if causal:
        i = torch.arange(Sq, device="cuda")[:, None]
        j = torch.arange(Skv, device="cuda")[None, :]
        s = s.masked_fill(j > i + (Skv - Sq), float("-inf"))
    ref = torch.matmul(torch.softmax(s, -1), vr)
    rq, rk, rv = torch.autograd.grad(ref, (qr, kr, vr), go.float())
    assert _rel(out, ref) < 1e-2
    assert gq.shape == q.shape and gk.shape == k.shape and gv.shape == v.shape
    assert _rel(gq, rq) < 2e-2, _rel(gq, rq)
    assert _rel(gk, rk) < 2e-2, _rel(gk, rk)
    assert _rel(gv, rv) < 2e-2, _rel(gv, rv)


def test_multi_head_attention_trains_through_the_blockwise_kernels():
    """Under autocast with head dimension 64 the module's training step uses the blockwise forward and backward
    (no S x S tensor is created); gradients of every projection agree with the fp32 reference module."""
    import ferrum_b200 as fb
    from ferrum_b200 import _lib
    from ferrum_b200.nn import MultiHeadAttention

    torch.manual_seed(8)
    B, S, E, H = 2, 256, 256, 4
    mha = MultiHeadAttention(E, H, device=fb.Device.Cuda(0))
    x = torch.randn(B, S, E, device="cuda", requires_grad=True)
    calls = []
    lib = _lib.cuda()
    orig = lib.fb_attention_bwd
    try:
        lib.fb_attention_bwd = lambda *a: (calls.append(1), orig(*a))[1]
        with fb.autocast():
            y = mha.forward_attn(x, x, x, causal=True)
        y.float().square().mean().backward()
    finally:
        lib.fb_attention_bwd = orig
    assert calls, "the blockwise backward kernel was not used"
    ref = torch.nn.MultiheadAttention(E, H, batch_first=True, device="cuda")
    with torch.no_grad():
        ref.in_proj_weight.copy_(torch.cat([mha.q_proj.weight, mha.k_proj.weight, mha.v_proj.weight]))
        ref.in_proj_bias.copy_(torch.cat([mha.q_proj.bias, mha.k_proj.bias, mha.v_proj.bias]))
        ref.out_proj.weight.copy_(mha.out_proj.weight)
        ref.out_proj.bias.copy_(mha.out_proj.bias)
    xr = x.detach().clone().requires_grad_(True)
    cm = torch.triu(torch.ones(S, S, device="cuda", dtype=torch.bool), 1)
    yr, _ = ref(xr, xr, xr, attn_mask=cm, need_weights=False)
    yr.square().mean().backward()
    assert _rel(y, yr) < 2e-2
    assert _rel(x.grad, xr.grad) < 4e-2
    gw = torch.cat([mha.q_proj.weight.grad, mha.k_proj.weight.grad, mha.v_proj.weight.grad])
    assert _rel(gw, ref.in_proj_weight.grad) < 4e-2


def test_backward_kernels_work_as_the_first_cuda_work_of_the_autograd_thread():
    """The backward's TMA maps are encoded on the autograd worker thread; in a fresh process that thread has made no
    CUDA runtime call before, and the driver's encoder refuses to work without a current context."""
    import subprocess
    import sys

    code = ("import torch\n"
            "from ferrum_b200.ops import functional as F\n"
            "q, k, v = (torch.randn(2, 1024, 16, 64, device='cuda').bfloat16().permute(0, 2, 1, 3).requires_grad_(True)"
            " for _ in range(3))\n"
            "g = torch.randn(2, 1024, 16, 64, device='cuda').bfloat16().permute(0, 2, 1, 3)\n"
            "dq, dk, dv = torch.autograd.grad(F.attention_blockwise(q, k, v, 0.125), (q, k, v), g)\n"
            "torch.cuda.synchronize()\n"
            "assert all(bool(torch.isfinite(t.float()).all()) for t in (dq, dk, dv))\n"
            "print('ok')\n")
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))     # the package lives beside tests/
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, cwd=root)
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr[-2000:]


def test_multihead_attention_head_dimension_128_uses_the_blockwise_forward():
    """Head dimension 128 under autocast: the blockwise kernels in inference and in training (``eff``: with
    ``memory_efficient`` set, which changes nothing where the blockwise backward applies) agree with the same module
    run through an explicit all-true mask, i.e. the batched-GEMM path."""
    import copy

    import ferrum_b200 as fb
    from ferrum_b200 import nn

    torch.manual_seed(5)
    ref = nn.MultiHeadAttention(256, 2, device=fb.Device.Cuda(0))
    eff = copy.deepcopy(ref)
    eff.memory_efficient = True
    x = torch.randn(2, 160, 256, device="cuda")
    with fb.autocast(), torch.no_grad():
        y_fast = eff(x).float()           # no gradient needed: the blockwise kernel
    outs, grads = [], []
    everything = torch.ones(160, 160, dtype=torch.bool, device="cuda")
    for m in (ref, eff):
        xi = x.clone().requires_grad_(True)
        with fb.autocast():
            y = m.forward_attn(xi, xi, xi, mask=everything) if m is ref else m(xi)
        (y.float() * torch.linspace(-1, 1, y.numel(), device="cuda").reshape(y.shape)).sum().backward()
        outs.append(y.float().detach())
        grads.append([xi.grad] + [p.grad for p in m.torch_parameters()])
    fb.utils.runtime.check_status()
    assert _rel(y_fast, outs[0]) < 2e-2 and _rel(outs[1], outs[0]) < 2e-2
    # (the key projection's bias has a zero gradient in exact arithmetic — a constant added to every key shifts all
    # scores of a row alike — so what both paths hold there is rounding noise: compare on the scale of all gradients)
    top = max(g.abs().max().item() for g in grads[0])
    for a, b in zip(grads[1], grads[0]):
        assert _rel(a, b) < 3e-2 or (a - b).abs().max().item() < 2e-3 * top, _rel(a, b)
