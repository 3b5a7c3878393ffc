"""Recurrent gate kernels, im2col / col2im convolution lowering and pooling kernels against PyTorch fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, tol=1e-4):
    assert a.shape == b.shape
    assert (a.float() - b.float()).abs().max().item() <= tol * max(1.0, b.float().abs().max().item())


def test_lstm_gate_kernel_matches_reference_formulas():
    from ferrum_b200.ops import functional as F

    torch.manual_seed(0)
    B, H = 37, 96
    xi, hh, c = (torch.randn(B, 4 * H, device="cuda", requires_grad=True),
                 torch.randn(B, 4 * H, device="cuda", requires_grad=True),
                 torch.randn(B, H, device="cuda", requires_grad=True))
    h2, c2 = F.lstm_gates(xi, hh, c)
    (h2.square().sum() + (c2 * 0.5).sum()).backward()
    xr, hr, cr = (t.detach().clone().requires_grad_(True) for t in (xi, hh, c))
    i, f, g, o = (xr + hr).chunk(4, -1)
    cref = torch.sigmoid(f) * cr + torch.sigmoid(i) * torch.tanh(g)
    href = torch.sigmoid(o) * torch.tanh(cref)
    (href.square().sum() + (cref * 0.5).sum()).backward()
    _close(h2, href), _close(c2, cref)
    _close(xi.grad, xr.grad), _close(hh.grad, hr.grad), _close(c.grad, cr.grad)


def test_gru_gate_kernel_matches_reference_formulas():
    from ferrum_b200.ops import functional as F

    torch.manual_seed(1)
    B, H = 29, 64
    xi, hh, h = (torch.randn(B, 3 * H, device="cuda", requires_grad=True),
                 torch.randn(B, 3 * H, device="cuda", requires_grad=True),
                 torch.randn(B, H, device="cuda", requires_grad=True))
    out = F.gru_gates(xi, hh, h)
    out.square().sum().backward()
    xr, hr, pr = (t.detach().clone().requires_grad_(True) for t in (xi, hh, h))
    a, b_, c_ = xr.chunk(3, -1)
    d, e, f = hr.chunk(3, -1)
    r, z = torch.sigmoid(a + d), torch.sigmoid(b_ + e)
    n = torch.tanh(c_ + r * f)
    ref = (1 - z) * n + z * pr
    ref.square().sum().backward()
    _close(out, ref)
    _close(xi.grad, xr.grad), _close(hh.grad, hr.grad), _close(h.grad, pr.grad)


@pytest.mark.parametrize("cls", ["LSTM", "GRU"])
def test_recurrent_modules_match_torch(cls):
    import ferrum_b200 as fb
    from ferrum_b200 import nn

    torch.manual_seed(2)
    T, B, Fi, H = 7, 5, 12, 16
    ours = getattr(nn, cls)(Fi, H, 2, device=fb.Device.Cuda(0))
    ref = getattr(torch.nn, cls)(Fi, H, 2).double()  # CPU float64: cuDNN's fp32 RNN may run on TF32
    for l, cell in enumerate(ours.cells):
        for ours_name, ref_name in (("weight_ih", f"weight_ih_l{l}"), ("weight_hh", f"weight_hh_l{l}"),
                                    ("bias_ih", f"bias_ih_l{l}"), ("bias_hh", f"bias_hh_l{l}")):
            getattr(ref, ref_name).data.copy_(getattr(cell, ours_name).data.double().cpu())
    x = torch.randn(T, B, Fi, device="cuda", requires_grad=True)
    xr = x.detach().double().cpu().requires_grad_(True)
    y = ours(x)
    yr, _ = ref(xr)
    _close(y.cpu(), yr, 1e-4)
    y.square().mean().backward()
    yr.square().mean().backward()
    _close(x.grad.cpu(), xr.grad, 1e-4)
    _close(ours.cells[0].weight_hh.grad.cpu(), ref.weight_hh_l0.grad, 1e-4)


@pytest.mark.parametrize("cfg", [(3, 8, 3, 1, 1, 1, 1), (4, 6, 5, 2, 2, 1, 2), (6, 4, 3, 1, 0, 2, 1), (2, 2, 2, 3, 1, 1, 1)])
def test_conv2d_forward_backward_matches_torch(cfg):
    import ferrum_b200 as fb
    from ferrum_b200 import nn

    cin, cout, k, stride, pad, dil, groups = cfg
    torch.manual_seed(3)
    conv = nn.Conv2d(cin, cout, k, stride, pad, dil, groups, device=fb.Device.Cuda(0))
    x = torch.randn(3, cin, 17, 13, device="cuda", requires_grad=True)
    xr = x.detach().clone().requires_grad_(True)
    y = conv(x)
    wr, br = conv.weight.detach().clone().requires_grad_(True), conv.bias.detach().clone().requires_grad_(True)
    yr = torch.nn.functional.conv2d(xr, wr, br, stride, pad, dil, groups)
    _close(y, yr, 1e-4)
    y.square().mean().backward()
    yr.square().mean().backward()
    _close(x.grad, xr.grad, 1e-4), _close(conv.weight.grad, wr.grad, 1e-4), _close(conv.bias.grad, br.grad, 1e-4)


@pytest.mark.parametrize("B,cin,cout,H,W,k,pad,dil", [
    (2, 3, 5, 17, 19, (3, 3), (1, 1), (1, 1)),          # RGB-like input: channels padded to 8
    (1, 64, 64, 56, 56, (3, 3), (1, 1), (1, 1)),        # the kernel benchmark's layer
    (2, 16, 200, 20, 33, (3, 5), (1, 2), (2, 1)),       # 256-column tile, rectangular dilated filter
    (2, 136, 72, 9, 70, (1, 1), (0, 0), (1, 1)),        # pointwise, three channel chunks, wide flat image
    (3, 24, 40, 12, 12, (5, 5), (2, 2), (1, 1)),
    (1, 8, 8, 5, 4, (3, 3), (0, 0), (1, 1)),            # output smaller than one patch
])
def test_conv2d_implicit_gemm_forward_backward_matches_fp32(B, cin, cout, H, W, k, pad, dil):
    """Under bf16 autocast a stride-1 convolution takes the implicit-GEMM kernels in all three directions; the result
    is compared with an fp32 PyTorch convolution of the bf16-rounded operands (products are exact in fp32, so only
    the accumulation order and the bf16 rounding of the incoming gradient differ)."""
    import ferrum_b200 as fb
    from ferrum_b200 import nn
    from ferrum_b200.ops import functional as F

    torch.manual_seed(11)
    conv = nn.Conv2d(cin, cout, k, 1, pad, dil, 1, device=fb.Device.Cuda(0))
    x = torch.randn(B, cin, H, W, device="cuda", requires_grad=True)
    with fb.autocast():
        assert F.conv_igemm_ok(x, (1, 1), dil, pad, k, 1)
        y = conv(x)
    fb.utils.runtime.check_status()
    r16 = lambda t: t.detach().bfloat16().float()
    xr, wr = r16(x).requires_grad_(True), r16(conv.weight).requires_grad_(True)
    br = conv.bias.detach().clone().requires_grad_(True)
    yr = torch.nn.functional.conv2d(xr, wr, br, 1, pad, dil, 1)
    assert y.dtype == torch.float32 and y.shape == yr.shape
    _close(y, yr, 2e-4)
    g = torch.randn_like(yr).bfloat16().float()         # a gradient that bf16 represents exactly
    y.backward(g)
    yr.backward(g)
    fb.utils.runtime.check_status()
    _close(x.grad, xr.grad, 2e-4), _close(conv.weight.grad, wr.grad, 2e-4), _close(conv.bias.grad, br.grad, 2e-4)


@pytest.mark.parametrize("B,cin,cout,H,W,k,stride,pad", [
    (2, 3, 5, 17, 19, (3, 3), (2, 2), (1, 1)),
    (1, 4, 6, 16, 16, (4, 4), (4, 4), (0, 0)),          # patch embedding: kernel = stride, one plain GEMM
    (2, 5, 7, 15, 20, (5, 3), (2, 3), (2, 1)),          # different strides per axis, kernel not a multiple of them
    (1, 3, 64, 56, 56, (7, 7), (2, 2), (3, 3)),         # a ResNet stem
    (2, 64, 128, 28, 28, (3, 3), (2, 2), (1, 1)),       # a down-sampling layer: 256 space-to-depth channels
])
def test_strided_conv2d_under_autocast_runs_through_space_to_depth(B, cin, cout, H, W, k, stride, pad):
    """Strided convolutions reach the implicit-GEMM kernels through the space-to-depth layout: forward, data gradient
    and weight gradient against an fp32 PyTorch convolution of the bf16-rounded operands."""
    import ferrum_b200 as fb
    from ferrum_b200 import nn
    from ferrum_b200.ops import functional as F

    torch.manual_seed(13)
    conv = nn.Conv2d(cin, cout, k, stride, pad, 1, 1, device=fb.Device.Cuda(0))
    x = torch.randn(B, cin, H, W, device="cuda", requires_grad=True)
    with fb.autocast():
        assert F.conv_igemm_ok(x, stride, (1, 1), pad, k, 1)
        y = conv(x)
    fb.utils.runtime.check_status()
    r16 = lambda t: t.detach().bfloat16().float()
    xr, wr = r16(x).requires_grad_(True), r16(conv.weight).requires_grad_(True)
    br = conv.bias.detach().clone().requires_grad_(True)
    yr = torch.nn.functional.conv2d(xr, wr, br, stride, pad, 1, 1)
    assert y.shape == yr.shape
    _close(y, yr, 2e-4)
    g = torch.randn_like(yr).bfloat16().float()
    y.backward(g)
    yr.backward(g)
    fb.utils.runtime.check_status()
    _close(x.grad, xr.grad, 2e-4), _close(conv.weight.grad, wr.grad, 2e-4), _close(conv.bias.grad, br.grad, 2e-4)


def test_conv1d_under_autocast_takes_the_implicit_gemm():
    """Conv1d is a one-row Conv2d: under autocast with stride 1 it runs on the implicit-GEMM kernels (patch 128 x 1)."""
    import ferrum_b200 as fb
    from ferrum_b200 import nn

    torch.manual_seed(12)
    conv = nn.Conv1d(24, 40, 5, 1, 2, 1, 1, device=fb.Device.Cuda(0))
    x = torch.randn(3, 24, 301, device="cuda", requires_grad=True)
    with fb.autocast():
        y = conv(x)
    r16 = lambda t: t.detach().bfloat16().float()
    xr, wr = r16(x).requires_grad_(True), r16(conv.weight).requires_grad_(True)
    br = conv.bias.detach().clone().requires_grad_(True)
    yr = torch.nn.functional.conv1d(xr, wr, br, 1, 2, 1, 1)
    _close(y, yr, 2e-4)
    g = torch.randn_like(yr).bfloat16().float()
    y.backward(g)
    yr.backward(g)
    fb.utils.runtime.check_status()
    _close(x.grad, xr.grad, 2e-4), _close(conv.weight.grad, wr.grad, 2e-4), _close(conv.bias.grad, br.grad, 2e-4)


def test_im2col_rows_are_gemm_ready():
    from ferrum_b200.ops import functional as F

    x = torch.randn(2, 3, 6, 5, device="cuda")
    cols = F.im2col(x, (3, 2), (1, 2), (1, 0), (1, 1))
    ref = torch.nn.functional.unfold(x, (3, 2), dilation=1, padding=(1, 0), stride=(1, 2))
    assert cols.is_contiguous() and cols.shape == (2 * ref.shape[2], 3 * 3 * 2)
    _close(cols, ref.transpose(1, 2).reshape(cols.shape), 0)


@pytest.mark.parametrize("C,k,stride,pad,dil", [(4, (3, 3), (1, 1), (1, 1), (1, 1)), (8, (3, 3), (2, 1), (0, 2), (1, 2)),
                                                 (2, (3, 2), (1, 2), (1, 0), (2, 1)), (12, (1, 1), (1, 1), (0, 0), (1, 1)),
                                                 (5, (2, 2), (1, 1), (1, 1), (1, 1)), (16, (5, 5), (2, 2), (2, 2), (1, 1))])
def test_im2col_warp_per_row_kernel_matches_unfold(C, k, stride, pad, dil):
    """Window matrices whose row length is a multiple of 4 take the warp-per-row kernel (vector stores, index
    arithmetic once per four columns); every geometry must reproduce torch's unfold exactly."""
    from ferrum_b200.ops import functional as F

    torch.manual_seed(C)
    x = torch.randn(3, C, 19, 14, device="cuda")
    cols = F.im2col(x, k, stride, pad, dil)
    ref = torch.nn.functional.unfold(x, k, dilation=dil, padding=pad, stride=stride)
    assert cols.shape == (3 * ref.shape[2], C * k[0] * k[1])
    assert torch.equal(cols, ref.transpose(1, 2).reshape(cols.shape))


@pytest.mark.parametrize("op", ["max", "avg"])
@pytest.mark.parametrize("k,s", [(2, 2), (3, 2), (3, 1)])
def test_pool2d_forward_backward(op, k, s):
    from ferrum_b200 import nn

    torch.manual_seed(4)
    x = torch.randn(2, 5, 11, 14, device="cuda", requires_grad=True)
    xr = x.detach().clone().requires_grad_(True)
    pool = (nn.MaxPool2d if op == "max" else nn.AvgPool2d).with_stride(k, s)
    y = pool(x)
    yr = (torch.nn.functional.max_pool2d if op == "max" else torch.nn.functional.avg_pool2d)(xr, k, s)
    _close(y, yr, 1e-6)
    (y * torch.arange(y.numel(), device="cuda").reshape(y.shape)).sum().backward()
    (yr * torch.arange(y.numel(), device="cuda").reshape(y.shape)).sum().backward()
    _close(x.grad, xr.grad, 1e-5)


def test_small_cnn_trains():
    import ferrum_b200 as fb
    from ferrum_b200 import nn, optim

    class Flatten(nn.Module):
        def forward(self, t):
            return t.reshape(t.shape[0], -1)

    torch.manual_seed(5)
    dev = fb.Device.Cuda(0)
    net = nn.Sequential(nn.Conv2d(1, 8, 3, 1, 1, device=dev), nn.ReLU(), nn.MaxPool2d(2), Flatten(),
                        nn.Linear(8 * 4 * 4, 3, device=dev))
    opt = optim.Adam(net.parameters(), optim.AdamConfig(lr=1e-2))
    x = torch.randn(24, 1, 8, 8, device="cuda")
    y = torch.randint(0, 3, (24,), device="cuda")
    losses = []
    for _ in range(40):
        opt.zero_grad()
        loss = nn.cross_entropy(net(x), y)
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert losses[-1] < 0.5 * losses[0]


def test_resnet18_under_autocast_matches_the_fp32_path():
    """Every convolution of the model zoo's ResNet-18 on the implicit-GEMM kernels (7 x 7 stride-2 stem on three
    channels, 3 x 3 stride-1 and stride-2 layers, 1 x 1 stride-2 shortcuts, no biases, feature maps down to 2 x 2):
    logits agree with the fp32 im2col path within bf16 accuracy, weight gradients in direction."""
    import copy

    import ferrum_b200 as fb
    from ferrum_b200.models.vision import ResNet

    torch.manual_seed(21)
    net = ResNet.resnet18(10, device=fb.Device.Cuda(0))
    ref = copy.deepcopy(net)
    x = torch.randn(4, 3, 64, 64, device="cuda")
    with fb.autocast():
        y = net(x)
    yr = ref(x)
    fb.utils.runtime.check_status()
    assert y.shape == yr.shape == (4, 10)
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()
    assert rel(y, yr) < 5e-2, rel(y, yr)
    g = torch.randn_like(yr)
    y.float().backward(g)
    yr.backward(g)
    fb.utils.runtime.check_status()
    # seventeen bf16 layers with ReLU and max-pool switches between the loss and the stem: the gradients agree in
    # direction, not digit by digit
    cos = lambda a, b: torch.nn.functional.cosine_similarity(a.flatten().float(), b.flatten().float(), dim=0).item()
    for a, b in ((net.conv1.weight.grad, ref.conv1.weight.grad),
                 (net.blocks[2].downsample.weight.grad, ref.blocks[2].downsample.weight.grad),
                 (net.fc.weight.grad, ref.fc.weight.grad)):
        assert torch.isfinite(a).all() and cos(a, b) > 0.8, cos(a, b)
