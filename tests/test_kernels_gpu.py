"""Every CUDA kernel family against a plain fp32 PyTorch statement of the same op (forward and backward)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

SIZES = [1, 31, 33, 127, 4097, 70001]


def _F():
    from ferrum_b200.ops import functional as F

    return F


def _ref_unary(x, op, a, b):
    from ferrum_b200.ops.functional import _unary_cpu

    return _unary_cpu(x, op, a, b)


UNARY_CASES = [("relu", 0, 0), ("gelu", 0, 0), ("silu", 0, 0), ("tanh", 0, 0), ("sigmoid", 0, 0),
               ("leaky_relu", 0.01, 0), ("elu", 1.0, 0), ("neg", 0, 0), ("exp", 0, 0), ("log", 0, 0),
               ("sqrt", 0, 0), ("abs", 0, 0), ("sin", 0, 0), ("cos", 0, 0), ("pow", 3.0, 0), ("add_scalar", 1.5, 0),
               ("mul_scalar", -2.0, 0), ("rsub_scalar", 1.0, 0), ("rdiv_scalar", 2.0, 0), ("affine", 2.0, -1.0),
               ("clamp", -0.5, 0.5)]


@pytest.mark.parametrize("op,a,b", UNARY_CASES)
@pytest.mark.parametrize("n", [33, 4097])
def test_unary_fwd_bwd_f32(op, a, b, n):
    F = _F()
    torch.manual_seed(0)
    x = torch.randn(n, device="cuda")
    if op in ("log", "sqrt", "rdiv_scalar"):
        x = x.abs() + 0.5
    x1 = x.clone().requires_grad_(True)
    x2 = x.clone().requires_grad_(True)
    y = F.unary(x1, op, a, b)
    yr = _ref_unary(x2, op, a, b)
    assert torch.allclose(y, yr, atol=1e-5, rtol=1e-5), op
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g)
    assert torch.allclose(x1.grad, x2.grad, atol=1e-4, rtol=1e-4), op


@pytest.mark.parametrize("op", ["relu", "gelu", "silu", "tanh"])
def test_unary_bf16(op):
    F = _F()
    x = torch.randn(4099, device="cuda").to(torch.bfloat16)
    y = F.unary(x, op)
    yr = _ref_unary(x.float(), op, 0, 0)
    assert y.dtype == torch.bfloat16
    assert torch.allclose(y.float(), yr, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div", "max", "min", "pow"])
@pytest.mark.parametrize("sa,sb", [((5, 7), (5, 7)), ((5, 7), (7,)), ((5, 1), (1, 7)), ((3, 1, 4), (2, 1)),
                                   ((4097,), (1,)), ((2, 3, 4, 5), (4, 1))])
def test_binary_broadcast(op, sa, sb):
    F = _F()
    torch.manual_seed(1)
    a = torch.rand(sa, device="cuda") + 0.5
    b = torch.rand(sb, device="cuda") + 0.5
    a1, b1 = a.clone().requires_grad_(True), b.clone().requires_grad_(True)
    a2, b2 = a.clone().requires_grad_(True), b.clone().requires_grad_(True)
    from ferrum_b200.ops.functional import _binary_cpu

    y = F.binary(a1, b1, op)
    yr = _binary_cpu(a2, b2, op)
    assert y.shape == yr.shape
    assert torch.allclose(y, yr, atol=1e-5, rtol=1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g)
    assert torch.allclose(a1.grad, a2.grad, atol=1e-4, rtol=1e-4)
    assert torch.allclose(b1.grad, b2.grad, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("op", ["sum", "mean", "max", "min", "prod"])
@pytest.mark.parametrize("shape,dim", [((7,), None), ((70001,), None), ((33, 65), 0), ((33, 65), 1), ((4, 5, 6), 1),
                                       ((3, 20000), 1), ((20000, 3), 0), ((1 << 20,), None)])
def test_reduce(op, shape, dim):
    F = _F()
    torch.manual_seed(2)
    x = torch.rand(shape, device="cuda") * 0.02 + 0.99 if op == "prod" else torch.randn(shape, device="cuda")
    if op == "prod" and x.numel() > 100000:
        pytest.skip("product of a million values is not a meaningful numeric check")
    x1 = x.clone().requires_grad_(True)
    x2 = x.clone().double().requires_grad_(True)
    y = F.reduce(x1, op, dim)
    if dim is None:
        yr = getattr(torch, op)(x2)
    elif op in ("max", "min"):
        yr = getattr(torch, op)(x2, dim=dim).values
    else:
        yr = getattr(torch, op)(x2, dim=dim)
    assert torch.allclose(y.double(), yr, atol=1e-3 if op == "sum" else 1e-4, rtol=1e-4)
    if op in ("sum", "mean"):
        g = torch.randn_like(y)
        y.backward(g)
        yr.backward(g.double())
        assert torch.allclose(x1.grad.double(), x2.grad, atol=1e-5)


@pytest.mark.parametrize("shape,dim", [((100,), None), ((33, 65), 1), ((33, 65), 0), ((4, 5, 6), 1)])
def test_argmax_argmin(shape, dim):
    F = _F()
    x = torch.randn(shape, device="cuda")
    for is_max in (True, False):
        got = F.arg_reduce(x, is_max, dim)
        ref = (torch.argmax if is_max else torch.argmin)(x) if dim is None else (
            torch.argmax if is_max else torch.argmin)(x, dim=dim)
        assert torch.equal(got, ref)


@pytest.mark.parametrize("rows,cols", [(5, 8), (128, 256), (33, 1024), (64, 4096), (7, 8192), (9, 1000), (3, 10),
                                       (4, 12000)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pre_act", [None, "gelu"])
def test_layernorm(rows, cols, dtype, pre_act):
    F = _F()
    torch.manual_seed(3)
    x = torch.randn(rows, cols, device="cuda").to(dtype)
    gamma = torch.rand(cols, device="cuda") + 0.5
    beta = torch.randn(cols, device="cuda")
    x1 = x.clone().requires_grad_(True)
    g1, b1 = gamma.clone().requires_grad_(True), beta.clone().requires_grad_(True)
    y = F.layer_norm(x1, g1, b1, 1e-5, pre_act)
    x2 = x.float().clone().requires_grad_(True)
    g2, b2 = gamma.clone().requires_grad_(True), beta.clone().requires_grad_(True)
    a = torch.nn.functional.gelu(x2, approximate="tanh") if pre_act else x2
    yr = torch.nn.functional.layer_norm(a, (cols,), g2, b2, 1e-5)
    tol = 1e-4 if dtype == torch.float32 else 4e-2
    assert torch.allclose(y.float(), yr, atol=tol, rtol=tol)
    go = torch.randn(rows, cols, device="cuda").to(dtype)
    y.backward(go)
    yr.backward(go.float())
    btol = 2e-3 if dtype == torch.float32 else 8e-2
    assert torch.allclose(x1.grad.float(), x2.grad, atol=btol, rtol=btol)
    scale = max(1.0, g2.grad.abs().max().item())
    assert (g1.grad - g2.grad).abs().max().item() < (2e-3 if dtype == torch.float32 else 8e-2) * scale
    assert (b1.grad - b2.grad).abs().max().item() < (2e-3 if dtype == torch.float32 else 8e-2) * max(
        1.0, b2.grad.abs().max().item())


@pytest.mark.parametrize("rows,cols", [(4, 10), (128, 10), (33, 1000), (5, 5000), (1, 1)])
@pytest.mark.parametrize("log_mode", [False, True])
def test_softmax(rows, cols, log_mode):
    F = _F()
    x = torch.randn(rows, cols, device="cuda") * 3
    x1 = x.clone().requires_grad_(True)
    x2 = x.clone().requires_grad_(True)
    y = (F.log_softmax if log_mode else F.softmax)(x1, -1)
    yr = (torch.log_softmax if log_mode else torch.softmax)(x2, -1)
    assert torch.allclose(y, yr, atol=1e-5, rtol=1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g)
    assert torch.allclose(x1.grad, x2.grad, atol=1e-5, rtol=1e-4)


def test_softmax_other_dim():
    F = _F()
    x = torch.randn(4, 7, 5, device="cuda")
    assert torch.allclose(F.softmax(x, 1), torch.softmax(x, 1), atol=1e-6)


@pytest.mark.parametrize("rows,cols", [(128, 10), (64, 1000), (7, 513)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_cross_entropy_fused(rows, cols, dtype):
    F = _F()
    torch.manual_seed(4)
    x = (torch.randn(rows, cols, device="cuda") * 2).to(dtype)
    labels = torch.randint(0, cols, (rows,), device="cuda")
    x1 = x.clone().requires_grad_(True)
    x2 = x.float().clone().requires_grad_(True)
    loss = F.cross_entropy_logits(x1, labels)
    ref = torch.nn.functional.cross_entropy(x2, labels)
    assert abs(loss.item() - ref.item()) < 1e-4 * max(1, abs(ref.item()))
    (loss * 2.0).backward()
    (ref * 2.0).backward()
    tol = 1e-6 if dtype == torch.float32 else 1e-3
    assert torch.allclose(x1.grad.float(), x2.grad, atol=tol, rtol=2e-2)


@pytest.mark.parametrize("kind", ["mse", "bce", "l1", "smooth_l1"])
def test_elementwise_losses(kind):
    F = _F()
    torch.manual_seed(5)
    p = torch.rand(37, 11, device="cuda") * 0.9 + 0.05
    t = (torch.rand(37, 11, device="cuda") > 0.5).float() if kind == "bce" else torch.randn(37, 11, device="cuda") * 2
    p1 = p.clone().requires_grad_(True)
    p2 = p.cpu().clone().requires_grad_(True)
    l1 = F.elementwise_loss(p1, t, kind)
    l2 = F.elementwise_loss(p2, t.cpu(), kind)
    assert abs(l1.item() - l2.item()) < 1e-5 * max(1, abs(l2.item()))
    l1.backward()
    l2.backward()
    assert torch.allclose(p1.grad.cpu(), p2.grad, atol=1e-6, rtol=1e-4)


def test_dropout_statistics_and_backward():
    F = _F()
    x = torch.ones(1 << 20, device="cuda", requires_grad=True)
    y = F.dropout(x, 0.25, True, seed=123)
    kept = (y != 0).float().mean().item()
    assert abs(kept - 0.75) < 5e-3
    assert torch.allclose(y[y != 0], torch.full_like(y[y != 0], 1 / 0.75))
    y.sum().backward()
    assert torch.equal(x.grad != 0, y != 0)
    y2 = F.dropout(x.detach(), 0.25, True, seed=123)
    assert not torch.equal(y2 != 0, y != 0)  # the offset advances between calls
    assert F.dropout(x, 0.25, False) is x


def test_embedding_fwd_bwd():
    F = _F()
    torch.manual_seed(6)
    w = torch.randn(50, 24, device="cuda")
    idx = torch.randint(0, 50, (7, 9), device="cuda")
    idx[0, 0] = 3
    w1 = w.clone().requires_grad_(True)
    w2 = w.clone().requires_grad_(True)
    y = F.embedding(w1, idx, padding_idx=3)
    yr = torch.nn.functional.embedding(idx, w2, padding_idx=3) * (idx != 3).unsqueeze(-1)
    assert torch.allclose(y, yr)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g)
    assert torch.allclose(w1.grad, w2.grad, atol=1e-5)


def test_embedding_mean_pool():
    F = _F()
    torch.manual_seed(7)
    w = torch.randn(1000, 64, device="cuda")
    idx = torch.randint(0, 30, (16, 40), device="cuda")  # heavy duplication
    w1 = w.clone().requires_grad_(True)
    w2 = w.clone().requires_grad_(True)
    y = F.embedding_mean_pool(w1, idx)
    yr = torch.nn.functional.embedding(idx, w2).mean(1)
    assert torch.allclose(y, yr, atol=1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g)
    assert torch.allclose(w1.grad, w2.grad, atol=1e-4)


def test_batchnorm_train_and_eval():
    F = _F()
    torch.manual_seed(8)
    x = torch.randn(64, 37, device="cuda") * 2 + 1
    gamma = torch.rand(37, device="cuda") + 0.5
    beta = torch.randn(37, device="cuda")
    rm, rv = torch.zeros(37, device="cuda"), torch.ones(37, device="cuda")
    rm2, rv2 = rm.clone(), rv.clone()
    x1 = x.clone().requires_grad_(True)
    g1, b1 = gamma.clone().requires_grad_(True), beta.clone().requires_grad_(True)
    y = F.batch_norm(x1, g1, b1, rm, rv, True, 0.1, 1e-5)
    x2 = x.clone().requires_grad_(True)
    g2, b2 = gamma.clone().requires_grad_(True), beta.clone().requires_grad_(True)
    yr = torch.nn.functional.batch_norm(x2, rm2, rv2, g2, b2, True, 0.1, 1e-5)
    assert torch.allclose(y, yr, atol=1e-4, rtol=1e-4)
    assert torch.allclose(rm, rm2, atol=1e-5) and torch.allclose(rv, rv2, atol=1e-4)
    go = torch.randn_like(y)
    y.backward(go)
    yr.backward(go)
    assert torch.allclose(x1.grad, x2.grad, atol=1e-4, rtol=1e-3)
    assert torch.allclose(g1.grad, g2.grad, atol=1e-3, rtol=1e-3)
    assert torch.allclose(b1.grad, b2.grad, atol=1e-4, rtol=1e-3)
    ye = F.batch_norm(x, gamma, beta, rm, rv, False, 0.1, 1e-5)
    yer = torch.nn.functional.batch_norm(x, rm2, rv2, gamma, beta, False, 0.1, 1e-5)
    assert torch.allclose(ye, yer, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("rows,cols,offset", [(8192, 1024, 0.0), (4100, 130, 300.0), (33, 7, -50.0)])
def test_batchnorm_one_pass_statistics_survive_a_large_mean(rows, cols, offset):
    """The statistics come from one pass over the shifted data x - x[0]; a column mean far from zero must not cost
    the variance its digits (sum of squares minus squared sum of the raw data would)."""
    F = _F()
    torch.manual_seed(9)
    x = torch.randn(rows, cols, device="cuda") * 0.5 + offset
    rm, rv = torch.zeros(cols, device="cuda"), torch.ones(cols, device="cuda")
    y = F.batch_norm(x, None, None, rm, rv, True, 1.0, 1e-5)
    xd = x.double()
    ref = (xd - xd.mean(0)) / torch.sqrt(xd.var(0, unbiased=False) + 1e-5)
    assert (y.double() - ref).abs().max().item() < 2e-3
    assert torch.allclose(rm.double(), xd.mean(0), atol=1e-4 * max(1.0, abs(offset)))
    assert torch.allclose(rv.double(), xd.var(0, unbiased=True), rtol=2e-3)


def test_cast_transpose_gather_colsum():
    F = _F()
    x = torch.randn(130, 77, device="cuda")
    xb = F.raw_cast(x, torch.bfloat16)
    assert torch.equal(xb, x.to(torch.bfloat16))
    assert torch.equal(F.raw_cast(xb, torch.float32), xb.float())
    assert torch.equal(F.transpose_2d(x), x.t().contiguous())
    assert torch.equal(F.transpose_2d(xb), xb.t().contiguous())
    idx = torch.randint(0, 130, (50,), device="cuda")
    assert torch.equal(F.gather_rows(x, idx), x[idx])
    assert torch.equal(F.gather_rows(xb, idx), xb[idx])
    big = torch.randn(8192, 520, device="cuda")
    assert torch.allclose(F.raw_colsum(big), big.sum(0), atol=2e-3)
    assert torch.allclose(F.raw_colsum(big.to(torch.bfloat16)), big.to(torch.bfloat16).float().sum(0), atol=2e-2)


def _adam_ref(p, g, m, v, t, lr, b1, b2, eps, wd):
    p = p - lr * wd * p
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    mh = m / (1 - b1 ** t)
    vh = v / (1 - b2 ** t)
    return p - lr * mh / (vh.sqrt() + eps), m, v


def test_adam_and_sgd_steps_match_reference_rules():
    from ferrum_b200 import optim

    torch.manual_seed(9)
    shapes = [(33,), (64, 64), (4097,), (5, 7)]
    ps = [torch.randn(s, device="cuda", requires_grad=True) for s in shapes]
    ref = [p.detach().clone() for p in ps]
    m = [torch.zeros_like(p) for p in ref]
    v = [torch.zeros_like(p) for p in ref]
    opt = optim.Adam(ps, optim.AdamConfig(lr=1e-2, weight_decay=0.1))
    for t in range(1, 4):
        for i, p in enumerate(ps):
            p.grad = torch.randn_like(p)
            ref[i], m[i], v[i] = _adam_ref(ref[i], p.grad, m[i], v[i], t, 1e-2, 0.9, 0.999, 1e-8, 0.1)
        opt.step()
    for p, r in zip(ps, ref):
        assert torch.allclose(p.detach(), r, atol=1e-5, rtol=1e-5)

    ps = [torch.randn(s, device="cuda", requires_grad=True) for s in shapes]
    ref = [p.detach().clone() for p in ps]
    vel = [None] * len(ps)
    opt = optim.SGD(ps, optim.SGDConfig(lr=0.1, momentum=0.9, weight_decay=1e-2, nesterov=True))
    for t in range(3):
        for i, p in enumerate(ps):
            p.grad = torch.randn_like(p)
            g = p.grad + 1e-2 * ref[i]
            vel[i] = g.clone() if vel[i] is None else 0.9 * vel[i] + g
            ref[i] = ref[i] - 0.1 * (g + 0.9 * vel[i])
        opt.step()
    for p, r in zip(ps, ref):
        assert torch.allclose(p.detach(), r, atol=1e-5, rtol=1e-5)


def test_amp_kernels():
    from ferrum_b200 import optim

    gs = [torch.randn(1000, device="cuda") * 4, torch.randn(33, 7, device="cuda") * 4]
    ref = [g.clone() for g in gs]
    sc = optim.GradScaler.with_scale(8.0)
    assert sc.unscale_gradients(gs) is True
    for g, r in zip(gs, ref):
        assert torch.allclose(g, r / 8.0)
    gs[0][5] = float("inf")
    assert sc.step(gs) is False and sc.get_scale() == 4.0
    gs = [torch.randn(1000, device="cuda"), torch.randn(33, 7, device="cuda")]
    ref = [g.clone() for g in gs]
    total = math.sqrt(sum((g ** 2).sum().item() for g in ref))
    got = optim.clip_grad_norm(gs, 1.0)
    assert abs(got - total) < 1e-3 * total
    for g, r in zip(gs, ref):
        assert torch.allclose(g, r * (1.0 / (total + 1e-6)), atol=1e-6)
    optim.clip_grad_value(gs, 0.01)
    assert all(g.abs().max().item() <= 0.01 + 1e-9 for g in gs)


@pytest.mark.parametrize("low", [False, True])
def test_linear_fwd_bwd(low):
    from ferrum_b200 import config
    F = _F()
    torch.manual_seed(10)
    x = torch.randn(96, 136, device="cuda")
    w = torch.randn(72, 136, device="cuda") * 0.1
    b = torch.randn(72, device="cuda")
    x1, w1, b1 = (t.clone().requires_grad_(True) for t in (x, w, b))
    x2, w2, b2 = (t.clone().requires_grad_(True) for t in (x, w, b))
    with config.autocast(torch.bfloat16, enabled=low):
        y = F.linear(x1, w1, b1, act=None if low else "relu")
    yr = torch.nn.functional.linear(x2, w2, b2)
    if not low:  # a bf16 forward flips the ReLU mask of near-zero outputs, so the mask is tested in fp32 only
        yr = torch.relu(yr)
    tol = 5e-2 if low else 1e-4
    assert torch.allclose(y.float(), yr, atol=tol, rtol=tol)
    g = torch.randn_like(yr)
    y.backward(g.to(y.dtype))
    yr.backward(g)
    assert torch.allclose(x1.grad, x2.grad, atol=tol * 2, rtol=tol)
    assert torch.allclose(w1.grad, w2.grad, atol=tol * 8, rtol=tol)
    assert torch.allclose(b1.grad, b2.grad, atol=tol * 8, rtol=tol)


@pytest.mark.parametrize("low", [False, True])
def test_fused_linear_gelu_layernorm_block(low):
    """Sequential's fused Linear-GELU-LayerNorm node equals the composition of the three layers."""
    import ferrum_b200 as fb
    from ferrum_b200 import nn

    torch.manual_seed(11)
    dev = fb.Device.Cuda(0)
    blk = nn.Sequential(nn.Linear(136, 264, device=dev), nn.GELU(), nn.LayerNorm([264], device=dev))
    with torch.no_grad():
        blk[2].weight.uniform_(0.5, 1.5)
        blk[2].bias.normal_()
    x = torch.randn(200, 136, device="cuda")
    x1 = x.clone().requires_grad_(True)
    with fb.autocast(enabled=low):
        y = blk(x1)
    x2 = x.clone().requires_grad_(True)
    ref = torch.nn.functional.layer_norm(
        torch.nn.functional.gelu(torch.nn.functional.linear(x2, blk[0].weight, blk[0].bias), approximate="tanh"),
        (264,), blk[2].weight, blk[2].bias, 1e-5)
    tol = 6e-2 if low else 2e-4
    assert torch.allclose(y.float(), ref, atol=tol, rtol=tol)
    g = torch.randn_like(ref)
    y.backward(g.to(y.dtype))
    mine = [x1.grad] + [p.grad.clone() for p in blk.torch_parameters()]
    blk.zero_grad()
    ref.backward(g)
    theirs = [x2.grad] + [p.grad for p in blk.torch_parameters()]
    for a, b in zip(mine, theirs):
        scale = max(1.0, b.abs().max().item())
        assert (a.float() - b).abs().max().item() < (0.15 if low else 2e-3) * scale


@pytest.mark.parametrize("rows,cols", [(300, 4096), (150, 2560), (64, 4000), (70, 1024), (33, 264)])
@pytest.mark.parametrize("with_act_grad", [False, True])
def test_layernorm_bwd_with_stored_activation_derivative(rows, cols, with_act_grad):
    """LayerNorm backward on bf16 rows where the activation derivative comes as a tensor: the 512-thread
    streaming kernel for 2056..4096 columns, the register-tiled kernels otherwise."""
    from ferrum_b200 import _lib

    lib = _lib.cuda()
    torch.manual_seed(rows + cols)
    a = torch.randn(rows, cols, device="cuda").bfloat16()
    dy = torch.randn(rows, cols, device="cuda").bfloat16()
    da = (torch.rand(rows, cols, device="cuda") * 1.5).bfloat16() if with_act_grad else None
    gamma = torch.rand(cols, device="cuda") + 0.5
    af = a.float().requires_grad_(True)
    gr = gamma.clone().requires_grad_(True)
    br = torch.zeros(cols, device="cuda", requires_grad=True)
    yr = torch.nn.functional.layer_norm(af, (cols,), gr, br, 1e-5)
    yr.backward(dy.float())
    ref_dx = af.grad * (da.float() if with_act_grad else 1.0)
    mean = a.float().mean(1)
    rstd = torch.rsqrt(a.float().var(1, unbiased=False) + 1e-5)
    dx = torch.empty_like(a)
    nblk = lib.fb_layernorm_bwd_blocks(rows, cols)
    partial = torch.empty(max(nblk, 1), 3, cols, device="cuda")
    stats = torch.zeros(3, cols, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    rc = lib.fb_layernorm_bwd(dy.data_ptr(), a.data_ptr(), da.data_ptr() if with_act_grad else None, gamma.data_ptr(),
                              mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(), partial.data_ptr(), stats.data_ptr(),
                              rows, cols, 0, 3, nblk, 1, st)
    assert rc == 0
    torch.cuda.synchronize()
    scale = max(1.0, ref_dx.abs().max().item())
    assert (dx.float() - ref_dx).abs().max().item() < 2e-2 * scale
    assert torch.allclose(stats[0], gr.grad, atol=2e-2 * max(1.0, gr.grad.abs().max().item()))
    assert torch.allclose(stats[1], br.grad, atol=2e-2 * max(1.0, br.grad.abs().max().item()))
    ref_cs = ref_dx.sum(0)
    assert torch.allclose(stats[2], ref_cs, atol=3e-2 * max(1.0, ref_cs.abs().max().item()))


@pytest.mark.parametrize("act", ["gelu", "relu", "silu", "tanh", "sigmoid"])
@pytest.mark.parametrize("M,N,K", [(640, 512, 128), (200, 264, 136), (1024, 1000, 64)])
def test_gemm_epilogue_stores_activation_and_derivative(act, M, N, K):
    from ferrum_b200.ops import gemm

    torch.manual_seed(M + N)
    a = (torch.randn(M, K, device="cuda") * 0.3).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.3).bfloat16()
    bias = torch.randn(N, device="cuda")
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    der = torch.empty_like(out)
    gemm.gemm_bf16(a, b, bias=bias, act=act, out=out, act_grad=der)
    z = (a.float() @ b.float().t() + bias).requires_grad_(True)
    fn = {"gelu": lambda t: torch.nn.functional.gelu(t, approximate="tanh"), "relu": torch.relu,
          "silu": torch.nn.functional.silu, "tanh": torch.tanh, "sigmoid": torch.sigmoid}[act]
    val = fn(z)
    val.sum().backward()
    assert (out.float() - val).abs().max().item() < 3e-2 * max(1.0, val.abs().max().item())
    mism = (der.float() - z.grad).abs()
    if act == "relu":  # pre-activations within rounding of zero may land on either side
        assert (mism > 1e-2).float().mean().item() < 1e-3
    else:
        assert mism.max().item() < 2e-2


@pytest.mark.parametrize("op", ["sum", "mean", "max", "min", "prod"])
@pytest.mark.parametrize("shape,dim", [((8192, 256), 0), ((3, 700, 132), 1), ((5000, 4), 0), ((2, 33, 8), 1)])
def test_reduce_columns_vectorised(op, shape, dim):
    F = _F()
    torch.manual_seed(7)
    x = torch.randn(*shape, device="cuda")
    if op == "prod":
        x = 1.0 + 0.001 * x
    got = F.raw_reduce(x, op, dim)
    xd = x.double()
    ref = {"sum": xd.sum(dim), "mean": xd.mean(dim), "max": xd.max(dim).values, "min": xd.min(dim).values,
           "prod": xd.prod(dim)}[op]
    assert got.shape == ref.shape
    assert torch.allclose(got.double(), ref, rtol=1e-4, atol=1e-3)


def test_cross_entropy_backward_scales_by_incoming_gradient_on_device():
    F = _F()
    torch.manual_seed(9)
    for dtype in (torch.float32, torch.bfloat16):
        x = torch.randn(257, 1000, device="cuda").to(dtype)
        labels = torch.randint(0, 1000, (257,), device="cuda")
        x1 = x.clone().requires_grad_(True)
        x2 = x.float().clone().requires_grad_(True)
        (F.cross_entropy_logits(x1, labels) * -3.5).backward()
        (torch.nn.functional.cross_entropy(x2, labels) * -3.5).backward()
        assert torch.allclose(x1.grad.float(), x2.grad, atol=1e-6 if dtype == torch.float32 else 2e-4, rtol=2e-2)


def test_layernorm_forward_ring_variant_in_subprocess():
    """The opt-in forward ring kernel (FERRUM_LN_RING_FWD=1, read once per process) against PyTorch."""
    import os
    import subprocess
    import sys

    code = r"""
import torch, sys
sys.path.insert(0, %r)
from ferrum_b200.ops import functional as F
torch.manual_seed(0)
for dtype, tol in ((torch.bfloat16, 4e-2), (torch.float32, 2e-4)):
    for rows, cols in ((300, 4096), (77, 2048), (5, 1024 if dtype == torch.float32 else 4000)):
        x = (torch.randn(rows, cols, device="cuda") * 2 + 0.7).to(dtype)
        g = torch.rand(cols, device="cuda") + 0.5
        b = torch.randn(cols, device="cuda")
        y = F.layer_norm(x, g, b, 1e-5)
        ref = torch.nn.functional.layer_norm(x.float(), (cols,), g, b, 1e-5)
        err = (y.float() - ref).abs().max().item()
        assert err < tol, (dtype, rows, cols, err)
from ferrum_b200.utils.runtime import check_status
check_status()
print("RING_OK")
""" % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, FERRUM_LN_RING_FWD="1")
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert "RING_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]
