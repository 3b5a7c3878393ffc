"""Layers, losses, optimizers, schedulers and AMP utilities on CPU (value-level, unlike the reference's
shape-only layer tests: ferrum-nn/src/*.rs tests, ferrum-optim/src/{scheduler,amp}.rs tests)."""
import ctypes
import math

import numpy as np
import pytest
import torch

import ferrum_b200 as fb
from ferrum_b200 import Tensor, nn, optim


def test_linear_shapes_init_and_values():
    l = nn.Linear(64, 32)
    assert l.in_features() == 64 and l.out_features() == 32 and l.num_parameters() == 64 * 32 + 32
    bound = math.sqrt(6 / 64)
    assert l.weight.abs().max().item() <= bound + 1e-6 and l.bias.abs().max().item() <= 1 / 8 + 1e-6
    assert nn.Linear.with_bias(4, 3, False).bias is None and len(nn.Linear(4, 3, bias=False).parameters()) == 1
    x = Tensor.randn([5, 64])
    y = l(x)
    assert y.shape == (5, 32)
    assert torch.allclose(y.torch(), x.torch() @ l.weight.t() + l.bias, atol=1e-5)
    assert l(Tensor.randn([2, 3, 64])).shape == (2, 3, 32)
    with pytest.raises(fb.ShapeMismatch):
        l(Tensor.randn([5, 63]))


def test_sequential_container():
    m = nn.Sequential.new()
    assert m.is_empty() and m.len() == 0
    m.add(nn.Linear(4, 8)).add(nn.ReLU()).add_boxed(nn.Linear(8, 2))
    assert m.len() == 3 and len(m.parameters()) == 4 and m.name() == "Sequential"
    assert m(Tensor.randn([3, 4])).shape == (3, 2)
    assert m.is_training()
    m.eval()
    assert not m.is_training() and not m[0].is_training()
    m.train()
    assert m[2].is_training()
    assert set(m.state_dict().keys()) == {"0.weight", "0.bias", "2.weight", "2.bias"}


def test_activations_at_known_points():
    x = Tensor.from_slice([-2.0, 0.0, 3.0])
    assert nn.ReLU()(x).to_vec() == [0, 0, 3]
    assert abs(nn.Sigmoid()(x).to_vec()[1] - 0.5) < 1e-7
    assert nn.Tanh()(x).to_vec()[1] == 0
    assert nn.LeakyReLU(0.01)(x).to_vec()[0] == pytest.approx(-0.02)
    assert nn.ELU(1.0)(x).to_vec()[0] == pytest.approx(math.exp(-2) - 1)
    g = nn.GELU()(x).to_vec()
    ref = [0.5 * v * (1 + math.tanh(0.7978845608028654 * (v + 0.044715 * v ** 3))) for v in (-2.0, 0.0, 3.0)]
    assert g == pytest.approx(ref, abs=1e-6)
    assert nn.SiLU()(x).to_vec()[2] == pytest.approx(3 / (1 + math.exp(-3)))


def test_softmax_is_per_row_and_stable():
    x = Tensor.from_slice([[1.0, 2.0, 3.0], [1000.0, 1000.0, 1000.0]])
    s = nn.Softmax(-1)(x)
    assert s.sum_dim(1).to_vec() == pytest.approx([1.0, 1.0])
    assert s.to_vec()[3:] == pytest.approx([1 / 3] * 3)
    ls = nn.LogSoftmax(-1)(x)
    assert ls.exp().sum_dim(1).to_vec() == pytest.approx([1.0, 1.0])
    assert nn.softmax(x, 0).sum_dim(0).to_vec() == pytest.approx([1.0] * 3)


def test_layernorm_is_per_row_with_trainable_affine():
    ln = nn.LayerNorm([8])
    x = Tensor.randn([4, 8]).mul_scalar(3).add_scalar(5)
    y = ln(x)
    assert y.mean_dim(1).to_vec() == pytest.approx([0.0] * 4, abs=1e-5)
    assert all(p.requires_grad() for p in ln.parameters()) and len(ln.parameters()) == 2
    assert nn.LayerNorm(8, 1e-6).eps == 1e-6
    ref = torch.nn.functional.layer_norm(x.torch(), (8,), ln.weight, ln.bias, 1e-5)
    assert torch.allclose(y.torch(), ref, atol=1e-5)
    y2 = nn.LayerNorm([2, 4])(Tensor.randn([3, 2, 4]))
    assert y2.shape == (3, 2, 4)


def test_batchnorm_training_updates_running_stats_and_eval_uses_them():
    bn = nn.BatchNorm1d(3)
    x = Tensor.from_slice(np.random.RandomState(0).randn(16, 3).astype("float32") * 2 + 1)
    y = bn(x)
    assert y.mean_dim(0).to_vec() == pytest.approx([0.0] * 3, abs=1e-5)
    assert bn.running_mean.abs().sum().item() > 0  # never updated in the reference
    bn.eval()
    y2 = bn(x)
    ref = (x.torch() - bn.running_mean) / torch.sqrt(bn.running_var + 1e-5)
    assert torch.allclose(y2.torch(), ref, atol=1e-5)


def test_dropout_is_inverted_and_identity_in_eval():
    d = nn.Dropout(0.5)
    x = Tensor.ones([10000])
    y = d(x).to_vec()
    assert set(round(v, 4) for v in y) <= {0.0, 2.0} and 0.4 < sum(1 for v in y if v) / 10000 < 0.6
    d.eval()
    assert d(x).to_vec() == x.to_vec()
    with pytest.raises(fb.FerrumError):
        nn.Dropout(1.5)


def test_embedding():
    e = nn.Embedding(10, 4)
    assert e.weight.shape == (10, 4) and e.weight.requires_grad
    idx = Tensor.from_slice([[1, 2], [3, 1]], dtype=fb.DType.I64)
    out = e(idx)
    assert out.shape == (2, 2, 4) and torch.equal(out.torch()[0, 0], e.weight[1])
    out.sum().backward()
    assert e.weight.grad[1].tolist() == [2.0] * 4 and e.weight.grad[0].tolist() == [0.0] * 4
    ep = nn.Embedding(10, 4).with_padding_idx(0)
    assert ep(Tensor.from_slice([0, 5], dtype=fb.DType.I64)).to_vec()[:4] == [0.0] * 4
    with pytest.raises(fb.IndexOutOfBounds):
        e(Tensor.from_slice([10], dtype=fb.DType.I64))
    with pytest.raises(fb.FerrumError):
        e(Tensor.from_slice([1.0]))
    fp = nn.Embedding.from_pretrained(Tensor.ones([3, 2]), freeze=True)
    assert not fp.weight.requires_grad
    assert nn.MeanPoolEmbedding(10, 4)(idx).shape == (2, 4)


def test_losses_values():
    p = Tensor.from_slice([1.0, 2.0, 3.0])
    t = Tensor.from_slice([1.0, 2.0, 3.0])
    assert nn.mse_loss(p, t).item() == 0
    assert nn.mse_loss(Tensor.from_slice([1.0, 2.0, 3.0]), Tensor.from_slice([2.0, 4.0, 6.0])).item() == pytest.approx(
        14 / 3)
    assert nn.l1_loss(Tensor.from_slice([1.0, 2.0, 3.0]), Tensor.from_slice([3.0, 4.0, 5.0])).item() == 2
    assert nn.smooth_l1_loss(Tensor.from_slice([0.5, 3.0]), Tensor.from_slice([0.0, 0.0])).item() == pytest.approx(
        (0.125 + 2.5) / 2)
    pr, tg = Tensor.from_slice([0.8, 0.2, 0.9]), Tensor.from_slice([1.0, 0.0, 1.0])
    ref = -sum(math.log(v) for v in (0.8 + 1e-7, 1 - 0.2, 0.9 + 1e-7)) / 3
    assert nn.bce_loss(pr, tg).item() == pytest.approx(ref, rel=1e-5)
    logits = Tensor.from_slice([[1.0, 2.0, 0.5], [0.1, 0.2, 3.0]])
    lp = nn.log_softmax(logits, -1)
    onehot = Tensor.from_slice([[0.0, 1.0, 0.0], [0.0, 0.0, 1.0]])
    ce = nn.cross_entropy_loss(lp, onehot).item()
    assert ce == pytest.approx(-(lp.to_vec()[1] + lp.to_vec()[5]) / 6)  # mean over B*C like the reference
    labels = Tensor.from_slice([1, 2], dtype=fb.DType.I64)
    assert nn.nll_loss(lp, labels).item() == pytest.approx(-(lp.to_vec()[1] + lp.to_vec()[5]) / 2)
    assert nn.cross_entropy(logits, labels).item() == pytest.approx(nn.nll_loss(lp, labels).item(), rel=1e-6)
    with pytest.raises(fb.ShapeMismatch):
        nn.mse_loss(Tensor.ones([2, 3]), Tensor.ones([4]))


def test_bce_gradient_flows():  # severed in the reference (add_scalar records nothing)
    m = nn.Sequential(nn.Linear(2, 1), nn.Sigmoid())
    loss = nn.bce_loss(m(Tensor.from_slice([[0.0, 1.0]])), Tensor.from_slice([[1.0]]))
    loss.backward()
    assert all(p.grad() is not None and p.grad().torch().abs().sum() > 0 for p in m.parameters())


def test_init_functions():
    w = nn.init.xavier_uniform((100, 50), 50, 100)
    assert w.abs().max().item() <= math.sqrt(6 / 150) + 1e-6
    assert abs(nn.init.kaiming_normal((400, 100), 100).std().item() - math.sqrt(2 / 100)) < 0.02
    q = nn.init.orthogonal((8, 8))
    assert torch.allclose(q @ q.t(), torch.eye(8), atol=1e-5)
    assert nn.init.constant((2, 2), 3.0).tolist() == [[3, 3], [3, 3]] and nn.init.zeros((2,)).sum() == 0


def _host():
    from ferrum_b200 import _lib

    return _lib.host()


def test_sgd_and_adam_match_the_reference_loops():
    torch.manual_seed(0)
    for cfg in (optim.SGDConfig.new(0.1), optim.SGDConfig.new(0.1).with_momentum(0.9).with_weight_decay(1e-2),
                optim.SGDConfig(lr=0.05, momentum=0.8, nesterov=True)):
        p = torch.randn(37, requires_grad=True)
        ref = p.detach().clone().numpy()
        vel = np.zeros(37, dtype=np.float32)
        opt = optim.SGD([p], cfg)
        for step in range(3):
            g = torch.randn(37)
            p.grad = g.clone()
            gn = g.numpy().copy()
            _host().fb_ref_sgd_step(ref.ctypes.data, gn.ctypes.data, vel.ctypes.data, 37, cfg.lr, cfg.momentum,
                                    cfg.weight_decay, 1 if cfg.nesterov else 0, 1 if step == 0 else 0)
            opt.step()
        assert np.allclose(p.detach().numpy(), ref, atol=1e-6)
    p = torch.randn(53, requires_grad=True)
    ref = p.detach().clone().numpy()
    m, v = np.zeros(53, dtype=np.float32), np.zeros(53, dtype=np.float32)
    cfg = optim.AdamConfig.new(1e-2).with_betas(0.8, 0.95).with_weight_decay(0.1)
    opt = optim.Adam([p], cfg)
    for t in range(1, 5):
        g = torch.randn(53)
        p.grad = g.clone()
        gn = g.numpy().copy()
        _host().fb_ref_adam_step(ref.ctypes.data, gn.ctypes.data, m.ctypes.data, v.ctypes.data, 53, 1e-2, 0.8, 0.95,
                                 1e-8, 0.1, t)
        opt.step()
    assert np.allclose(p.detach().numpy(), ref, atol=1e-6)
    assert optim.AdamConfig(betas=(0.5, 0.6)).beta2 == 0.6 and opt.learning_rate() == 1e-2
    opt.set_learning_rate(0.5)
    assert opt.learning_rate() == 0.5 and opt.param_groups()[0]["lr"] == 0.5
    opt.zero_grad()
    assert p.grad is None


def test_schedulers_closed_form():
    s = optim.StepLR(0.1, 10, 0.1)
    assert s.get_lr() == pytest.approx(0.1)
    for _ in range(10):
        s.step()
    assert s.get_lr() == pytest.approx(0.01)
    for _ in range(10):
        s.step()
    assert s.get_lr() == pytest.approx(0.001) and s.current_step() == 20
    s.reset()
    assert s.get_lr() == pytest.approx(0.1)
    s = optim.MultiStepLR(0.1, [15, 5], 0.1)
    for _ in range(5):
        s.step()
    assert s.get_lr() == pytest.approx(0.01)
    for _ in range(10):
        s.step()
    assert s.get_lr() == pytest.approx(0.001)
    s = optim.ExponentialLR(1.0, 0.5)
    s.step(), s.step()
    assert s.get_lr() == pytest.approx(0.25)
    s = optim.CosineAnnealingLR(0.1, 100, 0.0)
    for _ in range(50):
        s.step()
    assert s.get_lr() == pytest.approx(0.05)
    for _ in range(60):
        s.step()
    assert s.get_lr() == pytest.approx(0.0, abs=1e-12)
    s = optim.CosineAnnealingWarmRestarts(0.1, 10, 2, 0.0)
    for _ in range(10):
        s.step()
    assert s.get_lr() == pytest.approx(0.1) and s.current_t_i == 20  # restarted
    s = optim.LinearWarmupLR(0.1, 10, 100)
    assert s.get_lr() == 0
    for _ in range(5):
        s.step()
    assert s.get_lr() == pytest.approx(0.05)
    for _ in range(5):
        s.step()
    assert s.get_lr() == pytest.approx(0.1)
    for _ in range(90):
        s.step()
    assert s.get_lr() == pytest.approx(0.0)
    s = optim.OneCycleLR.new_default(1.0, 100)
    assert s.get_lr() == pytest.approx(1 / 25)
    for _ in range(30):
        s.step()
    assert s.get_lr() == pytest.approx(1.0)
    for _ in range(100):
        s.step()
    assert s.get_lr() == pytest.approx(1 / 25 / 1e4) and s.current_step() == 100
    s = optim.ReduceLROnPlateau(0.1, optim.PlateauMode.Min, 0.5, 2, 0.01)
    s.step_with_metric(1.0), s.step_with_metric(1.0), s.step_with_metric(1.0)
    assert s.get_lr() == pytest.approx(0.05)
    s.step_with_metric(0.5)
    assert s.get_lr() == pytest.approx(0.05)
    opt = optim.SGD([torch.zeros(1, requires_grad=True)], optim.SGDConfig.new(1.0))
    sch = optim.StepLR(1.0, 1, 0.5).attach(opt)
    sch.step()
    assert opt.learning_rate() == 0.5


def test_amp_utilities():
    sc = optim.GradScaler.new()
    assert sc.get_scale() == 65536.0 and sc.is_enabled()
    assert sc.scale(Tensor.from_slice([2.0])).item() == 131072.0
    g = [Tensor.from_slice([65536.0, 131072.0])]
    assert sc.unscale_gradients(g) and g[0].to_vec() == [1.0, 2.0]
    sc.update(True)
    assert sc.get_scale() == 32768.0
    sc2 = optim.GradScaler(init_scale=4.0, growth_interval=2)
    sc2.update(False), sc2.update(False)
    assert sc2.get_scale() == 8.0
    bad = [Tensor.from_slice([1.0, float("inf")])]
    assert sc.step(bad) is False
    assert optim.has_inf_or_nan(Tensor.from_slice([1.0, float("nan")])) and not optim.has_inf_or_nan(Tensor.ones([2]))
    gs = [Tensor.from_slice([3.0, 4.0])]
    assert optim.clip_grad_norm(gs, 1.0) == pytest.approx(5.0)
    assert gs[0].to_vec() == pytest.approx([0.6, 0.8], rel=1e-5)
    gs = [Tensor.from_slice([-5.0, 0.5, 5.0])]
    optim.clip_grad_value(gs, 1.0)
    assert gs[0].to_vec() == [-1.0, 0.5, 1.0]
    assert optim.to_bfloat16(Tensor.ones([2])).dtype is fb.DType.BF16 and optim.to_half(Tensor.ones([2])).dtype is \
        fb.DType.F16
    assert optim.to_float(optim.to_bfloat16(Tensor.ones([2]))).dtype is fb.DType.F32
    ac = optim.Autocast.with_dtype(fb.DType.BF16)
    assert ac.is_enabled() and ac.cast(Tensor.ones([2])).dtype is fb.DType.BF16
    with ac:
        assert fb.config.low_precision_active()
    assert not fb.config.low_precision_active()


def test_xor_training_matches_the_cpu_restatement():
    """Config 1: Linear(2,8)-Tanh-Linear(8,1)-Sigmoid, bce, SGD lr 1.0, 2000 full-batch epochs, injected weights."""
    rs = np.random.RandomState(42)
    H = 8
    w1 = (rs.randn(2, H) * 0.5).astype("float32")
    b1 = np.zeros(H, dtype="float32")
    w2 = (rs.randn(H) * 0.5).astype("float32")
    b2 = np.zeros(1, dtype="float32")
    model = nn.Sequential(nn.Linear(2, H), nn.Tanh(), nn.Linear(H, 1), nn.Sigmoid())
    with torch.no_grad():
        model[0].weight.copy_(torch.from_numpy(w1.T.copy()))
        model[0].bias.zero_()
        model[2].weight.copy_(torch.from_numpy(w2.reshape(1, H).copy()))
        model[2].bias.zero_()
    x = Tensor.from_slice([[0.0, 0.0], [0.0, 1.0], [1.0, 0.0], [1.0, 1.0]])
    y = Tensor.from_slice([[0.0], [1.0], [1.0], [0.0]])
    opt = optim.SGD(model.parameters(), optim.SGDConfig.new(1.0))
    epochs = 2000
    mine = []
    for _ in range(epochs):
        opt.zero_grad()
        loss = nn.bce_loss(model(x), y)
        loss.backward()
        opt.step()
        mine.append(loss.item())
    ref = np.zeros(epochs, dtype="float32")
    _host().fb_ref_train_xor(w1.ctypes.data, b1.ctypes.data, w2.ctypes.data, b2.ctypes.data, H, 1.0, epochs, 1,
                             ref.ctypes.data)
    assert np.allclose(np.array(mine), ref, atol=1e-4)
    pred = model(x).to_vec()
    assert [round(v) for v in pred] == [0, 1, 1, 0]  # 4/4 accuracy
    assert mine[-1] < 0.01


def test_causal_attention_ignores_later_positions():
    """forward_attn(causal=True): the output at position t does not change when later positions change."""
    import torch

    import ferrum_b200 as fb

    torch.manual_seed(0)
    m = fb.nn.MultiHeadAttention(32, 2)
    x = torch.randn(2, 6, 32)
    x2 = x.clone()
    x2[:, 4:] += 1.0
    with fb.no_grad():
        y, y2 = m.forward_attn(x, x, x, causal=True), m.forward_attn(x2, x2, x2, causal=True)
        z, z2 = m.forward_attn(x, x, x), m.forward_attn(x2, x2, x2)
    y, y2, z, z2 = (t.torch() if hasattr(t, "torch") else t for t in (y, y2, z, z2))
    assert float((y[:, :4] - y2[:, :4]).abs().max()) == 0.0
    assert float((z[:, :4] - z2[:, :4]).abs().max()) > 0.0
