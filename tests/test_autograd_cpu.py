"""Backward formulas with closed-form expectations (the reference calls each *Backward struct directly:
ferrum-autograd/tests/integration_test.rs:6-279), tape plumbing and finite differences."""
import math

import pytest
import torch

import ferrum_b200 as fb
from ferrum_b200 import GradientTape, Tensor, autograd


def _leaf(vals, shape=None):
    return Tensor.from_slice(vals, shape).set_requires_grad(True)


def test_add_sub_mul_div_backward():
    a, b = _leaf([1.0, 2.0, 3.0]), _leaf([4.0, 5.0, 6.0])
    a.add(b).sum().backward()
    assert a.grad().to_vec() == [1, 1, 1] and b.grad().to_vec() == [1, 1, 1]
    a, b = _leaf([1.0, 2.0, 3.0]), _leaf([4.0, 5.0, 6.0])
    a.sub(b).sum().backward()
    assert b.grad().to_vec() == [-1, -1, -1]
    a, b = _leaf([1.0, 2.0, 3.0]), _leaf([4.0, 5.0, 6.0])
    a.mul(b).sum().backward()
    assert a.grad().to_vec() == [4, 5, 6] and b.grad().to_vec() == [1, 2, 3]
    a, b = _leaf([2.0, 4.0]), _leaf([1.0, 2.0])
    a.div(b).sum().backward()
    assert a.grad().to_vec() == [1, 0.5] and b.grad().to_vec() == [-2, -1]


def test_broadcast_gradient_reduces_to_operand_shape():
    a, b = _leaf([1.0] * 6, [2, 3]), _leaf([1.0, 2.0, 3.0])
    a.mul(b).sum().backward()
    assert b.grad().shape == (3,) and b.grad().to_vec() == [2, 2, 2]


def test_matmul_backward():
    a, b = _leaf([1.0, 2.0, 3.0, 4.0], [2, 2]), _leaf([5.0, 6.0, 7.0, 8.0], [2, 2])
    a.matmul(b).sum().backward()
    assert a.grad().to_vec() == [11, 15, 11, 15] and b.grad().to_vec() == [4, 4, 6, 6]


def test_unary_backward():
    x = _leaf([-1.0, 2.0])
    x.relu().sum().backward()
    assert x.grad().to_vec() == [0, 1]
    x = _leaf([0.0])
    x.sigmoid().sum().backward()
    assert abs(x.grad().item() - 0.25) < 1e-7
    x = _leaf([0.0])
    x.tanh().sum().backward()
    assert abs(x.grad().item() - 1.0) < 1e-7
    x = _leaf([1.0, 2.0])
    x.exp().sum().backward()
    assert abs(x.grad().to_vec()[1] - math.e ** 2) < 1e-4
    x = _leaf([2.0, 4.0])
    x.log().sum().backward()
    assert x.grad().to_vec() == [0.5, 0.25]
    x = _leaf([3.0])
    x.pow(2).sum().backward()
    assert x.grad().item() == 6
    x = _leaf([4.0])
    x.sqrt().sum().backward()
    assert x.grad().item() == 0.25
    x = _leaf([1.0, -2.0])
    x.neg().sum().backward()
    assert x.grad().to_vec() == [-1, -1]


def test_sum_mean_backward_reach_leaves():
    x = _leaf([1.0, 2.0, 3.0, 4.0])
    x.sum().backward()
    assert x.grad().to_vec() == [1, 1, 1, 1]  # the reference leaves this None (empty saved_tensors)
    x = _leaf([1.0, 2.0, 3.0, 4.0])
    x.mean().backward()
    assert x.grad().to_vec() == [0.25] * 4
    x = _leaf([1.0, 2.0, 3.0, 4.0], [2, 2])
    x.sum_dim(0).sum().backward()
    assert x.grad().to_vec() == [1, 1, 1, 1]


def test_scalar_ops_are_differentiable():
    x = _leaf([1.0, 2.0])
    x.add_scalar(3).mul_scalar(2).sum().backward()
    assert x.grad().to_vec() == [2, 2]


def test_cat_backward():
    a, b = _leaf([1.0, 2.0]), _leaf([3.0])
    Tensor.cat([a, b], 0).mul(Tensor.from_slice([1.0, 2.0, 3.0])).sum().backward()
    assert a.grad().to_vec() == [1, 2] and b.grad().to_vec() == [3]


def test_tape_plumbing():
    tape = GradientTape.new()
    assert tape.is_recording() and tape.is_empty()
    tape.stop()
    assert not tape.is_recording() and not autograd.is_grad_enabled()
    tape.start()
    assert autograd.is_grad_enabled()
    assert GradientTape.current() is None

    def body(t):
        assert GradientTape.current() is t
        x = _leaf([2.0])
        y = x.mul(x)
        t.record(y)
        assert t.len() >= 1
        return t.gradient(y.sum(), [x])[0].item()

    assert GradientTape.with_tape(body) == 4.0
    assert GradientTape.current() is None
    with autograd.no_grad():
        assert not autograd.is_grad_enabled()
    assert autograd.no_grad(lambda: autograd.is_grad_enabled()) is False
    g = autograd.NoGradGuard()
    assert not autograd.is_grad_enabled()
    g.release()
    assert autograd.is_grad_enabled()


def test_backward_function_and_graph():
    x = _leaf([1.0, 2.0])
    y = x.mul(x).sum()
    graph = autograd.ComputationGraph(y)
    assert graph.len() >= 2 and not graph.is_empty()
    autograd.backward(y, graph)
    assert x.grad().to_vec() == [2, 4]
    with pytest.raises(fb.AutogradError):
        autograd.backward(x.mul(x))


def test_finite_differences():
    chk = autograd.GradChecker()
    x = Tensor.from_slice([0.5, -1.5, 2.0])
    assert chk.check(lambda t: t.mul(t), x)
    assert chk.check(lambda t: t.exp(), x)
    assert autograd.quick_gradcheck(lambda t: t.mul_scalar(2.0), x)
    assert autograd.check_gradients(lambda t: t.tanh().mul(t.sigmoid()), [x])


def test_every_layer_gradchecks_in_fp64():
    import ferrum_b200.ops.functional as F

    x = torch.randn(4, 6, dtype=torch.float64, requires_grad=True)
    g = torch.rand(6, dtype=torch.float64, requires_grad=True)
    b = torch.randn(6, dtype=torch.float64, requires_grad=True)
    assert torch.autograd.gradcheck(lambda x, g, b: F.layer_norm(x, g, b, 1e-5, "gelu"), (x, g, b))
    assert torch.autograd.gradcheck(lambda x: F.softmax(x, -1), (x,))
    assert torch.autograd.gradcheck(lambda x: F.log_softmax(x, 0), (x,))
    for op in ("gelu", "silu", "elu", "leaky_relu"):
        assert torch.autograd.gradcheck(lambda x: F.unary(x, op, 0.3), (x,))
    p = torch.rand(5, 3, dtype=torch.float64, requires_grad=True)
    t = (torch.rand(5, 3, dtype=torch.float64) > 0.5).double()
    for kind in ("mse", "bce", "smooth_l1"):
        assert torch.autograd.gradcheck(lambda p: F.elementwise_loss(p * 0.8 + 0.1, t, kind), (p,))
