"""Core types on CPU: the assertions of the reference's unit tests (ferrum-core shape.rs:444-549,
tensor.rs:2662-2899, storage.rs) restated against this package."""
import math

import pytest
import torch

import ferrum_b200 as fb
from ferrum_b200 import DType, Device, Shape, Tensor


def test_dtype_table():
    assert [int(d) for d in (DType.F32, DType.F64, DType.F16, DType.BF16, DType.I32, DType.I64, DType.U8,
                             DType.Bool)] == list(range(8))
    assert DType.F32.size_of() == 4 and DType.BF16.size_of() == 2 and DType.I64.size_of() == 8
    assert DType.F32.supports_grad() and not DType.I32.supports_grad()
    assert DType.I32.is_integer() and DType.I32.is_signed() and not DType.U8.is_signed()
    assert DType.default_float() is DType.F32 and DType.default_int() is DType.I64
    assert str(DType.BF16) == "bf16" and DType.from_torch(torch.float64) is DType.F64


def test_device():
    assert Device.Cpu.is_cpu() and not Device.Cpu.is_gpu() and Device.Cpu.index() is None
    c = Device.Cuda(1)
    assert c.is_cuda() and c.is_gpu() and c.index() == 1 and str(c) == "cuda:1" and str(Device.Metal(1)) == "metal:1"
    assert Device.default() == Device.Cpu and Device.Cuda(0) == Device.Cuda(0) and Device.Cuda(0) != Device.Cuda(1)
    assert fb.cuda_is_available() == torch.cuda.is_available()


def test_shape_basics():
    s = Shape([2, 3, 4])
    assert s.ndim() == 3 and s.numel() == 24 and s.dims() == [2, 3, 4] and s.dim(-1) == 4 and s[0] == 2
    assert s.strides_contiguous() == [12, 4, 1] and s.is_contiguous([12, 4, 1]) and not s.is_contiguous([1, 2, 6])
    assert Shape.scalar().is_scalar() and Shape.scalar().numel() == 1
    assert str(Shape([2, 3])) == "[2, 3]" and s() is s and s == (2, 3, 4)
    with pytest.raises(fb.InvalidAxis):
        s.dim(3)


def test_shape_broadcast():
    assert Shape([3, 1]).broadcast([1, 4]) == (3, 4)
    assert Shape([5, 3, 1]).broadcast([3, 4]) == (5, 3, 4)
    assert Shape([]).broadcast([2, 2]) == (2, 2)
    with pytest.raises(fb.BroadcastError):
        Shape([3, 2]).broadcast([4, 2])
    assert Shape([3, 1]).broadcast_strides([1, 1], [2, 3, 4]) == [0, 1, 0]


def test_shape_transforms():
    s = Shape([2, 3, 4])
    assert s.transpose([2, 0, 1]) == (4, 2, 3)
    assert s.unsqueeze(0) == (1, 2, 3, 4) and s.unsqueeze(-1) == (2, 3, 4, 1)
    assert Shape([1, 3, 1]).squeeze() == (3,) and Shape([1, 3, 1]).squeeze(0) == (3, 1)
    assert s.can_reshape_to([6, 4]) and not s.can_reshape_to([5, 5])
    with pytest.raises(fb.InvalidShape):
        s.transpose([0, 0, 1])


def test_factories():
    assert Tensor.zeros([2, 3]).to_vec() == [0.0] * 6
    assert Tensor.ones([2]).to_vec() == [1.0, 1.0]
    assert Tensor.full([2], 3.5).to_vec() == [3.5, 3.5]
    assert Tensor.eye(2).to_vec() == [1, 0, 0, 1]
    assert Tensor.arange(0, 5).to_vec() == [0, 1, 2, 3, 4]
    assert Tensor.arange(5).shape == (5,)
    lin = Tensor.linspace(0, 1, 5).to_vec()
    assert lin[0] == 0 and lin[-1] == 1 and abs(lin[2] - 0.5) < 1e-6
    t = Tensor.from_slice([1.0, 2.0, 3.0, 4.0], [2, 2])
    assert t.shape == (2, 2) and t.dtype is DType.F32 and t.device == Device.Cpu
    with pytest.raises(fb.ShapeMismatch):
        Tensor.from_slice([1.0, 2.0, 3.0], [2, 2])
    r = Tensor.randn([1000])
    assert abs(sum(r.to_vec()) / 1000) < 0.2
    u = Tensor.uniform([1000], -1.0, 1.0).to_vec()
    assert min(u) >= -1.0 and max(u) <= 1.0
    n = Tensor.normal([2000], 3.0, 0.1).to_vec()
    assert abs(sum(n) / 2000 - 3.0) < 0.05


def test_properties_and_views_share_storage():
    t = Tensor.arange(0, 6).reshape([2, 3])
    assert t.ndim() == 2 and t.numel() == 6 and t.strides() == [3, 1] and t.size(1) == 3 and t.is_contiguous()
    r = t.reshape([3, 2])
    assert r.tensor_id == t.tensor_id
    r.torch()[0, 0] = 42.0
    assert t.to_vec()[0] == 42.0  # a view, not a copy
    tt = t.t()
    assert tt.shape == (3, 2) and not tt.is_contiguous() and tt.contiguous().to_vec() == [42, 3, 1, 4, 2, 5]
    assert t.transpose(0, 1).shape == (3, 2) and t.permute(1, 0).shape == (3, 2)
    assert t.unsqueeze(0).shape == (1, 2, 3) and t.unsqueeze(0).squeeze(0).shape == (2, 3)
    assert Tensor.ones([1, 3]).expand([4, 3]).shape == (4, 3)
    assert t.narrow(1, 1, 2).to_vec() == [3, 1, 4, 5] or t.narrow(1, 1, 2).shape == (2, 2)
    assert t.flatten().shape == (6,)
    with pytest.raises(fb.ReshapeError):
        t.reshape([4, 2])
    with pytest.raises(fb.IndexOutOfBounds):
        t.narrow(0, 1, 5)
    with pytest.raises(fb.InvalidShape):
        Tensor.ones([2, 2, 2]).t()


def test_item_convert_display():
    assert Tensor.from_slice([7.0]).item() == 7.0
    with pytest.raises(fb.InvalidShape):
        Tensor.ones([2]).item()
    assert Tensor.from_slice([1.5, 2.5]).to_dtype(DType.I32).to_vec() == [1, 2]
    assert Tensor.from_slice([1, 2], dtype=DType.I32).to_dtype(DType.F64).dtype is DType.F64
    s = repr(Tensor.from_slice([1.0, 2.0]))
    assert s == "Tensor(shape=[2], dtype=f32, data=[1.0000, 2.0000])"
    assert "..." in repr(Tensor.zeros([20]))
    with pytest.raises(fb.NotImplemented_):
        Tensor.ones([1]).to_device(Device.Metal(0))


def test_arithmetic_and_broadcast():
    a = Tensor.from_slice([1.0, 2.0, 3.0, 4.0], [2, 2])
    b = Tensor.from_slice([10.0, 20.0], [2])
    assert a.add(b).to_vec() == [11, 22, 13, 24]
    assert (a - b).to_vec() == [-9, -18, -7, -16] and (a * 2).to_vec() == [2, 4, 6, 8] and (a / 2).to_vec() == [
        0.5, 1, 1.5, 2]
    assert (1 - a).to_vec() == [0, -1, -2, -3] and (-a).to_vec() == [-1, -2, -3, -4]
    assert a.add_scalar(1).to_vec() == [2, 3, 4, 5] and a.mul_scalar(0.5).to_vec() == [0.5, 1, 1.5, 2]
    with pytest.raises(fb.BroadcastError):
        a.add(Tensor.ones([3]))
    assert a.pow(2).to_vec() == [1, 4, 9, 16]
    assert abs(a.sqrt().to_vec()[3] - 2) < 1e-6 and abs(a.exp().log().to_vec()[2] - 3) < 1e-5
    x = Tensor.from_slice([-1.0, 0.0, 2.0])
    assert x.relu().to_vec() == [0, 0, 2]
    assert abs(x.sigmoid().to_vec()[1] - 0.5) < 1e-7 and abs(x.tanh().to_vec()[1]) < 1e-7
    assert a.sub_inplace(Tensor.ones([2, 2])).to_vec() == [0, 1, 2, 3]
    with pytest.raises(fb.ShapeMismatch):
        a.add_inplace(Tensor.ones([2]))


def test_reductions():
    t = Tensor.from_slice([1.0, 2.0, 3.0, 4.0, 5.0, 6.0], [2, 3])
    assert t.sum().item() == 21 and t.mean().item() == 3.5
    assert t.sum_dim(0).to_vec() == [5, 7, 9] and t.sum_dim(1).to_vec() == [6, 15]
    assert t.mean_dim(1).to_vec() == [2, 5] and t.sum_dim(1, keepdim=True).shape == (2, 1)
    assert t.max_dim(1).to_vec() == [3, 6] and t.min_dim(0).to_vec() == [1, 2, 3]
    assert t.argmax(1).to_vec() == [2, 2] and t.argmin(1).to_vec() == [0, 0] and t.argmax().item() == 5
    assert t.max().item() == 6 and t.min().item() == 1
    with pytest.raises(fb.InvalidAxis):
        t.sum_dim(2)


def test_matmul_forms():
    a = Tensor.ones([2, 3])
    b = Tensor.ones([3, 4])
    assert a.matmul(b).to_vec() == [3.0] * 8 and (a @ b).shape == (2, 4)
    assert a.matmul(Tensor.ones([3])).to_vec() == [3, 3]
    assert Tensor.ones([3]).matmul(b).to_vec() == [3, 3, 3, 3]
    assert Tensor.ones([5, 2, 3]).matmul(Tensor.ones([5, 3, 4])).shape == (5, 2, 4)
    with pytest.raises(fb.ShapeMismatch):
        a.matmul(Tensor.ones([4, 2]))


def test_cat_stack():
    a, b = Tensor.ones([2, 3]), Tensor.zeros([2, 3])
    assert Tensor.cat([a, b], 0).shape == (4, 3) and Tensor.cat([a, b], 1).shape == (2, 6)
    assert Tensor.stack([a, b], 0).shape == (2, 2, 3)
    with pytest.raises(fb.InvalidShape):
        Tensor.cat([])


def test_grad_api():
    t = Tensor.ones([2]).set_requires_grad(True)
    assert t.requires_grad() and t.grad() is None
    with pytest.raises(fb.UnsupportedDType):
        Tensor.ones([2], DType.I32).set_requires_grad(True)
    t.accumulate_grad(Tensor.full([2], 2.0))
    t.accumulate_grad(Tensor.full([2], 3.0))
    assert t.grad().to_vec() == [5, 5]
    t.zero_grad()
    assert t.grad() is None
    assert not t.detach().requires_grad()
    with pytest.raises(fb.AutogradError):
        Tensor.ones([2]).set_requires_grad(True).mul_scalar(2).backward()


def test_error_messages():
    assert str(fb.ShapeMismatch("matmul", "[2, 3]", "[4]")) == "Shape mismatch: matmul expects [2, 3], got [4]"
    assert str(fb.InvalidAxis(3, 2)) == "Invalid axis 3 for tensor with 2 dimensions"
    assert str(fb.NotImplemented_("x")) == "Not implemented: x"
    assert issubclass(fb.ReshapeError, fb.FerrumError)
    assert "Blackwell" in fb.banner()


def test_gpu_tensor_vocabulary_of_the_reference():
    """ptr / size_bytes / to_host / to_f32 / to_f64 / sum_axis / mean_axis (ferrum-cuda/src/tensor.rs:120-159,
    266-279) exist on the one tensor class and agree with the plain accessors."""
    import struct

    t = Tensor.from_slice([1.0, 2.0, 3.0, 4.0, 5.0, 6.0], [2, 3])
    assert t.ptr() != 0 and t.size_bytes() == 24
    assert struct.unpack("<6f", t.to_host()) == (1.0, 2.0, 3.0, 4.0, 5.0, 6.0)
    assert t.to_f32() == [1.0, 2.0, 3.0, 4.0, 5.0, 6.0] and t.to_f64() == t.to_f32()
    assert t.transpose(0, 1).to_host() == Tensor.from_slice([1.0, 4.0, 2.0, 5.0, 3.0, 6.0], [3, 2]).to_host()
    assert t.sum_axis(0).to_vec() == [5.0, 7.0, 9.0] and t.sum_axis(1).to_vec() == [6.0, 15.0]
    assert t.mean_axis(1).to_vec() == [2.0, 5.0] and t.mean_axis(-2).shape == (3,)
