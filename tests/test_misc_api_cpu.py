"""Storage / allocators, the named backward formulas (ferrum-autograd/tests/integration_test.rs calls them
directly), the functional op namespace, the prelude, secondary layers, profiler plumbing."""
import pytest
import torch

import ferrum_b200 as fb
from ferrum_b200 import DType, Storage, Tensor, nn, ops
from ferrum_b200 import autograd_functions as AF


def test_storage_sharing_and_copy_on_write():
    s = Storage.zeros(16)
    assert s.size() == 16 and s.read_as(DType.F32) == [0.0] * 4 and s.device() == fb.Device.Cpu
    s = Storage.from_slice([1.0, 2.0, 3.0])
    assert s.is_unique() and s.ref_count() == 1
    s2 = s.share()
    assert not s.is_unique() and s2.ref_count() == 2 and s2.as_ptr() == s.as_ptr()
    s2.make_unique()
    s2.write_as([9.0], DType.F32)
    assert s.read_as(DType.F32) == [1.0, 2.0, 3.0] and s2.read_as(DType.F32) == [9.0, 2.0, 3.0]
    assert s.is_unique() and Storage.uninit(0).size() == 0
    assert Storage.from_bytes(b"\x00\x00\x80\x3f").read_as(DType.F32) == [1.0]
    assert s.as_tensor(DType.F32, [3]).to_vec() == [1.0, 2.0, 3.0]
    buf = fb.CpuAllocator().alloc(100)
    assert buf.data_ptr() % 64 == 0 and buf.numel() == 100


def test_named_backward_functions():
    a, b = Tensor.from_slice([1.0, 2.0, 3.0]), Tensor.from_slice([4.0, 5.0, 6.0])
    g = Tensor.ones([3])
    assert [t.to_vec() for t in AF.AddBackward(a, b).backward(g)] == [[1, 1, 1], [1, 1, 1]]
    assert AF.SubBackward(a, b).backward(g)[1].to_vec() == [-1, -1, -1]
    assert [t.to_vec() for t in AF.MulBackward(a, b).backward(g)] == [[4, 5, 6], [1, 2, 3]]
    ga, gb = AF.DivBackward(Tensor.from_slice([2.0, 4.0]), Tensor.from_slice([1.0, 2.0])).backward(Tensor.ones([2]))
    assert ga.to_vec() == [1, 0.5] and gb.to_vec() == [-2, -1]
    ga, gb = AF.MatMulBackward(Tensor.from_slice([[1.0, 2.0], [3.0, 4.0]]),
                               Tensor.from_slice([[5.0, 6.0], [7.0, 8.0]])).backward(Tensor.ones([2, 2]))
    assert ga.to_vec() == [11, 15, 11, 15] and gb.to_vec() == [4, 4, 6, 6]
    assert AF.ReLUBackward(Tensor.from_slice([-1.0, 2.0])).backward(Tensor.ones([2]))[0].to_vec() == [0, 1]
    assert AF.SigmoidBackward(Tensor.from_slice([0.5])).backward(Tensor.ones([1]))[0].item() == 0.25
    assert AF.TanhBackward(Tensor.from_slice([0.0])).backward(Tensor.ones([1]))[0].item() == 1.0
    assert AF.ExpBackward(Tensor.from_slice([2.0])).backward(Tensor.from_slice([3.0]))[0].item() == 6.0
    assert AF.LogBackward(Tensor.from_slice([4.0])).backward(Tensor.ones([1]))[0].item() == 0.25
    assert AF.PowBackward(Tensor.from_slice([3.0]), 2.0).backward(Tensor.ones([1]))[0].item() == 6.0
    assert AF.SqrtBackward(Tensor.from_slice([2.0])).backward(Tensor.ones([1]))[0].item() == 0.25
    assert AF.NegBackward().backward(Tensor.ones([2]))[0].to_vec() == [-1, -1]
    assert AF.SumBackward([2, 2]).backward(Tensor.from_slice(2.0))[0].to_vec() == [2, 2, 2, 2]
    assert AF.MeanBackward([2, 2]).backward(Tensor.from_slice(1.0))[0].to_vec() == [0.25] * 4
    assert AF.SumDimBackward([2, 3], 0).backward(Tensor.ones([3]))[0].shape == (2, 3)
    parts = AF.CatBackward([2, 1], 0).backward(Tensor.from_slice([1.0, 2.0, 3.0]))
    assert parts[0].to_vec() == [1, 2] and parts[1].to_vec() == [3]
    assert AF.AddBackward(Tensor.ones([2, 3]), Tensor.ones([3])).backward(Tensor.ones([2, 3]))[1].to_vec() == [2, 2, 2]
    assert AF.MulBackward(a, b).name() == "MulBackward"
    assert AF.reduce_gradient(Tensor.ones([4, 3]), [1, 3]).to_vec() == [4, 4, 4]


def test_ops_namespace_and_prelude():
    a, b = Tensor.from_slice([[1.0, 2.0], [3.0, 4.0]]), Tensor.ones([2, 2])
    assert ops.add(a, b).to_vec() == [2, 3, 4, 5] and ops.matmul(a, b).to_vec() == [3, 3, 7, 7]
    assert ops.matmul_tiled(a, b).to_vec() == ops.matmul_blas(a, b).to_vec() == ops.matmul_parallel(a, b).to_vec()
    assert ops.sum_dim(a, 0).to_vec() == [4, 6] and ops.argmax(a, 1).to_vec() == [1, 1]
    assert ops.bmm(Tensor.ones([2, 2, 3]), Tensor.ones([2, 3, 2])).shape == (2, 2, 2)
    assert ops.stack([a, b]).shape == (2, 2, 2) and ops.neg(a).to_vec()[0] == -1
    ns = {}
    exec("from ferrum_b200.prelude import *", ns)
    for name in ("Tensor", "DType", "Device", "Linear", "Sequential", "GELU", "LayerNorm", "Adam", "AdamConfig",
                 "SGD", "StepLR", "OneCycleLR", "DataLoader", "DistributedSampler", "save", "load", "GradientTape",
                 "no_grad", "DistributedDataParallel", "ReduceOp", "mse_loss", "nll_loss", "init_process_group"):
        assert name in ns, name
    # the whole public checklist of the reference's facade: prelude names and the per-crate extras
    import ferrum_b200 as fb

    prelude_names = ("DType Device FerrumError Shape Tensor backward GradientTape AutogradTensor NoGradGuard no_grad "
                     "Linear Module ReLU Sequential Sigmoid Tanh GELU SiLU Softmax LogSoftmax LeakyReLU ELU LayerNorm "
                     "BatchNorm1d Dropout Embedding bce_loss cross_entropy_loss l1_loss log_softmax mse_loss nll_loss "
                     "smooth_l1_loss softmax Adam AdamConfig Optimizer SGDConfig SGD LRScheduler StepLR MultiStepLR "
                     "ExponentialLR CosineAnnealingLR CosineAnnealingWarmRestarts LinearWarmupLR OneCycleLR "
                     "ReduceLROnPlateau PlateauMode load save DataLoader Dataset TensorDataset Subset train_test_split "
                     "RandomSampler SequentialSampler DistributedSampler init_process_group get_rank get_world_size "
                     "is_main_process barrier Backend ProcessGroup DistributedDataParallel ReduceOp").split()
    assert [n for n in prelude_names if n not in ns] == []
    extras = {"nn": "Conv2d LSTM MultiHeadAttention ResNet MLP VGG BasicBlock init",
              "optim": "GradScaler Autocast clip_grad_norm",
              "data": "BatchSampler WeightedRandomSampler SubsetRandomSampler MapDataset ConcatDataset Compose Normalize",
              "distributed": "init_process_group_from_env destroy_process_group get_world is_initialized BackendConfig "
                             "new_group GradientBucket"}
    for mod, names in extras.items():
        assert [n for n in names.split() if not hasattr(getattr(fb, mod), n)] == [], mod
    assert callable(fb.banner) and hasattr(fb, "cuda")
    assert fb.nn.MLP.new([4, 8, 2])(Tensor.ones([3, 4])).shape == (3, 2)


def test_conv_pool_rnn_transformer_shapes_and_values():
    x = Tensor.randn([2, 3, 8, 8])
    c = nn.Conv2d.new(3, 4, 3).padding(1)
    assert torch.allclose(c(x).torch(), torch.nn.functional.conv2d(x.torch(), c.weight, c.bias, padding=1), atol=1e-5)
    assert nn.MaxPool2d.new(2)(x).shape == (2, 3, 4, 4) and nn.AvgPool2d.new(2)(x).shape == (2, 3, 4, 4)
    assert nn.AdaptiveAvgPool2d.square(1)(x).shape == (2, 3, 1, 1)
    assert nn.Conv1d.new(3, 5, 3)(Tensor.randn([2, 3, 10])).shape == (2, 5, 8)
    out, h = nn.RNN.new(4, 6, 2).forward_seq(Tensor.randn([5, 3, 4]))
    assert out.shape == (5, 3, 6) and h.shape == (2, 3, 6)
    out, (h, cc) = nn.LSTM.new(4, 6, 1).forward_seq(Tensor.randn([5, 3, 4]))
    assert out.shape == (5, 3, 6) and cc.shape == (1, 3, 6)
    assert nn.GRUCell.new(4, 6)(Tensor.randn([3, 4]), Tensor.zeros([3, 6])).shape == (3, 6)
    loss = nn.GRU.new(4, 6, 1)(Tensor.randn([5, 3, 4])).sum()
    loss.backward()  # recurrent layers are differentiable (host-only math without autograd in the reference)
    xs = Tensor.randn([2, 5, 16])
    assert nn.MultiHeadAttention.new(16, 4)(xs).shape == (2, 5, 16)
    assert nn.TransformerEncoderLayer.new(16, 4, 32)(xs).shape == (2, 5, 16)
    pe = nn.PositionalEncoding.new(16, 10)
    assert torch.allclose(pe(Tensor.zeros([1, 3, 16])).torch()[0, 0, 1::2], torch.ones(8))
    from ferrum_b200.models import MLP, BasicBlock

    assert MLP.new([4, 8, 2])(Tensor.randn([3, 4])).shape == (3, 2) and len(MLP([4, 8, 8, 2])) == 5
    assert BasicBlock.new(4, 8, 2)(Tensor.randn([1, 4, 8, 8])).shape == (1, 8, 4, 4)


def test_step_timer_and_peaks_file():
    from ferrum_b200.utils import StepTimer
    from ferrum_b200.utils.profiler import measured_peaks

    lines = []
    t = StepTimer(every=2, flops_per_sample=1e6, sink=lines.append)
    for _ in range(4):
        with t.step(8):
            pass
    assert len(lines) == 2 and "samples_per_s" in lines[0] and len(t.history) == 2
    pk = measured_peaks()
    assert pk is None or "hbm_gbs" in pk


def test_core_autograd_hook_names():
    from ferrum_b200 import autograd as ag

    a, b = ag.new_tensor_id(), ag.new_tensor_id()
    assert b == a + 1
    n1, n2 = ag.NodeId.new(), ag.NodeId.new()
    assert n2 == n1 + 1 and isinstance(n1, int)
    seen = []
    ag.register_autograd_callbacks(lambda *a, **k: seen.append(("rec", a)), lambda out: seen.append(("bwd", out)))
    ag.record_operation("add", 1, 2)
    ag.execute_backward("loss")
    with ag.no_grad():
        ag.record_operation("skipped")
    ag.unregister_autograd_callbacks()
    ag.record_operation("ignored")
    assert seen == [("rec", ("add", 1, 2)), ("bwd", "loss")]
    assert ag.is_autograd_enabled()
    ag.set_autograd_enabled(False)
    assert not ag.is_autograd_enabled()
    ag.set_autograd_enabled(True)


def test_new_switches_are_inert_without_a_gpu():
    """Options added for the GPU paths must not disturb CPU use: the blockwise attention is not selected for CPU
    tensors, the engine's push mode and guard bands stay off."""
    import torch

    import ferrum_b200 as fb
    from ferrum_b200.ops import functional as F
    from ferrum_b200.parallel import Backend, DistributedDataParallel, ProcessGroup

    q = torch.randn(1, 2, 16, 64)
    assert not F.flash_attention_ok(q, q, q)
    model = fb.nn.Sequential(fb.nn.Linear(4, 3))
    ddp = DistributedDataParallel(model, ProcessGroup(Backend.Gloo, 0, 1))
    assert ddp.push_gradients(True) is ddp
    assert ddp.check_guard_bands() == 0
    mha = fb.nn.MultiHeadAttention(128, 2, memory_efficient=True)
    y = mha(torch.randn(2, 5, 128))
    assert tuple(y.shape) == (2, 5, 128)


def test_space_to_depth_filters_reproduce_a_strided_convolution():
    """The host-side half of the strided implicit-GEMM convolution, on the CPU: with the input rearranged as
    z[b, I, J, (rh, rw, c)] = x_padded[b, c, I * sh + rh, J * sw + rw] and the filters rearranged by
    ``_ConvS2dFn._filters``, a stride-1 convolution of z equals the strided convolution of x; the weight-gradient
    mapping back is the exact inverse."""
    import torch.nn.functional as TF

    from ferrum_b200.ops.functional import _ConvS2dFn, conv_igemm_ok

    torch.manual_seed(0)
    for (B, C, O, H, W, k, s, p) in [(2, 3, 5, 17, 19, (3, 3), (2, 2), (1, 1)), (1, 4, 6, 16, 16, (4, 4), (4, 4), (0, 0)),
                                     (2, 5, 7, 15, 20, (5, 3), (2, 3), (2, 1)), (1, 3, 4, 14, 14, (7, 7), (2, 2), (3, 3))]:
        x, w = torch.randn(B, C, H, W), torch.randn(O, C, *k)
        (sh, sw), (ph, pw) = s, p
        Ho, Wo, k2h, k2w, Hz, Wz, Cz = _ConvS2dFn._geometry(x.shape, w.shape, s, p)
        assert (Ho, Wo) == tuple(TF.conv2d(x, w, None, s, p).shape[2:]) and Cz % 8 == 0 and Cz >= sh * sw * C
        xp = TF.pad(x, (pw, Wz * sw, ph, Hz * sh))[:, :, :Hz * sh, :Wz * sw]       # zero outside the image
        z = xp.reshape(B, C, Hz, sh, Wz, sw).permute(0, 2, 4, 3, 5, 1).reshape(B, Hz, Wz, sh * sw * C)
        w2 = _ConvS2dFn._filters(w, s, k2h, k2w, Cz)
        assert w2.shape == (O, k2h, k2w, Cz) and not w2[..., sh * sw * C:].any()
        y = TF.conv2d(z.permute(0, 3, 1, 2), w2[..., :sh * sw * C].permute(0, 3, 1, 2))
        assert torch.allclose(y, TF.conv2d(x, w, None, s, p), atol=1e-4)
        back = w2[..., :sh * sw * C].reshape(O, k2h, k2w, sh, sw, C).permute(0, 5, 1, 3, 2, 4)
        assert torch.equal(back.reshape(O, C, k2h * sh, k2w * sw)[:, :, :k[0], :k[1]], w)
        assert not conv_igemm_ok(x, s, (1, 1), p, k, 1)      # host tensors never take the tensor-core path
