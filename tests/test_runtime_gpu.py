"""CUDA runtime surface (ferrum-cuda tests run on host memory under `simulate`; these run on the device):
device properties, memory pool, buffers, streams / events, the eight kernel entry points, Tensor on Device.Cuda."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_device_properties_are_real():
    from ferrum_b200 import cuda

    assert cuda.cuda_available() and cuda.device_count() >= 1 and cuda.init_cuda() >= 1
    p = cuda.get_device_properties(0)
    assert "B200" in p.name or p.compute_capability_major >= 9
    assert p.multiprocessor_count > 68 and p.total_memory > 10 * 2 ** 30  # not the reference's fake RTX-3080
    assert p.warp_size == 32 and p.max_threads_per_block == 1024 and p.shared_memory_per_block_optin >= 200 * 1024
    d = cuda.CudaDevice.new(0)
    assert d.id() == 0 and d.name() == p.name and 0 < d.free_memory() <= d.total_memory()
    d.set_current()
    d.synchronize()
    m = cuda.CudaDeviceManager.initialize()
    assert m.device_count() == cuda.device_count() and m.current_device() == 0 and m.get_device(0).id() == 0
    with pytest.raises(cuda.CudaError):
        cuda.CudaDevice(99)


def test_memory_pool_buckets_and_buffers():
    from ferrum_b200 import cuda

    pool = cuda.MemoryPool()
    assert pool.round_size(1) == 256 and pool.round_size(257) == 512 and pool.round_size(3 << 20) == 4 << 20
    base = pool.allocated_bytes()
    b = pool.alloc(1000)
    assert b.size() == 1000 and b.ptr() != 0 and pool.allocated_bytes() - base == 1024
    ptr = b.ptr()
    pool.free(b)
    assert pool.cached_bytes() >= 1024
    b2 = pool.alloc(900)
    assert b2.ptr() == ptr  # served from the 1 KiB bucket
    payload = bytes(range(200)) * 4
    b2.copy_from_host(payload)
    assert b2.copy_to_host()[:800] == payload
    c = b2.clone()
    assert c.ptr() != b2.ptr() and c.copy_to_host()[:800] == payload
    c.zero()
    cuda.synchronize()
    assert c.copy_to_host()[:8] == b"\0" * 8
    b2.free(), c.free()
    pool.clear()
    assert pool.cached_bytes() == 0


def test_streams_and_events():
    from ferrum_b200 import cuda

    s = cuda.CudaStream.new()
    e0, e1 = cuda.CudaEvent.with_timing(), cuda.CudaEvent.with_timing()
    e0.record(s)
    with torch.cuda.stream(s.as_torch()):
        x = torch.randn(4096, 4096, device="cuda")
        y = x @ x
    e1.record(s)
    s.synchronize()
    assert s.query() and e1.query()
    assert e0.elapsed_time(e1) > 0.0  # the reference's simulated events return 0.0
    other = cuda.CudaStream.new()
    other.wait_event(s.record_event())
    other.synchronize()
    pool = cuda.StreamPool()
    a = pool.get()
    pool.put(a)
    assert pool.get() is a and cuda.CudaStream.default_stream().handle() == 0
    assert float(y[0, 0]) == float(y[0, 0])


def test_kernel_entry_points():
    import ferrum_b200 as fb
    from ferrum_b200 import kernels as K

    dev = fb.Device.Cuda(0)
    a = fb.Tensor.from_slice([[1.0, 2.0], [3.0, 4.0]], device=dev)
    b = fb.Tensor.from_slice([10.0, 20.0], device=dev)
    assert K.binary_op(a, b, K.BinaryOp.Add).cpu().to_vec() == [11, 22, 13, 24]  # real broadcasting
    assert K.binary_op(a, a, K.BinaryOp.Max).cpu().to_vec() == [1, 2, 3, 4]
    assert K.unary_op(fb.Tensor.from_slice([-1.0, 2.0], device=dev), K.UnaryOp.Relu).cpu().to_vec() == [0, 2]
    assert K.unary_op(fb.Tensor.from_slice([-1.0], device=dev), K.UnaryOp.LeakyRelu).cpu().to_vec() == pytest.approx(
        [-0.01])
    assert K.scalar_op(a, 2.0, K.ScalarOp.Mul).cpu().to_vec() == [2, 4, 6, 8]
    assert K.scalar_op(a, 1.0, K.ScalarOp.Sub).cpu().to_vec() == [0, 1, 2, 3]
    assert K.reduce_op(a, K.ReduceKind.Sum).cpu().item() == 10
    assert K.reduce_op(a, K.ReduceKind.Max, axis=0).cpu().to_vec() == [3, 4]
    assert K.reduce_op(a, K.ReduceKind.Mean, axis=1).cpu().to_vec() == [1.5, 3.5]
    assert K.matmul(a, a).cpu().to_vec() == [7, 10, 15, 22]
    assert K.transpose(a).cpu().to_vec() == [1, 3, 2, 4]
    sm = K.softmax(a).cpu()
    assert sm.sum_dim(1).to_vec() == pytest.approx([1, 1])
    assert K.log_softmax(a).exp().cpu().to_vec() == pytest.approx(sm.to_vec(), abs=1e-6)
    big_a = fb.Tensor.randn([256, 128], device=dev).to_dtype(fb.DType.BF16)
    big_b = fb.Tensor.randn([128, 64], device=dev).to_dtype(fb.DType.BF16)
    ref = big_a.torch().float() @ big_b.torch().float()
    assert (K.matmul(big_a, big_b).torch().float() - ref).abs().max().item() < 0.5  # tcgen05 path


def test_tensor_lives_on_cuda_and_trains():
    import ferrum_b200 as fb
    from ferrum_b200.cuda import CudaTensor

    t = CudaTensor.from_host([1.0, 2.0, 3.0, 4.0], [2, 2])
    assert t.device == fb.Device.Cuda(0) and t.device.is_cuda()
    assert t.add(t).sum().item() == 20 and t.matmul(t).cpu().to_vec() == [7, 10, 15, 22]
    assert t.to_device(fb.Device.Cpu).device.is_cpu() and t.cpu().cuda().to_vec() == [1, 2, 3, 4]
    w = fb.Tensor.randn([4, 3], device=fb.Device.Cuda(0)).set_requires_grad(True)
    x = fb.Tensor.randn([5, 4], device=fb.Device.Cuda(0))
    loss = x.matmul(w).tanh().pow(2).mean()
    loss.backward()
    g = w.grad().torch()
    xr, wr = x.torch().cpu().double(), w.torch().detach().cpu().double().requires_grad_(True)
    (xr @ wr).tanh().pow(2).mean().backward()
    assert torch.allclose(g.cpu().double(), wr.grad, atol=1e-5)
    with fb.no_grad():
        assert not x.matmul(w).requires_grad()


def test_profiler_collects_kernel_timings():
    import ferrum_b200 as fb
    from ferrum_b200.utils import profile

    x = fb.Tensor.randn([512, 512], device=fb.Device.Cuda(0))
    with profile() as prof:
        y = x.relu().add(x).sum_dim(0)
    rep = prof.report()
    assert "fb_unary_fwd" in rep and "fb_binary_fwd" in rep and "fb_reduce" in rep
    assert all(v["total_ms"] >= 0 and v["calls"] >= 1 for v in rep.values())
    assert "fb_unary_fwd" in prof.table()
    assert y.shape == (512,)


def test_device_prefetcher_delivers_batches_in_order():
    import ferrum_b200 as fb

    host = [(torch.full((1024, 64), float(i)).pin_memory(), torch.tensor([i])) for i in range(5)]
    seen = []
    for x, y in fb.data.DevicePrefetcher(iter(host), device=fb.Device.Cuda(0)):
        assert x.is_cuda and y.is_cuda
        seen.append((float(x.mean()), int(y)))
    assert seen == [(float(i), i) for i in range(5)]
    wrapped = [fb.Tensor(torch.ones(4) * i) for i in range(3)]
    out = [t.to_vec()[0] for t in fb.data.DevicePrefetcher(iter(wrapped), device=fb.Device.Cuda(0))]
    assert out == [0.0, 1.0, 2.0]


@pytest.mark.parametrize("which", ["adam", "sgd"])
def test_graphed_step_matches_eager_training(which):
    """A step recorded in a CUDA graph (capturable optimizer: device-side lr and bias corrections) follows the
    eager trajectory, including a learning-rate change between replays."""
    import copy

    import ferrum_b200 as fb
    from ferrum_b200 import nn, optim

    torch.manual_seed(0)
    dev = fb.Device.Cuda(0)
    ref = nn.Sequential(nn.Linear(32, 64, device=dev), nn.ReLU(), nn.LayerNorm([64], device=dev),
                        nn.Linear(64, 10, device=dev), nn.LogSoftmax(-1))
    cap = copy.deepcopy(ref)

    def make(ps):
        if which == "adam":
            return optim.Adam(ps, optim.AdamConfig(lr=1e-2))
        return optim.SGD(ps, optim.SGDConfig(lr=0.05, momentum=0.9))

    opt_ref, opt_cap = make(ref.parameters()), make(cap.parameters())
    xs = [torch.randn(48, 32, device="cuda") for _ in range(9)]
    ys = [torch.randint(0, 10, (48,), device="cuda") for _ in range(9)]

    def train_on(model, opt):
        def fn(x, y):
            opt.zero_grad()
            loss = nn.nll_loss(model(x), y)
            loss.backward()
            opt.step()
            return loss
        return fn

    eager, fn_cap = train_on(ref, opt_ref), train_on(cap, opt_cap)
    graphed = fb.cuda.GraphedStep(fn_cap, (xs[0], ys[0]), optimizer=opt_cap, warmup=2)   # 2 eager steps on batch 0
    for _ in range(2):
        eager(xs[0], ys[0])
    losses_e, losses_g = [], []
    for i in range(1, 9):
        if i == 5:
            opt_ref.set_learning_rate(opt_ref.learning_rate() * 0.5)
            opt_cap.set_learning_rate(opt_cap.learning_rate() * 0.5)
        losses_e.append(float(eager(xs[i], ys[i])))
        losses_g.append(float(graphed(xs[i], ys[i])))
    assert opt_cap.step_count == opt_ref.step_count == 10
    assert losses_g == pytest.approx(losses_e, rel=1e-4, abs=1e-5)
    for a, b in zip(ref.torch_parameters(), cap.torch_parameters()):
        assert torch.allclose(a, b, atol=1e-5, rtol=1e-4)


def test_graphed_step_draws_fresh_dropout_masks():
    import ferrum_b200 as fb
    from ferrum_b200.ops import functional as F

    x = torch.ones(4096, device="cuda")
    outs = []

    def fn(t):
        return F.dropout(t, 0.5, True, seed=7)

    try:
        g = fb.cuda.GraphedStep(fn, (x,), optimizer=None, warmup=1)
        for _ in range(3):
            outs.append(g(x).clone())
    finally:
        F.set_capturable_rng(False)
    assert not torch.equal(outs[0], outs[1]) and not torch.equal(outs[1], outs[2])
    for o in outs:
        kept = (o != 0).float().mean().item()
        assert 0.4 < kept < 0.6 and torch.all((o == 0) | (o == 2.0))
