"""Single-process assertions of ferrum-distributed's unit tests (lib.rs:132-166, backend.rs:133-163,
process_group.rs:124-147, collectives.rs:131-148, ddp.rs:200-237) plus the bucket planner."""
import ctypes

import pytest
import torch

import ferrum_b200 as fb
from ferrum_b200 import distributed as d


@pytest.fixture(autouse=True)
def _clean():
    d.destroy_process_group()
    yield
    d.destroy_process_group()


def test_init_destroy_and_getters():
    assert not d.is_initialized() and d.get_rank() == 0 and d.get_world_size() == 1 and d.is_main_process()
    assert d.get_world() is None
    d.barrier()  # no-op when uninitialised
    pg = d.init_process_group(d.Backend.Gloo, 0, 1)
    assert d.is_initialized() and d.get_world() is pg and pg.is_main() and pg.backend() is d.Backend.Gloo
    with pytest.raises(d.AlreadyInitialized):
        d.init_process_group(d.Backend.Gloo, 0, 1)
    d.destroy_process_group()
    assert not d.is_initialized()


def test_invalid_rank_and_backend_parsing():
    with pytest.raises(d.InvalidRank, match="Invalid rank 4 for world size 4"):
        d.ProcessGroup.new(d.Backend.Gloo, 4, 4)
    assert d.Backend.from_str("NCCL") is d.Backend.Nccl and d.Backend.from_str("gloo").name_str() == "gloo"
    assert str(d.Backend.Nvlink) == "nvlink" and d.Backend.Gloo.is_available() and not d.Backend.Mpi.is_available()
    with pytest.raises(d.UnsupportedBackend):
        d.Backend.from_str("smoke-signals")
    with pytest.raises(d.UnsupportedBackend):
        d.ProcessGroup(d.Backend.Mpi, 0, 2)


def test_backend_config(monkeypatch):
    c = d.BackendConfig()
    assert (c.master_addr, c.master_port, c.timeout_seconds, c.num_threads) == ("127.0.0.1", 29500, 1800, 4)
    c2 = c.with_master_addr("10.0.0.1").with_master_port(1234).with_timeout(60)
    assert (c2.master_addr, c2.master_port, c2.timeout_seconds) == ("10.0.0.1", 1234, 60) and c.master_port == 29500
    monkeypatch.setenv("MASTER_ADDR", "1.2.3.4")
    monkeypatch.setenv("MASTER_PORT", "4321")
    monkeypatch.setenv("DIST_TIMEOUT", "5")
    e = d.BackendConfig.from_env()
    assert (e.master_addr, e.master_port, e.timeout_seconds) == ("1.2.3.4", 4321, 5)
    assert e.device_wait_ns() == 5_000_000_000 and d.BackendConfig().device_wait_ns() == 10_000_000_000


def test_from_env(monkeypatch):
    monkeypatch.setenv("RANK", "0")
    monkeypatch.setenv("WORLD_SIZE", "1")
    monkeypatch.setenv("DIST_BACKEND", "gloo")
    pg = d.init_process_group_from_env()
    assert pg.rank() == 0 and pg.world_size() == 1 and pg.backend() is d.Backend.Gloo


def test_reduce_op_apply():
    assert d.ReduceOp.Sum.apply(2, 3) == 5 and d.ReduceOp.Product.apply(2, 3) == 6
    assert d.ReduceOp.Min.apply(2, 3) == 2 and d.ReduceOp.Max.apply(2, 3) == 3 and d.ReduceOp.Average.apply(2, 4) == 6


def test_world_of_one_collectives_are_identities():
    pg = d.ProcessGroup.new(d.Backend.Gloo, 0, 1)
    t = fb.Tensor.from_slice([1.0, 2.0])
    pg.all_reduce(t, d.ReduceOp.Average)
    pg.broadcast(t, 0)
    pg.reduce(t, 0, d.ReduceOp.Sum)
    assert t.to_vec() == [1, 2]
    out = [fb.Tensor.zeros([2])]
    pg.all_gather(out, t)
    assert out[0].to_vec() == [1, 2]
    pg.gather(out, t.mul_scalar(2), 0)
    assert out[0].to_vec() == [2, 4]
    o = fb.Tensor.zeros([2])
    pg.scatter(o, [t], 0)
    pg.reduce_scatter(o, [t], d.ReduceOp.Sum)
    assert o.to_vec() == [1, 2]
    pg.barrier()
    assert pg.sequence_number() == 8
    with pytest.raises(d.InvalidRank):
        pg.broadcast(t, 3)
    with pytest.raises(d.InvalidConfiguration):
        pg.all_gather([], t)
    with pytest.raises(d.NotInitialized):
        d.new_group([0])
    d.init_process_group(d.Backend.Gloo, 0, 1)
    assert d.new_group([0]).world_size() == 1


def test_gradient_bucket_bookkeeping():
    b = d.GradientBucket.new()
    assert not b.is_ready() and b.size_bytes() == 0
    b.add_gradient(0, [1.0, 2.0, 3.0])
    b.add_gradient(2, fb.Tensor.ones([2]))
    assert b.param_indices == [0, 2] and b.sizes == [3, 2] and b.size_bytes() == 20
    b.mark_ready()
    assert b.is_ready()
    h = d.GradientHook.new(None, 3)
    assert len(h.buckets) == 3 and not h.all_ready()


def test_bucket_planner_layout():
    from ferrum_b200.parallel.ddp import _plan

    sizes = [1000, 10, 5000, 20, 300]
    total, offs, bof, bstart, blen = _plan(sizes, 4096, 16, 32)
    assert bof[4] == 0 and bof[3] == 0 and offs[4] == 0       # reverse registration order: last parameter first
    assert bof[2] == 1 and blen[1] >= 5000                     # a tensor above the cap gets a bucket of its own
    assert bof[0] == bof[1] == 2
    assert all(o % 32 == 0 for o in offs) and all(l % 16 == 0 for l in blen)
    spans = sorted((offs[i], offs[i] + sizes[i]) for i in range(5))
    assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))  # slots do not overlap
    assert total == bstart[-1] + blen[-1]
    for i in range(5):
        assert bstart[bof[i]] <= offs[i] and offs[i] + sizes[i] <= bstart[bof[i]] + blen[bof[i]]
    lo, hi = ctypes.c_longlong(), ctypes.c_longlong()
    from ferrum_b200 import _lib

    cover = []
    for r in range(3):
        _lib.host().fb_plan_shard(1000, 3, r, ctypes.byref(lo), ctypes.byref(hi))
        cover.append((lo.value, hi.value))
    assert cover[0][0] == 0 and cover[-1][1] == 1000 and all(a[1] == b[0] for a, b in zip(cover, cover[1:]))


def test_ddp_wraps_a_module_and_trains_in_a_world_of_one():
    pg = d.ProcessGroup.new(d.Backend.Gloo, 0, 1)
    model = fb.nn.Sequential(fb.nn.Linear(4, 8), fb.nn.ReLU(), fb.nn.Linear(8, 2))
    ddp = d.DistributedDataParallel.new(model, pg).bucket_size_mb(25).broadcast_buffers(True).find_unused_parameters(
        False)
    assert ddp.module() is model and ddp.process_group() is pg and ddp.module_mut() is model
    ref = fb.nn.Sequential(fb.nn.Linear(4, 8), fb.nn.ReLU(), fb.nn.Linear(8, 2))
    ref.load_state_dict(model.state_dict())
    opt = fb.optim.SGD(model.parameters(), fb.optim.SGDConfig.new(0.1).with_momentum(0.9))
    ropt = fb.optim.SGD(ref.parameters(), fb.optim.SGDConfig.new(0.1).with_momentum(0.9))
    ddp.fuse_optimizer(opt)
    x, y = fb.Tensor.randn([6, 4]), fb.Tensor.randn([6, 2])
    for _ in range(3):
        for net, o in ((ddp, opt), (ref, ropt)):
            o.zero_grad()
            fb.nn.mse_loss(net(x), y).backward()
            o.step()
    for p, q in zip(model.torch_parameters(), ref.torch_parameters()):
        assert torch.allclose(p, q, atol=1e-6)
    grads = [fb.Tensor.ones([3])]
    ddp.sync_gradients(grads)
    ddp.broadcast_parameters([fb.Tensor.ones([3])])
    assert ddp.into_inner() is model
