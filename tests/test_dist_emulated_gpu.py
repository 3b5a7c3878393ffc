"""Inter-GPU kernels with all ranks emulated on ONE GPU as a single cooperative launch.

The same device code runs in the multi-process path; here the "peers" are further arenas on the same device,
so the handshake protocol, the shard arithmetic and the fused optimizer update are checked without a second GPU.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(world, nfloats_total):
    from ferrum_b200 import _lib
    from ferrum_b200._lib_dist import DistCtx
    from ferrum_b200.parallel.symm import SymmetricArena

    arenas = SymmetricArena.emulated(nfloats_total * 4, world)
    ctxs = (DistCtx * world)(*[a.ctx for a in arenas])
    return _lib.cuda(), arenas, ctxs


def _stream():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("n", [8 * 4, 8 * 4 * 333, 1 << 20])
def test_allreduce_average_emulated(world, n):
    from ferrum_b200.utils.runtime import check_status

    lib, arenas, ctxs = _setup(world, n)
    off = arenas[0].data_offset()
    torch.manual_seed(world * 31 + n)
    data = [torch.randn(n, device="cuda") for _ in range(world)]
    for a, d in zip(arenas, data):
        a.view(off, (n,), torch.float32).copy_(d)
    rc = lib.fb_dist_allreduce_emulated(ctxs, world, 0, 0, 1, off, 0, -1, n, 4, 1.0 / world, None, None, None, None,
                                        1, 4, 256, _stream())
    assert rc == 0
    check_status()
    ref = torch.stack(data).sum(0) / world
    for a in arenas:
        assert torch.allclose(a.view(off, (n,), torch.float32), ref, atol=1e-5, rtol=1e-5)
    for a in arenas:
        a.close()


@pytest.mark.parametrize("world,n,blocks", [(2, 1000, 1), (4, 4097, 5), (8, 65536, 16), (3, 1, 1)])
@pytest.mark.parametrize("op", [0, 3, 4])
def test_oneshot_allreduce_emulated(world, n, blocks, op):
    """Latency form of the all-reduce: one handshake, every rank reads all regions and reduces for itself.  Four
    calls in a row alternate between the two slots (no exit handshake protects a slot: its reuse is safe only
    because a whole collective lies between two uses), sum / max / average, tensors that are their own output."""
    from ferrum_b200.utils.runtime import check_status

    slot_bytes = (n * 4 + 255) // 256 * 256
    lib, arenas, ctxs = _setup(world, 2 * slot_bytes // 4 + 64)
    off = arenas[0].data_offset()
    torch.manual_seed(world * 7 + n + op)
    epoch = 1
    for call in range(4):
        data = [torch.randn(n, device="cuda") for _ in range(world)]
        stack = torch.stack([d.clone() for d in data])
        ref = stack.max(0).values if op == 3 else stack.sum(0) / (world if op == 4 else 1)
        ptrs = (ctypes.c_void_p * world)(*[d.data_ptr() for d in data])
        rc = lib.fb_dist_allreduce_oneshot_emulated(ctxs, world, 0, epoch, off + (call % 2) * slot_bytes, n, op,
                                                    1.0 / world if op == 4 else 1.0, ptrs, ptrs, blocks, 256,
                                                    _stream())
        assert rc == 0
        epoch += 2
        check_status()
        for d in data:
            assert torch.allclose(d, ref, atol=1e-5, rtol=1e-5)
    for a in arenas:
        a.close()


@pytest.mark.parametrize("world,n_valid,offset", [(2, 8000, 0), (4, 4097, 0), (8, 333, 1), (3, 1, 3)])
def test_staged_allreduce_emulated(world, n_valid, offset):
    """All-reduce of tensors that live outside the arena: the kernel stages them in and out itself (ragged
    lengths, tensors that do not start on a 16-byte boundary)."""
    from ferrum_b200.utils.runtime import check_status

    n = (n_valid + 4 * world - 1) // (4 * world) * (4 * world)
    lib, arenas, ctxs = _setup(world, n)
    off = arenas[0].data_offset()
    torch.manual_seed(world + n_valid)
    bufs = [torch.randn(n_valid + offset + 5, device="cuda") for _ in range(world)]
    data = [b[offset:offset + n_valid] for b in bufs]
    before = [b.clone() for b in bufs]
    ref = torch.stack([d.clone() for d in data]).sum(0) / world
    ptrs = (ctypes.c_void_p * world)(*[d.data_ptr() for d in data])
    for epoch in (1, 3):  # twice: the second round reduces the first round's results
        rc = lib.fb_dist_allreduce_staged_emulated(ctxs, world, 0, epoch, off, n, 4, 1.0 / world, ptrs, ptrs,
                                                   n_valid, 3, 128, _stream())
        assert rc == 0
        check_status()
        for d in data:
            assert torch.allclose(d, ref, atol=1e-5, rtol=1e-5)
    for b, b0 in zip(bufs, before):  # nothing outside [offset, offset + n_valid) was touched
        assert torch.equal(b[:offset], b0[:offset]) and torch.equal(b[offset + n_valid:], b0[offset + n_valid:])
    for a in arenas:
        a.close()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("fuse,publish_master", [(2, 1), (2, 0), (1, 1)])
def test_reduce_scatter_then_shard_update_emulated(world, fuse, publish_master):
    """The two-kernel form of the gradient reduction: a reduce-scatter per bucket (each rank sums its shard over
    all ranks, 1 / world folded in, result left in its own arena) and one update kernel over all buckets (Adam or
    SGD-momentum on the shard, new fp32 / bf16 weights stored into every rank's arena).  Three buckets of ragged
    lengths inside one arena layout, three steps, against a float reference of the whole thing."""
    from ferrum_b200 import _lib as L
    from ferrum_b200.utils.runtime import check_status

    lens = [4 * world * 257, 4 * world * 3, 4 * world * 1031]
    starts = [0, lens[0], lens[0] + lens[1]]
    n = sum(lens)
    lib, arenas, ctxs = _setup(world, n * 3)
    base = arenas[0].data_offset()
    off_p, off_g, off_s = base, base + n * 4, base + n * 8
    torch.manual_seed(17 + world)
    p0 = torch.randn(n, device="cuda")
    for a in arenas:
        a.view(off_p, (n,), torch.float32).copy_(p0)
    pers = [ln // world for ln in lens]
    soffs = [0, pers[0], pers[0] + pers[1]]
    ms = [torch.zeros(sum(pers), device="cuda") for _ in range(world)]
    vs = [torch.zeros(sum(pers), device="cuda") for _ in range(world)]
    mp = (ctypes.c_void_p * world)(*[m.data_ptr() for m in ms])
    vp = (ctypes.c_void_p * world)(*[v.data_ptr() for v in vs])
    # the middle bucket always publishes fp32 (a bucket of biases under sharded master weights)
    pub = [publish_master, 1, publish_master]
    table = torch.tensor([[starts[k], lens[k], soffs[k], pub[k]] for k in range(3)], dtype=torch.int64,
                         device="cuda")
    lr, b1, b2, eps, wd, mu = 1e-2, 0.9, 0.999, 1e-8, 0.05, 0.9
    ref_p, ref_m, ref_v = p0.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    e_rs, e_up = 1, 1
    for t in (1, 2, 3):
        grads = [torch.randn(n, device="cuda") for _ in range(world)]
        for a, g in zip(arenas, grads):
            a.view(off_g, (n,), torch.float32).copy_(g)
        for k in range(3):
            rc = lib.fb_dist_reduce_scatter_shard_emulated(ctxs, world, 2, e_rs, off_g + starts[k] * 4, lens[k],
                                                           1.0 / world, 3, 256, _stream())
            assert rc == 0
            e_rs += 2
        if fuse == 2:
            h = L.AdamH(lr, b1, b2, eps, wd, 1 - b1 ** t, 1 - b2 ** t, 1.0)
            rc = lib.fb_dist_shard_update_emulated(ctxs, world, 2, 4, e_up, off_g, off_p, off_s, table.data_ptr(), 3,
                                                   ctypes.byref(h), None, mp, vp, 5, 256, _stream())
        else:
            h = L.SgdH(lr, mu, wd, 1.0, 0, 1 if t == 1 else 0)
            rc = lib.fb_dist_shard_update_emulated(ctxs, world, 1, 4, e_up, off_g, off_p, off_s, table.data_ptr(), 3,
                                                   None, ctypes.byref(h), mp, None, 5, 256, _stream())
        assert rc == 0
        e_up += 2
        g = torch.stack(grads).sum(0) / world
        if fuse == 2:
            ref_p = ref_p - lr * wd * ref_p
            ref_m = b1 * ref_m + (1 - b1) * g
            ref_v = b2 * ref_v + (1 - b2) * g * g
            ref_p = ref_p - lr * (ref_m / (1 - b1 ** t)) / ((ref_v / (1 - b2 ** t)).sqrt() + eps)
        else:
            g = g + wd * ref_p
            ref_m = g if t == 1 else mu * ref_m + g
            ref_p = ref_p - lr * ref_m
    check_status()
    owner_p = torch.empty(n, device="cuda")
    for k in range(3):          # the owner of a shard always holds its current fp32 values
        for r in range(world):
            lo, hi = starts[k] + r * pers[k], starts[k] + (r + 1) * pers[k]
            owner_p[lo:hi] = arenas[r].view(off_p, (n,), torch.float32)[lo:hi]
    assert torch.allclose(owner_p, ref_p, atol=2e-5, rtol=1e-5), (owner_p - ref_p).abs().max().item()
    for a in arenas:
        assert torch.equal(a.view(off_s, (n,), torch.bfloat16), owner_p.bfloat16())
        got = a.view(off_p, (n,), torch.float32)
        for k in range(3):
            if pub[k]:
                assert torch.equal(got[starts[k]:starts[k] + lens[k]], owner_p[starts[k]:starts[k] + lens[k]])
    got_m = torch.empty(n, device="cuda")
    for k in range(3):
        for r in range(world):
            got_m[starts[k] + r * pers[k]:starts[k] + (r + 1) * pers[k]] = ms[r][soffs[k]:soffs[k] + pers[k]]
    assert torch.allclose(got_m, ref_m, atol=1e-5)
    for a in arenas:
        a.close()


@pytest.mark.parametrize("world", [2, 4])
def test_fused_allreduce_adam_emulated(world):
    from ferrum_b200 import _lib as L
    from ferrum_b200.utils.runtime import check_status

    n = 4 * world * 1000
    lib, arenas, ctxs = _setup(world, n * 3)
    base = arenas[0].data_offset()
    off_p, off_g, off_s = base, base + n * 4, base + n * 8
    torch.manual_seed(5)
    p0 = torch.randn(n, device="cuda")
    grads = [torch.randn(n, device="cuda") for _ in range(world)]
    for a, g in zip(arenas, grads):
        a.view(off_p, (n,), torch.float32).copy_(p0)
        a.view(off_g, (n,), torch.float32).copy_(g)
    per = n // world
    ms = [torch.zeros(per, device="cuda") for _ in range(world)]
    vs = [torch.zeros(per, device="cuda") for _ in range(world)]
    mp = (ctypes.c_void_p * world)(*[m.data_ptr() for m in ms])
    vp = (ctypes.c_void_p * world)(*[v.data_ptr() for v in vs])
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.999, 1e-8, 0.05
    ref_p, ref_m, ref_v = p0.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    epoch = 1
    for t in (1, 2, 3):
        h = L.AdamH(lr, b1, b2, eps, wd, 1 - b1 ** t, 1 - b2 ** t, 1.0 / world)
        rc = lib.fb_dist_allreduce_emulated(ctxs, world, 2, 0, epoch, off_g, off_p, off_s, n, 0, 1.0,
                                            ctypes.byref(h), None, mp, vp, 1, 3, 256, _stream())
        assert rc == 0
        epoch += 2
        g = torch.stack(grads).sum(0) / world
        ref_p = ref_p - lr * wd * ref_p
        ref_m = b1 * ref_m + (1 - b1) * g
        ref_v = b2 * ref_v + (1 - b2) * g * g
        ref_p = ref_p - lr * (ref_m / (1 - b1 ** t)) / ((ref_v / (1 - b2 ** t)).sqrt() + eps)
    check_status()
    for a in arenas:
        assert torch.allclose(a.view(off_p, (n,), torch.float32), ref_p, atol=1e-5, rtol=1e-5)
        assert torch.equal(a.view(off_s, (n,), torch.bfloat16), ref_p_bf16(a, off_p, n))
    assert torch.allclose(torch.cat(ms), ref_m, atol=1e-6)
    for a in arenas:
        a.close()


def ref_p_bf16(arena, off_p, n):
    return arena.view(off_p, (n,), torch.float32).to(torch.bfloat16)


def test_fused_allreduce_sgd_momentum_emulated():
    from ferrum_b200 import _lib as L
    from ferrum_b200.utils.runtime import check_status

    world, n = 4, 16 * 257
    lib, arenas, ctxs = _setup(world, n * 3)
    base = arenas[0].data_offset()
    off_p, off_g, off_s = base, base + n * 4, base + n * 8
    p0 = torch.randn(n, device="cuda")
    grads = [torch.randn(n, device="cuda") for _ in range(world)]
    for a, g in zip(arenas, grads):
        a.view(off_p, (n,), torch.float32).copy_(p0)
        a.view(off_g, (n,), torch.float32).copy_(g)
    per = ((n + world - 1) // world + 3) // 4 * 4
    vel = [torch.zeros(per, device="cuda") for _ in range(world)]
    mp = (ctypes.c_void_p * world)(*[v.data_ptr() for v in vel])
    ref_p, ref_v = p0.clone(), None
    epoch = 1
    for step in range(3):
        h = L.SgdH(0.1, 0.9, 1e-4, 1.0 / world, 0, 1 if step == 0 else 0)
        rc = lib.fb_dist_allreduce_emulated(ctxs, world, 1, 0, epoch, off_g, off_p, off_s, n, 0, 1.0, None,
                                            ctypes.byref(h), mp, None, 1, 2, 128, _stream())
        assert rc == 0
        epoch += 2
        g = torch.stack(grads).sum(0) / world + 1e-4 * ref_p
        ref_v = g.clone() if ref_v is None else 0.9 * ref_v + g
        ref_p = ref_p - 0.1 * ref_v
    check_status()
    for a in arenas:
        assert torch.allclose(a.view(off_p, (n,), torch.float32), ref_p, atol=1e-5, rtol=1e-5)
    for a in arenas:
        a.close()


def test_pull_collectives_emulated():
    from ferrum_b200.utils.runtime import check_status

    world, n = 4, 1000
    lib, arenas, ctxs = _setup(world, n * (2 + 2 * world))
    base = arenas[0].data_offset()
    in_off, out_off = base, base + n * world * 4
    data = [torch.randn(n * world, device="cuda") for _ in range(world)]

    def load():
        for a, d in zip(arenas, data):
            a.view(in_off, (n * world,), torch.float32).copy_(d)

    epoch = 1
    # broadcast from rank 2 (in place)
    load()
    assert lib.fb_dist_collective_emulated(ctxs, world, 0, 0, epoch, 2, in_off, in_off, n * 4, 0, 1.0, 2, _stream()) == 0
    epoch += 2
    for a in arenas:
        assert torch.equal(a.view(in_off, (n,), torch.float32), data[2][:n])
    # all-gather of the first n floats of every rank
    load()
    assert lib.fb_dist_collective_emulated(ctxs, world, 1, 0, epoch, 0, in_off, out_off, n * 4, 0, 1.0, 2, _stream()) == 0
    epoch += 2
    want = torch.cat([d[:n] for d in data])
    for a in arenas:
        assert torch.equal(a.view(out_off, (n * world,), torch.float32), want)
    # scatter from rank 1
    load()
    assert lib.fb_dist_collective_emulated(ctxs, world, 3, 0, epoch, 1, in_off, out_off, n * 4, 0, 1.0, 2, _stream()) == 0
    epoch += 2
    for r, a in enumerate(arenas):
        assert torch.equal(a.view(out_off, (n,), torch.float32), data[1][r * n:(r + 1) * n])
    # reduce-scatter (sum)
    load()
    assert lib.fb_dist_collective_emulated(ctxs, world, 4, 0, epoch, 0, in_off, out_off, n * 4, 0, 1.0, 2, _stream()) == 0
    epoch += 2
    tot = torch.stack(data).sum(0)
    for r, a in enumerate(arenas):
        assert torch.allclose(a.view(out_off, (n,), torch.float32), tot[r * n:(r + 1) * n], atol=1e-5)
    # reduce (max) to rank 3
    load()
    assert lib.fb_dist_collective_emulated(ctxs, world, 5, 0, epoch, 3, in_off, out_off, n * 4, 3, 1.0, 2, _stream()) == 0
    epoch += 2
    assert torch.equal(arenas[3].view(out_off, (n,), torch.float32), torch.stack(data).max(0).values[:n])
    check_status()
    for a in arenas:
        a.close()


@pytest.mark.parametrize("world,n,shift", [(4, 1000, 0), (4, 333, 1), (3, 5, 0), (8, 4099, 3)])
def test_staged_pull_collectives_emulated(world, n, shift):
    """The pull collectives on tensors outside the arena: the kernel stages the inputs itself and writes results
    straight to the destination.  Chunk sizes that are not multiples of 16 bytes and pointers that are only
    4-byte aligned take the element-wise paths."""
    from ferrum_b200.utils.runtime import check_status

    lib, arenas, ctxs = _setup(world, n * world + 16)
    in_off = arenas[0].data_offset()
    torch.manual_seed(world * 7 + n)
    src = [torch.randn(n * world + shift, device="cuda")[shift:] for _ in range(world)]
    outs = [torch.full((n * world + shift + 3,), -7.0, device="cuda") for _ in range(world)]
    VP = ctypes.c_void_p * world
    none = VP(*[None] * world)

    def run(mode, root, ins, dsts, epoch, op=0):
        rc = lib.fb_dist_collective_staged_emulated(ctxs, world, mode, 0, epoch, root, in_off, n * 4, op, 1.0,
                                                    ins, dsts, 2, _stream())
        assert rc == 0
        check_status()

    def reset():
        for o in outs:
            o.fill_(-7.0)

    o_ptr = VP(*[o[shift:].data_ptr() for o in outs])
    s_ptr = VP(*[x.data_ptr() for x in src])
    root = world - 1
    # broadcast: only the root contributes, everybody else receives
    reset()
    run(0, root, VP(*[src[r].data_ptr() if r == root else None for r in range(world)]),
        VP(*[None if r == root else outs[r][shift:].data_ptr() for r in range(world)]), 1)
    for r in range(world):
        if r != root:
            assert torch.equal(outs[r][shift:shift + n], src[root][:n])
            assert (outs[r][shift + n:] == -7).all() and (outs[r][:shift] == -7).all()
    # all-gather of the first n floats of every rank
    reset()
    run(1, 0, s_ptr, o_ptr, 3)
    want = torch.cat([x[:n] for x in src])
    for o in outs:
        assert torch.equal(o[shift:shift + n * world], want) and (o[shift + n * world:] == -7).all()
    # gather to the root only
    reset()
    run(2, root, s_ptr, VP(*[outs[r][shift:].data_ptr() if r == root else None for r in range(world)]), 5)
    assert torch.equal(outs[root][shift:shift + n * world], want)
    assert all((outs[r] == -7).all() for r in range(world) if r != root)
    # scatter from rank 0
    reset()
    run(3, 0, VP(*[src[0].data_ptr() if r == 0 else None for r in range(world)]), o_ptr, 7)
    for r in range(world):
        assert torch.equal(outs[r][shift:shift + n], src[0][r * n:(r + 1) * n]) and (outs[r][shift + n:] == -7).all()
    # reduce-scatter (sum) and reduce (max) to the root
    reset()
    run(4, 0, s_ptr, o_ptr, 9)
    tot = torch.stack([x[:n * world] for x in src]).sum(0)
    for r in range(world):
        assert torch.allclose(outs[r][shift:shift + n], tot[r * n:(r + 1) * n], atol=1e-5)
    reset()
    run(5, root, s_ptr, VP(*[outs[r][shift:].data_ptr() if r == root else None for r in range(world)]), 11, op=3)
    assert torch.equal(outs[root][shift:shift + n], torch.stack([x[:n] for x in src]).max(0).values)
    assert (outs[root][shift + n:] == -7).all()
    del none
    for a in arenas:
        a.close()


def test_bounded_wait_reports_timeout_and_context_survives():
    """A handshake whose peer never signals gives up after the configured bound and reports it."""
    from ferrum_b200 import _lib
    from ferrum_b200._lib_dist import DistCtx
    from ferrum_b200.parallel.symm import SymmetricArena
    from ferrum_b200.utils import runtime as rt

    arena = SymmetricArena.emulated(4096, 1, wait_ns=50_000_000)[0]
    ctx = DistCtx()
    ctx.rank, ctx.world = 0, 2
    ctx.arena[0] = arena.local_ptr
    ctx.arena[1] = arena.local_ptr  # "rank 1" never writes its slot: nothing else is launched
    ctx.status = rt.status_ptr()
    ctx.timeout_ns = 50_000_000
    rt.read_status(clear=True)
    assert _lib.cuda().fb_dist_barrier(ctx, 3, 7, _stream()) == 0
    torch.cuda.synchronize()
    code, where, peer, epoch = rt.read_status(clear=True)
    assert code == 2 and peer == 1 and epoch == 7
    with pytest.raises(rt.DeviceStatusError):
        _lib.cuda().fb_dist_barrier(ctx, 3, 9, _stream())
        rt.check_status()
    x = torch.ones(1024, device="cuda")
    assert float((x * 2).sum()) == 2048.0  # the context is still usable
    arena.close()


def test_sharded_master_weights_and_inplace_all_gather_emulated():
    """publish_master = 0: peers receive only the bf16 copy; the in-place all-gather then restores fp32 everywhere."""
    from ferrum_b200 import _lib as L
    from ferrum_b200.utils.runtime import check_status

    world = 4
    n = 4 * world * 500
    lib, arenas, ctxs = _setup(world, n * 3)
    base = arenas[0].data_offset()
    off_p, off_g, off_s = base, base + n * 4, base + n * 8
    p0 = torch.randn(n, device="cuda")
    grads = [torch.randn(n, device="cuda") for _ in range(world)]
    for a, g in zip(arenas, grads):
        a.view(off_p, (n,), torch.float32).copy_(p0)
        a.view(off_g, (n,), torch.float32).copy_(g)
    per = n // world
    vel = [torch.zeros(per, device="cuda") for _ in range(world)]
    mp = (ctypes.c_void_p * world)(*[v.data_ptr() for v in vel])
    h = L.SgdH(0.1, 0.0, 0.0, 1.0 / world, 0, 1)
    assert lib.fb_dist_allreduce_emulated(ctxs, world, 1, 0, 1, off_g, off_p, off_s, n, 0, 1.0, None, ctypes.byref(h),
                                          mp, None, 0, 2, 128, _stream()) == 0
    ref = p0 - 0.1 * torch.stack(grads).sum(0) / world
    for r, a in enumerate(arenas):
        mine = a.view(off_p, (n,), torch.float32)
        assert torch.allclose(mine[r * per:(r + 1) * per], ref[r * per:(r + 1) * per], atol=1e-6)
        other = (r + 1) % world
        assert torch.equal(mine[other * per:(other + 1) * per], p0[other * per:(other + 1) * per])  # still stale
        assert torch.allclose(a.view(off_s, (n,), torch.bfloat16).float(), ref, atol=2e-2, rtol=1e-2)  # bf16 current
    assert lib.fb_dist_collective_emulated(ctxs, world, 6, 0, 3, 0, off_p, 0, per * 4, 0, 1.0, 2, _stream()) == 0
    check_status()
    for a in arenas:
        assert torch.allclose(a.view(off_p, (n,), torch.float32), ref, atol=1e-6)
        a.close()


@pytest.mark.parametrize("schedule", ["update after backward", "update in backward", "single kernel"])
def test_single_rank_engine_overlaps_optimizer_and_matches_plain_training(schedule):
    """World size 1 with a fused optimizer, in the engine's three schedules (one update kernel after backward,
    an update kernel per bucket behind each weight gradient, the single all-reduce + update kernel per bucket);
    the trajectory must equal plain Adam / SGD on the same model."""
    import copy

    import ferrum_b200 as fb
    from ferrum_b200 import nn, optim
    from ferrum_b200.parallel import Backend, DistributedDataParallel, ProcessGroup

    dev = fb.Device.Cuda(0)
    for make_opt in (lambda ps: optim.Adam(ps, optim.AdamConfig(lr=1e-2)),
                     lambda ps: optim.SGD(ps, optim.SGDConfig(lr=0.05, momentum=0.9))):
        torch.manual_seed(5)
        ref = nn.Sequential(nn.Linear(64, 256, device=dev), nn.GELU(), nn.LayerNorm([256], device=dev),
                            nn.Linear(256, 264, device=dev), nn.ReLU(), nn.Linear(264, 10, device=dev))
        eng_model = copy.deepcopy(ref)
        opt_ref = make_opt(ref.parameters())
        opt_eng = make_opt(eng_model.parameters())
        pg = ProcessGroup(Backend.Nvlink, 0, 1)
        eng = DistributedDataParallel(eng_model, pg).bucket_size_mb(0.1)
        eng.fuse_optimizer(opt_eng)
        if schedule == "update in backward":
            eng.update_in_backward(True)
        elif schedule == "single kernel":
            eng.defer_update(False)
        x = torch.randn(96, 64, device="cuda")
        y = torch.randint(0, 10, (96,), device="cuda")
        for step in range(4):
            for net, opt in ((ref, opt_ref), (eng, opt_eng)):
                opt.zero_grad()
                with fb.autocast():
                    loss = nn.cross_entropy(net(x), y)
                loss.backward()
                opt.step()
        torch.cuda.synchronize()
        fb.utils.runtime.check_status()
        for a, b in zip(ref.torch_parameters(), eng_model.torch_parameters()):
            assert torch.allclose(a, b, atol=2e-3, rtol=2e-2), (a - b).abs().max().item()
        eng.shutdown()


def _two_branch_model(dev):
    import ferrum_b200 as fb
    from ferrum_b200 import nn

    class TwoBranch(nn.Module):
        def __init__(self):
            super().__init__()
            self.a = nn.Linear(32, 48, device=dev)
            self.b = nn.Linear(32, 48, device=dev)
            self.head = nn.Linear(48, 6, device=dev)

        def forward(self, x, use_b=True):
            h = self.a(x)
            if use_b:
                h = h + self.b(x)
            return self.head(h)

    return TwoBranch()


def test_engine_weight_without_gradient_takes_a_zero_gradient():
    """A Linear weight whose GEMM did not run in a step must not be updated with the previous step's gradient
    (its arena slot is overwritten by the GEMM, never zeroed): with plain SGD it stays exactly where it was, and
    with Adam the trajectory equals an unfused run in which the skipped weight is given an explicit zero gradient."""
    import copy

    import ferrum_b200 as fb
    from ferrum_b200 import nn, optim
    from ferrum_b200.parallel import Backend, DistributedDataParallel, ProcessGroup

    dev = fb.Device.Cuda(0)
    x = torch.randn(64, 32, device="cuda")
    y = torch.randint(0, 6, (64,), device="cuda")
    for kind in ("sgd", "adam"):
        torch.manual_seed(3)
        ref = _two_branch_model(dev)
        model = copy.deepcopy(ref)
        mk = (lambda ps: optim.SGD(ps, optim.SGDConfig(lr=0.1))) if kind == "sgd" else (
            lambda ps: optim.Adam(ps, optim.AdamConfig(lr=1e-2)))
        opt, ropt = mk(model.parameters()), mk(ref.parameters())
        eng = DistributedDataParallel(model, ProcessGroup(Backend.Nvlink, 0, 1)).bucket_size_mb(0.002)
        eng.fuse_optimizer(opt)
        for step in range(4):
            use_b = step % 2 == 0
            before = model.b.weight.detach().clone()
            opt.zero_grad()
            nn.cross_entropy(eng(x, use_b=use_b), y).backward()
            opt.step()
            ropt.zero_grad(set_to_none=False)
            nn.cross_entropy(ref(x, use_b=use_b), y).backward()
            for p in ref.torch_parameters():
                if p.grad is None:
                    p.grad = torch.zeros_like(p)
            ropt.step()
            torch.cuda.synchronize()
            if kind == "sgd" and not use_b:
                assert torch.equal(model.b.weight.detach(), before)
        for a, b in zip(model.torch_parameters(), ref.torch_parameters()):
            assert torch.allclose(a, b, atol=1e-5, rtol=1e-4), (kind, (a - b).abs().max().item())
        eng.shutdown()


@pytest.mark.parametrize("capturable", [False, True])
def test_engine_checkpoint_resume_matches_uninterrupted_run(tmp_path, capturable):
    """save_checkpoint with a fused engine stores the moments that live in the engine's shards; a fresh model +
    engine that loads the file continues exactly like the run that was never interrupted (also with the step
    factors kept in device memory)."""
    import copy

    import ferrum_b200 as fb
    from ferrum_b200 import nn, optim, serialize
    from ferrum_b200.parallel import Backend, DistributedDataParallel, ProcessGroup

    dev = fb.Device.Cuda(0)
    x = torch.randn(64, 32, device="cuda")
    y = torch.randint(0, 6, (64,), device="cuda")

    def build(seed):
        torch.manual_seed(seed)
        m = nn.Sequential(nn.Linear(32, 64, device=dev), nn.GELU(), nn.LayerNorm([64], device=dev),
                          nn.Linear(64, 6, device=dev))
        o = optim.Adam(m.parameters(), optim.AdamConfig(lr=1e-2, weight_decay=0.01))
        e = DistributedDataParallel(m, ProcessGroup(Backend.Nvlink, 0, 1)).bucket_size_mb(0.004)
        e.fuse_optimizer(o)
        if capturable:
            e.capturable(True)
        return m, o, e

    def steps(e, o, n):
        for _ in range(n):
            o.zero_grad()
            nn.cross_entropy(e(x), y).backward()
            o.step()

    m1, o1, e1 = build(1)
    steps(e1, o1, 3)
    path = tmp_path / "ck.ferrum"
    serialize.save_checkpoint(path, model=m1, optimizer=o1)
    saved = serialize.load(path)
    assert any(k.startswith("optim.m.") for k in saved) and int(saved["optim.step"].item()) == 3
    assert sum(saved[k]._t.abs().sum().item() for k in saved if k.startswith("optim.v.")) > 0
    steps(e1, o1, 2)
    m2, o2, e2 = build(99)               # different init: everything must come from the file
    steps(e2, o2, 1)                     # its own state exists and gets replaced
    serialize.load_checkpoint(path, model=m2, optimizer=o2, device=dev)
    assert o2.step_count == 3
    steps(e2, o2, 2)
    torch.cuda.synchronize()
    for a, b in zip(m1.torch_parameters(), m2.torch_parameters()):
        assert torch.allclose(a, b, atol=1e-6, rtol=1e-5), (a - b).abs().max().item()
    e1.shutdown()
    e2.shutdown()


def test_into_inner_hands_back_a_module_that_trains_without_the_engine():
    import ferrum_b200 as fb
    from ferrum_b200 import nn, optim
    from ferrum_b200.parallel import Backend, DistributedDataParallel, ProcessGroup

    dev = fb.Device.Cuda(0)
    torch.manual_seed(4)
    model = nn.Sequential(nn.Linear(32, 64, device=dev), nn.ReLU(), nn.Linear(64, 6, device=dev))
    opt = optim.Adam(model.parameters(), optim.AdamConfig(lr=1e-2))
    eng = DistributedDataParallel(model, ProcessGroup(Backend.Nvlink, 0, 1)).bucket_size_mb(0.004)
    eng.fuse_optimizer(opt)
    x = torch.randn(64, 32, device="cuda")
    y = torch.randint(0, 6, (64,), device="cuda")
    for _ in range(2):
        opt.zero_grad()
        nn.cross_entropy(eng(x), y).backward()
        opt.step()
    inner = eng.into_inner()
    assert inner is model and opt._engine is None
    assert all(getattr(m, "grad_sink", None) is None for m in model.modules())
    assert opt.m[0] is not None and opt.m[0].abs().sum().item() > 0     # the moments moved back to the optimizer
    l0 = nn.cross_entropy(inner(x), y).item()
    for _ in range(5):
        opt.zero_grad()
        loss = nn.cross_entropy(inner(x), y)
        loss.backward()
        opt.step()
    assert opt.step_count == 7 and loss.item() < l0


def test_guard_bands_around_the_engine_arena_detect_a_stray_write(monkeypatch):
    """FERRUM_GUARD_BANDS=1: pattern-filled bands around the parameter / gradient / bf16 regions stay intact over
    training steps, and a write into one of them (made from the host side here) is reported with its position."""
    import ferrum_b200 as fb
    from ferrum_b200 import nn, optim
    from ferrum_b200.parallel import Backend, DistributedDataParallel, InternalError, ProcessGroup

    monkeypatch.setenv("FERRUM_GUARD_BANDS", "1")
    dev = fb.Device.Cuda(0)
    torch.manual_seed(2)
    model = nn.Sequential(nn.Linear(64, 256, device=dev), nn.GELU(), nn.LayerNorm([256], device=dev),
                          nn.Linear(256, 10, device=dev))
    opt = optim.Adam(model.parameters(), optim.AdamConfig(lr=1e-2))
    eng = DistributedDataParallel(model, ProcessGroup(Backend.Nvlink, 0, 1)).bucket_size_mb(0.1)
    eng.fuse_optimizer(opt)
    x = torch.randn(96, 64, device="cuda")
    y = torch.randint(0, 10, (96,), device="cuda")
    for _ in range(3):
        opt.zero_grad()
        with fb.autocast():
            loss = nn.cross_entropy(eng(x), y)
        loss.backward()
        opt.step()
    assert eng.check_guard_bands() == 4
    name, band = eng._guards[1]
    band[123] = 7  # what a kernel writing past the end of the parameter region would do
    with pytest.raises(InternalError, match="byte 123"):
        eng.check_guard_bands()
    band[123] = 0xA5
    eng.shutdown()


@pytest.mark.parametrize("world,M,N,K,small", [(2, 512, 260, 128, 0), (4, 1024, 388, 64, 0), (2, 776, 128, 96, 0),
                                               (8, 520, 132, 64, 0)])
def test_wgrad_gemm_pushes_its_tiles_to_the_shard_owners_emulated(world, M, N, K, small):
    """GEMM + reduce-scatter in one kernel: every virtual rank runs the CTA-pair wgrad GEMM whose epilogue stores
    each 16-byte piece into the owner's bucket region (its own slot), then the bucket kernel reduces the pushed
    range from local memory only.  The bucket holds the one weight (plus alignment padding, pulled the ordinary
    way); shard boundaries fall inside rows and inside 32-column chunks."""
    from ferrum_b200 import _lib as L
    from ferrum_b200.utils.runtime import check_status

    wsz = M * N
    n = (wsz + small + 4 * world - 1) // (4 * world) * (4 * world)
    lib, arenas, ctxs = _setup(world, n * 3)
    base = arenas[0].data_offset()
    off_p, off_g, off_s = base, base + n * 4, base + n * 8
    torch.manual_seed(M + N + world)
    p0 = torch.randn(n, device="cuda")
    As = [(torch.randn(M, K, device="cuda") * 0.5).bfloat16() for _ in range(world)]
    Bs = [(torch.randn(N, K, device="cuda") * 0.5).bfloat16() for _ in range(world)]
    smalls = [torch.randn(n - wsz, device="cuda") for _ in range(world)]
    for a, sm in zip(arenas, smalls):
        a.view(off_p, (n,), torch.float32).copy_(p0)
        g = a.view(off_g, (n,), torch.float32)
        g.fill_(float("nan"))            # whatever the GEMMs do not overwrite must not be read for the weight
        g[wsz:].copy_(sm)                # alignment padding of the bucket: ordinary layout, pulled from the peers
    per = n // world
    for r in range(world):
        rc = lib.fb_gemm_bf16_2cta_push(As[r].data_ptr(), Bs[r].data_ptr(), M, N, K, K, K, N, 0, 0,
                                        ctypes.byref(ctxs[r]), off_g, 0, per, n, 0, None, _stream())
        assert rc == 0, rc
    # NaN fill survives only outside the slots: inside the pushed range every slot of every owner was written
    LLn = ctypes.c_longlong * 1
    assert lib.fb_dist_set_pushed_ranges(1, LLn(0), LLn(wsz)) == 0
    h = L.SgdH(0.5, 0.0, 0.0, 1.0 / world, 0, 1)
    rc = lib.fb_dist_allreduce_emulated(ctxs, world, 1, 0, 1, off_g, off_p, off_s, n, 0, 1.0, None, ctypes.byref(h),
                                        None, None, 1, 3, 256, _stream())
    assert rc == 0
    check_status()
    gw = torch.stack([a.float() @ b.float().t() for a, b in zip(As, Bs)]).sum(0).reshape(-1) / world
    ref = p0[:wsz] - 0.5 * gw
    for a in arenas:
        got = a.view(off_p, (n,), torch.float32)[:wsz]
        assert torch.isfinite(got).all()
        assert torch.allclose(got, ref, atol=2e-3, rtol=1e-3), (got - ref).abs().max().item()
    for a in arenas:
        a.close()
