"""Worker functions for the multi-process tests (spawned ranks import this module)."""
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _init(rank, world, port, backend="gloo", timeout=60):
    import ferrum_b200 as fb
    from ferrum_b200 import distributed as d

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"], os.environ["WORLD_SIZE"] = str(rank), str(world)
    cfg = d.BackendConfig.from_env().with_timeout(timeout)
    return fb, d, d.init_process_group(d.Backend.from_str(backend), rank, world, cfg)


def collectives_worker(rank, world, port, out_dir):
    fb, d, pg = _init(rank, world, port)
    ok = True
    t = torch.full((5,), float(rank + 1))
    pg.all_reduce(t, d.ReduceOp.Sum)
    ok &= bool(torch.allclose(t, torch.full((5,), float(sum(range(1, world + 1))))))
    t = torch.full((3,), float(rank + 1))
    pg.all_reduce(fb.Tensor(t), d.ReduceOp.Average)
    ok &= bool(torch.allclose(t, torch.full((3,), (world + 1) / 2.0)))
    t = torch.full((3,), float(rank + 2))
    pg.all_reduce(t, d.ReduceOp.Max)
    ok &= bool(torch.allclose(t, torch.full((3,), float(world + 1))))
    b = torch.arange(4.0) if rank == 1 else torch.zeros(4)
    pg.broadcast(b, 1)
    ok &= bool(torch.equal(b, torch.arange(4.0)))
    outs = [torch.zeros(2) for _ in range(world)]
    pg.all_gather(outs, torch.full((2,), float(rank)))
    ok &= all(bool(torch.equal(o, torch.full((2,), float(r)))) for r, o in enumerate(outs))
    g = [torch.zeros(2) for _ in range(world)] if rank == 0 else None
    pg.gather(g, torch.full((2,), float(rank * 10)), 0)
    if rank == 0:
        ok &= all(bool(torch.equal(o, torch.full((2,), float(r * 10)))) for r, o in enumerate(g))
    o = torch.zeros(2)
    pg.scatter(o, [torch.full((2,), float(r + 5)) for r in range(world)] if rank == 0 else None, 0)
    ok &= bool(torch.equal(o, torch.full((2,), float(rank + 5))))
    o = torch.zeros(2)
    pg.reduce_scatter(o, [torch.full((2,), float(r + rank)) for r in range(world)], d.ReduceOp.Sum)
    ok &= bool(torch.allclose(o, torch.full((2,), float(sum(rank + q for q in range(world))))))
    r_ = torch.full((2,), float(rank + 1))
    pg.reduce(r_, 0, d.ReduceOp.Sum)
    if rank == 0:
        ok &= bool(torch.allclose(r_, torch.full((2,), float(sum(range(1, world + 1))))))
    pg.barrier()
    pg.verify_in_step()
    d.destroy_process_group()
    open(os.path.join(out_dir, f"ok{rank}"), "w").write("1" if ok else "0")


def _make_model(fb, seed=7):
    torch.manual_seed(seed)
    return fb.nn.Sequential(fb.nn.Linear(6, 16), fb.nn.GELU(), fb.nn.LayerNorm([16]), fb.nn.Linear(16, 4))


def ddp_worker(rank, world, port, out_dir, backend="gloo", device="cpu"):
    """DDP over `world` ranks with batch b each must equal one process with batch world*b."""
    fb, d, pg = _init(rank, world, port, backend)
    if device == "cuda":
        torch.cuda.set_device(rank)
    dev = fb.Device.Cuda(rank) if device == "cuda" else fb.Device.Cpu
    model = _make_model(fb).to_device(dev)
    if rank != 0:  # perturb so that broadcast_parameters has something to fix
        with torch.no_grad():
            for p in model.torch_parameters():
                p.add_(1.0)
    opt = fb.optim.Adam(model.parameters(), fb.optim.AdamConfig(lr=1e-2))
    ddp = d.DistributedDataParallel(model, pg).bucket_size_mb(0.0005)
    ddp.fuse_optimizer(opt)
    g = torch.Generator().manual_seed(3)
    X = torch.randn(world * 8, 6, generator=g)
    Y = torch.randn(world * 8, 4, generator=g)
    xs = X[rank * 8:(rank + 1) * 8].to(dev.to_torch())
    ys = Y[rank * 8:(rank + 1) * 8].to(dev.to_torch())
    for _ in range(4):
        opt.zero_grad()
        loss = fb.nn.mse_loss(ddp(xs), ys)
        loss.backward()
        opt.step()
    params = [p.detach().cpu().clone() for p in model.torch_parameters()]
    nb = len(ddp.buckets)
    ddp.shutdown()
    d.destroy_process_group()
    torch.save({"params": params, "buckets": nb}, os.path.join(out_dir, f"params{rank}.pt"))


def single_reference(world, out_path):
    import ferrum_b200 as fb

    model = _make_model(fb)
    opt = fb.optim.Adam(model.parameters(), fb.optim.AdamConfig(lr=1e-2))
    g = torch.Generator().manual_seed(3)
    X = torch.randn(world * 8, 6, generator=g)
    Y = torch.randn(world * 8, 4, generator=g)
    for _ in range(4):
        opt.zero_grad()
        loss = fb.nn.mse_loss(model(X), Y)
        loss.backward()
        opt.step()
    torch.save([p.detach().clone() for p in model.torch_parameters()], out_path)


def late_rank_worker(rank, world, port, out_dir):
    """Rank 1 never joins the rendezvous: rank 0 must get a Timeout, not hang."""
    if rank == 1:
        time.sleep(0.1)
        return
    import ferrum_b200  # noqa: F401
    from ferrum_b200 import distributed as d

    t0 = time.time()
    try:
        _init(rank, world, port, timeout=3)
        res = "joined"
    except d.Timeout:
        res = "timeout"
    except d.CommunicationError:
        res = "commerror"
    open(os.path.join(out_dir, "late"), "w").write(f"{res} {time.time() - t0:.1f}")


def skipped_collective_worker(rank, world, port, out_dir):
    """Rank 1 skips one all_reduce: the host-side sequence check must flag it before anything hangs."""
    fb, d, pg = _init(rank, world, port, timeout=20)
    t = torch.ones(2)
    pg.all_reduce(t)
    if rank == 0:
        pg._seq += 1  # what issuing one more collective than the peer looks like to the bookkeeping
    try:
        pg.verify_in_step()
        res = "ok"
    except d.CommunicationError:
        res = "mismatch"
    d.destroy_process_group()
    open(os.path.join(out_dir, f"skip{rank}"), "w").write(res)


def leaving_rank_worker(rank, world, port, out_dir):
    """A rank leaves between steps and announces it through the store; the others stop before the next launch."""
    fb, d, pg = _init(rank, world, port, timeout=20)
    import torch.distributed as dist

    store = dist.distributed_c10d._get_default_store()
    res = "ran"
    for step in range(4):
        if rank == 1 and step == 2:
            store.set("left/1", "1")
            break
        gone = [r for r in range(world) if store.check([f"left/{r}"])] if step else []
        flag = torch.tensor([1.0 if (rank == 1 and step == 1) else 0.0])
        if gone:
            res = f"peer_left_at_{step}"
            break
        pg.all_reduce(flag, d.ReduceOp.Max)
        if flag.item() > 0 and rank != 1:
            # rank 1 announced on the previous step that it is about to leave
            time.sleep(0.3)
    open(os.path.join(out_dir, f"leave{rank}"), "w").write(res)
    if rank != 1:
        try:
            d.destroy_process_group()
        except Exception:
            pass


def recovery_worker(rank, world, port, out_dir):
    """Three ranks train with DDP and checkpoint; rank 2 leaves between steps.  The survivors get
    CommunicationError from the library at their next step, destroy the group, form a new one of two ranks, load
    the checkpoint and train on."""
    fb, d, pg = _init(rank, world, port, timeout=20)
    from ferrum_b200 import nn, optim, serialize

    def build():
        torch.manual_seed(7)
        m = nn.Sequential(nn.Linear(6, 16), nn.Tanh(), nn.Linear(16, 3))
        o = optim.Adam(m.parameters(), optim.AdamConfig(lr=1e-2))
        return m, o

    g = torch.Generator().manual_seed(11)
    X, Y = torch.randn(24, 6, generator=g), torch.randn(24, 3, generator=g)

    def step(ddp, opt, r, w):
        xs, ys = X[r::w], Y[r::w]
        opt.zero_grad()
        loss = nn.mse_loss(ddp(xs), ys)
        loss.backward()
        opt.step()
        return loss.item()

    model, opt = build()
    ddp = d.DistributedDataParallel(model, pg).fuse_optimizer(opt)
    for _ in range(2):
        step(ddp, opt, rank, world)
    ck = os.path.join(out_dir, "ck.ferrum")
    if rank == 0:
        serialize.save_checkpoint(ck, model=model, optimizer=opt)
    pg.barrier()
    if rank == 2:
        d.leave_process_group()          # between steps, nothing of this rank in flight
        open(os.path.join(out_dir, "rec2"), "w").write("left")
        return
    time.sleep(0.5)                      # the gap between two steps in which the departure becomes visible
    try:
        step(ddp, opt, rank, world)
        res = "no error"
    except d.CommunicationError as exc:  # raised on the host, before anything was launched
        res = "detected" if "left the job" in str(exc) else f"other: {exc}"
    d.destroy_process_group()
    # the survivors regroup: same rank order, a fresh rendezvous next to the old one
    new_world, new_rank = world - 1, rank
    cfg = d.BackendConfig(master_addr="127.0.0.1", master_port=port + 1, timeout_seconds=20)
    pg2 = d.init_process_group(d.Backend.Gloo, new_rank, new_world, cfg)
    model2, opt2 = build()
    with torch.no_grad():
        for p in model2.torch_parameters():
            p.add_(1.0)                   # nothing of the fresh model may survive the load
    serialize.load_checkpoint(ck, model=model2, optimizer=opt2)
    ddp2 = d.DistributedDataParallel(model2, pg2).fuse_optimizer(opt2)
    l0 = step(ddp2, opt2, new_rank, new_world)
    for _ in range(5):
        l1 = step(ddp2, opt2, new_rank, new_world)
    flat = torch.cat([p.detach().reshape(-1) for p in model2.torch_parameters()])
    both = [torch.empty_like(flat) for _ in range(new_world)]
    pg2.all_gather(both, flat)
    same = all(torch.equal(both[0], b) for b in both)
    d.destroy_process_group()
    open(os.path.join(out_dir, f"rec{rank}"), "w").write(
        f"{res} steps={opt2.step_count} same={same} improved={l1 < l0}")


def silent_death_worker(rank, world, port, out_dir):
    """Rank 1 exits without announcing anything; rank 0's next collective ends with Timeout / CommunicationError
    after the (short) process-group timeout instead of hanging."""
    fb, d, pg = _init(rank, world, port, timeout=4)
    t = torch.ones(3)
    pg.all_reduce(t)
    if rank == 1:
        os._exit(0)
    time.sleep(0.5)
    t0 = time.time()
    try:
        pg.all_reduce(t)
        res = "no error"
    except (d.Timeout, d.CommunicationError) as exc:
        res = type(exc).__name__
    open(os.path.join(out_dir, "silent0"), "w").write(f"{res} {time.time() - t0:.1f}")
    os._exit(0)  # the group cannot be shut down cleanly any more
