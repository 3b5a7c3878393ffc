"""Comparison baseline: the same MLP trained with stock PyTorch — ``torch.nn`` layers, cuBLAS GEMMs under bf16
autocast, ``torch.optim.Adam(fused=True)`` and, for more than one GPU, ``DistributedDataParallel`` over NCCL with
25 MB buckets.  None of this package's kernels run on this path."""
from __future__ import annotations


def build(model_cfg, depth, width, device):
    import torch

    layers, d = [], model_cfg["in_features"]
    for _ in range(depth):
        layers += [torch.nn.Linear(d, width), torch.nn.GELU(approximate="tanh"), torch.nn.LayerNorm(width)]
        d = width
    layers.append(torch.nn.Linear(d, model_cfg["num_classes"]))
    return torch.nn.Sequential(*layers).to(device)


def run(args, model_cfg, lr, dist_env, timed_steps, ClockSampler, merge_clocks=None):
    import torch

    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    own_group = False
    if world > 1:
        import torch.distributed as dist

        if not dist.is_initialized():  # bench.py's own arm may have left its rendezvous (gloo + NCCL) up
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            own_group = True
    torch.manual_seed(1234)
    model = build(model_cfg, args.depth, args.width, "cuda")
    net = model
    if world > 1:
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], bucket_cap_mb=25,
                                                        gradient_as_bucket_view=True)
    opt = torch.optim.Adam(model.parameters(), lr=lr, fused=True)
    B = args.batch
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    x_dev = torch.randn(B, model_cfg["in_features"], device="cuda", generator=g)
    y_dev = torch.randint(0, model_cfg["num_classes"], (B,), device="cuda", generator=g)
    x_pin, y_pin = x_dev.cpu().pin_memory(), y_dev.cpu().pin_memory()

    def train_step(x, y):
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = torch.nn.functional.cross_entropy(net(x), y)
        loss.backward()
        opt.step()
        return loss

    losses = []

    def step_device():
        train_step(x_dev, y_dev)

    # same read-back discipline as the other arm: the loss is copied to pinned host memory behind its step and read
    # one step later, so the host never drains the GPU's queue
    slots = [torch.empty((), dtype=torch.float32).pin_memory() for _ in range(3)]
    events = [torch.cuda.Event() for _ in range(3)]
    inflight = []
    counter = [0]

    def pop_loss():
        i = inflight.pop(0)
        events[i].synchronize()
        losses.append(float(slots[i]))

    def step_e2e():
        loss = train_step(x_pin.to("cuda", non_blocking=True), y_pin.to("cuda", non_blocking=True))
        i = counter[0] % 3
        counter[0] += 1
        slots[i].copy_(loss.detach().float(), non_blocking=True)
        events[i].record()
        inflight.append(i)
        if len(inflight) > 1:
            pop_loss()

    def drain_e2e():
        while inflight:
            pop_loss()

    if world > 1:
        barrier = dist.barrier
    else:
        def barrier():
            return None

    for _ in range(max(args.warmup, 3)):
        step_device()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    ms = timed_steps(step_device, args.steps, world, barrier)
    clocks = sampler.stop()
    if merge_clocks is not None:
        clocks = merge_clocks(clocks, world)
    e2e = None
    if not args.no_e2e:
        for _ in range(2):
            step_e2e()
        drain_e2e()
        ms2 = timed_steps(step_e2e, args.steps, world, barrier, finish=drain_e2e)
        e2e = {"value": args.steps * B * world / (ms2 / 1e3), "unit": "samples/s", "ms_per_step": ms2 / args.steps,
               "h2d_bytes_per_step": x_pin.numel() * 4 + y_pin.numel() * 8, "d2h_bytes_per_step": 4,
               "final_loss": losses[-1] if losses else None}
    if own_group:
        dist.destroy_process_group()
    return ms, 0, clocks, e2e, "torch-ddp-nccl" if world > 1 else "torch-single"
