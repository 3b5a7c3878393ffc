"""CPU model of the flag / epoch handshake that the inter-GPU kernels use, with an exhaustive interleaving
checker.

The kernels of ``csrc/dist/collectives.cu`` synchronise per (channel, block): block ``b`` of every rank stores an
epoch into slot ``[channel][b][its rank]`` of every peer's flag region (``st.release.sys``) and waits until its own
region shows that epoch from every peer (``ld.acquire.sys``, wrap-safe signed comparison, bounded by a timeout).
A fused all-reduce runs

    entry handshake (epoch e)  ->  read the own shard of every peer's gradients, write the result into every
    peer's parameters           ->  exit handshake (epoch e + 1)

and consecutive collectives on a channel use e, e + 2, e + 4, ...  Blocks with different indices never talk to each
other, so one block per rank is the whole protocol.  This module states that protocol as a small program per rank,
explores EVERY interleaving of the ranks' memory operations (sequentially consistent memory, which the release /
acquire pairs provide for the flag-then-data pattern), and checks:

* no rank reads a peer's gradients before the peer wrote them for this step, or after the peer overwrote them for
  the next one;
* after its exit handshake a rank sees this step's parameters from every owner;
* no reachable state is stuck (deadlock freedom), also across the 32-bit wrap of the epoch counter;
* when a rank never arrives, every other rank gives up through the timeout path, reports it, and touches no peer
  data afterwards.

``variant`` selects deliberately broken protocols (no exit handshake, exit epoch equal to the entry epoch, plain
unsigned comparison) that the checker must reject; they show that the properties are not vacuous.  The reference
has no counterpart (its collectives are no-ops: ferrum-distributed/src/collectives.rs:74-129); this is the
race-detection stand-in for the device protocol, runnable without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass

MASK = 0xFFFFFFFF


def _reached(flag: int, epoch: int, wrap_safe: bool) -> bool:
    if wrap_safe:  # the device test: (int32)(flag - epoch) >= 0
        d = (flag - epoch) & MASK
        return d < 0x80000000
    return flag >= epoch


@dataclass
class Result:
    ok: bool
    states: int
    violation: str | None = None
    trace: tuple = ()
    # for every terminal state: which ranks left through the timeout path
    finals: frozenset = frozenset()


def _program(rank: int, world: int, steps: int, base_epoch: int, variant: str):
    """The micro-operations of one rank: tuples (op, a, b)."""
    ops = []
    for k in range(steps):
        e = (base_epoch + 2 * k) & MASK
        e_exit = e if variant == "same_exit_epoch" else (e + 1) & MASK
        ops.append(("wgrad", k, 0))                       # earlier kernels of the stream: this step's gradients
        for p in range(world):
            ops.append(("sflag", p, e))
        for p in range(world):
            ops.append(("wait", p, e))
        for p in range(world):
            ops.append(("rgrad", p, k))                   # own shard of every rank's gradients
        for p in range(world):
            ops.append(("wparam", p, k))                  # the updated shard goes to every rank
        if variant != "no_exit_handshake":
            for p in range(world):
                ops.append(("sflag", p, e_exit))
            for p in range(world):
                ops.append(("wait", p, e_exit))
        ops.append(("check", k, 0))                       # later kernels of the stream read all parameters
    return tuple(ops)


def check(world: int = 2, steps: int = 2, base_epoch: int = 1, variant: str = "ok", absent: int | None = None,
          max_states: int = 2_000_000) -> Result:
    """Explore every interleaving.  ``absent``: a rank that never runs.  A wait whose flag can no longer be stored
    (its writer is absent or has already returned) leaves through the timeout transition: the rank is marked as
    timed out and executes nothing further, like a block that reports and returns."""
    wrap_safe = variant != "plain_compare"
    progs = [_program(r, world, steps, base_epoch, variant) for r in range(world)]
    ends = tuple(len(p) for p in progs)
    init_flag = (base_epoch - 1) & MASK  # what the previous collective left behind
    # state: (pcs, flags[dst*world+src], grads[r], params[r*world+owner], timed_out[r])
    init = (tuple(0 for _ in range(world)), tuple(init_flag for _ in range(world * world)),
            tuple(-1 for _ in range(world)), tuple(-1 for _ in range(world * world)),
            tuple(False for _ in range(world)))
    seen = {init}
    stack = [(init, ())]
    finals = set()
    n = 0
    while stack:
        state, trace = stack.pop()
        n += 1
        if n > max_states:
            return Result(False, n, "state budget exceeded", trace)
        pcs, flags, grads, params, dead = state
        moved = False
        all_done = True
        for r in range(world):
            if r == absent or dead[r] or pcs[r] >= ends[r]:
                continue
            all_done = False
            op, a, b = progs[r][pcs[r]]
            nflags, ngrads, nparams, ndead = flags, grads, params, dead
            npc = pcs[r] + 1
            if op == "wgrad":
                ngrads = grads[:r] + (a,) + grads[r + 1:]
            elif op == "sflag":
                i = a * world + r
                nflags = flags[:i] + (b,) + flags[i + 1:]
            elif op == "wait":
                if not _reached(flags[r * world + a], b, wrap_safe):
                    if a == absent or dead[a] or pcs[a] >= ends[a]:
                        # nobody will ever store this flag: the bounded wait runs out, the block reports and returns
                        ndead = dead[:r] + (True,) + dead[r + 1:]
                        npc = ends[r]
                    else:
                        continue  # not enabled yet
            elif op == "rgrad":
                if grads[a] != b:
                    what = "before it was written" if grads[a] < b else "after it was overwritten"
                    return Result(False, n, f"rank {r} read rank {a}'s gradients of step {b} {what} "
                                            f"(found step {grads[a]})", trace + ((r, op, a, b),))
            elif op == "wparam":
                i = a * world + r
                nparams = params[:i] + (b,) + params[i + 1:]
            elif op == "check":
                for owner in range(world):
                    if params[r * world + owner] != a:
                        return Result(False, n, f"rank {r} left step {a} without rank {owner}'s shard "
                                                f"(found step {params[r * world + owner]})",
                                      trace + ((r, op, a, b),))
            nxt = (pcs[:r] + (npc,) + pcs[r + 1:], nflags, ngrads, nparams, ndead)
            moved = True
            if nxt not in seen:
                seen.add(nxt)
                stack.append((nxt, trace + ((r, op, a, b),) if len(trace) < 64 else trace))
        if all_done:
            finals.add(dead)
        elif not moved:
            return Result(False, n, "deadlock: no rank can move", trace)
    return Result(True, n, finals=frozenset(finals))
