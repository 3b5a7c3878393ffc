"""Address arithmetic of the push mode (GEMM + reduce-scatter in one kernel), restated on the CPU.

In push mode the epilogue of a weight-gradient GEMM (``fb_gemm_bf16_2cta_push``, csrc/gemm/tcgen05_gemm_2cta.cu)
does not write a local matrix: element ``e`` of the bucket belongs to shard ``o = e // per`` (``per`` = bucket
length / world), and source rank ``s`` stores its value at element ``s * per + (e - o * per)`` of rank ``o``'s
bucket region.  The bucket kernel (``allreduce_body``, csrc/dist/collectives.cu) then reduces element ``e`` of its
own shard from the ``world`` local positions ``r * per + (e - o * per)``.  Elements outside the pushed ranges keep
the ordinary layout (element ``e`` at position ``e`` of every rank, pulled from the peers).

These functions model both sides so that the layout can be checked exhaustively without a GPU: every pushed element
is delivered exactly once per source, nothing is written twice, and — the reason why push mode is limited to buckets
that hold a single tensor — slots must not alias ordinarily laid-out data of the same bucket.
"""
from __future__ import annotations


def push_destination(e: int, source: int, per: int) -> tuple[int, int]:
    """(owner rank, element position inside the owner's bucket region) of source's value for bucket element e."""
    owner = e // per
    return owner, source * per + (e - owner * per)


def owner_reads(e: int, world: int, per: int) -> list[int]:
    """Positions of its own bucket region that the owner of pushed element e sums."""
    j = e - (e // per) * per
    return [r * per + j for r in range(world)]


def check_layout(world: int, bucket_len: int, pushed: list[tuple[int, int]]) -> list[str]:
    """Problems of pushing the ranges ``pushed`` ([lo, hi) element ranges) of a bucket of ``bucket_len`` elements:
    an empty list means the layout is sound."""
    problems = []
    if bucket_len % (4 * world):
        return [f"bucket length {bucket_len} is not a multiple of 4 * world"]
    per = bucket_len // world
    is_pushed = [False] * bucket_len
    for lo, hi in pushed:
        if lo % 4 or hi % 4 or not 0 <= lo <= hi <= bucket_len:
            problems.append(f"range [{lo}, {hi}) is not 4-aligned inside the bucket")
            continue
        for e in range(lo, hi):
            is_pushed[e] = True
    # what every position of every rank's region holds: ("slot", source, element) or ("plain", element)
    holds = [dict() for _ in range(world)]
    for e in range(bucket_len):
        if is_pushed[e]:
            for s in range(world):
                o, pos = push_destination(e, s, per)
                if pos in holds[o]:
                    problems.append(f"rank {o} position {pos}: {holds[o][pos]} and slot of source {s} element {e}")
                holds[o][pos] = ("slot", s, e)
    for e in range(bucket_len):
        if not is_pushed[e]:
            for r in range(world):  # every rank keeps its local value of e at position e; the owner pulls them
                if e in holds[r] and holds[r][e][0] == "slot":
                    problems.append(f"rank {r} position {e}: ordinary element {e} aliases {holds[r][e]}")
    for e in range(bucket_len):
        if is_pushed[e]:
            o = e // per
            got = sorted(holds[o].get(pos, (None,)) for pos in owner_reads(e, world, per))
            want = sorted(("slot", s, e) for s in range(world))
            if got != want:
                problems.append(f"owner {o} would not find all contributions of element {e}")
    return problems[:20]
