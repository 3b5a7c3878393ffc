"""Exhaustive interleaving check of the inter-GPU flag / epoch handshake on a CPU model
(ferrum_b200/parallel/protocol_model.py); the device kernels are in csrc/dist/collectives.cu."""
import pytest

from ferrum_b200.parallel.protocol_model import check


@pytest.mark.parametrize("world,steps", [(2, 3), (3, 2), (4, 1)])
def test_protocol_is_race_and_deadlock_free(world, steps):
    res = check(world=world, steps=steps)
    assert res.ok, (res.violation, res.trace[-12:])
    assert res.states > 100
    assert res.finals == {tuple(False for _ in range(world))}  # everybody completes, nobody times out


def test_protocol_survives_epoch_wraparound():
    # entry / exit epochs 0xFFFFFFFE, 0xFFFFFFFF, then 0 and 1: the signed-difference test keeps working
    res = check(world=2, steps=3, base_epoch=0xFFFFFFFE)
    assert res.ok, res.violation


@pytest.mark.parametrize("variant", ["no_exit_handshake", "same_exit_epoch"])
def test_checker_rejects_protocols_without_a_real_exit_handshake(variant):
    res = check(world=2, steps=2, variant=variant)
    assert not res.ok
    assert "gradients" in res.violation or "shard" in res.violation


def test_checker_rejects_plain_unsigned_comparison_at_the_wrap():
    res = check(world=2, steps=3, base_epoch=0xFFFFFFFE, variant="plain_compare")
    assert not res.ok


@pytest.mark.parametrize("world,absent", [(2, 1), (3, 0), (4, 2)])
def test_absent_rank_makes_everyone_time_out_not_hang(world, absent):
    res = check(world=world, steps=2, absent=absent)
    assert res.ok, res.violation  # no deadlock, no read of data that never arrived
    for final in res.finals:
        assert all(final[r] for r in range(world) if r != absent), final


# ---- layout of the push mode (GEMM epilogue stores into the shard owners' memory)
from ferrum_b200.parallel.push_layout import check_layout, owner_reads, push_destination  # noqa: E402


@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_push_layout_of_a_single_tensor_bucket_is_sound(world):
    n = 4 * world * 37
    assert check_layout(world, n, [(0, n)]) == []
    # with alignment padding behind the tensor (ordinary layout): the padding belongs to no parameter, but its
    # positions are slot positions too, which the checker reports — harmless only because nothing reads padding
    assert check_layout(world, n, [(0, n - 4 * world)]) != []


def test_push_layout_rejects_a_bucket_shared_with_ordinarily_laid_out_tensors():
    # a pushed weight followed by small tensors in the same bucket: the last source's slot in every other owner's
    # region lands on the small tensors' positions
    problems = check_layout(2, 4 * 2 * 100, [(0, 4 * 2 * 90)])
    assert problems and "aliases" in " ".join(problems)


def test_push_destination_and_owner_reads_agree():
    world, per = 4, 24
    for e in range(world * per):
        o = e // per
        assert sorted(push_destination(e, s, per)[1] for s in range(world)) == owner_reads(e, world, per)
        assert all(push_destination(e, s, per)[0] == o for s in range(world))


def test_host_epoch_counter_wraps_with_the_device_modulus():
    """``SymmetricArena.next_epoch`` advances modulo 2^32, like the device-side counter and the kernels' wrap-safe
    comparison: through the wrap every entry epoch is 'not reached' by the previous exit flag and 'reached' by
    its own, which a 31-bit host counter broke (a stale flag satisfied the first collective after the wrap)."""
    from ferrum_b200.parallel.protocol_model import _reached
    from ferrum_b200.parallel.symm import SymmetricArena

    arena = SymmetricArena.__new__(SymmetricArena)
    arena._epochs = {2: 0xFFFFFFF9}
    flag = (0xFFFFFFF9 - 1) & 0xFFFFFFFF          # exit epoch of the collective before
    for _ in range(8):
        e = arena.next_epoch(2)
        assert 0 <= e <= 0xFFFFFFFF and e % 2 == 1
        assert not _reached(flag, e, True)        # nobody has arrived yet: the old flag must not pass
        assert _reached(e, e, True)
        flag = (e + 1) & 0xFFFFFFFF               # what the exit handshake leaves behind
        assert _reached(flag, (e + 1) & 0xFFFFFFFF, True)
    assert arena._epochs[2] == 0xFFFFFFF9 + 16 - (1 << 32)
