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
