"""Multi-process behaviour on CPU ranks (gloo): collectives, DDP equivalence, and failure detection made on
the host — a rank that never joins, a skipped collective, a rank that leaves between steps."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from tests import _dist_workers as W


def _port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _spawn(fn, world, tmp_path, *extra):
    mp.spawn(fn, args=(world, _port(), str(tmp_path), *extra), nprocs=world, join=True)


@pytest.mark.timeout(180)
@pytest.mark.parametrize("world", [2, 3])
def test_collectives_gloo(world, tmp_path):
    _spawn(W.collectives_worker, world, tmp_path)
    for r in range(world):
        assert (tmp_path / f"ok{r}").read_text() == "1"


@pytest.mark.timeout(180)
def test_ddp_equals_large_batch(tmp_path):
    world = 2
    _spawn(W.ddp_worker, world, tmp_path)
    W.single_reference(world, str(tmp_path / "ref.pt"))
    ref = torch.load(tmp_path / "ref.pt")
    outs = [torch.load(tmp_path / f"params{r}.pt") for r in range(world)]
    assert outs[0]["buckets"] > 1  # the tiny bucket size splits the model into several buckets
    for r in range(world):
        for p, q in zip(outs[r]["params"], ref):
            assert torch.allclose(p, q, atol=2e-5, rtol=1e-4)
    for p, q in zip(outs[0]["params"], outs[1]["params"]):
        assert torch.equal(p, q)


@pytest.mark.timeout(120)
def test_rank_that_never_joins_times_out(tmp_path):
    _spawn(W.late_rank_worker, 2, tmp_path)
    res, secs = (tmp_path / "late").read_text().split()
    assert res in ("timeout", "commerror")
    assert float(secs) < 60


@pytest.mark.timeout(120)
def test_skipped_collective_is_detected(tmp_path):
    _spawn(W.skipped_collective_worker, 2, tmp_path)
    assert (tmp_path / "skip0").read_text() == "mismatch"
    assert (tmp_path / "skip1").read_text() == "mismatch"


@pytest.mark.timeout(120)
def test_rank_leaving_between_steps_is_noticed(tmp_path):
    _spawn(W.leaving_rank_worker, 2, tmp_path)
    assert (tmp_path / "leave0").read_text().startswith("peer_left_at_")


@pytest.mark.timeout(240)
def test_survivors_regroup_and_resume_from_the_checkpoint(tmp_path):
    """The whole recovery path on host ranks: a rank leaves between steps -> the library raises
    CommunicationError at the survivors' next step -> destroy_process_group -> init_process_group with the
    remaining world -> load_checkpoint -> training continues, replicas identical."""
    _spawn(W.recovery_worker, 3, tmp_path)
    assert (tmp_path / "rec2").read_text() == "left"
    for r in (0, 1):
        assert (tmp_path / f"rec{r}").read_text() == "detected steps=8 same=True improved=True"


@pytest.mark.timeout(120)
def test_rank_that_dies_silently_ends_the_next_collective_with_an_error(tmp_path):
    _spawn(W.silent_death_worker, 2, tmp_path)
    res, secs = (tmp_path / "silent0").read_text().split()
    assert res in ("Timeout", "CommunicationError") and float(secs) < 60
