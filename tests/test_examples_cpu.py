"""The example programs run end to end on CPU and reach their stated results."""
import importlib.util
import os

import pytest

EX = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")


def _load(name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(EX, name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_simple_autograd_example():
    gx, gy = _load("simple_autograd").main()
    assert gx == [6.0, 9.0, 12.0] and gy == [1.0, 2.0, 3.0]


def test_tape_xor_example_learns_xor():
    pred = _load("train_xor_tape").main()
    assert [round(p) for p in pred] == [0, 1, 1, 0]


def test_optimizer_xor_example_converges():
    assert _load("train_xor_autograd").main() < 1e-2


def test_simple_nn_example_classifies():
    assert _load("simple_nn").main() > 0.95


def test_feature_tour_runs(capsys):
    _load("new_features_demo").main()
    out = capsys.readouterr().out
    for word in ("conv + pool", "LSTM", "attention", "embedding", "batch sizes"):
        assert word in out


def test_ddp_example_runs_as_two_gloo_ranks(tmp_path):
    """The data-parallel example as two CPU processes over gloo: both ranks finish and the loss falls."""
    import subprocess
    import sys

    import socket

    with socket.socket() as sock:  # a free port, so that parallel test runs do not collide
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(EX, "train_ddp_mlp.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("world 2:")]
    assert line, r.stdout[-2000:]
    first, last = (float(v) for v in line[0].split("loss")[1].split("after")[0].split("->"))
    assert last < first
