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
