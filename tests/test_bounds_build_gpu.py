"""The debug kernel library (-DFERRUM_BOUNDS=1, selected with FERRUM_BOUNDS=1 at import time): device-side index
checks record {site, index, limit} in the status block and skip the access — nothing traps, the context stays
usable.  Stands in for compute-sanitizer runs.  Each case runs in a child process because the library is chosen
when the package is first used."""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu

needs_gpu = pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _child(body: str, bounds: bool = True) -> str:
    env = dict(os.environ)
    env["FERRUM_BOUNDS"] = "1" if bounds else "0"
    env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
    r = subprocess.run([sys.executable, "-c", textwrap.dedent(body)], capture_output=True, text=True, env=env,
                       timeout=600)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    return r.stdout


@needs_gpu
def test_bounds_build_reports_bad_label_and_keeps_working():
    out = _child("""
        import torch
        import ferrum_b200 as fb
        from ferrum_b200 import _lib
        from ferrum_b200.ops import functional as F
        from ferrum_b200.utils import runtime as rt
        assert _lib.bounds_build_active()
        rt.status_ptr()
        torch.manual_seed(0)
        logits = torch.randn(64, 1000, device="cuda").bfloat16().requires_grad_(True)
        labels = torch.randint(0, 1000, (64,), device="cuda")
        good = F.cross_entropy_logits(logits, labels)
        rt.check_status()                       # in-range labels: nothing reported
        labels[5] = 1000                        # one past the last class
        bad = F.cross_entropy_logits(logits, labels)
        torch.cuda.synchronize()
        code, where, i0, i1 = rt.read_status(clear=True)
        print("STATUS", code, where, i0, i1)
        # the bad row contributed nothing and the context still works
        again = F.cross_entropy_logits(logits, labels.clamp(max=999))
        rt.check_status()
        print("FINITE", bool(torch.isfinite(bad).item()), bool(torch.isfinite(again).item()))
    """)
    assert "STATUS 3 41 1000 1000" in out, out
    assert "FINITE True True" in out, out


@needs_gpu
def test_normal_build_does_not_report_the_bad_label():
    out = _child("""
        import torch
        from ferrum_b200 import _lib
        from ferrum_b200.ops import functional as F
        from ferrum_b200.utils import runtime as rt
        assert not _lib.bounds_build_active()
        rt.status_ptr()
        logits = torch.randn(64, 1000, device="cuda").bfloat16()
        labels = torch.randint(0, 1000, (64,), device="cuda")
        labels[5] = 1000
        F.cross_entropy_logits(logits, labels)
        torch.cuda.synchronize()
        print("STATUS", *rt.read_status(clear=True))
    """, bounds=False)
    assert "STATUS 0" in out, out


@needs_gpu
def test_row_gather_reports_and_zero_fills_an_index_outside_the_source():
    # this check is part of every build: the indices come from user code
    from ferrum_b200.ops import functional as F
    from ferrum_b200.utils import runtime as rt

    rt.status_ptr()
    src = torch.arange(40, device="cuda", dtype=torch.float32).reshape(10, 4)
    idx = torch.tensor([3, 10, 0, -1], device="cuda")
    out = F.gather_rows(src, idx)
    torch.cuda.synchronize()
    code, where, i0, i1 = rt.read_status(clear=True)
    assert code == 3 and where == 11 and (i0, i1) in ((1, 10), (3, -1))
    assert torch.equal(out[0], src[3]) and torch.equal(out[2], src[0])
    assert out[1].abs().sum().item() == 0 and out[3].abs().sum().item() == 0


@needs_gpu
def test_embedding_backward_drops_rows_of_ids_outside_the_table():
    from ferrum_b200.ops import functional as F
    from ferrum_b200.utils import runtime as rt

    rt.status_ptr()
    w = torch.randn(16, 8, device="cuda", requires_grad=True)
    idx = torch.tensor([[1, 2, 16, 3]], device="cuda")  # 16 is outside the table
    out = F.embedding(w, idx)
    out.sum().backward()
    torch.cuda.synchronize()
    code, where, _, i1 = rt.read_status(clear=True)
    assert code == 3 and where == 10 and i1 == 16
    g = w.grad
    assert torch.isfinite(g).all()
    assert g[1].sum().item() == 8 and g[2].sum().item() == 8 and g[3].sum().item() == 8
    assert g.sum().item() == 24  # nothing else was written
