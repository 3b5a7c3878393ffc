"""The host library (bucket planner, samplers, checkpoint reader / writer, CPU restatements) under gcc's
sanitizers: its sources are compiled with a C++ driver that calls every entry point with ragged and boundary
sizes — once with AddressSanitizer + UndefinedBehaviorSanitizer, once with ThreadSanitizer and several concurrent
callers.  Stands in for the reference's reliance on Rust ownership / RwLock (ferrum-core/src/storage.rs:46-47,
232-234) on the native side; needs no GPU."""
import shutil
import subprocess

import pytest

from ferrum_b200 import _build


def _run(exe, scratch, threads):
    r = subprocess.run([str(exe), str(scratch), str(threads)], capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-4000:]
    assert "selftest ok" in r.stdout
    assert "Sanitizer" not in out and "runtime error" not in out, out[-4000:]


def _build_or_skip(tmp_path, sanitizer):
    try:
        return _build.build_host_selftest(tmp_path, sanitizer)
    except _build.SanitizerUnavailable as e:
        pytest.skip(f"sanitizer runtime not installed: {str(e)[:200]}")


@pytest.mark.skipif(shutil.which(_build.CXX) is None, reason="no C++ compiler")
def test_host_library_under_asan_ubsan(tmp_path):
    exe = _build_or_skip(tmp_path, "address,undefined")
    _run(exe, tmp_path, 1)


@pytest.mark.skipif(shutil.which(_build.CXX) is None, reason="no C++ compiler")
def test_host_library_concurrent_callers_under_tsan(tmp_path):
    exe = _build_or_skip(tmp_path, "thread")
    _run(exe, tmp_path, 4)
