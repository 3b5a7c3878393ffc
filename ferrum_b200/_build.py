"""In-tree native build of the two shared libraries of this package.

``lib/libferrum_b200_cuda.so``
    every ``.cu`` / ``.cpp`` under ``csrc/`` except ``csrc/host`` — the sm_100a
    kernels and the CUDA runtime wrappers, compiled with
    ``nvcc -gencode arch=compute_100a,code=sm_100a`` (cross-compiles without a GPU).
``lib/libferrum_b200_host.so``
    ``csrc/host/*.cpp`` — checkpoint serializer, samplers, bucket planner and the
    plain-C++ CPU reference loops; no CUDA dependency, so it loads anywhere.

Both expose a C ABI that the Python layer reaches through :mod:`ctypes`, which
keeps the build free of framework headers (a full rebuild takes well under a
minute) and lets non-Python callers link the same entry points.

Objects are cached by a hash of the source, the headers under ``csrc/`` and the
flags, so ``build()`` is incremental.  Run ``python -m ferrum_b200._build``.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "_obj"
LIB = ROOT / "lib"
CUDA_LIB = LIB / "libferrum_b200_cuda.so"
OBJ_BOUNDS = ROOT / "_obj_bounds"
CUDA_LIB_BOUNDS = LIB / "libferrum_b200_cuda_bounds.so"  # debug build with device-side index checks
HOST_LIB = LIB / "libferrum_b200_host.so"

CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.environ.get("NVCC") or shutil.which("nvcc") or f"{CUDA_HOME}/bin/nvcc"
CXX = os.environ.get("CXX", "g++")

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function"]


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.rglob("*")):
        if p.suffix in (".h", ".cuh", ".hpp"):
            h.update(p.name.encode())
            h.update(p.read_bytes())
    return h.hexdigest()


def _compile_one(src: Path, flags_key: str, hdr: str, verbose: bool, bounds: bool = False) -> Path:
    rel = src.relative_to(CSRC)
    extra = ["-DFERRUM_BOUNDS=1"] if bounds else []
    flags_key += " ".join(extra)
    obj = (OBJ_BOUNDS if bounds else OBJ) / (str(rel).replace("/", "__") + ".o")
    stamp = obj.with_suffix(".hash")
    key = hashlib.sha256((flags_key + hdr).encode() + src.read_bytes()).hexdigest()
    if obj.exists() and stamp.exists() and stamp.read_text() == key:
        return obj
    if src.suffix == ".cu":
        cmd = [NVCC, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    else:
        cmd = [CXX, *CXX_FLAGS, *extra, "-I", str(CSRC), "-I", f"{CUDA_HOME}/include", "-c", str(src), "-o",
               str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    log = obj.with_suffix(".log")
    log.write_text(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {src}\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(f"[ferrum_b200 build] {rel}")
    stamp.write_text(key)
    return obj


def _link(objs: list[Path], out: Path, cuda: bool) -> None:
    out.parent.mkdir(parents=True, exist_ok=True)
    tmp = out.with_suffix(".so.tmp")
    if cuda:
        cmd = [NVCC, "-shared", "-o", str(tmp), *map(str, objs), "-cudart", "static", "-Xcompiler", "-fPIC",
               "-lpthread", "-ldl", "-lrt"]
    else:
        cmd = [CXX, "-shared", "-o", str(tmp), *map(str, objs), "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed: {out}\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, out)


def sources() -> tuple[list[Path], list[Path]]:
    host = sorted(p for p in (CSRC / "host").glob("*.cpp") if p.name != "selftest.cpp")
    cuda = sorted(p for p in CSRC.rglob("*") if p.suffix in (".cu", ".cpp") and (CSRC / "host") not in p.parents)
    return cuda, host


def build_bounds(verbose: bool = True, jobs: int | None = None) -> None:
    """The kernel library again with ``-DFERRUM_BOUNDS=1`` (device-side index checks that report and skip);
    loaded instead of the normal one when ``FERRUM_BOUNDS=1`` is set at import time."""
    OBJ_BOUNDS.mkdir(exist_ok=True)
    cuda_src, _ = sources()
    hdr = _headers_digest()
    jobs = jobs or min(8, os.cpu_count() or 4)
    with ThreadPoolExecutor(jobs) as ex:
        futs = [ex.submit(_compile_one, s, " ".join(NVCC_FLAGS if s.suffix == ".cu" else CXX_FLAGS), hdr, verbose,
                          True) for s in cuda_src]
        objs = [f.result() for f in futs]
    if (not CUDA_LIB_BOUNDS.exists()) or any(o.stat().st_mtime > CUDA_LIB_BOUNDS.stat().st_mtime for o in objs):
        _link(objs, CUDA_LIB_BOUNDS, cuda=True)
        if verbose:
            print(f"[ferrum_b200 build] linked {CUDA_LIB_BOUNDS.name}")


def build(verbose: bool = True, jobs: int | None = None) -> None:
    """Compile every native source for sm_100a and link the two libraries."""
    OBJ.mkdir(exist_ok=True)
    cuda_src, host_src = sources()
    hdr = _headers_digest()
    nv_key = " ".join(NVCC_FLAGS)
    cx_key = " ".join(CXX_FLAGS)
    jobs = jobs or min(8, os.cpu_count() or 4)
    with ThreadPoolExecutor(jobs) as ex:
        cuda_futs = [ex.submit(_compile_one, s, nv_key if s.suffix == ".cu" else cx_key, hdr, verbose)
                     for s in cuda_src]
        host_futs = [ex.submit(_compile_one, s, cx_key, hdr, verbose) for s in host_src]
        cuda_objs = [f.result() for f in cuda_futs]
        host_objs = [f.result() for f in host_futs]

    def newer(objs: list[Path], lib: Path) -> bool:
        return (not lib.exists()) or any(o.stat().st_mtime > lib.stat().st_mtime for o in objs)

    if cuda_objs and newer(cuda_objs, CUDA_LIB):
        _link(cuda_objs, CUDA_LIB, cuda=True)
        if verbose:
            print(f"[ferrum_b200 build] linked {CUDA_LIB.name}")
    if host_objs and newer(host_objs, HOST_LIB):
        _link(host_objs, HOST_LIB, cuda=False)
        if verbose:
            print(f"[ferrum_b200 build] linked {HOST_LIB.name}")


def build_host_selftest(out_dir, sanitizer: str = "address,undefined") -> Path:
    """Compile the host library's sources together with ``csrc/host/selftest.cpp`` under a gcc sanitizer
    (``"address,undefined"`` or ``"thread"``) into ``out_dir/selftest_<sanitizer>`` and return the path.
    The binary takes a scratch directory and a thread count; it needs no GPU."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    exe = out_dir / ("selftest_" + sanitizer.replace(",", "_"))
    srcs = [str(p) for p in sorted((CSRC / "host").glob("*.cpp"))]
    # The configured compiler may ship without the sanitizer runtimes; the system g++ is tried next.
    tried, last = [], None
    for cxx in (CXX, shutil.which("g++"), "/usr/bin/g++"):
        if not cxx or cxx in tried or shutil.which(cxx) is None:
            continue
        tried.append(cxx)
        cmd = [cxx, "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", f"-fsanitize={sanitizer}",
               "-fno-sanitize-recover=all", "-pthread", *srcs, "-o", str(exe)]
        last = subprocess.run(cmd, capture_output=True, text=True)
        if last.returncode == 0:
            return exe
        if "sanitize" not in last.stderr and "asan" not in last.stderr and "tsan" not in last.stderr \
                and "ubsan" not in last.stderr:
            break  # a genuine compile error, not a missing runtime
    missing = last is not None and any(k in last.stderr for k in ("-lasan", "-ltsan", "-lubsan", "preinit"))
    err = SanitizerUnavailable if missing else RuntimeError
    raise err(f"self-test build failed with {tried}\n{last.stdout if last else ''}\n{last.stderr if last else ''}")


class SanitizerUnavailable(RuntimeError):
    """No compiler on this machine can link the requested sanitizer runtime."""


def ptxas_report() -> str:
    """Registers / spills / shared memory per kernel, as printed by ``-Xptxas -v``."""
    out = []
    for log in sorted(OBJ.glob("*.log")):
        txt = log.read_text()
        if "ptxas info" in txt:
            out.append(f"== {log.stem}")
            out.extend(l for l in txt.splitlines() if "ptxas info" in l and ("Used" in l or "Compiling" in l
                                                                           or "spill" in l))
    return "\n".join(out)


if __name__ == "__main__":
    build(verbose=True)
    if os.environ.get("FERRUM_BOUNDS") == "1" or "--bounds" in sys.argv:
        build_bounds(verbose=True)
    if "--ptxas" in sys.argv:
        print(ptxas_report())
