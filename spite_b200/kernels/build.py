"""Compile the CUDA sources under `spite_b200/csrc` into shared libraries for
sm_100a and load them with ctypes.

One library per source file, built in-tree under `csrc/_build/` at first use and
reused while the sources (and the flags) are unchanged.  Only what a model asks
for is compiled.  There is no fallback: if a library is neither built nor
buildable, the call raises.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import threading
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
BUILD_DIR = CSRC / "_build"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

#: library name -> source files (relative to csrc/), extra flags
LIBRARIES = {
    "elementwise": (["elementwise.cu"], []),
    "gemm_simt": (["gemm_simt.cu"], []),
    "gemm_skinny": (["gemm_skinny.cu"], []),
    "gemm_tc": (["gemm_tc.cu"], []),
    "gemm_tc_pair": (["gemm_tc_pair.cu"], []),
    "gemm_tc_experts": (["gemm_tc_experts.cu"], []),
    "gemm_stream": (["gemm_stream.cu"], []),
    "attention": (["attention.cu"], []),
    "attention_mma": (["attention_mma.cu"], []),
    "attention_decode": (["attention_decode.cu"], []),
    "attention_rows": (["attention_rows.cu"], []),
    "attention_tc": (["attention_tc.cu"], []),
    "moe": (["moe.cu"], []),
    "sampling": (["sampling.cu"], []),
}

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def _nvcc() -> str | None:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    return None


def _signature(name: str) -> str:
    sources, extra = LIBRARIES[name]
    h = hashlib.sha256()
    for f in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    for s in sources:
        h.update(s.encode())
        h.update((CSRC / s).read_bytes())
    h.update(" ".join(NVCC_FLAGS + extra).encode())
    return h.hexdigest()


def library_path(name: str) -> Path:
    return BUILD_DIR / f"libspite_{name}.so"


def is_current(name: str) -> bool:
    so, sig = library_path(name), library_path(name).with_suffix(".sig")
    return so.is_file() and sig.is_file() and sig.read_text().strip() == _signature(name)


def _say(msg: str):
    print(f"[spite_b200] {msg}", file=sys.stderr, flush=True)


def _compile(name: str):
    nvcc = _nvcc()
    if nvcc is None:
        raise KernelBuildError(
            f"kernel library {name!r} is not built and nvcc was not found; "
            f"run `python -c 'import __graft_entry__ as g; g.build()'` where the CUDA toolkit is installed")
    sources, extra = LIBRARIES[name]
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    out = library_path(name)
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-o", str(tmp)] + [str(CSRC / s) for s in sources]
    _say(f"compiling {', '.join(sources)} for sm_100a")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    lines = []

    def pump():
        for line in proc.stdout:
            lines.append(line)
    reader = threading.Thread(target=pump, daemon=True)
    reader.start()
    while proc.poll() is None:
        try:
            proc.wait(timeout=10)
        except subprocess.TimeoutExpired:
            _say(f"  still compiling {name} ({time.time() - t0:.0f} s)")
    reader.join()
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise KernelBuildError(f"nvcc failed for {name}:\n{' '.join(cmd)}\n{''.join(lines)}")
    os.replace(tmp, out)
    out.with_suffix(".sig").write_text(_signature(name))
    _say(f"  built {out.name} in {time.time() - t0:.1f} s")


def ensure_built(names=None, parallel: bool = True):
    """Compile every named library that is missing or stale (all of them by default)."""
    names = list(LIBRARIES) if names is None else list(names)
    todo = [n for n in names if not is_current(n)]
    if not todo:
        return
    errors = []

    def work(n):
        try:
            _compile(n)
        except Exception as e:          # noqa: BLE001 - reported below
            errors.append(e)
    if parallel and len(todo) > 1:
        threads = [threading.Thread(target=work, args=(n,)) for n in todo]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
    else:
        for n in todo:
            work(n)
    if errors:
        raise errors[0]


def load(name: str) -> ctypes.CDLL:
    """The loaded library `name`, compiled first if needed."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            if name not in LIBRARIES:
                raise KernelBuildError(f"unknown kernel library {name!r}")
            if not is_current(name):
                _compile(name)
            lib = ctypes.CDLL(str(library_path(name)))
            _loaded[name] = lib
        return lib
