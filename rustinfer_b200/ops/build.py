"""Compiling the CUDA sources for sm_100a, in the tree, when they are first needed.

Each library is one `nvcc -shared` of a few `.cu` files of `csrc/` (no torch headers, so a
library builds in seconds) and lands in `rustinfer_b200/_build/`.  A stamp beside it holds a
hash of sources and flags; a library is rebuilt only when that changes.  Only what a model
needs is built: the attention kernels are compiled for the one head size in use.  There
is no fallback: if nvcc is missing or a source does not compile, the error is raised.

RustInfer compiles its kernels ahead of time from build.rs for a detected architecture
(crates/infer-backend-cuda/build.rs:122-153); this engine targets sm_100a alone.
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import Iterable, Optional, Sequence

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[rustinfer_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("RUSTINFER_B200_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $RUSTINFER_B200_NVCC, PATH, $CUDA_HOME/bin, "
                     "/usr/local/cuda/bin); the sm_100a kernels cannot be built and there is no fallback")


def build_dir() -> str:
    """`rustinfer_b200/_build` when it can be written, else a per-user folder under the
    system's temporary directory."""
    override = os.environ.get("RUSTINFER_B200_BUILD_DIR")
    cands = [override] if override else []
    cands.append(os.path.join(os.path.dirname(CSRC), "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"rustinfer_b200_build_{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".probe_{os.getpid()}")
            with open(probe, "w"):
                pass
            os.unlink(probe)
            return d
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {cands}")


def _digest(sources: Sequence[str], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cuh", ".h")):
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(f.encode()); h.update(fh.read())
    for s in sources:
        with open(os.path.join(CSRC, s), "rb") as fh:
            h.update(s.encode()); h.update(fh.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:24]


def build_library(name: str, sources: Sequence[str], defines: Iterable[str] = (),
                  extra_flags: Iterable[str] = (), libs: Iterable[str] = ()) -> str:
    """Path of `lib<name>.so`, compiled now if it is absent or stale."""
    flags = ARCH_FLAGS + BASE_FLAGS + [f"-D{d}" for d in defines] + list(extra_flags)
    link = [f"-l{l}" for l in libs]
    want = _digest(sources, flags + link)
    bdir = build_dir()
    out = os.path.join(bdir, f"lib{name}.so")
    stamp = out + ".stamp"

    def fresh() -> bool:
        try:
            with open(stamp) as f:
                return os.path.isfile(out) and f.read().strip() == want
        except OSError:
            return False

    if fresh():
        return out
    nvcc = find_nvcc()
    with open(os.path.join(bdir, f".{name}.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if fresh():                                   # another process built it meanwhile
                return out
            tmp = os.path.join(bdir, f".lib{name}.{os.getpid()}.so")
            cmd = [nvcc] + flags + ["-I", CSRC, "-o", tmp] + [os.path.join(CSRC, s) for s in sources] + link
            _say(f"compiling {name} ({', '.join(sources)}) for sm_100a ...")
            t0 = time.time()
            env = dict(os.environ)
            env.setdefault("TMPDIR", tempfile.gettempdir())
            proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env, text=True)
            nxt = 10.0
            while True:
                try:
                    log, _ = proc.communicate(timeout=1.0)
                    break
                except subprocess.TimeoutExpired:
                    if time.time() - t0 >= nxt:
                        _say(f"... still compiling {name} ({time.time() - t0:.0f} s)")
                        nxt += 10.0
            if proc.returncode != 0:
                if os.path.exists(tmp):
                    os.unlink(tmp)
                raise BuildError(f"nvcc failed for {name} (exit {proc.returncode}):\n{' '.join(cmd)}\n{log}")
            os.replace(tmp, out)
            with open(stamp, "w") as f:
                f.write(want)
            _say(f"compiled {name} in {time.time() - t0:.1f} s")
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return out
