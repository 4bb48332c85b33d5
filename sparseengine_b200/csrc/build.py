"""Compile the CUDA sources of this folder for sm_100a and load them as one library.

There is no install step: the first call compiles what is stale (one ``nvcc`` process
per source, in parallel) into ``_build/`` beside the sources and links
``libsparseengine_b200.so``; later calls find the objects by the hash of their source
and flags.  The sources use no framework headers, so a cold build takes well under a
minute.  If the package folder is not writable the build goes to a per-user folder
under the system's temporary directory.  There is no fallback: if the library cannot
be built or loaded, importing the ops raises.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor

_HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
                           "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]
NVCC_FLAGS += os.environ.get("SPARSEENGINE_NVCC_FLAGS", "").split()     # e.g. -D switches for experiments
LIB_NAME = "libsparseengine_b200.so"

_lock = threading.Lock()
_lib = None


def _say(msg: str) -> None:
    print(f"[sparseengine_b200] {msg}", file=sys.stderr, flush=True)


def sources() -> list[str]:
    return sorted(f for f in os.listdir(_HERE) if f.endswith(".cu"))


def _headers_digest() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(_HERE)):
        if f.endswith((".cuh", ".h")):
            with open(os.path.join(_HERE, f), "rb") as fh:
                h.update(f.encode() + b"\0" + fh.read())
    return h.hexdigest()


def find_nvcc() -> str:
    for cand in (os.environ.get("SPARSEENGINE_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise RuntimeError("nvcc not found (set CUDA_HOME or SPARSEENGINE_NVCC); the CUDA kernels "
                       "of sparseengine_b200 have to be compiled and there is no fallback")


def build_dir() -> str:
    want = os.environ.get("SPARSEENGINE_BUILD_DIR") or os.path.join(_HERE, "_build")
    try:
        os.makedirs(want, exist_ok=True)
        probe = os.path.join(want, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return want
    except OSError:
        alt = os.path.join(tempfile.gettempdir(), f"sparseengine_b200_build_{os.getuid()}")
        os.makedirs(alt, exist_ok=True)
        return alt


def _object_name(src: str, hdr: str) -> str:
    with open(os.path.join(_HERE, src), "rb") as f:
        digest = hashlib.sha256(f.read() + hdr.encode() + " ".join(NVCC_FLAGS).encode()).hexdigest()[:16]
    return f"{os.path.splitext(src)[0]}.{digest}.o"


def _compile_one(nvcc: str, src: str, obj: str) -> None:
    tmp = f"{obj}.tmp{os.getpid()}"
    cmd = [nvcc, *NVCC_FLAGS, "-I", _HERE, "-c", os.path.join(_HERE, src), "-o", tmp]
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    r = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, obj)


def build(verbose: bool = True) -> str:
    """Compile stale sources, link, return the library's path."""
    out = build_dir()
    hdr = _headers_digest()
    srcs = sources()
    objs = [os.path.join(out, _object_name(s, hdr)) for s in srcs]
    stale = [(s, o) for s, o in zip(srcs, objs) if not os.path.isfile(o)]
    link_digest = hashlib.sha256("\n".join(os.path.basename(o) for o in objs).encode()).hexdigest()[:16]
    lib = os.path.join(out, LIB_NAME)
    stamp = os.path.join(out, "link.stamp")
    linked = os.path.isfile(lib) and os.path.isfile(stamp) and open(stamp).read().strip() == link_digest
    if not stale and linked:
        return lib
    nvcc = find_nvcc()
    if stale:
        t0 = time.time()
        if verbose:
            _say(f"compiling {len(stale)} CUDA source(s) for sm_100a into {out} (first use only)")
        done = 0
        with ThreadPoolExecutor(max_workers=min(len(stale), os.cpu_count() or 4)) as pool:
            futs = {pool.submit(_compile_one, nvcc, s, o): s for s, o in stale}
            pending = set(futs)
            while pending:
                finished = {f for f in pending if f.done()}
                for f in finished:
                    f.result()
                    done += 1
                    if verbose:
                        _say(f"  compiled {futs[f]} ({done}/{len(stale)}, {time.time() - t0:.0f}s)")
                pending -= finished
                if pending:
                    time.sleep(0.5)
                    if verbose and int(time.time() - t0) % 10 == 0 and time.time() - t0 > 9.5:
                        _say(f"  still compiling ({len(pending)} left, {time.time() - t0:.0f}s)")
                        time.sleep(0.6)
    tmp = f"{lib}.tmp{os.getpid()}"
    cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    with open(stamp, "w") as f:
        f.write(link_digest)
    for f in os.listdir(out):   # drop objects of older source versions
        if f.endswith(".o") and os.path.join(out, f) not in objs:
            try:
                os.remove(os.path.join(out, f))
            except OSError:
                pass
    if verbose:
        _say(f"linked {lib}")
    return lib


def load() -> ctypes.CDLL:
    """Build if needed and load the library (once per process)."""
    global _lib
    with _lock:
        if _lib is None:
            _lib = ctypes.CDLL(build(), mode=ctypes.RTLD_GLOBAL)
        return _lib
