"""Compile the CUDA sources under ``csrc/`` for sm_100a into one shared library.

The reference compiles its ``.cu`` files at run time through NVRTC and keeps a PTX cache
on disk (crates/cuda/src/nvrtc.rs:27-120).  Here ``nvcc`` builds a shared library the
first time it is needed and whenever a source changes; the library lives beside the
sources (``csrc/_build``), or under the system temporary folder when the checkout is not
writable.  A line is printed for every file so a first call is not silent.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
LIB_NAME = "libinfero_b200.so"


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[infero_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    cands = [os.environ.get("INFERO_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"]
    for c in cands:
        if c and os.path.exists(c):
            return c
    raise BuildError("nvcc not found (looked at $INFERO_NVCC, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels cannot be built and there is no other path")


def sources() -> List[str]:
    """CUDA files, and plain C++ files of the host side (nvcc hands those to the host compiler)."""
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def source_digest(extra: str = "") -> str:
    h = hashlib.sha256()
    for f in sources() + _headers():
        h.update(f.encode())
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + COMMON_FLAGS).encode())
    h.update(extra.encode())
    return h.hexdigest()[:16]


def variant_defines() -> List[str]:
    """INFERO_TIMELINE=1 builds the variant whose kernels log when each of their blocks ran
    (tools/timeline.py); it lives in a build folder of its own beside the ordinary library."""
    return ["-DINFERO_TIMELINE"] if os.environ.get("INFERO_TIMELINE", "0") == "1" else []


def build_dir() -> str:
    """A folder this user can write: csrc/_build, else a per-user folder under the temp dir."""
    env = os.environ.get("INFERO_BUILD_DIR")
    suffix = "_timeline" if variant_defines() else ""
    cands = [env + suffix] if env else []
    cands.append(os.path.join(CSRC, "_build" + suffix))
    cands.append(os.path.join(tempfile.gettempdir(), f"infero_b200_build{suffix}_{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}")
            with open(probe, "w") as fh:
                fh.write("x")
            os.remove(probe)
            return d
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {cands}")


def _compile_one(nvcc: str, src: str, obj: str, defines: List[str]) -> None:
    cmd = [nvcc] + ARCH_FLAGS + COMMON_FLAGS + defines + ["-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"nvcc failed on {src}:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")


def ensure_built(verbose: bool = True) -> str:
    """Return the path of an up-to-date shared library, compiling what is stale."""
    d = build_dir()
    defines = variant_defines()
    digest = source_digest(" ".join(defines))
    lib = os.path.join(d, LIB_NAME)
    stamp = os.path.join(d, "digest.txt")
    if os.path.exists(lib) and os.path.exists(stamp):
        with open(stamp) as fh:
            if fh.read().strip() == digest:
                return lib
    nvcc = find_nvcc()
    srcs = sources()
    t0 = time.time()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {d} (first call or sources changed)")
    objs = []
    jobs = []
    workers = max(1, min(len(srcs), (os.cpu_count() or 2)))
    with ThreadPoolExecutor(max_workers=workers) as ex:
        for s in srcs:
            with open(os.path.join(CSRC, s), "rb") as fh:
                sh = hashlib.sha256(fh.read() + digest.encode()).hexdigest()[:12]
            obj = os.path.join(d, f"{os.path.splitext(s)[0]}.{sh}.o")
            objs.append(obj)
            if os.path.exists(obj):
                continue
            jobs.append((ex.submit(_compile_one, nvcc, s, obj + f".tmp{os.getpid()}.o", defines), s, obj))
        done = 0
        for fut, s, obj in [(j[0], j[1], j[2]) for j in jobs]:
            fut.result()
            os.replace(obj + f".tmp{os.getpid()}.o", obj)
            done += 1
            if verbose:
                _say(f"  {s} done ({done}/{len(jobs)}, {time.time() - t0:.0f}s)")
    tmp = lib + f".tmp{os.getpid()}"
    cmd = [nvcc] + ARCH_FLAGS + ["-shared", "-o", tmp] + objs
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"link failed:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    with open(stamp, "w") as fh:
        fh.write(digest)
    # drop objects of older source versions
    keep = set(objs)
    for f in os.listdir(d):
        p = os.path.join(d, f)
        if f.endswith(".o") and p not in keep:
            try:
                os.remove(p)
            except OSError:
                pass
    if verbose:
        _say(f"built {lib} in {time.time() - t0:.0f}s")
    return lib
