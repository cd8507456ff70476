"""Compiles the CUDA sources of ``csrc/`` for sm_100a into one shared library.

The library is plain CUDA with ``extern "C"`` launchers (no Python or torch headers),
so a build takes seconds per file.  It is built at the first call that needs it and
kept beside the package under ``_build/``, named by a hash of the sources and flags;
when that folder cannot be written (a read-only install) a per-user folder under the
system's temporary directory is used.  While it compiles it prints a line per file to
standard error.
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

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir, "csrc")
CSRC = os.path.normpath(CSRC)

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("TIS_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $TIS_NVCC, PATH and /usr/local/cuda/bin): the CUDA kernels of "
                     "this engine have to be compiled and there is no other implementation to fall back to")


#: sources compiled once per head size (-DTIS_HD=<hd>) into libraries of their own
PER_HEAD_SIZE = ("attention_mma.cu", "attention_tc.cu")


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu") and f not in PER_HEAD_SIZE)


def _digest() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_root() -> str:
    pkg = os.path.normpath(os.path.join(CSRC, os.pardir, "_build"))
    try:
        os.makedirs(pkg, exist_ok=True)
        probe = os.path.join(pkg, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return pkg
    except OSError:
        alt = os.path.join(tempfile.gettempdir(), f"tis_build_{os.getuid()}")
        os.makedirs(alt, exist_ok=True)
        return alt


def library_path() -> str:
    return os.path.join(_build_root(), f"libtis_kernels_{_digest()}.so")


def _say(msg: str) -> None:
    print(f"[tiny_inference_server_b200] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: str, obj: str, defines=()) -> None:
    t0 = time.time()
    cmd = [nvcc, *NVCC_FLAGS, *defines, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise BuildError(f"nvcc failed on {src}:\n{p.stdout}\n{p.stderr}")
    _say(f"compiled {src} ({time.time() - t0:.1f} s)")


def build(verbose: bool = True) -> str:
    """Build the library if it is not there yet; return its path."""
    out = library_path()
    if os.path.isfile(out):
        return out
    nvcc = _nvcc()
    root = os.path.dirname(out)
    work = tempfile.mkdtemp(prefix="tis_obj_", dir=root)
    try:
        srcs = sources()
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out} (first call only)")
        objs = [os.path.join(work, s[:-3] + ".o") for s in srcs]
        with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
            list(ex.map(lambda so: _compile_one(nvcc, *so), zip(srcs, objs)))
        tmp_so = os.path.join(work, "lib.so")
        p = subprocess.run([nvcc, "-shared", "-o", tmp_so, *objs], capture_output=True, text=True)
        if p.returncode != 0:
            raise BuildError(f"link failed:\n{p.stdout}\n{p.stderr}")
        os.replace(tmp_so, out)       # atomic: a concurrent builder ends with the same file
        _say("library ready")
    finally:
        shutil.rmtree(work, ignore_errors=True)
    return out


def attention_library_path(head_dim: int) -> str:
    return os.path.join(_build_root(), f"libtis_attn_hd{head_dim}_{_digest()}.so")


def build_attention(head_dim: int) -> str:
    """The tensor-core attention kernels for one head size (what a model needs is compiled
    when the model first runs)."""
    if head_dim % 16 or not (16 <= head_dim <= 256):
        raise BuildError(f"head size {head_dim}: the attention kernels take multiples of 16 from 16 to 256")
    out = attention_library_path(head_dim)
    if os.path.isfile(out):
        return out
    nvcc = _nvcc()
    root = os.path.dirname(out)
    work = tempfile.mkdtemp(prefix="tis_obj_", dir=root)
    try:
        _say(f"compiling the attention kernels for head size {head_dim} (first call only)")
        jobs = [(src, os.path.join(work, src[:-3] + ".o"), (f"-DTIS_HD={head_dim}",)) for src in PER_HEAD_SIZE]
        jobs.append(("errors.cu", os.path.join(work, "errors.o"), ()))
        with ThreadPoolExecutor(max_workers=len(jobs)) as ex:
            list(ex.map(lambda j: _compile_one(nvcc, *j), jobs))
        tmp_so = os.path.join(work, "lib.so")
        p = subprocess.run([nvcc, "-shared", "-o", tmp_so, *[j[1] for j in jobs]], capture_output=True, text=True)
        if p.returncode != 0:
            raise BuildError(f"link failed:\n{p.stdout}\n{p.stderr}")
        os.replace(tmp_so, out)
    finally:
        shutil.rmtree(work, ignore_errors=True)
    return out
