"""Builds the CUDA libraries for sm_100a with nvcc and loads them with ctypes.

Sources live in `tandemllm_b200/csrc/`; each library is a list of `.cu` files compiled to objects in
parallel and linked into `csrc/_build/lib<name>-<digest>.so`, the digest taken over the sources, the
shared headers and the flags, so an edited source is rebuilt and a built one is found again (the
reference names its builds by a hash of the text too, engine/native_build.py:26-59). A library is
built at its first use, and only the libraries a run asks for are built. While nvcc runs, a line goes
to stderr for every file. There is no fallback: without nvcc and without a built library the load
fails with the reason.

The sources include no torch header, so a file compiles in seconds; tensors cross as raw pointers and
the stream as a handle.
"""

from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor

from ..settings import SETTINGS

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]

LIBRARIES: dict[str, list[str]] = {
    # every kernel of the 32-bit path, and the plain bfloat16 variants of the same kernels
    "core": ["rows.cu", "gemm_simt.cu", "conv.cu", "attention_simt.cu", "attention_split.cu", "moe_route.cu",
             "sampling.cu", "graphs.cu"],
    # the tcgen05 / TMA kernels of the bfloat16 path; a 32-bit run never builds or loads them
    "tensorcore": ["tc_gemm.cu", "tc_gemm_pair.cu", "attention_mma.cu", "attention_tc.cu", "gemm_skinny_mma.cu"],
}
HEADERS = ["common.cuh", "route.cuh", "attention_noalloc.h", "tma.cuh"]

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class ExtensionError(RuntimeError):
    """The CUDA library is missing and could not be built."""


def say(text: str) -> None:
    print(f"[tandemllm_b200] {text}", file=sys.stderr, flush=True)


def find_nvcc() -> str | None:
    for cand in (SETTINGS.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    return None


def build_dir() -> str:
    """`csrc/_build` in the tree; where the tree cannot be written, a per-user folder under the temp dir."""
    want = SETTINGS.get("BUILD_DIR") or os.path.join(CSRC, "_build")
    try:
        os.makedirs(want, exist_ok=True)
        probe = os.path.join(want, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return want
    except OSError:
        alt = os.path.join(tempfile.gettempdir(), f"tandemllm_b200-build-{os.getuid()}")
        os.makedirs(alt, exist_ok=True)
        return alt


def digest(name: str) -> str:
    h = hashlib.sha1()
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    for f in HEADERS + LIBRARIES[name]:
        h.update(f.encode())
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:12]


def library_path(name: str, folder: str | None = None) -> str:
    return os.path.join(folder or build_dir(), f"lib{name}-{digest(name)}.so")


def _compile(nvcc: str, src: str, obj: str) -> None:
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise ExtensionError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")


def build(name: str, force: bool = False) -> str:
    """Compile library `name` if its file is not there yet; returns the path of the .so."""
    folder = build_dir()
    out = library_path(name, folder)
    if os.path.isfile(out) and not force:
        return out
    nvcc = find_nvcc()
    if nvcc is None:
        raise ExtensionError(
            f"the CUDA library {os.path.basename(out)} is not built and nvcc was not found "
            "(looked at $TANDEMLLM_NVCC, PATH and /usr/local/cuda/bin/nvcc); this engine has no other path")
    with open(os.path.join(folder, f".{name}.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.isfile(out) and not force:
                return out
            srcs = LIBRARIES[name]
            tag = digest(name)
            t0 = time.time()
            say(f"building {os.path.basename(out)} for sm_100a: {len(srcs)} files with {nvcc}")
            objs = [os.path.join(folder, f"{name}-{tag}-{os.path.splitext(s)[0]}.o") for s in srcs]
            done = [0]

            def one(pair):
                src, obj = pair
                _compile(nvcc, src, obj)
                done[0] += 1
                say(f"  compiled {src} ({done[0]}/{len(srcs)}, {time.time() - t0:.0f} s)")

            with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as pool:
                list(pool.map(one, zip(srcs, objs)))
            tmp = out + f".tmp{os.getpid()}"
            r = subprocess.run([nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs], capture_output=True, text=True)
            if r.returncode != 0:
                raise ExtensionError(f"linking {out} failed:\n{r.stdout}\n{r.stderr}")
            os.replace(tmp, out)
            for old in os.listdir(folder):          # builds of earlier source texts are of no use any more
                if old.startswith(f"lib{name}-") and old.endswith(".so") and os.path.join(folder, old) != out:
                    try:
                        os.remove(os.path.join(folder, old))
                    except OSError:
                        pass
            for o in objs:
                try:
                    os.remove(o)
                except OSError:
                    pass
            say(f"built {os.path.basename(out)} in {time.time() - t0:.0f} s")
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return out


def load(name: str) -> ctypes.CDLL:
    """The loaded library `name`, built first if need be."""
    with _lock:
        if name not in _loaded:
            path = build(name)
            try:
                _loaded[name] = ctypes.CDLL(path)
            except OSError as e:
                raise ExtensionError(f"{path} could not be loaded: {e}") from None
        return _loaded[name]


def build_all() -> list[str]:
    return [build(name) for name in LIBRARIES]
