"""Builds the kernel library with nvcc for sm_100a and loads it with ctypes.

The sources are plain CUDA with `extern "C"` entry points (no torch headers), so a
cold build is a handful of nvcc processes run side by side.  The library lands in
`csrc/_build/` inside the package when that folder can be written, else in a per-user
folder under the system temp directory; a stamp of the source hashes decides whether a
rebuild is needed.  There is no fallback: if the library cannot be built or loaded the
import of any kernel raises `KernelBuildError`.
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
from pathlib import Path

CSRC = Path(__file__).resolve().parent
SOURCES = ["elementwise.cu", "norm.cu", "rope_cache.cu", "attention.cu", "sampling.cu",
           "linear_small.cu", "linear_tma.cu", "linear_tc5.cu", "attention_mma.cu", "attention_mma_odd.cu",
           "attention_mma_prefill.cu", "attention_tc5.cu", "attention_decode_tma.cu", "device_error.cu"]
HEADERS = ["common.cuh", "no_alloc.h", "tensor_map.h", "attention_decode.cuh", "attention_mma.cuh", "device_error.h"]
LIB_NAME = "libmll_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr"]


class KernelBuildError(RuntimeError):
    pass


def _say(message: str) -> None:
    print(f"[cpp_minilamma_b200] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            candidates.append(Path(os.environ[var]) / "bin" / "nvcc")
    candidates.append(Path("/usr/local/cuda/bin/nvcc"))
    for c in candidates:
        if c.is_file():
            return str(c)
    found = shutil.which("nvcc")
    if found:
        return found
    raise KernelBuildError("nvcc not found (looked in CUDA_HOME, /usr/local/cuda/bin and PATH); "
                           "the kernels cannot be built and there is no fallback")


def existing_sources():
    return [s for s in SOURCES if (CSRC / s).is_file()]


def source_stamp() -> str:
    digest = hashlib.sha256()
    for name in HEADERS + existing_sources():
        digest.update(name.encode())
        digest.update((CSRC / name).read_bytes())
    digest.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return digest.hexdigest()


def _writable_dir(path: Path) -> bool:
    try:
        path.mkdir(parents=True, exist_ok=True)
        probe = path / f".probe_{os.getpid()}"
        probe.write_text("x")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    override = os.environ.get("MLL_BUILD_DIR")
    if override:
        path = Path(override)
        if not _writable_dir(path):
            raise KernelBuildError(f"MLL_BUILD_DIR={override} cannot be written")
        return path
    in_tree = CSRC / "_build"
    if _writable_dir(in_tree):
        return in_tree
    fallback = Path(tempfile.gettempdir()) / f"cpp_minilamma_b200_build_{os.getuid()}"
    if _writable_dir(fallback):
        return fallback
    raise KernelBuildError(f"neither {in_tree} nor {fallback} can be written; nowhere to build the kernels")


def _compile_one(nvcc, src: Path, obj: Path, verbose_ptxas: bool, errors: list) -> None:
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose_ptxas:
        cmd.insert(1, "-Xptxas=-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        errors.append(f"{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    elif verbose_ptxas:
        (obj.parent / (obj.stem + ".ptxas.txt")).write_text(proc.stderr)


def build(force: bool = False, verbose_ptxas: bool = False) -> Path:
    """Compile (if needed) and return the path of the shared library."""
    out_dir = build_dir()
    lib = out_dir / LIB_NAME
    stamp_file = out_dir / "stamp.txt"
    stamp = source_stamp()
    if not force and lib.is_file() and stamp_file.is_file() and stamp_file.read_text().strip() == stamp:
        return lib
    nvcc = find_nvcc()
    sources = existing_sources()
    _say(f"building {len(sources)} CUDA sources for sm_100a into {out_dir} (first call only)")
    started = time.time()
    errors: list = []
    threads = []
    objects = []
    for name in sources:
        obj = out_dir / (Path(name).stem + ".o")
        objects.append(obj)
        t = threading.Thread(target=_compile_one, args=(nvcc, CSRC / name, obj, verbose_ptxas, errors))
        t.start()
        threads.append(t)
    while any(t.is_alive() for t in threads):
        for t in threads:
            t.join(timeout=10.0 / len(threads))
        if any(t.is_alive() for t in threads):
            alive = sum(t.is_alive() for t in threads)
            _say(f"  still compiling: {alive} of {len(threads)} files, {time.time() - started:.0f} s")
    if errors:
        raise KernelBuildError("nvcc failed:\n" + "\n".join(errors))
    tmp_lib = out_dir / f".{LIB_NAME}.{os.getpid()}"
    link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp_lib), *map(str, objects), "-lcudart"]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise KernelBuildError(f"link failed: {' '.join(link)}\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp_lib, lib)
    stamp_file.write_text(stamp + "\n")
    _say(f"kernels built in {time.time() - started:.0f} s")
    return lib


_LIB = None
_LOCK = threading.Lock()


def load_library() -> ctypes.CDLL:
    """Build if needed, load once, and return the ctypes handle."""
    global _LIB
    with _LOCK:
        if _LIB is None:
            path = build()
            try:
                _LIB = ctypes.CDLL(str(path))
            except OSError as exc:
                raise KernelBuildError(f"cannot load {path}: {exc}") from None
        return _LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose_ptxas="--ptxas" in sys.argv))
