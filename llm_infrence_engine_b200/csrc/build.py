"""Builds the package's CUDA library for sm_100a with nvcc and loads it with ctypes.

The library is built at the first call that needs it and kept next to the sources (``_build/``,
which version control ignores), or in a per-user folder under the system's temporary directory
when the source tree cannot be written. Its file name carries a hash of all sources, so an edit
rebuilds and an old library is never loaded by mistake. While nvcc runs, a line goes to stderr now
and then. There is no fallback: without nvcc the error says so.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import List, Optional

HERE = Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

_lib: Optional[ctypes.CDLL] = None
_lib_path: Optional[Path] = None


class BuildError(RuntimeError):
    pass


def sources() -> List[Path]:
    return sorted(HERE.glob("*.cu"))


def _headers() -> List[Path]:
    return sorted(HERE.glob("*.cuh")) + sorted(HERE.glob("*.h"))


def _digest() -> str:
    h = hashlib.sha256()
    for p in sources() + _headers():
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def find_nvcc() -> str:
    for cand in (os.environ.get("LLMIE_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $LLMIE_NVCC, PATH, $CUDA_HOME/bin and /usr/local/cuda/bin); "
                     "the kernels of this package have no other implementation")


def _build_dirs() -> List[Path]:
    dirs = []
    if os.environ.get("LLMIE_BUILD_DIR"):
        dirs.append(Path(os.environ["LLMIE_BUILD_DIR"]))
    dirs.append(HERE / "_build")
    dirs.append(Path(tempfile.gettempdir()) / f"llm_infrence_engine_b200_build_{os.getuid()}")
    return dirs


def _writable(d: Path) -> bool:
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".probe_{os.getpid()}"
        probe.write_text("x")
        probe.unlink()
        return True
    except OSError:
        return False


def _say(msg: str) -> None:
    print(f"[llm_infrence_engine_b200] {msg}", file=sys.stderr, flush=True)


def library_path(build: bool = True) -> Path:
    """The path of the built library; builds it first if it is not there yet."""
    name = f"libllmie_kernels_{_digest()}.so"
    for d in _build_dirs():
        if (d / name).is_file():
            return d / name
    if not build:
        raise BuildError(f"{name} has not been built")
    out_dir = next((d for d in _build_dirs() if _writable(d)), None)
    if out_dir is None:
        raise BuildError("no writable folder for the CUDA library (tried " + ", ".join(map(str, _build_dirs())) + ")")
    nvcc = find_nvcc()
    srcs = sources()
    work = Path(tempfile.mkdtemp(prefix="obj_", dir=out_dir))
    _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out_dir} (first call only) ...")
    t0 = time.time()

    def compile_one(src: Path) -> Path:
        obj = work / (src.stem + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(HERE), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
        return obj

    try:
        with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as pool:
            futures = [pool.submit(compile_one, s) for s in srcs]
            while True:
                done = sum(f.done() for f in futures)
                if done == len(futures):
                    break
                time.sleep(1.0)
                if int(time.time() - t0) % 10 == 0:
                    _say(f"... still compiling ({int(time.time() - t0)} s, {done} of {len(futures)} files done)")
            objs = [f.result() for f in futures]
        tmp = work / name
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *map(str, objs), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"linking the CUDA library failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, out_dir / name)
        for old in out_dir.glob("libllmie_kernels_*.so"):  # libraries of earlier source states are never loaded again
            if old.name != name:
                old.unlink(missing_ok=True)
    finally:
        shutil.rmtree(work, ignore_errors=True)
    _say(f"built {name} in {time.time() - t0:.0f} s")
    return out_dir / name


def load_library() -> ctypes.CDLL:
    global _lib, _lib_path
    if _lib is None:
        _lib_path = library_path()
        _lib = ctypes.CDLL(str(_lib_path))
    return _lib


def loaded_path() -> Optional[Path]:
    return _lib_path
