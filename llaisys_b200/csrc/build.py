"""Compiles the CUDA modules of this package for sm_100a and loads them with ctypes.

A module is one `.cu` file of this folder plus a set of -D definitions (the attention kernels
are compiled per head size).  Its shared library is cached under `_build/` beside the sources,
or, where that folder cannot be written, under a per-user folder in the system's temporary
directory; the cache key covers the sources, the headers, the definitions and the flags, so a
changed file is rebuilt.  Only what a model asks for is compiled, at its first use, and a line
is printed to stderr for every compilation so that a first call does not look hung.
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

SRC_DIR = Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr", "--extended-lambda"]

_lock = threading.RLock()
_loaded: dict[str, ctypes.CDLL] = {}
_loaded_fast: dict = {}      # (source, definitions) -> handle, found without forming the module name


class BuildError(RuntimeError):
    pass


def page_tokens() -> int:
    """Tokens of a cache page: the one constant LLB_PAGE of common.cuh, read from the source so that
    the host side and the kernels cannot disagree."""
    import re
    m = re.search(r"constexpr\s+int\s+LLB_PAGE\s*=\s*(\d+)\s*;", (SRC_DIR / "common.cuh").read_text())
    if not m:
        raise BuildError("common.cuh does not define LLB_PAGE")
    return int(m.group(1))


def find_nvcc() -> str:
    for cand in (os.environ.get("LLAISYS_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise BuildError("nvcc not found (set LLAISYS_NVCC or put the CUDA toolkit on PATH); "
                     "the CUDA kernels of llaisys_b200 cannot be built")


_build_dir_cache = None


def _build_dir() -> Path:
    global _build_dir_cache
    with _lock:
        if _build_dir_cache is None:
            _build_dir_cache = _find_build_dir()
        return _build_dir_cache


def _find_build_dir() -> Path:
    override = os.environ.get("LLAISYS_BUILD_DIR")
    cands = [Path(override)] if override else []
    cands.append(SRC_DIR / "_build")
    cands.append(Path(tempfile.gettempdir()) / f"llaisys_b200-build-{os.getuid()}")
    for d in cands:
        try:
            d.mkdir(parents=True, exist_ok=True)
            with tempfile.NamedTemporaryFile(dir=d, prefix=".probe"):
                pass
            return d
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {[str(c) for c in cands]}")


def _tag(source: str, defines: dict) -> str:
    h = hashlib.sha256()
    for f in [SRC_DIR / source, *sorted(SRC_DIR.glob("*.cuh"))]:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(repr(sorted(defines.items())).encode())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def module_name(source: str, defines: dict | None = None) -> str:
    defines = defines or {}
    stem = Path(source).stem
    suffix = "".join(f"_{k.lower().replace('llb_', '')}{v}" for k, v in sorted(defines.items()))
    return f"{stem}{suffix}"


def compile_module(source: str, defines: dict | None = None, verbose: bool = True) -> Path:
    """Builds (if needed) and returns the shared library of `source` with `defines`."""
    defines = defines or {}
    name = module_name(source, defines)
    out_dir = _build_dir()
    so = out_dir / f"libllb_{name}.{_tag(source, defines)}.so"
    if so.exists():
        return so
    nvcc = find_nvcc()
    tmp = so.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *[f"-D{k}={v}" for k, v in sorted(defines.items())],
           f"-I{SRC_DIR}", str(SRC_DIR / source), "-o", str(tmp)]
    if verbose:
        print(f"[llaisys_b200] compiling {name} for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            out, _ = proc.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[llaisys_b200] ... still compiling {name} ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise BuildError(f"nvcc failed for {name}:\n{' '.join(cmd)}\n{out}")
    os.replace(tmp, so)
    for old in out_dir.glob(f"libllb_{name}.*.so"):       # superseded builds of this module
        if old != so and ".tmp" not in old.name:
            old.unlink(missing_ok=True)
    if verbose:
        print(f"[llaisys_b200] compiled {name} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return so


def load_module(source: str, defines: dict | None = None) -> ctypes.CDLL:
    """The ctypes handle of a module, compiling it first if its library is missing or stale."""
    fast = (source, tuple(sorted(defines.items())) if defines else ())
    lib = _loaded_fast.get(fast)
    if lib is not None:
        return lib
    key = module_name(source, defines)
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            lib = ctypes.CDLL(str(compile_module(source, defines)))
            _loaded[key] = lib
        _loaded_fast[fast] = lib
        return lib


# The modules that serving the usual head sizes (64 and 128) needs, in both precisions.  Any other
# head size is compiled when a model first asks for it; tests name the sizes they need themselves.
DEFAULT_MODULES = [
    ("basic.cu", {}), ("gemm_simt.cu", {}), ("gemm_tc.cu", {}), ("gemm_tc2.cu", {}), ("mlp_tc.cu", {}), ("sampling.cu", {}), ("random_init.cu", {}),
    *[("attention_simt.cu", {"LLB_HEAD_DIM": d}) for d in (64, 128)],
    *[("attention_mma.cu", {"LLB_HEAD_DIM": d}) for d in (64, 128)],
    *[("attention_tc.cu", {"LLB_HEAD_DIM": d}) for d in (64, 128)],
]


# Builds with cycle stamps (bench.py --stamps): the three kernels of a decode step that carry them.
STAMP_MODULES = [("gemm_tc.cu", {"LLB_STAMPS": 1}), ("gemm_tc2.cu", {"LLB_STAMPS": 1}), ("mlp_tc.cu", {"LLB_STAMPS": 1}),
                 ("attention_mma.cu", {"LLB_HEAD_DIM": 128, "LLB_STAMPS": 1})]


def build_all(modules=None, jobs: int | None = None) -> list[Path]:
    from concurrent.futures import ThreadPoolExecutor
    modules = modules or DEFAULT_MODULES
    with ThreadPoolExecutor(max_workers=jobs or min(8, os.cpu_count() or 1)) as ex:
        return list(ex.map(lambda m: compile_module(*m), modules))


if __name__ == "__main__":
    for p in build_all():
        print(p)
