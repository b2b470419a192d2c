"""In-tree build of the native libraries.

Two artefacts land in ``eredu_b200/lib/``:

* ``liberedu_cuda.so`` - every ``csrc/kernels/*.cu`` and ``csrc/comm/*.cu`` compiled by nvcc for
  sm_100a only (``-gencode arch=compute_100a,code=sm_100a``); a C ABI (``eredu_*``) consumed through
  ctypes, the counterpart of the reference's ``mlx_*`` C shim (safemlx-sys/src/mlx-c/mlx/c/*.cpp).
* ``_eredu_host*.so`` - the host-side C++ runtime (GGUF / SafeTensors codecs, quantisers, topology
  planner, scheduler, consensus, KV block manager) as a pybind11 module; no CUDA needed.

Objects are cached by source hash so that rebuilding after an edit recompiles one file.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "_build"
LIB = ROOT / "lib"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]
# extra nvcc flags for one-off builds, e.g. EREDU_NVCC_EXTRA="-DEREDU_TRACE_FINE" for sub-step timeline marks
NVCC_FLAGS += os.environ.get("EREDU_NVCC_EXTRA", "").split()
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function", "-fvisibility=hidden"]


def _nvcc() -> str | None:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def _digest(path: Path, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    h.update(path.read_bytes())
    for inc in sorted((CSRC / "common").glob("*")):
        h.update(inc.read_bytes())
    for pattern in ("*.h", "*.hpp", "*.cuh"):      # headers that sit next to the source
        for inc in sorted(path.parent.glob(pattern)):
            h.update(inc.read_bytes())
    return h.hexdigest()[:16]


def _compile(cmd: list[str], src: Path, obj: Path, stamp: str, verbose: bool) -> tuple[Path, str]:
    stamp_file = obj.with_suffix(obj.suffix + ".stamp")
    if obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return obj, ""
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    stamp_file.write_text(stamp)
    log = proc.stderr if verbose else ""
    (obj.with_suffix(obj.suffix + ".log")).write_text(proc.stderr)
    return obj, log


def cuda_sources() -> list[Path]:
    return sorted((CSRC / "kernels").glob("*.cu")) + sorted((CSRC / "comm").glob("*.cu"))


def host_sources() -> list[Path]:
    return sorted((CSRC / "host").glob("*.cpp"))


def build_cuda(verbose: bool = False) -> Path:
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build liberedu_cuda.so")
    OBJ.mkdir(exist_ok=True)
    LIB.mkdir(exist_ok=True)
    jobs = []
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        for src in cuda_sources():
            obj = OBJ / (src.stem + ".o")
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            jobs.append(pool.submit(_compile, cmd, src, obj, _digest(src, " ".join(NVCC_FLAGS)), verbose))
        objs = []
        for j in jobs:
            obj, log = j.result()
            objs.append(obj)
            if log:
                print(log, file=sys.stderr)
    out = LIB / "liberedu_cuda.so"
    newest = max(o.stat().st_mtime for o in objs)
    if not out.exists() or out.stat().st_mtime < newest:
        cmd = [nvcc, "-shared", "-o", str(out), *map(str, objs)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed: {proc.stderr}")
    return out


def build_host(verbose: bool = False) -> Path:
    import pybind11

    if not host_sources():
        return LIB
    OBJ.mkdir(exist_ok=True)
    LIB.mkdir(exist_ok=True)
    cxx = os.environ.get("CXX", "g++")
    incs = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", str(CSRC)]
    jobs = []
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        for src in host_sources():
            obj = OBJ / ("host_" + src.stem + ".o")
            cmd = [cxx, *CXX_FLAGS, *incs, "-c", str(src), "-o", str(obj)]
            jobs.append(pool.submit(_compile, cmd, src, obj, _digest(src, " ".join(CXX_FLAGS)), verbose))
        objs = [j.result()[0] for j in jobs]
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    out = LIB / ("_eredu_host" + suffix)
    newest = max(o.stat().st_mtime for o in objs)
    if not out.exists() or out.stat().st_mtime < newest:
        cmd = [cxx, "-shared", "-o", str(out), *map(str, objs), "-lpthread"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed: {proc.stderr}")
    return out


def build_all(verbose: bool = False) -> None:
    build_host(verbose)
    build_cuda(verbose)


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv)
    print("built:", *sorted(p.name for p in LIB.iterdir()))
