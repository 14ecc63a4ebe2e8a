"""In-tree native build: nvcc for the sm_100a kernel library, g++ for the host runtime library.

Two shared objects are produced next to this file:
  * ``libsllm_b200_kernels.so`` - every ``csrc/*.cu`` translation unit (CUDA kernels + launchers)
  * ``libsllm_b200_host.so``    - every ``csrc/host/*.cpp`` translation unit (page pool, grammar,
    sampler chain, batch planner; no CUDA dependency, usable on a GPU-less machine)

Objects are rebuilt only when their source (or a header) is newer.  nvcc cross-compiles for
sm_100a without a GPU.  The role matches the reference's CMake + build.rs pair
(native/hip/CMakeLists.txt:245-266, crates/sllm-hip-sys/build.rs), with one exact target.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "build"
KERNEL_LIB = ROOT / "libsllm_b200_kernels.so"
HOST_LIB = ROOT / "libsllm_b200_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wextra", "-Werror", "-pthread"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the kernel library cannot be built")
    return exe


def _newest_header() -> float:
    hs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((CSRC / "host").glob("*.h"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _stale(src: Path, obj: Path, hdr_time: float) -> bool:
    return (not obj.exists()) or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("build step failed: " + " ".join(cmd))
    if proc.stderr.strip() and os.environ.get("SLLM_BUILD_VERBOSE"):
        sys.stderr.write(proc.stderr)


def _source_hash(files) -> str:
    import hashlib
    h = hashlib.sha256()
    for f in sorted(files):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def _up_to_date(lib: Path, files) -> bool:
    """True when `lib` was built from exactly these sources (content hash, robust to copied trees
    whose mtimes were not preserved)."""
    tag = lib.with_suffix(".so.srchash")
    return lib.exists() and tag.exists() and tag.read_text().strip() == _source_hash(files)


def _stamp(lib: Path, files) -> None:
    lib.with_suffix(".so.srchash").write_text(_source_hash(files))


def build_kernels(force: bool = False, verbose_ptxas: bool = False) -> Path:
    srcs = sorted(CSRC.glob("*.cu"))
    deps = srcs + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    if not force and not verbose_ptxas and _up_to_date(KERNEL_LIB, deps):
        return KERNEL_LIB
    OBJ.mkdir(exist_ok=True)
    hdr = _newest_header()
    jobs = []
    for s in srcs:
        o = OBJ / (s.stem + ".o")
        if force or _stale(s, o, hdr):
            cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(s), "-o", str(o)]
            if verbose_ptxas:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(_run, jobs))
    objs = [str(OBJ / (s.stem + ".o")) for s in srcs]
    if jobs or not KERNEL_LIB.exists():
        _run([_nvcc(), "-shared", "-o", str(KERNEL_LIB), *objs, "-lcudart"])
    _stamp(KERNEL_LIB, deps)
    return KERNEL_LIB


def build_host(force: bool = False) -> Path:
    srcs = sorted((CSRC / "host").glob("*.cpp"))
    if not srcs:
        return HOST_LIB
    deps = srcs + sorted((CSRC / "host").glob("*.h"))
    if not force and _up_to_date(HOST_LIB, deps):
        return HOST_LIB
    OBJ.mkdir(exist_ok=True)
    hdr = _newest_header()
    cxx = shutil.which("g++") or "g++"
    jobs = []
    for s in srcs:
        o = OBJ / ("host_" + s.stem + ".o")
        if force or _stale(s, o, hdr):
            jobs.append([cxx, *CXX_FLAGS, "-I", str(CSRC), "-c", str(s), "-o", str(o)])
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(_run, jobs))
    objs = [str(OBJ / ("host_" + s.stem + ".o")) for s in srcs]
    if jobs or not HOST_LIB.exists():
        _run([cxx, "-shared", "-pthread", "-o", str(HOST_LIB), *objs])
    _stamp(HOST_LIB, deps)
    return HOST_LIB


def build_all(force: bool = False) -> None:
    build_host(force)
    build_kernels(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    if "--ptxas" in sys.argv:
        build_kernels(force=True, verbose_ptxas=True)
    print("built", KERNEL_LIB.name, HOST_LIB.name if HOST_LIB.exists() else "")
