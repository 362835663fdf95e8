"""In-tree build of the native extension ``mccl_b200/_C.so`` for sm_100a.

Uses ``torch.utils.cpp_extension`` (ninja) with an explicit
``-gencode arch=compute_100a,code=sm_100a`` so the result does not depend on a
visible GPU; nvcc cross-compiles.  Objects live in ``mccl_b200/_build``; the
linked library is copied next to the package so that a plain import finds it and
it travels with the source tree.

    python -m mccl_b200._build          # build if sources changed
    python -m mccl_b200._build --force  # rebuild everything
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = ROOT / "csrc"
BUILD_DIR = PKG / "_build"
TARGET = PKG / "_C.so"

CPP_SOURCES = [
    "binding.cpp",
    "backend/process_group.cpp",
    "backend/process_group_cuda.cpp",
    "backend/work.cpp",
    "runtime/metrics.cpp",
    "runtime/watchdog.cpp",
    "runtime/arena.cpp",
    "transport/host_transport.cpp",
    "compression/compressor.cpp",
    "cpu/reduce.cpp",
    "transforms/stft.cpp",
    "p2p/nccl_p2p.cpp",
]
CUDA_SOURCES = [
    "kernels/ew.cu",
    "kernels/collectives.cu",
    "kernels/reduce_ws2.cu",
    "kernels/reduce_ws4.cu",
    "kernels/reduce_ws8.cu",
    "kernels/topk.cu",
    "kernels/stft.cu",
    "kernels/adamw.cu",
    "kernels/noalloc.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xptxas", "-v",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fvisibility=hidden", "-Wall", "-Wno-unused-function", "-DMCCL_WITH_STFT"]


def sources():
    out = []
    for rel in CPP_SOURCES + CUDA_SOURCES:
        p = CSRC / rel
        if p.exists():
            out.append(str(p))
    return out


def nccl_include_dirs():
    """nccl.h matching torch's bundled NCCL (only send/recv use it, through torch's ProcessGroupNCCL)."""
    out = []
    try:
        import nvidia.nccl
        for base in list(getattr(nvidia.nccl, "__path__", [])):
            if (Path(base) / "include" / "nccl.h").exists():
                out.append(str(Path(base) / "include"))
    except Exception:
        pass
    if not out and Path("/usr/include/nccl.h").exists():
        out.append("/usr/include")
    return out


def newest_source_mtime() -> float:
    newest = 0.0
    for p in CSRC.rglob("*"):
        if p.suffix in (".cpp", ".cu", ".h", ".cuh"):
            newest = max(newest, p.stat().st_mtime)
    return newest


def is_stale() -> bool:
    return not TARGET.exists() or TARGET.stat().st_mtime < newest_source_mtime()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles every native source for sm_100a and installs ``_C.so`` in the package."""
    if force and BUILD_DIR.exists():
        shutil.rmtree(BUILD_DIR)
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    # A relocated compiler whose libstdc++.so link is dangling links libstdc++
    # statically; a second copy of the C++ runtime inside the extension crashes in
    # iostream locale code.  Prefer the system compiler, which links it shared.
    if os.environ.get("MCCL_KEEP_CXX") != "1" and os.path.exists("/usr/bin/g++"):
        os.environ["CXX"] = "/usr/bin/g++"
        os.environ["CC"] = "/usr/bin/gcc"
    from torch.utils import cpp_extension

    cflags = list(CXX_FLAGS)
    if not (CSRC / "transforms" / "stft.cpp").exists():
        cflags.remove("-DMCCL_WITH_STFT")
    cpp_extension.load(
        name="_C",
        sources=sources(),
        extra_cflags=cflags,
        extra_cuda_cflags=NVCC_FLAGS,
        extra_include_paths=[str(CSRC)] + nccl_include_dirs(),
        build_directory=str(BUILD_DIR),
        with_cuda=True,
        is_python_module=False,
        verbose=verbose,
    )
    built = BUILD_DIR / "_C.so"
    if not built.exists():
        raise RuntimeError(f"build finished but {built} is missing")
    tmp = TARGET.with_suffix(".so.tmp")
    shutil.copy2(built, tmp)
    os.replace(tmp, TARGET)
    return TARGET


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv or "--verbose" in sys.argv)
    print(path)
