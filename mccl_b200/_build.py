"""In-tree build of the native extension ``mccl_b200/_C.so`` for sm_100a.

Uses ``torch.utils.cpp_extension`` (ninja) with an explicit
``-gencode arch=compute_100a,code=sm_100a`` so the result does not depend on a
visible GPU; nvcc cross-compiles.  Objects live in ``mccl_b200/_build``; the
linked library is copied next to the package so that a plain import finds it and
it travels with the source tree.

    python -m mccl_b200._build          # build if sources changed
    python -m mccl_b200._build --force  # rebuild everything

``MCCL_SANITIZE=address`` (or ``thread``) builds a second, instrumented library
``mccl_b200/_C_asan.so`` / ``_C_tsan.so`` next to the regular one (host code compiled with
``-fsanitize``; objects in their own directory).  It is loaded instead of ``_C.so`` when
``MCCL_NATIVE_LIB`` points at it and the sanitizer runtime is preloaded, which is what
``tests/test_sanitized_runtime.py`` does for the CPU-rank tests.
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
    "runtime/nvls.cpp",
    "runtime/nvls_pool.cpp",
    "transport/host_transport.cpp",
    "compression/compressor.cpp",
    "cpu/reduce.cpp",
    "transforms/stft.cpp",
    "p2p/nccl_p2p.cpp",
]
CUDA_SOURCES = [
    "kernels/ew.cu",
    "kernels/collectives.cu",
    "kernels/nvls.cu",
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


SANITIZERS = {"address": "asan", "thread": "tsan"}


def sanitized_target(kind: str) -> Path:
    return PKG / f"_C_{SANITIZERS[kind]}.so"


def sanitizer_runtime(kind: str) -> str:
    """Path of the sanitizer runtime that has to be preloaded into an uninstrumented python."""
    import subprocess
    name = {"address": "libasan.so", "thread": "libtsan.so"}[kind]
    cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
    def find(lib):
        out = subprocess.run([cc, f"-print-file-name={lib}"], capture_output=True, text=True).stdout.strip()
        return out if out and os.path.isabs(out) and os.path.exists(out) else ""

    rt = find(name)
    if not rt:
        return ""
    # libstdc++ has to be in the initial library list as well: the runtime resolves the real
    # __cxa_throw when it starts, and python itself does not link the C++ runtime
    cxx = find("libstdc++.so.6") or find("libstdc++.so")
    return f"{rt}:{cxx}" if cxx else rt


def build(force: bool = False, verbose: bool = False, sanitize: str = "") -> Path:
    """Compiles every native source for sm_100a and installs ``_C.so`` in the package.

    ``sanitize`` ("address" / "thread", default from ``MCCL_SANITIZE``) builds the instrumented
    variant instead and leaves the regular library alone.
    """
    sanitize = sanitize or os.environ.get("MCCL_SANITIZE", "")
    if sanitize and sanitize not in SANITIZERS:
        raise ValueError(f"MCCL_SANITIZE must be one of {sorted(SANITIZERS)}, got {sanitize!r}")
    build_dir = PKG / f"_build_{SANITIZERS[sanitize]}" if sanitize else BUILD_DIR
    target = sanitized_target(sanitize) if sanitize else TARGET
    if sanitize and os.environ.get("MCCL_SANITIZE_CHILD") != "1":
        # The build helper loads the fresh library into the (uninstrumented) interpreter once.  The
        # sanitizer runtime reads its options from the environment the process STARTED with, so the
        # build runs in a child whose initial environment tells it to tolerate not being first in
        # the library list.
        import subprocess
        env = dict(os.environ, MCCL_SANITIZE=sanitize, MCCL_SANITIZE_CHILD="1", MCCL_NO_AUTOBUILD="1")
        env["ASAN_OPTIONS"] = "verify_asan_link_order=0:detect_leaks=0:protect_shadow_gap=0"
        env["TSAN_OPTIONS"] = "report_bugs=0"
        cmd = [sys.executable, "-m", "mccl_b200._build"] + (["--force"] if force else []) + (["-v"] if verbose else [])
        subprocess.run(cmd, env=env, cwd=str(ROOT), check=True)
        if not target.exists():
            raise RuntimeError(f"sanitized build finished but {target} is missing")
        return target
    if force and build_dir.exists():
        shutil.rmtree(build_dir)
    build_dir.mkdir(parents=True, exist_ok=True)
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    # A relocated compiler whose libstdc++.so link is dangling links libstdc++
    # statically; a second copy of the C++ runtime inside the extension crashes in
    # iostream locale code.  Prefer the system compiler, which links it shared.
    if os.environ.get("MCCL_KEEP_CXX") != "1" and os.path.exists("/usr/bin/g++"):
        os.environ["CXX"] = "/usr/bin/g++"
        os.environ["CC"] = "/usr/bin/gcc"
    from torch.utils import cpp_extension

    cflags = list(CXX_FLAGS)
    ldflags = []
    if not (CSRC / "transforms" / "stft.cpp").exists():
        cflags.remove("-DMCCL_WITH_STFT")
    if sanitize:
        san = [f"-fsanitize={sanitize}", "-fno-omit-frame-pointer", "-g"]
        cflags = [f for f in cflags if f != "-O3"] + ["-O1"] + san
        ldflags = [f"-fsanitize={sanitize}"]
    built = build_dir / "_C.so"
    try:
        cpp_extension.load(
            name="_C",
            sources=sources(),
            extra_cflags=cflags,
            extra_cuda_cflags=NVCC_FLAGS,
            extra_ldflags=ldflags,
            extra_include_paths=[str(CSRC)] + nccl_include_dirs(),
            build_directory=str(build_dir),
            with_cuda=True,
            is_python_module=False,
            verbose=verbose,
        )
    except OSError:
        # An instrumented library may refuse to load into an interpreter that did not start with the
        # sanitizer runtime (static TLS); the link step has succeeded by then, which is all we need.
        if not (sanitize and built.exists()):
            raise
    if not built.exists():
        raise RuntimeError(f"build finished but {built} is missing")
    tmp = target.with_suffix(".so.tmp")
    shutil.copy2(built, tmp)
    os.replace(tmp, target)
    return target


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv or "--verbose" in sys.argv)
    print(path, flush=True)
    if os.environ.get("MCCL_SANITIZE_CHILD") == "1":
        # the instrumented library was loaded into an interpreter whose earlier allocations the
        # sanitizer never saw: skip the exit-time destructors, the build product is already in place
        os._exit(0)
