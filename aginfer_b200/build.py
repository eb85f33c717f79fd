"""Build the native parts in-tree: the loader library and the sm_100a kernel bundle.

    python -m aginfer_b200.build            # both, only what is out of date
    python -m aginfer_b200.build --force

Outputs (git-ignored): ``aginfer_b200/_lib/libaginfer_b200.so`` (g++, no CUDA link
dependency: the driver is resolved with dlopen at run time) and
``aginfer_b200/_lib/sm100/kernels.cubin`` (``nvcc -cubin -arch=sm_100a``; a CUBIN holds
SASS only, which is what an AIM kernel bundle must be).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REPO = HERE.parent
LIB_DIR = HERE / "_lib"
RUNTIME_SRC = HERE / "csrc" / "runtime"
KERNEL_SRC = HERE / "csrc" / "kernels"
LIBRARY = LIB_DIR / "libaginfer_b200.so"
CUBIN = LIB_DIR / "sm100" / "kernels.cubin"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))


def _stale(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return True
    built = target.stat().st_mtime
    return any(s.stat().st_mtime > built for s in sources)


def _run(cmd: list[str]) -> None:
    done = subprocess.run(cmd, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(cmd)}\n{done.stdout}\n{done.stderr}")
    if done.stderr.strip() and os.environ.get("AGI_BUILD_VERBOSE"):
        print(done.stderr, file=sys.stderr)


def build_runtime(force: bool = False) -> Path:
    sources = sorted(RUNTIME_SRC.glob("*.cc"))
    device_sources = sorted(RUNTIME_SRC.glob("*.cu"))   # entry points that launch kernels through the CUDA runtime
    deps = sources + device_sources + sorted(RUNTIME_SRC.glob("*.h")) + sorted(KERNEL_SRC.glob("*.cuh")) + \
        [REPO / "include" / "aginfer_b200.h"]
    if force or _stale(LIBRARY, deps):
        LIB_DIR.mkdir(parents=True, exist_ok=True)
        objects = []
        for src in device_sources:
            obj = LIB_DIR / (src.stem + ".o")
            _run([nvcc(), "-c", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
                  "-Xcompiler", "-fPIC,-fvisibility=hidden", f"-I{REPO / 'include'}", f"-I{RUNTIME_SRC}",
                  "-o", str(obj), str(src)])
            objects.append(str(obj))
        link = ["-ldl", "-lpthread"]
        if objects:  # the CUDA runtime is linked statically; it finds the driver by itself at first use
            link = [f"-L{CUDA_HOME / 'lib64'}", "-lcudart_static", "-lrt", *link]
        _run(["g++", "-std=c++20", "-O2", "-fPIC", "-shared", "-Wall", "-Wextra", "-Wpedantic", "-fvisibility=hidden",
              f"-I{REPO / 'include'}", f"-I{CUDA_HOME / 'include'}", *map(str, sources), *objects, "-o", str(LIBRARY),
              *link])
    return LIBRARY


def nvcc() -> str:
    found = shutil.which("nvcc") or str(CUDA_HOME / "bin" / "nvcc")
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; set CUDA_HOME")
    return found


def build_kernels(force: bool = False, extra: tuple[str, ...] = ()) -> Path:
    main = KERNEL_SRC / "kernels.cu"
    deps = [main] + sorted(KERNEL_SRC.glob("*.cuh"))
    if force or _stale(CUBIN, deps):
        CUBIN.parent.mkdir(parents=True, exist_ok=True)
        _run([nvcc(), "-cubin", "-arch=sm_100a", "-O3", "-std=c++17", "-Xptxas", "-v", f"-I{KERNEL_SRC}", *extra, "-o", str(CUBIN), str(main)])
    return CUBIN


def build_all(force: bool = False) -> tuple[Path, Path]:
    return build_runtime(force), build_kernels(force)


if __name__ == "__main__":
    lib, cubin = build_all("--force" in sys.argv)
    print(lib, lib.stat().st_size)
    print(cubin, cubin.stat().st_size)
