"""Builds libiom_b200.so (the C-ABI kernel library) in-tree with nvcc for sm_100a.

Usage: ``python -m iom_b200.build [--force] [--verbose]``. nvcc cross-compiles
without a GPU. Floating-point contraction is disabled for every translation
unit (``--fmad=false``): the kernels must round each multiply and add exactly
like the reference codec does.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
LIBRARY = PACKAGE_DIR / "libiom_b200.so"
SOURCES = ["host.cu", "binary.cu", "rmsnorm.cu", "rmsnorm_long.cu", "copy.cu", "gather.cu", "sumsq.cu", "silu.cu", "rope.cu", "sdpa.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--fmad=false", "-ftz=false", "-prec-div=true", "-prec-sqrt=true",
    "-Xcompiler", "-fPIC",
]


def find_nvcc() -> str:
    candidate = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(candidate).exists():
        raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")
    return candidate


def sources() -> list[Path]:
    return [CSRC / name for name in SOURCES]


def is_stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    inputs = list(CSRC.glob("*")) + [PACKAGE_DIR.parent / "include" / "iom_b200.h", Path(__file__)]
    return any(path.stat().st_mtime > built for path in inputs)


def build(force: bool = False, verbose: bool = False, defines: tuple = (),
          library: Path = LIBRARY, build_dir_name: str = "build") -> Path:
    """`defines` (e.g. ("IOMB_PACKED_BF16=1",)) with another `library` / `build_dir_name`
    gives a variant build beside the default one."""
    if not force and not defines and not is_stale():
        return library
    nvcc = find_nvcc()
    objects = []
    build_dir = PACKAGE_DIR / build_dir_name
    build_dir.mkdir(exist_ok=True)
    procs = []
    for source in sources():
        obj = build_dir / (source.stem + ".o")
        objects.append(obj)
        command = [nvcc, *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-c", str(source), "-o", str(obj)]
        if verbose:
            command[1:1] = ["-Xptxas", "-v"]
            print(" ".join(command), flush=True)
        procs.append((source, subprocess.Popen(command, stdout=subprocess.PIPE,
                                               stderr=subprocess.STDOUT, text=True)))
    failed = False
    for source, proc in procs:
        output, _ = proc.communicate()
        if verbose or proc.returncode != 0:
            print(output, flush=True)
        if proc.returncode != 0:
            failed = True
            print(f"nvcc failed on {source}", file=sys.stderr)
    if failed:
        raise RuntimeError("libiom_b200.so build failed")
    link = [nvcc, "-shared", "-o", str(library), *map(str, objects),
            "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
    subprocess.run(link, check=True)
    return library


# ---- the C++ backend (needs the reference checkout: it subclasses the reference's classes) ----

BACKEND_LIBRARY = PACKAGE_DIR / "libiom_b200_backend.so"
BACKEND_ARCHIVE = PACKAGE_DIR / "libiom_b200_backend.a"
BACKEND_SOURCES = ["b200_backend.cpp", "b200_capi.cpp"]
# The reference's backend-neutral sources a backend links with (its "common op layer"),
# compiled unmodified from where they lie; flags follow the reference's CMake configuration
# (C++20 ISO mode, -O2, no fast-math: CMakeLists.txt:60-63).
REFERENCE_COMMON = ["device_ops", "device_ops_copy", "device_ops_binary", "device_ops_cache_append",
                    "device_ops_rmsnorm", "device_ops_embedding", "device_ops_neural", "workspace",
                    "tensor", "tensor_view", "alloc"]


def build_backend(reference: Path, force: bool = False) -> Path:
    """Builds libiom_b200_backend.a (the backend's own objects: what a maintainer of the
    reference adds to its build) and libiom_b200_backend.so (those objects, the reference's
    common sources and the C driver interface of include/iom_b200_backend_c.h, linked
    against libiom_b200.so)."""
    reference = Path(reference)
    if not (reference / "include" / "iom" / "iom.hpp").exists():
        raise RuntimeError(f"{reference} is not a checkout of the reference")
    build(force=False)
    backend_dir = PACKAGE_DIR / "backend"
    inputs = [backend_dir / name for name in BACKEND_SOURCES] + [
        PACKAGE_DIR.parent / "include" / name
        for name in ("iom_b200.h", "iom_b200_backend.hpp", "iom_b200_backend_c.h")]
    if (not force and BACKEND_LIBRARY.exists()
            and all(path.stat().st_mtime <= BACKEND_LIBRARY.stat().st_mtime for path in inputs)
            and LIBRARY.stat().st_mtime <= BACKEND_LIBRARY.stat().st_mtime):
        return BACKEND_LIBRARY
    cuda_home = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    out_dir = PACKAGE_DIR / "build" / "backend"
    out_dir.mkdir(parents=True, exist_ok=True)
    cxx = os.environ.get("CXX", "g++")
    flags = ["-std=c++20", "-O2", "-fPIC", f"-I{reference / 'include'}", f"-I{reference / 'src'}",
             f"-I{PACKAGE_DIR.parent / 'include'}", f"-I{cuda_home / 'include'}"]
    jobs = []
    own, common = [], []
    for name in BACKEND_SOURCES:
        obj = out_dir / (Path(name).stem + ".o")
        own.append(obj)
        jobs.append((name, subprocess.Popen([cxx, *flags, "-c", str(backend_dir / name), "-o", str(obj)])))
    for name in REFERENCE_COMMON:
        obj = out_dir / f"reference_{name}.o"
        common.append(obj)
        jobs.append((name, subprocess.Popen([cxx, *flags, "-c", str(reference / "src" / f"{name}.cpp"),
                                             "-o", str(obj)])))
    for name, proc in jobs:
        if proc.wait() != 0:
            raise RuntimeError(f"compiling {name} failed")
    if BACKEND_ARCHIVE.exists():
        BACKEND_ARCHIVE.unlink()
    subprocess.run(["ar", "rcs", str(BACKEND_ARCHIVE), str(own[0])], check=True)
    subprocess.run([cxx, "-shared", "-o", str(BACKEND_LIBRARY), *map(str, own), *map(str, common),
                    f"-L{PACKAGE_DIR}", "-liom_b200", "-Wl,-rpath,$ORIGIN",
                    f"-L{cuda_home / 'lib64'}", "-lcudart_static", "-ldl", "-lrt", "-lpthread"],
                   check=True)
    return BACKEND_LIBRARY


if __name__ == "__main__":
    backend = [a.split("=", 1)[1] for a in sys.argv if a.startswith("--backend=")]
    if backend:
        # --backend=<reference checkout> builds the C++ backend against that checkout
        print(build_backend(Path(backend[0]), force="--force" in sys.argv))
        sys.exit(0)
    variant = [a.split("=", 1)[1] for a in sys.argv if a.startswith("--variant=")]
    if variant:
        # --variant=name:DEFINE=1[,DEFINE2=..] builds libiom_b200_<name>.so with those defines
        name, _, defs = variant[0].partition(":")
        path = build(force=True, verbose="--verbose" in sys.argv,
                     defines=tuple(d for d in defs.split(",") if d),
                     library=PACKAGE_DIR / f"libiom_b200_{name}.so", build_dir_name=f"build_{name}")
    else:
        path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
