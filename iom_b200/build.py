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


if __name__ == "__main__":
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
