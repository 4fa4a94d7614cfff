"""Build `libkrn_b200.so` for sm_100a with nvcc: `python -m krn_b200.csrc.build`.

nvcc cross-compiles without a GPU. The library lands beside the package (`krn_b200/libkrn_b200.so`), which
is where `krn_b200.hw.Libraries` looks for the logical name "krn_b200".
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUTPUT = HERE.parent / "libkrn_b200.so"
SOURCES = ("host.cu", "gemm_tn.cu", "gemm_fp8.cu", "gemm_mxfp8.cu", "attn_fwd.cu", "attn_decode.cu", "scatter.cu")
FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC")


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found: the kernel library needs the CUDA toolkit to build")
    return found


def stale() -> bool:
    if not OUTPUT.exists():
        return True
    built = OUTPUT.stat().st_mtime
    inputs = [*HERE.glob("*.cu"), *HERE.glob("*.cuh"), HERE.parent.parent / "include" / "krn_b200.h"]
    return any(path.stat().st_mtime > built for path in inputs)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every kernel source into one shared library; a no-op when it is up to date."""
    if not force and not stale():
        return OUTPUT
    sources = [HERE / name for name in SOURCES if (HERE / name).exists()]
    objects = []
    build_dir = HERE / "build"
    build_dir.mkdir(exist_ok=True)
    jobs = []
    for source in sources:
        obj = build_dir / (source.stem + ".o")
        objects.append(obj)
        command = [nvcc(), *FLAGS, *(("-Xptxas", "-v") if verbose else ()), "-c", str(source), "-o", str(obj)]
        jobs.append((source, subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for source, job in jobs:
        output, _ = job.communicate()
        if verbose or job.returncode != 0:
            sys.stderr.write(output)
        if job.returncode != 0:
            raise RuntimeError(f"nvcc failed on {source.name}")
    temporary = OUTPUT.with_suffix(".so.tmp")
    # the CUDA runtime is linked statically (nvcc's default): the library has no libcudart.so dependency
    link = [nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", str(temporary), *map(str, objects)]
    subprocess.run(link, check=True)
    os.replace(temporary, OUTPUT)
    return OUTPUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
