"""Builds libcake_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
LIB_DIR = PACKAGE_DIR / "lib"
LIBRARY = LIB_DIR / "libcake_b200.so"
SOURCES = ("cake_runtime.cu", "matmul_rs_sm100.cu", "rpa_decode_sm100.cu")
NVCC_FLAGS = (
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
)


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found: libcake_b200.so cannot be built")
    return found


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(dep.stat().st_mtime > stamp for dep in deps)


def build(*, force: bool = False, verbose: bool = False) -> Path:
    """Compiles every translation unit to an object and links the shared library."""
    LIB_DIR.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh"))
    headers.append(PACKAGE_DIR.parent / "include" / "cake_abi.h")
    objects: list[Path] = []
    procs: list[tuple[subprocess.Popen, Path]] = []
    for name in SOURCES:
        source = CSRC / name
        obj = LIB_DIR / (source.stem + ".o")
        objects.append(obj)
        if force or _stale(obj, [source, *headers]):
            cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(source), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            procs.append((subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True), obj))
    for proc, obj in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed for {obj.name}:\n{out}")
        if verbose and out:
            print(out)
    if force or procs or _stale(LIBRARY, objects):
        cmd = [_nvcc(), "-shared", "-o", str(LIBRARY), *map(str, objects)]
        result = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"link failed:\n{result.stdout}")
    return LIBRARY


PUSH_RATE_PROGRAM = LIB_DIR / "peer_push_rate"


def build_push_rate_program(*, force: bool = False) -> Path:
    """Compiles ``csrc/peer_push_rate.cu``, the stand-alone measurement of the all-to-all push rate
    between the GPUs of a node (the link-side denominator of the fused matmul + reduce-scatter)."""
    LIB_DIR.mkdir(exist_ok=True)
    source = CSRC / "peer_push_rate.cu"
    if force or _stale(PUSH_RATE_PROGRAM, [source]):
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-o", str(PUSH_RATE_PROGRAM), str(source)]
        result = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"nvcc failed for {source.name}:\n{result.stdout}")
    return PUSH_RATE_PROGRAM


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv or bool(os.environ.get("CAKE_VERBOSE")))
    print(path)
    print(build_push_rate_program(force="--force" in sys.argv))
