"""Builds libishizuki_cuda.so in-tree with nvcc for sm_100a (no JIT cache, no torch extension)."""
from __future__ import annotations

import os
import pathlib
import shutil
import subprocess

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libishizuki_cuda.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]
OBJ = CSRC / "_obj"  # object files, one per translation unit, rebuilt only when stale


def sources() -> list[pathlib.Path]:
    return sorted(CSRC.glob("*.cu"))


def stale() -> bool:
    if not LIB.exists():
        return True
    built = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    deps.append(PKG.parent / "include" / "ishizuki_cuda.h")
    return any(d.stat().st_mtime > built for d in deps)


def _headers_mtime() -> float:
    deps = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [PKG.parent / "include" / "ishizuki_cuda.h"]
    return max(d.stat().st_mtime for d in deps)


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    """Compiles every .cu under csrc/ (the translation units side by side) and links them into one
    shared library. Needs nvcc, not a GPU."""
    if not force and not stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: libishizuki_cuda.so cannot be built on this machine")
    OBJ.mkdir(exist_ok=True)
    newest_header = _headers_mtime()
    jobs = []
    objects = []
    for src in sources():
        obj = OBJ / (src.stem + ".o")
        objects.append(obj)
        if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, newest_header):
            continue
        # ISHI_NVCC_EXTRA: extra compiler flags of a diagnostic build (e.g. -DISHI_TRACE)
        cmd = [nvcc, *NVCC_FLAGS, *os.environ.get("ISHI_NVCC_EXTRA", "").split(), "-c", "-o", str(obj), str(src)]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
        jobs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
    for src, proc in jobs:
        out, err = proc.communicate()
        if proc.returncode != 0:
            for _, other in jobs:
                if other.poll() is None:
                    other.kill()
            raise RuntimeError(f"nvcc failed on {src.name}:\n{out}\n{err}")
        if verbose:
            print(err)
    link = subprocess.run([nvcc, "-shared", "-o", str(LIB), *map(str, objects), "-ldl"], capture_output=True, text=True)
    if link.returncode != 0:
        raise RuntimeError(f"link failed:\n{link.stdout}\n{link.stderr}")
    return LIB


if __name__ == "__main__":
    import sys

    print(build(force=True, verbose="-v" in sys.argv))
