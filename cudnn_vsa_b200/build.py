"""Build ``libvsa_b200.so`` (sm_100a only) in-tree with nvcc.

``python -m cudnn_vsa_b200.build`` compiles every ``csrc/*.cu`` into
``cudnn_vsa_b200/lib/libvsa_b200.so``.  nvcc cross-compiles without a GPU.  Objects are
rebuilt only when a source or header is newer.
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
LIB_DIR = ROOT / "lib"
LIB = LIB_DIR / "libvsa_b200.so"
OBJ_DIR = ROOT / "build"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def nvcc_path() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; the VSA kernels need the CUDA 12.9 toolchain")
    return found


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > stamp for d in deps)


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile the library if any source is newer than it; return its path."""
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + sorted(
        (ROOT.parent / "include").glob("*.h"))
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    nvcc = nvcc_path()

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            done = subprocess.run(cmd, capture_output=True, text=True)
            if verbose:
                sys.stderr.write(done.stderr)
            if done.returncode:
                raise RuntimeError(f"nvcc failed on {src.name}:\n{done.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objects = list(pool.map(compile_one, sources))
    if force or _stale(LIB, objects):
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(LIB), *map(str, objects)]
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode:
            raise RuntimeError(f"link failed:\n{done.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
