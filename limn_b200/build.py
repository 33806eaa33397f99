"""Build liblimn_b200.so for sm_100a with nvcc, in-tree next to this file.

    python -m limn_b200.build            # build if any source is newer than the library
    python -m limn_b200.build --force

nvcc cross-compiles, so this runs on a machine without a GPU. The library links the CUDA
runtime statically and looks the one driver entry point it needs (tensor-map encoding) up
at run time, so it has no link-time dependency on libcuda.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
LIB = HERE / "liblimn_b200.so"
SOURCES = ["capi.cu", "sdpa_general.cu", "sdpa_general_tiled.cu", "dispatch_sm100.cu", "sdpa_fwd_sm100.cu", "sdpa_bwd_sm100.cu", "sdpa_decode.cu", "static_scratch.cu", "wait_probe.cu", "nccl_gather.cpp"]
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
    "--expt-relaxed-constexpr",
]


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; limn_b200 has no prebuilt fallback")
    return found


def stale() -> bool:
    if not LIB.exists():
        return True
    built = LIB.stat().st_mtime
    deps = list(CSRC.glob("*")) + [HERE.parent / "include" / "limn_b200.h", Path(__file__)]
    return any(dep.stat().st_mtime > built for dep in deps)


def compile_one(source: str) -> tuple[str, str]:
    obj = OBJ / (source + ".o")
    cmd = [nvcc(), *FLAGS, "-c", str(CSRC / source), "-o", str(obj)]
    done = subprocess.run(cmd, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"nvcc failed on {source}:\n{done.stdout}\n{done.stderr}")
    return str(obj), done.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIB
    OBJ.mkdir(exist_ok=True)
    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as pool:
        results = list(pool.map(compile_one, SOURCES))
    (OBJ / "ptxas.log").write_text("\n".join(log for _, log in results))
    if verbose:
        print("\n".join(log for _, log in results))
    link = [nvcc(), "-shared", "-o", str(LIB), *[obj for obj, _ in results], "-cudart", "static", "-ldl"]
    done = subprocess.run(link, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"linking liblimn_b200.so failed:\n{done.stdout}\n{done.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
