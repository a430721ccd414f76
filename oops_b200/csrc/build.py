"""Builds liboops_ta_sm100.so in-tree with nvcc for sm_100a (no GPU needed).

    python -m oops_b200.csrc.build [--force]

The shared library lands in oops_b200/lib/.  It is a plain C-ABI library
(include/oops_ta.h); nothing in it links against Python or PyTorch.
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
ROOT = CSRC.parent.parent
LIB_DIR = CSRC.parent / "lib"
LIB_PATH = LIB_DIR / "liboops_ta_sm100.so"
SOURCES = ("ta_api.cu", "ta_generic.cu", "ta_gate.cu", "ta_mask.cu", "ta_layer_norm.cu", "ta_tensor_sm100.cu", "ta_tensor_bwd_sm100.cu")
NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
)


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    candidate = Path(cuda_home) / "bin" / "nvcc"
    return str(candidate) if candidate.exists() else "nvcc"


# Kernels that keep tensor-memory loads in flight under arithmetic: a load writes its destination registers when the
# data arrives, so a spill (or copy) of such a register between issue and wait would save stale data.  ptxas must
# report no spill stores for them; the build fails otherwise.
NO_SPILL_KERNELS = ("ta_bwd_fused_kernel", "ta_bwd_dbias_kernel")


def _spilling_entries(ptxas_log: str, kernels) -> list:
    """Entry functions of `kernels` for which `ptxas -v` reports spill stores."""
    found, current = [], None
    for line in ptxas_log.splitlines():
        if "Compiling entry function" in line:
            current = line.split("'")[1] if "'" in line else line
        elif "bytes spill stores" in line and current is not None:
            stores = int(line.split("bytes stack frame,")[1].split("bytes spill stores")[0])
            if stores > 0 and any(k in current for k in kernels):
                found.append(f"{current}: {stores} bytes")
            current = None
    return found


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > stamp for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    LIB_DIR.mkdir(exist_ok=True)
    obj_dir = LIB_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    headers = [CSRC / "ta_internal.h", ROOT / "include" / "oops_ta.h", *CSRC.glob("*.cuh")]

    def compile_one(name: str):
        src = CSRC / name
        obj = obj_dir / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(ROOT / "include"), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            done = subprocess.run(cmd, capture_output=True, text=True)
            log = obj_dir / (src.stem + ".ptxas.log")
            log.write_text(done.stdout + done.stderr)
            if done.returncode != 0:
                raise RuntimeError(f"nvcc failed for {name}:\n{done.stdout}\n{done.stderr}")
            spilled = _spilling_entries(done.stdout + done.stderr, NO_SPILL_KERNELS)
            if spilled:
                obj.unlink(missing_ok=True)
                raise RuntimeError(f"{name}: register spills in kernels that keep tensor-memory loads in flight: {spilled}")
            if verbose:
                print(done.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objects = list(pool.map(compile_one, SOURCES))
    if force or _stale(LIB_PATH, objects):
        cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *map(str, objects), "-lcudart"]
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"link failed:\n{done.stdout}\n{done.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
