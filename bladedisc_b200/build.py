"""Builds libdisc_b200_ral.so in-tree with nvcc for sm_100a.

The library is compiled from the sources under ``csrc/`` into ``_lib/`` next to
this file.  Object files are cached by source content so that an unchanged
translation unit is not recompiled.
"""
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "_lib"
LIB = OUT / "libdisc_b200_ral.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]
SOURCES = [
    "kernels/qgemm_sm100.cu",
    "kernels/rowops.cu",
    "ral/context.cc",
    "ral/pdl_attr.cc",
    "ral/nccl_dyn.cc",
    "kernels/woq_gemm.cu",
    "kernels/woq_gemm_tc.cu",
    "kernels/qconv.cu",
    "kernels/observer.cu",
    "kernels/attention.cu",
    "ral/conv_plan.cc",
    "ral/metadata.cc",
    "ral/cu_driver_dyn.cc",
    "ral/views.cc",
    "ral/selfcheck_calls.cc",
    "ral/calls.cc",
    "c_api.cc",
]
HEADERS = [
    "kernels/qgemm.h", "kernels/rowops.h", "kernels/woq_gemm.h", "kernels/qconv.h", "kernels/observer.h", "kernels/attention.h", "ral/conv_plan.h", "kernels/sm100_ptx.cuh", "kernels/device_info.h", "kernels/tensor_map.h",
    "kernels/qgemm_pair.inl", "kernels/qgemm_gemv.inl", "kernels/qgemm_skinny.inl",
    "kernels/rownorm_staged.inl",
    "ral/abi.h", "ral/context.h", "ral/pdl_attr.h", "ral/nccl_dyn.h", "ral/metadata.h", "ral/cu_driver_dyn.h",
    "../../include/disc_b200_ral.h",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; it is required to build the sm_100a kernels")


def _digest(src: Path) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(src.read_bytes())
    for hd in HEADERS:
        h.update((CSRC / hd).read_bytes())
    return h.hexdigest()[:16]


# no device code and heavy on templates: the host compiler alone (through nvcc for the CUDA include paths)
HOST_ONLY = {"ral/views.cc", "ral/selfcheck_calls.cc"}


def _compile(nvcc: str, rel: str, obj: Path, verbose: bool) -> None:
    src = CSRC / rel
    if rel in HOST_ONLY:
        cmd = [nvcc, "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-c", str(src), "-o", str(obj)]
    else:
        cmd = [nvcc, *NVCC_FLAGS, "-x", "cu", "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compiles (if needed) and returns the path of the shared library."""
    from concurrent.futures import ThreadPoolExecutor
    OUT.mkdir(exist_ok=True)
    nvcc = _nvcc()
    objs = []
    todo = []
    for rel in SOURCES:
        obj = OUT / (rel.replace("/", "_") + "." + _digest(CSRC / rel) + ".o")
        objs.append(obj)
        if obj.exists() and not force:
            continue
        for stale in OUT.glob(rel.replace("/", "_") + ".*.o"):
            stale.unlink()
        todo.append((rel, obj))
    if todo:
        with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 1, 8)) as pool:
            for f in [pool.submit(_compile, nvcc, rel, obj, verbose) for rel, obj in todo]:
                f.result()
    if todo or not LIB.exists() or force:
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB), *map(str, objs), "-ldl"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(path)
