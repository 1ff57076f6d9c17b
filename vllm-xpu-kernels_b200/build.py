"""In-tree build of the sm_100a kernels and their torch registration libraries.

Outputs (all inside ``vllm_xpu_kernels/`` next to this file, git-ignored):

* ``libb200moe.so`` - the C ABI of ``include/b200moe.h`` (nvcc, no torch);
* ``_C.so``, ``_moe_C.so``, ``_xpu_C.so`` - one TORCH_LIBRARY registration
  library per op namespace, linked against ``libb200moe.so``.

Run ``python build.py`` (add ``--force`` to rebuild everything, ``--no-torch``
to build only the C ABI library).  nvcc cross-compiles for sm_100a without a
GPU being present.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
PKG = HERE / "vllm_xpu_kernels"
OBJ = HERE / "build"
INCLUDE = HERE.parent / "include"

CU_SOURCES = ["abi.cu", "routing.cu", "permute.cu", "ep.cu", "elementwise.cu", "fused_quant.cu", "gemm.cu",
              "gemm_check.cu", "gemm_tc.cu", "gemm_tc_dq.cu", "gemm_tc_mx.cu", "gemm_tc_fp8t.cu"]
SHIMS = {"_C": "c_ops.cpp", "_moe_C": "moe_ops.cpp", "_xpu_C": "xpu_ops.cpp"}

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
              "-std=c++17", "-Xcompiler", "-fPIC", "--threads", "2"]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(d).stat().st_mtime <= t for d in deps)


def _run(cmd):
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(map(str, cmd)), res.stdout, res.stderr))


def build_abi(force: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [INCLUDE / "b200moe.h"]
    sources = list(CU_SOURCES)
    nvcc = _nvcc()
    jobs = []
    objs = []
    for src in sources:
        obj = OBJ / (src + ".o")
        objs.append(obj)
        if force or not _newer(obj, [CSRC / src] + headers):
            jobs.append([nvcc] + NVCC_FLAGS + ["-c", str(CSRC / src), "-o", str(obj)])
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        list(pool.map(_run, jobs))
    lib = PKG / "libb200moe.so"
    if force or jobs or not _newer(lib, objs):
        _run([nvcc, "-shared", "-o", str(lib)] + [str(o) for o in objs])
    return lib


def build_shims(force: bool = False) -> None:
    import torch  # noqa: F401  (only for the include / library paths)
    from torch.utils import cpp_extension as ce

    OBJ.mkdir(exist_ok=True)
    inc = []
    for p in ce.include_paths():
        inc += ["-I", p]
    inc += ["-I", sysconfig.get_paths()["include"], "-I", "/usr/local/cuda/include"]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    common = ["g++", "-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-DTORCH_API_INCLUDE_EXTENSION_H",
              f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-Wno-deprecated-declarations"] + inc
    headers = [CSRC / "torch" / "shim.h", INCLUDE / "b200moe.h"]
    jobs = []
    for name, src in SHIMS.items():
        out = PKG / f"{name}.so"
        srcp = CSRC / "torch" / src
        if force or not _newer(out, [srcp] + headers):
            jobs.append(common + ["-shared", str(srcp), "-o", str(out),
                                  "-fvisibility=default",
                                  "-L", str(PKG), "-lb200moe", "-L", torch_lib, "-ltorch", "-ltorch_cpu",
                                  "-lc10", "-lc10_cuda", "-ltorch_cuda",
                                  "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"])
    with ThreadPoolExecutor(max_workers=3) as pool:
        list(pool.map(_run, jobs))


def build(force: bool = False, torch_shims: bool = True) -> None:
    build_abi(force)
    if torch_shims:
        build_shims(force)


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--no-torch", action="store_true")
    a = ap.parse_args()
    build(force=a.force, torch_shims=not a.no_torch)
    print("built:", sorted(p.name for p in PKG.glob("*.so")))
