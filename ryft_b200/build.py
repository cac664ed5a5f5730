"""Builds the native libraries in-tree with nvcc for sm_100a.

  ryft_b200/lib/libpjrt-plugin-cuda-13.so   PJRT plugin; exports only `GetPjrtApi`
  ryft_b200/lib/libb2x_kernels.so           kernel-level C ABI (include/b2x_kernels.h) plus `b2x_plan_dump`

`python -m ryft_b200.build` rebuilds what is out of date.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
OBJ = ROOT / "build"
INCLUDE = ROOT.parent / "include"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CXXFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wno-unused-function"]

KERNEL_SOURCES = ["kernels/elementwise.cu", "kernels/reduce.cu", "kernels/gemm_simt.cu", "kernels/gemm_tc.cu", "kernels/gemm_tc_static.cu", "kernels/attention.cu", "kernels/wide.cu"]
HOST_SOURCES = ["frontend/parser.cc", "frontend/verify.cc", "frontend/canonicalize.cc", "runtime/planner.cc", "runtime/proto.cc", "runtime/nccl_dyn.cc",
                "runtime/executor.cc", "runtime/pjrt_plugin.cc", "runtime/debug_api.cc"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; the native libraries cannot be built")


def _headers() -> list[Path]:
    hs = list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return hs


def _stale(src: Path, obj: Path, newest_header: float) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    return src.stat().st_mtime > t or newest_header > t


def _compile(nvcc: str, src: Path, obj: Path, verbose: bool) -> None:
    cmd = [nvcc, *ARCH, *CXXFLAGS, "-I", str(CSRC), "-I", str(INCLUDE), "-I", "/usr/include", "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")


def build(verbose: bool = False, force: bool = False) -> dict:
    nvcc = _nvcc()
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    newest_header = max(h.stat().st_mtime for h in _headers())
    sources = [s for s in KERNEL_SOURCES + HOST_SOURCES if (CSRC / s).exists()]
    jobs = []
    objs = {}
    for s in sources:
        src = CSRC / s
        obj = OBJ / (s.replace("/", "_") + ".o")
        objs[s] = obj
        if force or _stale(src, obj, newest_header):
            jobs.append((src, obj))
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(lambda j: _compile(nvcc, j[0], j[1], verbose), jobs))

    kernel_objs = [str(objs[s]) for s in KERNEL_SOURCES if s in objs]
    host_objs = [str(objs[s]) for s in HOST_SOURCES if s in objs]
    plugin = LIB / "libpjrt-plugin-cuda-13.so"
    kernels = LIB / "libb2x_kernels.so"
    vs = OBJ / "plugin.lds"
    # the plugin exports exactly one symbol, like the reference's plugins do
    vs.write_text("{\n  global:\n    GetPjrtApi;\n  local:\n    *;\n};\n")
    ks = OBJ / "kernels.lds"
    ks.write_text("{\n  global:\n    b2x_*;\n  local:\n    *;\n};\n")
    relink = bool(jobs) or not plugin.exists() or not kernels.exists()
    if relink:
        common = [nvcc, *ARCH, "-shared", "-cudart", "static", "-Xlinker", "--no-undefined", "-ldl", "-lpthread"]
        for out, objects, script in ((plugin, host_objs + kernel_objs, vs), (kernels, host_objs + kernel_objs, ks)):
            cmd = common + ["-Xlinker", f"--version-script={script}", "-o", str(out)] + objects
            if verbose:
                print(" ".join(cmd), flush=True)
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"link failed for {out}:\n{r.stdout}\n{r.stderr}")
        # the name the reference's load_cuda_12_plugin() looks for
        alias = LIB / "libpjrt-plugin-cuda-12.so"
        shutil.copyfile(plugin, alias)
    return {"plugin": str(plugin), "kernels": str(kernels), "compiled": [str(j[0]) for j in jobs]}


if __name__ == "__main__":
    info = build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print("built:", info["plugin"], info["kernels"], f"({len(info['compiled'])} files compiled)")
