"""Builds libc0ven_moe.so, the CUDA library behind include/moe_layer.h, and libengine.so, the same objects behind
include/engine_abi.h with only the engine_* symbols exported (as the reference builds its libengine:
core/CMakeLists.txt:50-58), in-tree with nvcc for sm_100a.

    python -m c0ven_b200.build [--force]

nvcc cross-compiles without a GPU. The IQ3_S codebook header is generated first from gguf-py (csrc/gen_iq3s_grid.py).
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(ROOT, "build", "obj")
LIB = os.path.join(HERE, "libc0ven_moe.so")
ENGINE_LIB = os.path.join(HERE, "libengine.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-DMOE_API_EXPORT", "-DENGINE_API_EXPORT", "-I" + os.path.join(ROOT, "include"),
          "-I" + os.path.join(ROOT, "build"), "-I" + CSRC, "-ccbin", "g++",
          "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wno-unknown-pragmas"]


def sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src: str, force: bool, verbose: bool) -> str:
    obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers += [os.path.join(ROOT, "include", "moe_layer.h"), os.path.join(ROOT, "include", "engine_abi.h"), os.path.join(ROOT, "build", "iq3s_grid.h"),
                os.path.join(ROOT, "build", "iq4nl_values.h")]
    if force or _newer(obj, [os.path.join(CSRC, src)] + headers):
        cmd = [NVCC] + ARCH + COMMON + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    sys.path.insert(0, CSRC)
    import gen_iq3s_grid

    grid_h = os.path.join(ROOT, "build", "iq3s_grid.h")
    if not os.path.exists(grid_h) or not os.path.exists(os.path.join(ROOT, "build", "iq4nl_values.h")):
        gen_iq3s_grid.main(grid_h)
    with cf.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, verbose), sources()))
    # libc0ven_moe.so exports what the sources mark (moe_* and engine_*); libengine.so is the same objects linked with a
    # version script that keeps only the engine ABI's symbols global.
    vers = os.path.join(ROOT, "build", "engine.map")
    if not os.path.exists(vers):
        open(vers, "w").write("{ global: engine_*; local: *; };\n")
    for lib, extra in ((LIB, []), (ENGINE_LIB, ["-Xlinker", "--version-script=" + vers])):
        if force or _newer(lib, objs):
            cmd = [NVCC] + ARCH + ["-shared", "-o", lib] + objs + ["-ccbin", "g++", "-Xlinker", "--exclude-libs,ALL"] + extra
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
