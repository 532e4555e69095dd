"""Builds libh3_b200.so (CUDA kernels + C ABI + the plain-C DiT host) in-tree for sm_100a.

    python -m h3c_b200.build [--force]

nvcc cross-compiles without a GPU; the built library sits next to this file so that it
travels with the source tree.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "_obj"
LIB = HERE / "libh3_b200.so"
SDPA_PLUGIN = HERE / "libh3_b200_sdpa.so"   # the attention kernel behind the reference's dlopen plugin ABI
PROBE = HERE / "libh3_b200_probe.so"        # tensor-pipe rate probe used by the bench (not part of the product)

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]
GCC_FLAGS = ["-std=c11", "-O2", "-fPIC", "-Wall", "-Wextra", "-D_GNU_SOURCE"]


def _sources():
    cu = sorted(CSRC.glob("*.cu"))
    c = sorted(CSRC.glob("*.c"))
    hdr = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + sorted((HERE.parent / "include").glob("*.h"))
    return cu, c, hdr


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _compile(src: Path, hdr, force: bool) -> Path:
    obj = OBJ / (src.name + ".o")
    if force or _stale(obj, [src] + hdr):
        if src.suffix == ".cu":
            cmd = ["nvcc"] + NVCC_FLAGS + ["-c", str(src), "-o", str(obj)]
        else:
            cmd = ["gcc"] + GCC_FLAGS + ["-I/usr/local/cuda/include", "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"{' '.join(cmd)}\n{res.stdout}{res.stderr}")
    return obj


def build(force: bool = False) -> Path:
    cu, c, hdr = _sources()
    OBJ.mkdir(exist_ok=True)
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(lambda s: _compile(s, hdr, force), cu + c))
    if force or _stale(LIB, objs):
        cmd = ["nvcc", "-shared", "-o", str(LIB)] + [str(o) for o in objs] + ["-lpthread", "-ldl", "-Xlinker", "-Bsymbolic"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"{' '.join(cmd)}\n{res.stdout}{res.stderr}")
    plugin_src = CSRC / "plugin" / "h3b_sdpa_plugin.c"
    if force or _stale(SDPA_PLUGIN, [plugin_src, LIB] + hdr):
        cmd = ["gcc"] + GCC_FLAGS + ["-shared", "-I/usr/local/cuda/include", str(plugin_src), "-o", str(SDPA_PLUGIN),
                                     f"-L{HERE}", "-lh3_b200", "-Wl,-rpath,$ORIGIN", "-L/usr/local/cuda/lib64", "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"{' '.join(cmd)}\n{res.stdout}{res.stderr}")
    probe_src = CSRC / "probe" / "h3b_peak.cu"
    if force or _stale(PROBE, [probe_src, LIB] + hdr):
        cmd = ["nvcc"] + NVCC_FLAGS + ["-shared", str(probe_src), "-o", str(PROBE), f"-L{HERE}", "-lh3_b200", "-Xlinker",
                                       "-rpath=$ORIGIN"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"{' '.join(cmd)}\n{res.stdout}{res.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
