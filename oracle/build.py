"""Builds the checker libraries used by the test-suite (never by the product):

  oracle/_build/libh3_oracle.so      -- this repository's CPU restatement (h3_oracle.c)
  oracle/_ref/libh3_ref.so           -- the reference's own CPU functions, compiled from the
                                        h3.c sources where they lie (read-only, nothing copied)
  oracle/_ref/cuda/libh3_refcuda.so  -- the reference's own CUDA operator library for sm_100a
                                        (cuBLASLt / cuDNN inside): the same-precision checker
  oracle/_ref/libh3_refhost.so       -- the reference's unmodified DiT host linked on top of the
                                        product library (the drop-in check)

The reference's DiT source file also contains its CUDA orchestration, so it has many
undefined h3_cuda_* / cuda* symbols.  Its CPU functions never reach them; they are given
aborting stubs generated from `nm -u` so the shared object loads without a CUDA runtime.

Usage: python oracle/build.py [--ref-root PATH]   (default PATH: $H3_REFERENCE_ROOT, else the directory
"reference" beside this repository)
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
BUILD = HERE / "_build"
REF_OUT = HERE / "_ref"

# Reference translation units that hold the CPU side of the DiT block path.
REF_SOURCES = [
    "h3_w4a8_dequant.c",
    "h3_w4a8.c",
    "h3_safetensors.c",
    "h3_ulysses.c",
    "h3_dit_int8.c",
    "h3_dit_nvfp4.c",
    "h3_nvfp4.c",
    "h3_lora.c",
    "h3_w4a8_cache.c",
    "h3_dit_w4a8.c",
    "h3_sdpa_registry.c",
    "h3_cuda_device_caps.c",
]


def default_ref_root() -> Path:
    """Where the h3.c tree is looked for: $H3_REFERENCE_ROOT, else a directory "reference" beside this repository."""
    env = os.environ.get("H3_REFERENCE_ROOT")
    return Path(env) if env else HERE.parent.parent / "reference"


def _run(cmd: list[str]) -> None:
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
        raise RuntimeError(f"command failed: {cmd[0]}")


def _newer(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(s.exists() and s.stat().st_mtime <= t for s in sources)


def build_oracle(force: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    out = BUILD / "libh3_oracle.so"
    srcs = [HERE / "h3_oracle.c", HERE / "h3_oracle.h"]
    if not force and _newer(out, srcs):
        return out
    _run(["gcc", "-std=c11", "-O2", "-fPIC", "-shared", "-o", str(out), str(HERE / "h3_oracle.c"),
          "-lm", "-lpthread"])
    return out


def build_ref(ref_root: Path, force: bool = False) -> Path | None:
    """Returns the path of libh3_ref.so, or None when the reference tree is absent
    and no prebuilt copy exists."""
    out = REF_OUT / "libh3_ref.so"
    if not ref_root.is_dir():
        return out if out.exists() else None
    if out.exists() and not force:
        return out
    REF_OUT.mkdir(exist_ok=True)
    cuda_inc = "/usr/local/cuda/include"
    objs = []
    for name in REF_SOURCES:
        obj = REF_OUT / (Path(name).stem + ".o")
        _run(["gcc", "-std=c11", "-O2", "-fPIC", "-D_GNU_SOURCE", "-w", f"-I{ref_root}",
              f"-I{cuda_inc}", "-c", str(ref_root / name), "-o", str(obj)])
        objs.append(str(obj))
    shim = REF_OUT / "ref_shim.o"
    _run(["gcc", "-std=c11", "-O2", "-fPIC", "-D_GNU_SOURCE", "-w", f"-I{ref_root}", "-c",
          str(HERE / "ref_shim.c"), "-o", str(shim)])
    objs.append(str(shim))
    # Relocatable link, then stub whatever is still undefined and is not libc/libm/pthread.
    merged = REF_OUT / "merged.o"
    _run(["ld", "-r", "-o", str(merged)] + objs)
    undefined = subprocess.run(["nm", "-u", str(merged)], capture_output=True, text=True,
                               check=True).stdout.split()
    undefined = [s for s in undefined if s not in ("U", "w")]
    stub_names = sorted(s for s in set(undefined)
                        if s.startswith(("h3_", "cuda", "cu", "cublas", "nccl")))
    stub_c = REF_OUT / "stubs.c"
    with open(stub_c, "w") as f:
        f.write("/* generated: aborting stand-ins for the GPU entry points the reference's CPU\n"
                " * functions never reach */\n#include <stdio.h>\n#include <stdlib.h>\n")
        for s in stub_names:
            f.write(f'void {s}(void) {{ fprintf(stderr, "libh3_ref: GPU entry point {s} '
                    f'reached on the CPU checker\\n"); abort(); }}\n')
    _run(["gcc", "-O0", "-fPIC", "-w", "-c", str(stub_c), "-o", str(REF_OUT / "stubs.o")])
    _run(["gcc", "-shared", "-o", str(out), str(merged), str(REF_OUT / "stubs.o"), "-lm",
          "-lpthread", "-ldl"])
    return out


def build_ref_cuda(ref_root: Path, force: bool = False) -> Path | None:
    """The reference's CUDA operator library compiled for sm_100a from its own sources where they lie:
    h3_gpu_cuda.cu (cuBLASLt int8 / fp4 linears, activation quantisers, in-tree flash attention) and its cuDNN
    attention shim, with --use_fast_math as the reference's build sets it.  Output:
    oracle/_ref/cuda/libh3_refcuda.so, the same-precision checker that oracle/ref_cuda_worker.py drives in a
    process of its own.  Returns None when the reference tree is absent and nothing was built before."""
    out_dir = REF_OUT / "cuda"
    out = out_dir / "libh3_refcuda.so"
    if not ref_root.is_dir():
        return out if out.exists() else None
    if out.exists() and not force:
        return out
    out_dir.mkdir(parents=True, exist_ok=True)
    cuda_home = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    cudnn_inc = "/usr/include/x86_64-linux-gnu"
    have_cudnn = Path(cudnn_inc, "cudnn.h").exists()
    defs = ["-DH3_HAVE_CUDNN=1", "-DH3_HAVE_CUDNN_FRONTEND=1"] if have_cudnn else []
    objs = []
    obj = out_dir / "h3_gpu_cuda.o"
    _run(["nvcc", "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "--use_fast_math", "-w",
          "-Xcompiler", "-fPIC", f"-I{ref_root}", f"-I{cudnn_inc}"] + defs +
         ["-c", str(ref_root / "h3_gpu_cuda.cu"), "-o", str(obj)])
    objs.append(str(obj))
    if have_cudnn:
        obj = out_dir / "h3_gpu_cuda_sdpa_cudnn.o"
        _run(["g++", "-std=c++17", "-O2", "-fPIC", "-w", f"-I{ref_root}",
              f"-I{ref_root / 'third_party' / 'cudnn_frontend' / 'include'}", f"-I{cudnn_inc}",
              f"-I{cuda_home / 'include'}"] + defs +
             ["-c", str(ref_root / "h3_gpu_cuda_sdpa_cudnn.cpp"), "-o", str(obj)])
        objs.append(str(obj))
    for name in ("h3_w4a8_dequant.c", "h3_w4a8.c", "h3_safetensors.c", "h3_sdpa_registry.c", "h3_cuda_device_caps.c"):
        obj = out_dir / (Path(name).stem + ".o")
        _run(["gcc", "-std=c11", "-O2", "-fPIC", "-D_GNU_SOURCE", "-w", f"-I{ref_root}",
              f"-I{cuda_home / 'include'}", "-c", str(ref_root / name), "-o", str(obj)])
        objs.append(str(obj))
    # two launchers of the reference's VAE library are referenced but never reached from the DiT operators
    stub_c = out_dir / "vae_stubs.c"
    stub_c.write_text("void h3_cuda_vae_launch_f16_unpad(void) {}\nvoid h3_cuda_vae_launch_qkv_rope_f16_in(void) {}\n")
    _run(["gcc", "-fPIC", "-c", str(stub_c), "-o", str(out_dir / "vae_stubs.o")])
    objs.append(str(out_dir / "vae_stubs.o"))
    lib64 = cuda_home / "lib64"
    _run(["g++", "-shared", "-Wl,-z,defs", "-o", str(out)] + objs +
         [f"-L{lib64}", f"-L{lib64 / 'stubs'}", f"-Wl,-rpath,{lib64}", "-lcublas", "-lcublasLt", "-lcudart"] +
         (["-lcudnn"] if have_cudnn else []) + ["-lcuda", "-ldl", "-lpthread", "-lm"])
    return out


# Reference translation units of the DiT host and of the weight formats beneath it (no GPU code): together
# with libh3_b200.so in place of the reference's CUDA operator library they are the reference's whole DiT stack.
REF_HOST_OBJECTS = ["h3_dit_w4a8", "h3_w4a8_cache", "h3_w4a8_dequant", "h3_w4a8", "h3_safetensors", "h3_dit_int8",
                    "h3_dit_nvfp4", "h3_nvfp4", "h3_lora", "h3_sdpa_registry", "h3_cuda_device_caps"]


def build_ref_host(ref_root: Path, product_lib: Path, force: bool = False) -> Path | None:
    """Links the reference's UNMODIFIED DiT host objects (compiled by build_ref from the sources where they lie)
    against the product library, refusing any undefined symbol: oracle/_ref/libh3_refhost.so.  That the link
    succeeds is the drop-in check; the GPU tests then drive the reference's own h3_dit_w4a8_* entry points
    through it.  Returns None when neither the reference tree nor prebuilt objects exist."""
    out = REF_OUT / "libh3_refhost.so"
    objs = [REF_OUT / f"{name}.o" for name in REF_HOST_OBJECTS]
    if not all(o.exists() for o in objs):
        if not ref_root.is_dir() or build_ref(ref_root, force) is None:
            return out if out.exists() else None
    if not all(o.exists() for o in objs):
        return None
    if not force and _newer(out, objs + [product_lib]):
        return out
    cuda_lib = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "lib64"
    _run(["gcc", "-shared", "-Wl,-z,defs", "-o", str(out)] + [str(o) for o in objs] +
         [f"-L{product_lib.parent}", "-lh3_b200", "-Wl,-rpath,$ORIGIN/../../h3c_b200", f"-L{cuda_lib}",
          f"-Wl,-rpath,{cuda_lib}", "-lcudart", "-lm", "-lpthread", "-ldl"])
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-root", default=str(default_ref_root()))
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args()
    print("oracle:", build_oracle(args.force))
    print("ref   :", build_ref(Path(args.ref_root), args.force))
    print("refcuda:", build_ref_cuda(Path(args.ref_root), args.force))
    print("refhost:", build_ref_host(Path(args.ref_root), HERE.parent / "h3c_b200" / "libh3_b200.so", args.force))


if __name__ == "__main__":
    main()
