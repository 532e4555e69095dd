"""Builds the two checker libraries used by the test-suite (never by the product):

  oracle/_build/libh3_oracle.so  -- this repository's CPU restatement (h3_oracle.c)
  oracle/_ref/libh3_ref.so       -- the reference's own CPU functions, compiled from the
                                    h3.c sources where they lie (read-only, nothing copied)

The reference's DiT source file also contains its CUDA orchestration, so it has many
undefined h3_cuda_* / cuda* symbols.  Its CPU functions never reach them; they are given
aborting stubs generated from `nm -u` so the shared object loads without a CUDA runtime.

Usage: python oracle/build.py [--ref-root PATH]   (default PATH: $H3_REFERENCE_ROOT or /root/reference)
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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-root", default=os.environ.get("H3_REFERENCE_ROOT", "/root/reference"))
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args()
    print("oracle:", build_oracle(args.force))
    print("ref   :", build_ref(Path(args.ref_root), args.force))


if __name__ == "__main__":
    main()
