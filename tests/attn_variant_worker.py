"""Child process of tests/test_gpu_attn_variants.py: the attention kernel variant is chosen by H3B_ATTN_EMU when the
library first launches the kernel, so each variant gets a process of its own.  Prints one JSON object: the relative L2
error against f64 attention for every shape given on the command line as lq,lk,heads."""
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import h3c_b200  # noqa: E402


def main():
    dtype = torch.float16 if sys.argv[1] == "f16" else torch.bfloat16
    cuda = h3c_b200.Cuda(0)
    g = torch.Generator(device="cuda")
    g.manual_seed(0)
    out = {}
    for spec in sys.argv[2:]:
        lq, lk, heads = (int(v) for v in spec.split(","))
        q = torch.randn((lq, heads, 128), generator=g, device="cuda").to(dtype)
        k = torch.randn((lk, heads, 128), generator=g, device="cuda").to(dtype)
        v = torch.randn((lk, heads, 128), generator=g, device="cuda").to(dtype)
        o = cuda.sdpa(q, k, v)
        s = torch.einsum("qhd,khd->hqk", q.double(), k.double()) * 128 ** -0.5
        want = torch.einsum("hqk,khd->qhd", torch.softmax(s, dim=-1), v.double()).reshape(lq, -1)
        out[spec] = float((o.double() - want).norm() / want.norm())
    cuda.check()
    cuda.close()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
