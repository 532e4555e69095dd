"""Single-kernel cases on synthetic data: times one operator of the library with CUDA events and prints
achieved TFLOP/s or GB/s.  Also the small, self-contained commands used for ncu captures.

    python -m h3c_b200.cases gemm --m 6144 --n 9216 --k 3072 [--epi plain|gate|gelu|swiglu]
    python -m h3c_b200.cases attn --lq 6144 --lk 6144 --heads 24
    python -m h3c_b200.cases norm --m 6144 --k 3072 [--plain-quant]
    python -m h3c_b200.cases rope --m 6144 --heads 24
    python -m h3c_b200.cases gemm_fp4 --m 6144 --n 9216 --k 3072
    python -m h3c_b200.cases peak            # tensor-pipe rate, burst and sustained
"""
from __future__ import annotations

import argparse
import json

import numpy as np


def _time(fn, iters, warmup=3):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    import torch
    import h3c_b200
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "gemm_fp4", "attn", "norm", "rope", "peak", "sides"])
    ap.add_argument("--m", type=int, default=6144)
    ap.add_argument("--n", type=int, default=9216)
    ap.add_argument("--k", type=int, default=3072)
    ap.add_argument("--lq", type=int, default=6144)
    ap.add_argument("--lk", type=int, default=0)
    ap.add_argument("--heads", type=int, default=24)
    ap.add_argument("--epi", default="plain", choices=["plain", "gate", "gelu", "swiglu", "qkv"])
    ap.add_argument("--plain-quant", action="store_true")
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    cuda = h3c_b200.Cuda(0)
    g = torch.Generator(device="cuda")
    g.manual_seed(0)
    out = {"case": a.case}
    if a.case == "gemm":
        w_i8 = np.random.default_rng(0).integers(-127, 128, (a.n, a.k), dtype=np.int8)
        w = cuda.weight_from_i8(w_i8, np.full(a.n, 1e-3, np.float32))
        x = torch.randint(-127, 128, (a.m, a.k), generator=g, device="cuda", dtype=torch.int8)
        s = torch.full((a.m,), 0.01, device="cuda")
        if a.epi == "qkv":   # QKV projection with QK-norm and RoPE in the epilogue (N = 3 * heads * 128)
            qn = torch.ones(128, device="cuda")
            cos = torch.rand((a.m, 64), generator=g, device="cuda")
            sin = torch.rand((a.m, 64), generator=g, device="cuda")
            ms = _time(lambda: cuda.gemm_i8_qkv_rope(w, x, s, qn, qn, cos, sin, 64), a.iters)
            out.update(m=a.m, n=a.n, k=a.k, epi=a.epi, ms=ms, tops=2.0 * a.m * a.n * a.k / ms / 1e9)
            print(json.dumps(out))
            return
        kind = {"plain": h3c_b200.EPI_PLAIN, "gate": h3c_b200.EPI_GATE, "gelu": h3c_b200.EPI_GELU,
                "swiglu": h3c_b200.EPI_SWIGLU}[a.epi]
        n_out = a.n // 2 if a.epi == "swiglu" else a.n
        y = torch.empty((a.m, n_out), dtype=torch.bfloat16, device="cuda")
        res = torch.zeros_like(y) if a.epi == "gate" else None
        ms = _time(lambda: cuda.gemm_i8(w, x, s, kind=kind, residual=res, out=y), a.iters)
        out.update(m=a.m, n=a.n, k=a.k, epi=a.epi, ms=ms, tops=2.0 * a.m * a.n * a.k / ms / 1e9)
    elif a.case == "peak":
        import ctypes as C
        from .lib import call
        for kind, name in ((0, "int8"), (1, "bf16"), (2, "nvfp4"), (3, "bf16_n128_ss"), (4, "bf16_n128_ts"), (5, "nvfp4_n128")):
            v = C.c_double(0)
            call("h3b_umma_peak_dev", cuda.h, kind, 20000, C.byref(v))     # ~10 ms of MMAs: burst clocks
            out[name + "_burst_tops"] = v.value
            call("h3b_umma_peak_dev", cuda.h, kind, 2000000, C.byref(v))   # ~1 s: under the power limit
            out[name + "_sustained_tops"] = v.value
    elif a.case == "sides":   # patch embedding, final head and Euler update of a.m tokens (f32, hidden = a.n)
        lat = torch.randn((a.m, 96), generator=g, device="cuda")
        pw, pb = torch.randn((a.n, 96), generator=g, device="cuda"), torch.randn(a.n, generator=g, device="cuda")
        x = torch.randn((a.m, a.n), generator=g, device="cuda")
        nw, mod = torch.ones(a.n, device="cuda"), torch.zeros((2, a.n), device="cuda")
        fw, fb = torch.randn((96, a.n), generator=g, device="cuda"), torch.randn(96, generator=g, device="cuda")
        vel = torch.randn((a.m, 96), generator=g, device="cuda")
        out.update(m=a.m, hidden=a.n,
                   patch_embed_ms=_time(lambda: cuda.dense_f32(lat, pw, pb), a.iters),
                   final_head_ms=_time(lambda: cuda.final_head_f32(x, nw, mod, fw, fb), a.iters),
                   euler_ms=_time(lambda: cuda.euler_step_f32(lat, vel, 0.8, 0.7), a.iters))
    elif a.case == "gemm_fp4":
        x4 = torch.randint(0, 256, (a.m, a.k // 2), generator=g, device="cuda", dtype=torch.uint8)
        w4 = torch.randint(0, 256, (a.n, a.k // 2), generator=g, device="cuda", dtype=torch.uint8)
        sfb = lambda rows: int(h3c_b200.load().h3_cuda_nvfp4_sf_bytes(rows, a.k))
        sfx = torch.full((sfb(a.m),), 0x38, device="cuda", dtype=torch.uint8)
        sfw = torch.full((sfb(a.n),), 0x38, device="cuda", dtype=torch.uint8)
        ms = _time(lambda: cuda.gemm_fp4(w4, sfw, x4, sfx, out_dtype=torch.bfloat16), a.iters)
        out.update(m=a.m, n=a.n, k=a.k, ms=ms, tflops=2.0 * a.m * a.n * a.k / ms / 1e9)
    elif a.case == "attn":
        lk = a.lk or a.lq
        q = torch.randn((a.lq, a.heads, 128), generator=g, device="cuda").to(torch.bfloat16)
        k = torch.randn((lk, a.heads, 128), generator=g, device="cuda").to(torch.bfloat16)
        v = torch.randn((lk, a.heads, 128), generator=g, device="cuda").to(torch.bfloat16)
        o = torch.empty((a.lq, a.heads * 128), dtype=torch.bfloat16, device="cuda")
        ms = _time(lambda: cuda.sdpa_bf16(q, k, v, out=o), a.iters)
        out.update(lq=a.lq, lk=lk, heads=a.heads, ms=ms, tflops=4.0 * a.lq * lk * a.heads * 128 / ms / 1e9)
    elif a.case == "norm":
        x = torch.randn((a.m, a.k), generator=g, device="cuda").to(torch.bfloat16)
        q = torch.empty((a.m, a.k), dtype=torch.int8, device="cuda")
        s = torch.empty(a.m, dtype=torch.float32, device="cuda")
        if a.plain_quant:
            ms = _time(lambda: cuda.norm(x, identity=True, q=q, scales=s), a.iters)
        else:
            nw = torch.ones(a.k, device="cuda")
            mod = torch.zeros((1, 6, a.k), device="cuda")
            rm = torch.zeros(a.m, dtype=torch.int32, device="cuda")
            ms = _time(lambda: cuda.norm(x, norm_w=nw, modulation=mod, row_map=rm, slots=6, shift_slot=0, scale_slot=1,
                                         q=q, scales=s), a.iters)
        out.update(m=a.m, k=a.k, ms=ms, gbs=(a.m * a.k * 3 + a.m * 4) / ms / 1e6)
    else:
        qkv = torch.randn((a.m, 3 * a.heads * 128), generator=g, device="cuda").to(torch.bfloat16)
        qn = torch.ones(128, device="cuda")
        cos = torch.ones((a.m, 48), device="cuda")
        sin = torch.zeros((a.m, 48), device="cuda")
        ms = _time(lambda: cuda.qkv_rope(qkv, qn, qn, cos, sin, a.heads, 128, 48), a.iters)
        out.update(m=a.m, heads=a.heads, ms=ms, gbs=a.m * a.heads * 128 * 3 * 4 / ms / 1e6)
    cuda.check()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
