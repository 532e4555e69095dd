"""Generates tests/golden/*.npz by running the REFERENCE itself on seeded inputs.

Two sources, both read in place from the h3.c tree (nothing is copied):
  * oracle/_ref/libh3_ref.so -- the reference's C CPU functions (oracle/build.py builds it)
  * tools/quant_dit_nvfp4.py -- the reference's Python NVFP4 weight quantiser (imported)

Every file stores the inputs next to the reference's outputs, so the checks in
tests/test_golden.py need neither the reference tree nor a particular RNG.

Run where the reference tree is present:  python tests/golden/make_golden.py
"""
from __future__ import annotations

import importlib.util
import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

from oracle.pyoracle import Ref  # noqa: E402

REF_ROOT = Path(os.environ["H3_REFERENCE_ROOT"]) if os.environ.get("H3_REFERENCE_ROOT") else ROOT.parent / "reference"


def save(name, **arrays):
    np.savez_compressed(HERE / f"{name}.npz", **arrays)
    print(f"{name}.npz", {k: v.shape for k, v in arrays.items()})


def main():
    ref = Ref()
    rng = np.random.default_rng(0)

    # ---- scalar format tables
    e4m3 = np.array([ref.lib.h3_f8e4m3fn_to_f32(b) for b in range(256)], np.float32)
    save("f8e4m3fn_table", table=e4m3)

    # ---- W4A8 decode (packed nibbles + codebook + e4m3 group scales)
    n, k = 12, 128
    packed = rng.integers(-128, 128, size=(n, k // 2), dtype=np.int8)
    codebook = np.sort(rng.normal(0, 40, 16)).astype(np.float32)
    codebook[3] = 80.5  # forces a .5 tie after scaling by 1.0 and a clamp after scaling by 2
    s_rel = rng.integers(0x28, 0x48, size=(n, k // 16), dtype=np.uint8)  # e4m3 in [2^-2, 2^2)
    s_rel[0, 0] = 0x38  # exactly 1.0
    s_rel[0, 1] = 0x40  # exactly 2.0
    save("w4a8_decode", packed=packed, codebook=codebook, s_rel=s_rel,
         w_i8=ref.w4a8_dequant_to_int8(packed, codebook, s_rel, 16))

    # ---- Hadamard + ConvRot
    x = rng.normal(0, 1, (3, 512)).astype(np.float32)
    save("convrot", h16=ref.hadamard(16), h256_row3=ref.hadamard(256)[3], x=x, y=ref.convrot(x, 256),
         y_gs0=ref.convrot(x, 0))

    # ---- per-row INT8 activation quant: ties, a zero row, an outlier row
    x = rng.normal(0, 1, (6, 96)).astype(np.float32)
    x[1] = 0.0
    x[2, 5] = 50.0
    x[3] = np.round(x[3] * 4) / 4
    x[3, 0] = 127.0 / 4  # scale exactly 0.25 -> many exact .5 ties
    q, s = ref.quantize_act_int8(x)
    save("quantize_act_int8", x=x, q=q, scales=s)

    # ---- INT8 GEMM + dequant
    xi = rng.integers(-127, 128, (5, 64), dtype=np.int8)
    wi = rng.integers(-127, 128, (7, 64), dtype=np.int8)
    a = rng.uniform(0.01, 0.05, 5).astype(np.float32)
    sc = rng.uniform(0.001, 0.01, 7).astype(np.float32)
    save("gemm_i8_dequant", x=xi, w=wi, a=a, s=sc, y=ref.gemm_i8_dequant(xi, wi, a, sc))

    # ---- fused epilogues (with and without a LoRA delta)
    rows, width, slots = 4, 8, 6
    acc2 = rng.integers(-5000, 5000, (rows, 2 * width), dtype=np.int32)
    acc1 = np.ascontiguousarray(acc2[:, :width])
    a = rng.uniform(0.001, 0.01, rows).astype(np.float32)
    s2 = rng.uniform(0.01, 0.1, 2 * width).astype(np.float32)
    lora2 = rng.normal(0, 0.05, (rows, 2 * width)).astype(np.float32)
    res = rng.normal(0, 1, (rows, width)).astype(np.float32)
    mod = rng.normal(0, 0.5, (3, slots, width)).astype(np.float32)
    rmap = np.array([0, 2, 1, 0], np.uint32)
    save("epilogues", acc2=acc2, a=a, s2=s2, lora2=lora2, residual=res, modulation=mod, row_map=rmap,
         swiglu=ref.dequant_swiglu(acc2, a, s2), swiglu_lora=ref.dequant_swiglu(acc2, a, s2, lora2),
         gate=ref.dequant_gate(acc1, a, s2[:width], res, mod, rmap, slots, 5),
         gate_lora=ref.dequant_gate(acc1, a, s2[:width], res, mod, rmap, slots, 2,
                                    np.ascontiguousarray(lora2[:, :width])))

    # ---- row-wise ops
    rows, width = 5, 64
    x = rng.normal(0, 1.5, (rows, width)).astype(np.float32)
    br = rng.normal(0, 1, (rows, width)).astype(np.float32)
    nw = rng.normal(1, 0.1, width).astype(np.float32)
    mod = rng.normal(0, 0.3, (3, 6, width)).astype(np.float32)
    rmap = np.array([0, 1, 2, 1, 0], np.uint32)
    gated, normed = ref.gate_adaln(x, br, nw, mod, rmap, 6, 2, 3, 4)
    fused = rng.normal(0, 2, (rows, 2 * width)).astype(np.float32)
    save("rowwise", x=x, branch=br, norm_w=nw, modulation=mod, row_map=rmap, fused=fused,
         rms=ref.rms_norm(x, nw), adaln=ref.adaln(x, nw, mod, rmap, 6, 0, 1),
         adaln_identity_map=ref.adaln(x[:3], nw, mod, None, 6, 3, 4),
         gate=ref.gate(x, br, mod, rmap, 6, 2), gated=gated, normed=normed, swiglu=ref.swiglu(fused))

    # ---- positions, RoPE tables, QK-norm + RoPE
    inv_freq = (1.0 / (10000.0 ** (np.arange(16) / 16.0))).astype(np.float32)
    pt, ph, pw = ref.fill_video_pos(256, 3, 8, 12)
    cos, sin = ref.rope_tables(inv_freq, pt, ph, pw, 1.0)
    seq, heads, hd = len(pt), 2, 128
    qkv = rng.normal(0, 1, (seq, 3 * heads * hd)).astype(np.float32)
    qn = rng.normal(1, 0.1, hd).astype(np.float32)
    kn = rng.normal(1, 0.1, hd).astype(np.float32)
    q, kk, v = ref.qkv_rope(qkv, qn, kn, cos, sin, heads, hd, 48)
    q0, k0, v0 = ref.qkv_rope(qkv[:4], qn, kn, None, None, heads, hd, 0)
    save("rope", inv_freq=inv_freq, pos_t=pt, pos_h=ph, pos_w=pw, cos=cos, sin=sin, qkv=qkv, q_norm=qn,
         k_norm=kn, q=q, k=kk, v=v, q_norope=q0, k_norope=k0)

    # ---- SDPA
    seq, heads, hd = 11, 3, 16
    q = rng.normal(0, 1, (seq, heads, hd)).astype(np.float32)
    kk = rng.normal(0, 1, (seq, heads, hd)).astype(np.float32)
    v = rng.normal(0, 1, (seq, heads, hd)).astype(np.float32)
    save("sdpa", q=q, k=kk, v=v, out=ref.sdpa(q, kk, v))

    # ---- Ulysses helpers (the cases tests/test_h3_ulysses.c checks, plus a sweep)
    cases = [(56, 64, 1, 1, 1), (56, 64, 1, 2, 1), (56, 64, 1, 4, 1), (56, 64, 1, 8, 1), (56, 64, 1, 7, 1),
             (56, 64, 1, 3, 1), (56, 64, 2, 4, 1), (56, 64, 4, 4, 1), (24, 64, 1, 8, 1), (24, 64, 1, 16, 1),
             (0, 64, 1, 2, 1), (24, 60, 1, 8, 1), (24, 64, 1, 2, 2)]
    valid = np.array([ref.ulysses_validate(*c) for c in cases], np.int32)
    seqs = np.array([15973, 50220, 6144, 64, 1, 0], np.uint64)
    pads = np.array([ref.lib.h3_ulysses_pad_seq(int(s), 64) for s in seqs], np.uint64)
    local = np.array([[ref.lib.h3_ulysses_local_rows(int(p), u, r) for r in range(-1, 9)]
                      for p in (16000, 50240, 10) for u in (1, 2, 4, 8)], np.uint64)
    save("ulysses_helpers", cases=np.array(cases, np.int32), valid=valid, seqs=seqs, pads=pads, local=local)

    # ---- misc host helpers pinned by tests/test_h3_dit_act_f16.c and test_h3_dit_fused_epi.c
    amax = np.array([0.0, 1.0, 1e5, 3000.0, 4000.0, 65504.0], np.float32)
    pre = np.array([[ref.lib.ref_act_f16_pre_scale(float(a), gs) for gs in (3, 32, 256)] for a in amax], np.float32)
    for var in ("H3_INT8_GEMM_TILE_M", "H3_INT8_GEMM_ACC_MIB"):
        os.environ.pop(var, None)
    tiles = np.array([ref.lib.ref_int8_gemm_tile_rows(m, n) for m, n in ((39000, 5376), (39000, 28672), (100, 64))],
                     np.uint64)
    save("host_helpers", absmax=amax, pre_scale=pre, tile_rows=tiles)

    # ---- reference-geometry block, composed exactly as tools/h3_dit_w4a8_block_probe.c:360-441
    D, H, hd, F, seq = 256, 2, 128, 512, 24
    def lin(nn, kk_):
        w = rng.normal(0, 0.05, (nn, kk_)).astype(np.float32)
        wi, ws = ref.quantize_act_int8(w)  # per-row symmetric int8 == per-channel weight quant
        return wi, ws
    W = {"qkv": lin(3 * D, D), "out": lin(D, D), "fc1": lin(2 * F, D), "fc2": lin(D, F)}
    x = rng.normal(0, 1, (seq, D)).astype(np.float32)
    mod = rng.normal(0, 0.3, (3, 6, D)).astype(np.float32)
    rmap = (np.arange(seq) % 3).astype(np.uint32)
    n1 = rng.normal(1, 0.1, D).astype(np.float32)
    n2 = rng.normal(1, 0.1, D).astype(np.float32)
    qn = rng.normal(1, 0.1, hd).astype(np.float32)
    kn = rng.normal(1, 0.1, hd).astype(np.float32)
    pt, ph, pw = ref.fill_video_pos(8, 2, 6, 8)
    cos, sin = ref.rope_tables(inv_freq, pt, ph, pw, 1.0)
    assert len(pt) == seq
    out = {}
    for gs in (0, 256):
        def clin(name, inp):
            wi, ws = W[name]
            q_, s_ = ref.quantize_act_int8(ref.convrot(inp, gs))
            return ref.gemm_i8_dequant(q_, wi, s_, ws)
        a_ = ref.adaln(x, n1, mod, rmap, 6, 0, 1)
        q_, k_, v_ = ref.qkv_rope(clin("qkv", a_), qn, kn, cos, sin, H, hd, 48)
        att = ref.sdpa(q_, k_, v_)
        x1 = ref.gate(x, clin("out", att), mod, rmap, 6, 2)
        a2 = ref.adaln(x1, n2, mod, rmap, 6, 3, 4)
        act = ref.swiglu(clin("fc1", a2))
        out[gs] = ref.gate(x1, clin("fc2", act), mod, rmap, 6, 5)
    save("block_r", x=x, modulation=mod, row_map=rmap, norm1=n1, norm2=n2, q_norm=qn, k_norm=kn, cos=cos, sin=sin,
         y_gs0=out[0], y_gs256=out[256], checksum_gs0=np.array([ref.checksum_f32(out[0])], np.uint64),
         **{f"w_{k_}": v_[0] for k_, v_ in W.items()}, **{f"s_{k_}": v_[1] for k_, v_ in W.items()})

    # ---- NVFP4 weight quantiser (Python reference)
    spec = importlib.util.spec_from_file_location("ref_quant_dit_nvfp4", REF_ROOT / "tools" / "quant_dit_nvfp4.py")
    mod_q = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod_q)
    w_i8 = rng.integers(-127, 128, (130, 128), dtype=np.int8)
    w_i8[5, :16] = 0
    scale = rng.uniform(1e-4, 2e-2, (130, 1)).astype(np.float32)
    scale[7] = 1e-7  # drives the UE4M3 subnormal/underflow clamp
    packed, sf = mod_q.quant_linear(w_i8, scale)
    vals = np.concatenate([np.float32(2.0) ** np.arange(-12, 10), rng.uniform(1e-4, 500, 64)]).astype(np.float32)
    save("nvfp4_weight", w_i8=w_i8, scale=scale, packed=packed, sf=sf, ue4m3_in=vals,
         ue4m3_bytes=mod_q.f32_to_ue4m3(vals), ue4m3_table=mod_q.ue4m3_to_f32(np.arange(0x7F, dtype=np.uint8)))

    step_sides(ref)
    step_tables(ref)


def step_sides(ref):
    """The step on either side of the block chain (own seed, so that it can be generated alone):
    patch embedding, final head = adaLN with one modulation row + dense, Euler update."""
    rng = np.random.default_rng(77)
    seq, hidden, patch = 70, 256, 96
    lat = rng.normal(0, 1, (seq, patch)).astype(np.float32)
    pw = rng.normal(0, 0.1, (hidden, patch)).astype(np.float32)
    pb = rng.normal(0, 0.1, hidden).astype(np.float32)
    x = rng.normal(0, 1, (seq, hidden)).astype(np.float32)
    norm_w = rng.normal(1, 0.1, hidden).astype(np.float32)
    mod = rng.normal(0, 0.2, (1, 2, hidden)).astype(np.float32)
    fw = rng.normal(0, 0.05, (patch, hidden)).astype(np.float32)
    fb = rng.normal(0, 0.1, patch).astype(np.float32)
    normed = ref.adaln(x, norm_w, mod, np.zeros(seq, np.uint32), 2, 0, 1)
    vel = ref.dense(normed, fw, fb)
    save("step_sides", latent=lat, patch_w=pw, patch_b=pb, embedded=ref.dense(lat, pw, pb), x=x, norm_w=norm_w,
         modulation=mod, final_w=fw, final_b=fb, velocity=vel, sigma=np.array([0.8, 0.55], np.float32),
         stepped=ref.euler_step(lat, vel, 0.8, 0.55))


def step_tables(ref):
    """Positions, RoPE tables and time-table rows of the three benchmark grids, as the reference computes
    them.  The tables are large (50,220 x 48), so the file keeps their FNV-1a checksums (the reference's own
    h3_dit_w4a8_checksum_f32) plus the first and last rows."""
    import ctypes as C
    inv_freq = (1.0 / (10000.0 ** (np.arange(16) / 16.0))).astype(np.float32)
    out = {"inv_freq": inv_freq, "grids": np.array([(6, 32, 32), (24, 32, 32), (31, 30, 54)], np.int32),
           "text_len": np.array([512], np.int64)}
    for i, g in enumerate(out["grids"]):
        pt, ph, pw = ref.fill_video_pos(512, int(g[0]), 2 * int(g[1]), 2 * int(g[2]))
        cos, sin = ref.rope_tables(inv_freq, pt, ph, pw, 1.0)
        out[f"sum_{i}"] = np.array([ref.checksum_f32(x) for x in (pt, ph, pw, cos, sin)], np.uint64)
        out[f"cos_head_{i}"], out[f"cos_tail_{i}"] = cos[:4], cos[-4:]
        out[f"sin_head_{i}"], out[f"sin_tail_{i}"] = sin[:4], sin[-4:]
    fn = ref.lib.h3_dit_w4a8_t_row_from_sigma
    fn.restype, fn.argtypes = C.c_size_t, [C.c_float, C.c_size_t]
    sig = np.concatenate([np.linspace(-0.25, 1.25, 61), [0.5, 0.49951171875, 0.999, 1e-4]]).astype(np.float32)
    out["sigma"] = sig
    out["t_rows"] = np.array([[fn(float(s), r) for r in (0, 1, 2, 1025)] for s in sig], np.uint64)
    out["span_sum"] = np.array([ref.lib.h3_dit_w4a8_video_span_sum(t) for t in range(0, 40)], np.float32) \
        if _span_ready(ref) else np.zeros(0, np.float32)
    save("step_tables", **out)


def _span_ready(ref):
    import ctypes as C
    ref.lib.h3_dit_w4a8_video_span_sum.restype = C.c_float
    ref.lib.h3_dit_w4a8_video_span_sum.argtypes = [C.c_int]
    return True


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "step_sides":
        step_sides(Ref())
    elif len(sys.argv) > 1 and sys.argv[1] == "step_tables":
        step_tables(Ref())
    else:
        main()
