"""The CPU restatement (oracle/h3_oracle.c) against vectors produced by the reference itself
(tests/golden/make_golden.py).  Integer/byte results must match bit for bit; float results
must match bit for bit as well where the restatement keeps the reference's operation order."""
import numpy as np

from tests.conftest import rel_l2


def test_f8e4m3fn_table(oracle, golden):
    g = golden("f8e4m3fn_table")["table"]
    mine = np.array([oracle.lib.ho_f8e4m3fn_to_f32(b) for b in range(256)], np.float32)
    assert np.array_equal(np.isnan(mine), np.isnan(g))
    ok = ~np.isnan(g)
    assert np.array_equal(mine[ok].view(np.uint32), g[ok].view(np.uint32))


def test_w4a8_decode(oracle, golden):
    g = golden("w4a8_decode")
    w = oracle.w4a8_dequant_to_int8(g["packed"], g["codebook"], g["s_rel"], 16)
    assert np.array_equal(w, g["w_i8"])
    assert w.min() >= -127 and w.max() <= 127


def test_convrot(oracle, golden):
    g = golden("convrot")
    assert np.array_equal(oracle.hadamard(16), g["h16"])
    assert np.array_equal(oracle.hadamard(256)[3], g["h256_row3"])
    assert np.array_equal(oracle.convrot(g["x"], 256), g["y"])
    assert np.array_equal(oracle.convrot(g["x"], 0), g["y_gs0"])
    # involution: applying the normalised Hadamard twice restores the input
    assert rel_l2(oracle.convrot(oracle.convrot(g["x"], 256), 256), g["x"]) < 1e-6


def test_quantize_act_int8(oracle, golden):
    g = golden("quantize_act_int8")
    q, s = oracle.quantize_act_int8(g["x"])
    assert np.array_equal(q, g["q"])
    assert np.array_equal(s.view(np.uint32), g["scales"].view(np.uint32))
    assert s[1] == 1.0 and not q[1].any()  # zero row -> scale 1, zero codes


def test_gemm_i8_dequant(oracle, golden):
    g = golden("gemm_i8_dequant")
    y = oracle.gemm_i8_dequant(g["x"], g["w"], g["a"], g["s"])
    assert np.array_equal(y.view(np.uint32), g["y"].view(np.uint32))
    acc = oracle.gemm_i8_i32(g["x"], g["w"])
    assert np.array_equal(acc, g["x"].astype(np.int32) @ g["w"].astype(np.int32).T)


def test_epilogues(oracle, golden):
    g = golden("epilogues")
    acc2, a, s2 = g["acc2"], g["a"], g["s2"]
    width = acc2.shape[1] // 2
    acc1 = np.ascontiguousarray(acc2[:, :width])
    assert np.array_equal(oracle.dequant_swiglu(acc2, a, s2), g["swiglu"])
    assert np.array_equal(oracle.dequant_swiglu(acc2, a, s2, g["lora2"]), g["swiglu_lora"])
    assert np.array_equal(oracle.dequant_gate(acc1, a, s2[:width], g["residual"], g["modulation"], g["row_map"], 6, 5),
                          g["gate"])
    assert np.array_equal(oracle.dequant_gate(acc1, a, s2[:width], g["residual"], g["modulation"], g["row_map"], 6, 2,
                                              np.ascontiguousarray(g["lora2"][:, :width])), g["gate_lora"])


def test_rowwise(oracle, golden):
    g = golden("rowwise")
    x, br, nw, mod, rmap = g["x"], g["branch"], g["norm_w"], g["modulation"], g["row_map"]
    assert np.array_equal(oracle.rms_norm(x, nw), g["rms"])
    assert np.array_equal(oracle.adaln(x, nw, mod, rmap, 6, 0, 1), g["adaln"])
    assert np.array_equal(oracle.adaln(x[:3], nw, mod, None, 6, 3, 4), g["adaln_identity_map"])
    assert np.array_equal(oracle.gate(x, br, mod, rmap, 6, 2), g["gate"])
    gated, normed = oracle.gate_adaln(x, br, nw, mod, rmap, 6, 2, 3, 4)
    assert np.array_equal(gated, g["gated"]) and np.array_equal(normed, g["normed"])
    assert np.array_equal(oracle.swiglu(g["fused"]), g["swiglu"])


def test_rope(oracle, golden):
    g = golden("rope")
    pt, ph, pw = oracle.fill_video_pos(256, 3, 8, 12)
    assert np.array_equal(pt, g["pos_t"]) and np.array_equal(ph, g["pos_h"]) and np.array_equal(pw, g["pos_w"])
    cos, sin = oracle.rope_tables(g["inv_freq"], pt, ph, pw, 1.0)
    assert np.array_equal(cos, g["cos"]) and np.array_equal(sin, g["sin"])
    q, k, v = oracle.qkv_rope(g["qkv"], g["q_norm"], g["k_norm"], cos, sin, 2, 128, 48)
    assert np.array_equal(q, g["q"]) and np.array_equal(k, g["k"]) and np.array_equal(v, g["v"])
    q0, k0, _ = oracle.qkv_rope(g["qkv"][:4], g["q_norm"], g["k_norm"], None, None, 2, 128, 0)
    assert np.array_equal(q0, g["q_norope"]) and np.array_equal(k0, g["k_norope"])


def test_sdpa(oracle, golden):
    g = golden("sdpa")
    assert np.array_equal(oracle.sdpa(g["q"], g["k"], g["v"]), g["out"])


def test_ulysses_helpers(oracle, golden):
    g = golden("ulysses_helpers")
    mine = np.array([oracle.lib.ho_ulysses_validate(*map(int, c)) for c in g["cases"]], np.int32)
    assert np.array_equal(mine, g["valid"])
    pads = np.array([oracle.lib.ho_ulysses_pad_seq(int(s), 64) for s in g["seqs"]], np.uint64)
    assert np.array_equal(pads, g["pads"])
    assert oracle.lib.ho_ulysses_pad_seq(15973, 64) == 16000  # tests/test_h3_ulysses.c "cafe pad"
    local = np.array([[oracle.lib.ho_ulysses_local_rows(int(p), u, r) for r in range(-1, 9)]
                      for p in (16000, 50240, 10) for u in (1, 2, 4, 8)], np.uint64)
    assert np.array_equal(local, g["local"])


def test_block_r(oracle, golden):
    g = golden("block_r")
    W = {k: (g[f"w_{k}"], g[f"s_{k}"]) for k in ("qkv", "out", "fc1", "fc2")}
    for k in ("norm1", "norm2", "q_norm", "k_norm", "modulation"):
        W[k] = g[k]
    for gs in (0, 256):
        y = oracle.block_r(W, g["x"], g["cos"], g["sin"], g["row_map"], heads=2, head_dim=128, ffn=512,
                           quantised=True, convrot_gs=gs)
        assert np.array_equal(y, g[f"y_gs{gs}"])
    assert oracle.checksum_f32(g["y_gs0"]) == int(g["checksum_gs0"][0])


def test_nvfp4_weight_quantiser(oracle, golden):
    """The reference's Python weight quantiser and its CUDA activation quantiser implement the same
    rule (tools/quant_dit_nvfp4.py:65-107, h3_gpu_cuda.cu:4539-4614); the restatement must reproduce
    the Python one byte for byte."""
    g = golden("nvfp4_weight")
    w = g["w_i8"].astype(np.float32) * g["scale"].astype(np.float32)
    packed, sf = oracle.quantize_nvfp4(w, rule=1)
    assert np.array_equal(packed, g["packed"])
    # the CUDA activation rule differs from the Python one only in the sign bit of zeros
    packed0, sf0 = oracle.quantize_nvfp4(w, rule=0)
    assert np.array_equal(sf0, sf)
    assert np.array_equal(oracle.dequant_nvfp4(packed0, sf0), oracle.dequant_nvfp4(packed, sf))
    assert np.array_equal(sf, g["sf"])
    # Scale bytes: the restatement follows the CUDA helper (h3_gpu_cuda.cu:4498).  The Python helper
    # differs from it only at the edges: once the rounded value reaches 256 (inputs from 240 up) the
    # CUDA helper returns 0x7E (it treats biased exponent 15 as out of range) while the Python one
    # clips the exponent to 14 and keeps the wrapped mantissa, and on subnormal
    # ties Python rounds half to even (np.rint) instead of half away (lroundf).  Inside [2^-6, 240)
    # the two agree and must be reproduced exactly.
    vin = g["ue4m3_in"]
    mine = np.array([oracle.lib.ho_f32_to_ue4m3(float(v)) for v in vin], np.uint8)
    normal = (vin >= 2.0 ** -6) & (vin < 240.0)
    assert normal.sum() > 20
    assert np.array_equal(mine[normal], g["ue4m3_bytes"][normal])
    assert all(b == 0x7E for b in mine[vin >= 256.0])
    assert oracle.lib.ho_f32_to_ue4m3(2.0 ** -10) == 1 and oracle.lib.ho_f32_to_ue4m3(0.0) == 0
    tab = np.array([oracle.lib.ho_ue4m3_to_f32(b) for b in range(0x7F)], np.float32)
    assert np.array_equal(tab, g["ue4m3_table"])


def test_nvfp4_sf_bytes(oracle):
    # tests/test_h3_nvfp4_sf_bytes.c
    assert oracle.nvfp4_sf_bytes(21504, 5376) == 168 * 84 * 512
    assert oracle.nvfp4_sf_bytes(5376, 14336) == 42 * 224 * 512
    assert oracle.nvfp4_sf_bytes(1, 64) == 512
    assert oracle.nvfp4_sf_bytes(256, 512) == 2 * 8 * 512
    assert oracle.nvfp4_sf_bytes(1, 63) == 0 and oracle.nvfp4_sf_bytes(0, 64) == 0


def test_step_sides(oracle, golden):
    """Patch embedding, final head and Euler update against vectors the reference's own functions produced
    (h3_dit_w4a8_dense_f32, h3_dit_w4a8_adaln_f32, h3_dit_w4a8_euler_step_f32)."""
    g = golden("step_sides")
    assert np.array_equal(oracle.dense(g["latent"], g["patch_w"], g["patch_b"]), g["embedded"])
    vel = oracle.final_head(g["x"], g["norm_w"], g["modulation"], g["final_w"], g["final_b"])
    assert np.array_equal(vel, g["velocity"])
    s0, s1 = (float(v) for v in g["sigma"])
    assert np.array_equal(oracle.euler_step(g["latent"], vel, s0, s1), g["stepped"])
