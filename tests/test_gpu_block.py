"""Whole-block and block-chain parity through the C ABI (h3b_dit_*) against the CPU oracle."""
import os

import numpy as np
import pytest

from tests.conftest import GOLDEN, rel_l2

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def cuda():
    import h3c_b200
    c = h3c_b200.Cuda(0)
    yield c
    c.check()
    c.close()


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def rope_for(oracle, text_len, t, h, w):
    inv_freq = (1.0 / (10000.0 ** (np.arange(16) / 16.0))).astype(np.float32)
    pt, ph, pw = oracle.fill_video_pos(text_len, t, 2 * h, 2 * w)
    return oracle.rope_tables(inv_freq, pt, ph, pw, 1.0)


def test_reference_block_f32_stream_against_reference_vectors(cuda, oracle):
    """The reference's block (SwiGLU, row map with three modalities), f32 residual stream, against the
    output the reference's own CPU functions produced (tests/golden/block_r.npz)."""
    from h3c_b200 import dit as D
    g = np.load(GOLDEN / "block_r.npz")
    for gs in (0, 256):
        geo = D.DitGeometry(dim=256, heads=2, head_dim=128, ffn=512, n_blocks=1, mod_rows=3, t_dim=8,
                            kind=D.BLOCK_REFERENCE, stream_dtype=D.F32, convrot_gs=gs)
        dit = D.Dit(cuda, geo)
        for name, slot in D.LIN_NAMES_REF.items():
            dit.set_linear(0, slot, cuda.weight_from_i8(g[f"w_{name}"], g[f"s_{name}"]))
        dit.set_block_aux(0, g["norm1"], g["norm2"], g["q_norm"], g["k_norm"])
        y = dit.block_forward(0, dev(g["x"]), dev(g["cos"]), dev(g["sin"]), modulation=dev(g["modulation"]),
                              row_map=dev(g["row_map"].view(np.int32)))
        cuda.check()
        err = rel_l2(y.cpu().numpy(), g[f"y_gs{gs}"])
        # attention runs in bf16 on the tensor cores; everything else is f32 / exact int32
        assert err < 2e-3, (gs, err)
        dit.close()


@pytest.mark.parametrize("fp4_linears,gs", [((0, 1, 2, 3), 0), ((0, 1, 2, 3), 256), ((2, 3), 256)])
def test_reference_block_with_nvfp4_linears(cuda, oracle, fp4_linears, gs):
    """Per-linear NVFP4 / INT8 choice in the reference block (the reference's nvfp4_gemm_dispatch,
    h3_dit_w4a8.c:3519-3590): the chosen linears run ConvRot -> NVFP4 activation quantisation -> block-scaled GEMM with
    the plain / SwiGLU / gate epilogue, the others stay INT8.  Checked against the same block put together from the
    CPU checker's operators, with the NVFP4 linears as its quantiser + block-scaled product.  Bound 3e-2 (measured 0.9e-2 to
    1.3e-2): the bf16 attention output differs from the checker's by 2e-3, and wherever that difference, carried along
    the residual stream, moves an input of a later NVFP4 linear across a 4-bit code boundary, that input changes by up
    to a sixth of its block maximum (the operator tests hold each NVFP4 linear to 1e-5 on identical inputs; the INT8
    block, whose codes are 1/127 apart, holds 2e-3).  The NVFP4 block sits 3.7e-2 to 4e-2 from the INT8 block."""
    from h3c_b200 import dit as D
    g = np.load(GOLDEN / "block_r.npz")
    dim, heads, hd, ffn, slots = 256, 2, 128, 512, 6
    geo = D.DitGeometry(dim=dim, heads=heads, head_dim=hd, ffn=ffn, n_blocks=1, mod_rows=3, t_dim=8,
                        kind=D.BLOCK_REFERENCE, stream_dtype=D.F32, convrot_gs=gs)
    dit = D.Dit(cuda, geo)
    names = ["qkv", "out", "fc1", "fc2"]
    fp4, handles = {}, []
    for i, name in enumerate(names):
        dit.set_linear(0, D.LIN_NAMES_REF[name], cuda.weight_from_i8(g[f"w_{name}"], g[f"s_{name}"]))
        if i in fp4_linears:
            w = g[f"w_{name}"].astype(np.float32) * g[f"s_{name}"][:, None]
            amax = float(np.abs(w).max())
            scale2 = np.float32(amax / (6.0 * 448.0))              # per-tensor second-level scale of the sidecar
            w4, sfw = oracle.quantize_nvfp4(w / scale2, rule=1)
            h = cuda.nvfp4_weight(w4, sfw, float(scale2), *w.shape)
            handles.append(h)
            dit.set_linear_nvfp4(0, D.LIN_NAMES_REF[name], h)
            fp4[name] = (w4, sfw, scale2)
    dit.set_block_aux(0, g["norm1"], g["norm2"], g["q_norm"], g["k_norm"])
    x, cos, sin, mod, rmap = g["x"], g["cos"], g["sin"], g["modulation"], g["row_map"]
    y = dit.block_forward(0, dev(x), dev(cos), dev(sin), modulation=dev(mod), row_map=dev(rmap.view(np.int32)))
    cuda.check()

    def linear(name, a):
        a = oracle.convrot(a, gs) if gs else a
        if name in fp4:
            w4, sfw, scale2 = fp4[name]
            a4, sfa = oracle.quantize_nvfp4(a)
            return oracle.gemm_nvfp4(a4, sfa, w4, sfw, scale2)
        codes, scales = oracle.quantize_act_int8(a)
        return oracle.gemm_i8_dequant(codes, g[f"w_{name}"], scales, g[f"s_{name}"])

    a = oracle.adaln(x, g["norm1"], mod, rmap, slots, 0, 1)
    q, k, v = oracle.qkv_rope(linear("qkv", a), g["q_norm"], g["k_norm"], cos, sin, heads, hd, 48)
    att = oracle.bf16_round(oracle.sdpa(q, k, v))                   # the kernel hands the out projection bf16 rows
    x1 = oracle.gate(x, linear("out", att.reshape(x.shape[0], -1)), mod, rmap, slots, 2)
    h1 = oracle.swiglu(linear("fc1", oracle.adaln(x1, g["norm2"], mod, rmap, slots, 3, 4)))
    want = oracle.gate(x1, linear("fc2", h1), mod, rmap, slots, 5)
    err = rel_l2(y.cpu().numpy(), want)
    far = rel_l2(y.cpu().numpy(), g[f"y_gs{gs}"])
    print(f"NVFP4 linears {fp4_linears}, ConvRot {gs}: rel-L2 vs the checker's NVFP4 block {err:.2e}, vs the INT8 block {far:.2e}")
    assert err < 3e-2, (fp4_linears, gs, err)
    # it is the NVFP4 block that ran (4-bit weights and activations sit percents away from the INT8 block), not INT8
    assert err < 0.5 * far < 0.2
    if 0 in fp4_linears:
        # QK-norm and RoPE in the NVFP4 QKV epilogue (the default) and as a stand-alone kernel give the same bits
        os.environ["H3B_FP4_QKV_ROPE"] = "0"
        try:
            y2 = dit.block_forward(0, dev(x), dev(cos), dev(sin), modulation=dev(mod), row_map=dev(rmap.view(np.int32)))
            cuda.check()
        finally:
            del os.environ["H3B_FP4_QKV_ROPE"]
        assert torch.equal(y, y2)
    dit.close()
    for h in handles:
        cuda.nvfp4_weight_free(h)


def make_cross_case(cuda, oracle, seed, grid, text_len, dim, heads, ffn, n_blocks=1):
    from h3c_b200 import dit as D
    geo = D.DitGeometry(dim=dim, heads=heads, head_dim=128, ffn=ffn, n_blocks=n_blocks, mod_rows=1, t_dim=32,
                        kind=D.BLOCK_CROSS_GELU, stream_dtype=D.BF16)
    dit, host = D.build_synthetic(cuda, geo, seed=seed, keep_host=True)
    rng = np.random.default_rng(seed + 100)
    seq = grid[0] * grid[1] * grid[2]
    x = rng.normal(0, 1, (seq, dim)).astype(np.float32)
    text = rng.normal(0, 1, (text_len, dim)).astype(np.float32)
    t_feat = rng.normal(0, 1, geo.t_dim).astype(np.float32)
    cos, sin = rope_for(oracle, text_len, *grid)
    return geo, dit, host, x, text, t_feat, cos, sin


def oracle_weights(oracle, rec, t_feat, quantised):
    W = {}
    for name in ("qkv", "o", "cq", "ckv", "co", "up", "down"):
        w_i8, s = oracle.w4g128_decode_to_int8(*rec[name])
        W[name] = (w_i8, s) if quantised else (w_i8.astype(np.float32) * s[:, None])
    for name in ("norm1", "norm_c", "norm2", "q_norm", "k_norm"):
        W[name] = rec[name]
    W["modulation"] = oracle.adaln_project(rec["adaln_w"], rec["adaln_b"], t_feat).reshape(6, -1)
    return W


def test_cross_gelu_block_bf16_stream(cuda, oracle):
    """The benchmark's block on its own grid shape in miniature: (4,8,8) tokens, 64 text tokens."""
    geo, dit, host, x, text, t_feat, cos, sin = make_cross_case(cuda, oracle, 1, (4, 8, 8), 64, 256, 2, 512)
    dit.project_modulation(dev(t_feat))
    mod = dit.modulation(0).cpu().numpy()
    W = oracle_weights(oracle, host[0], t_feat, True)
    assert rel_l2(mod.reshape(6, -1), W["modulation"]) < 1e-5
    xb = dev(x, torch.bfloat16)
    tb = dev(text, torch.bfloat16)
    # one modulation row shared by every token: the row map is all zeros (NULL would mean row r -> row r)
    rmap = torch.zeros(x.shape[0], dtype=torch.int32, device="cuda")
    y = dit.block_forward(0, xb, dev(cos), dev(sin), text=tb, row_map=rmap)
    cuda.check()
    xh, th = xb.float().cpu().numpy(), tb.float().cpu().numpy()
    kw = dict(heads=2, head_dim=128, ffn=512)
    same = oracle.block_b(W, xh, th, cos, sin, quantised=True, bf16_stream=True, **kw)
    e_same = rel_l2(y.float().cpu().numpy(), same)
    # same-precision oracle (int8 linears, bf16 stored tensors): <= 2e-3 relative L2
    assert e_same < 2e-3, e_same
    full = oracle.block_b(oracle_weights(oracle, host[0], t_feat, False), xh, th, cos, sin, quantised=False,
                          bf16_stream=False, **kw)
    e_full = rel_l2(y.float().cpu().numpy(), full)
    # fp32 CPU block (f32 weights, no activation quantisation): <= 2e-2 relative L2
    assert e_full < 2e-2, e_full
    dit.close()


def test_block_at_the_cpu_plumbing_config_shape(cuda, oracle):
    """The benchmark's first configuration at its stated shape: hidden 3072, 24 x 128 heads, FFN 12288 with
    tanh-GELU, 1,024 video tokens (16 x 16 patches x 4 latent frames) + 256 text tokens, seed 0.  The GPU block
    (int4 group-128 weights, int8 activations, bf16 stream) against the CPU block at the same precision and against
    the f32 CPU block; the f32 block's FNV-1a checksum (h3_dit_w4a8.c:8911) is printed for the record."""
    geo, dit, host, x, text, t_feat, cos, sin = make_cross_case(cuda, oracle, 0, (4, 16, 16), 256, 3072, 24, 12288)
    assert x.shape == (1024, 3072) and text.shape == (256, 3072)
    dit.project_modulation(dev(t_feat))
    xb, tb = dev(x, torch.bfloat16), dev(text, torch.bfloat16)
    rmap = torch.zeros(x.shape[0], dtype=torch.int32, device="cuda")
    y = dit.block_forward(0, xb, dev(cos), dev(sin), text=tb, row_map=rmap)
    cuda.check()
    xh, th = xb.float().cpu().numpy(), tb.float().cpu().numpy()
    kw = dict(heads=24, head_dim=128, ffn=12288)
    same = oracle.block_b(oracle_weights(oracle, host[0], t_feat, True), xh, th, cos, sin, quantised=True, bf16_stream=True, **kw)
    full = oracle.block_b(oracle_weights(oracle, host[0], t_feat, False), xh, th, cos, sin, quantised=False, bf16_stream=False, **kw)
    got = y.float().cpu().numpy()
    e_same, e_full = rel_l2(got, same), rel_l2(got, full)
    print(f"config 0 shape: rel-L2 {e_same:.2e} vs the same-precision CPU block, {e_full:.2e} vs the f32 CPU block; "
          f"FNV-1a of the f32 CPU block output 0x{oracle.checksum_f32(full):016x}")
    # the checker's "same precision" block keeps f32 attention probabilities where the kernel rounds them to bf16;
    # over 1,024 + 256 keys and 24 heads that is 4e-3 here (2e-3 on the miniature shapes of the other tests)
    assert e_same < 6e-3 and e_full < 2e-2
    dit.close()


def test_chain_host_entry_point_matches_device_chain(cuda, oracle):
    """h3b_dit_layers_forward_f32 (host buffers in/out) == cast + device chain, and two chained blocks
    agree with the oracle applied twice."""
    geo, dit, host, x, text, t_feat, cos, sin = make_cross_case(cuda, oracle, 2, (2, 8, 8), 32, 256, 2, 512, n_blocks=2)
    y_host = dit.layers_forward_f32(t_feat, x, cos, sin, text=text)
    dit.project_modulation(dev(t_feat))
    y_dev = dit.layers_forward(dev(x, torch.bfloat16), dev(cos), dev(sin), text=dev(text, torch.bfloat16),
                               row_map=torch.zeros(x.shape[0], dtype=torch.int32, device="cuda"))
    cuda.check()
    assert np.array_equal(y_host, y_dev.float().cpu().numpy())
    cur = dev(x, torch.bfloat16).float().cpu().numpy()
    th = dev(text, torch.bfloat16).float().cpu().numpy()
    for b in range(2):
        cur = oracle.block_b(oracle_weights(oracle, host[b], t_feat, True), cur, th, cos, sin, heads=2, head_dim=128,
                             ffn=512, quantised=True, bf16_stream=True)
    assert rel_l2(y_host, cur) < 3e-3
    assert dit.launches_per_block == 16
    dit.close()


def test_chain_as_cuda_graph_in_the_c_host(cuda, oracle):
    """h3b_dit_layers_forward_graph_dev: the C host captures the chain on the first call and replays it afterwards;
    replays follow a changed input, a re-projected modulation, and give the bits of the launched chain."""
    geo, dit, host, x, text, t_feat, cos, sin = make_cross_case(cuda, oracle, 7, (2, 8, 8), 32, 256, 2, 512, n_blocks=2)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        cuda.use_stream(side)            # capture needs a real stream
        d_x, d_text = dev(x, torch.bfloat16), dev(text, torch.bfloat16)
        d_cos, d_sin, d_t = dev(cos), dev(sin), dev(t_feat)
        rmap = torch.zeros(x.shape[0], dtype=torch.int32, device="cuda")
        out = torch.empty_like(d_x)
        dit.project_modulation(d_t)
        want = dit.layers_forward(d_x, d_cos, d_sin, text=d_text, row_map=rmap).clone()
        assert dit.graph_nodes == 0
        y1 = dit.layers_forward_graph(d_x, d_cos, d_sin, text=d_text, row_map=rmap, out=out).clone()     # eager + capture
        nodes = dit.graph_nodes
        assert nodes >= 2 * dit.launches_per_block
        cuda.launch_count(reset=True)
        y2 = dit.layers_forward_graph(d_x, d_cos, d_sin, text=d_text, row_map=rmap, out=out).clone()     # replay
        assert cuda.launch_count() == 0 and dit.graph_nodes == nodes       # nothing launched by the host code
        side.synchronize()
        assert torch.equal(y1, want) and torch.equal(y2, want)
        # same buffers, new contents and a new time feature: the replay must follow both
        d_x.copy_(dev(np.random.default_rng(8).normal(0, 1, x.shape).astype(np.float32), torch.bfloat16))
        d_t.copy_(dev((t_feat * 0.5).astype(np.float32)))
        dit.project_modulation(d_t)
        y3 = dit.layers_forward_graph(d_x, d_cos, d_sin, text=d_text, row_map=rmap, out=out).clone()
        want3 = dit.layers_forward(d_x, d_cos, d_sin, text=d_text, row_map=rmap)
        side.synchronize()
        cuda.check()
        assert torch.equal(y3, want3) and not torch.equal(y3, want)
    torch.cuda.current_stream().wait_stream(side)
    cuda.use_stream(torch.cuda.current_stream())
    dit.close()


def test_device_resident_denoise_step(cuda, oracle):
    """Patch embedding -> two blocks -> final adaLN head -> Euler update, all on the device, against the oracle's
    composition of the same pieces at the same precision (f32 heads, int8 linears, bf16 stream)."""
    geo, dit, host, _, text, t_feat, cos, sin = make_cross_case(cuda, oracle, 5, (2, 8, 8), 32, 256, 2, 512, n_blocks=2)
    rng = np.random.default_rng(321)
    seq, dim, patch = 128, 256, 96
    latent = rng.normal(0, 1, (seq, patch)).astype(np.float32)
    pw = rng.normal(0, 0.1, (dim, patch)).astype(np.float32)
    pb = rng.normal(0, 0.1, dim).astype(np.float32)
    fnorm = rng.normal(1, 0.1, dim).astype(np.float32)
    fmod = rng.normal(0, 0.2, (2, dim)).astype(np.float32)
    fw = rng.normal(0, 0.05, (patch, dim)).astype(np.float32)
    fb = rng.normal(0, 0.1, patch).astype(np.float32)
    dit.project_modulation(dev(t_feat))
    lat_dev = dev(latent)
    vel = dit.denoise_step(lat_dev, dev(pw), dev(pb), dev(fnorm), dev(fmod), dev(fw), dev(fb), dev(cos), dev(sin), 0.9, 0.6,
                           text=dev(text, torch.bfloat16), row_map=torch.zeros(seq, dtype=torch.int32, device="cuda"))
    cuda.check()
    cur = dev(oracle.dense(latent, pw, pb), torch.bfloat16).float().cpu().numpy()
    th = dev(text, torch.bfloat16).float().cpu().numpy()
    for b in range(2):
        cur = oracle.block_b(oracle_weights(oracle, host[b], t_feat, True), cur, th, cos, sin, heads=2, head_dim=128,
                             ffn=512, quantised=True, bf16_stream=True)
    want_vel = oracle.final_head(cur, fnorm, fmod, fw, fb)
    got_vel = vel.cpu().numpy()
    assert rel_l2(got_vel, want_vel) < 5e-3, rel_l2(got_vel, want_vel)
    # the Euler update itself is exact given the velocity the device computed
    assert np.array_equal(lat_dev.cpu().numpy(), oracle.euler_step(latent, got_vel, 0.9, 0.6))
    dit.close()
