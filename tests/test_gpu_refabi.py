"""Parity of the remaining entry points of the reference's operator surface (called through the C ABI): host
GEMM forms, the f16 ConvRot, ConvRot + requantise, the NVFP4 FC1 -> SwiGLU -> requantise -> FC2 chain, the f16
attention entry points with history keys / values, token-reduction pool / expand, and the answers of the
optional features this library does not have."""
import ctypes as C

from h3c_b200.lib import load

import numpy as np
import pytest

from tests.conftest import rel_l2

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


def host(t):
    return t.detach().float().cpu().numpy() if t.dtype in (torch.bfloat16, torch.float16) else t.detach().cpu().numpy()


def acts(rng, m, k):
    x = rng.normal(0, 1, (m, k)).astype(np.float32)
    x[rng.random((m, k)) < 0.001] *= 20
    return x


def call(name, *args):
    from h3c_b200.lib import call as c
    return c(name, *args)


def view_device(pointer, shape, typestr):
    """A torch view of device memory the library handed back as a raw pointer."""
    class Raw:
        __cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(pointer), False), "version": 2}
    return torch.as_tensor(Raw(), device="cuda")


def p(t):
    from h3c_b200.lib import ptr
    return ptr(t)


# ------------------------------------------------------------------ fused requant of the SwiGLU output (requant_mode 1)

def test_fc1_swiglu_requant_then_fc2_on_the_codes(cuda, oracle):
    """The reference's E2 option (h3_gpu_cuda.h:386-397, armed at h3_dit_w4a8.c:4058): FC1 with SwiGLU also hands back
    the int8 codes and row scales of its output (library scratch, rows padded to 128 with zeros), and FC2 runs on them
    through the pre-quantised entry point.  Codes and scales are the activation quantiser's applied to the f32 output
    the same call wrote, bit for bit; the gate forms of the option stay refused."""
    import h3c_b200
    from h3c_b200 import lib as L
    rng = np.random.default_rng(91)
    m, d, ffn = 300, 512, 768
    x = acts(rng, m, d)
    w1 = rng.integers(-127, 128, (2 * ffn, d), dtype=np.int8)
    s1 = rng.uniform(5e-5, 2e-4, 2 * ffn).astype(np.float32)
    w2 = rng.integers(-127, 128, (d, ffn), dtype=np.int8)
    s2 = rng.uniform(5e-5, 2e-4, d).astype(np.float32)
    W1, W2 = cuda.weight_from_i8(w1, s1), cuda.weight_from_i8(w2, s2)
    epi = L.DitGemmEpi()
    epi.swiglu, epi.requant_mode, epi.requant_gs = 1, 1, ffn
    xd = dev(x)
    y1 = torch.empty((m, ffn), dtype=torch.float32, device="cuda")
    backend = C.create_string_buffer(32)
    call("h3_cuda_gemm_i8_dequant_f32_w_act_dev_epi", cuda.h, W1.h, p(xd), 0, m, p(y1), None, None, backend, 32, C.byref(epi))
    cuda.check()
    assert epi.d_rq_x and epi.d_rq_act and epi.requant_rows == 384
    codes = view_device(epi.d_rq_x, (384, ffn), "|i1").cpu().numpy()
    scales = view_device(epi.d_rq_act, (384,), "<f4").cpu().numpy()
    qo, so = oracle.quantize_act_int8(host(y1))
    assert np.array_equal(codes[:m], qo) and np.array_equal(scales[:m], so)
    assert not codes[m:].any() and not scales[m:].any()
    # FC2 on those codes, plain epilogue
    y2 = torch.empty((m, d), dtype=torch.float32, device="cuda")
    call("h3_cuda_gemm_i8_dequant_f32_dev_pre_q", cuda.h, W2.h, epi.d_rq_x, epi.d_rq_act, m, p(y2), None, None, backend, 32, None)
    cuda.check()
    assert np.array_equal(host(y2), oracle.gemm_i8_dequant(qo, w2, so, s2))
    # wrong group size, and the gate forms
    bad = L.DitGemmEpi()
    bad.swiglu, bad.requant_mode, bad.requant_gs = 1, 1, ffn // 2
    with pytest.raises(h3c_b200.H3Error, match="requant gs"):
        call("h3_cuda_gemm_i8_dequant_f32_w_act_dev_epi", cuda.h, W1.h, p(xd), 0, m, p(y1), None, None, backend, 32, C.byref(bad))
    bad.requant_mode, bad.swiglu = 2, 0
    with pytest.raises(h3c_b200.H3Error, match="not supported"):
        call("h3_cuda_gemm_i8_dequant_f32_w_act_dev_epi", cuda.h, W1.h, p(xd), 0, m, p(y1), None, None, backend, 32, C.byref(bad))
    W1.free()
    W2.free()


# ------------------------------------------------------------------ f32 GEMM forms, f16 ConvRot, requantise helper

def test_host_and_mixed_f32_gemms(cuda):
    rng = np.random.default_rng(1)
    m, n, k = 70, 96, 200
    x, w = rng.normal(0, 1, (m, k)).astype(np.float32), rng.normal(0, 0.1, (n, k)).astype(np.float32)
    want = x.astype(np.float64) @ w.astype(np.float64).T
    y = np.empty((m, n), np.float32)
    call("h3_cuda_gemm_f32", cuda.h, x.ctypes.data, w.ctypes.data, m, n, k, y.ctypes.data, None)
    assert rel_l2(y, want) < 1e-5
    y2 = np.empty_like(y)
    dw = dev(w)
    call("h3_cuda_gemm_f32_dw", cuda.h, x.ctypes.data, p(dw), m, n, k, y2.ctypes.data, None)
    assert np.array_equal(y, y2)
    # f16 weights, y = alpha * x W^T + beta * y (the LoRA second GEMM)
    wh = dev(w, torch.float16)
    y0 = rng.normal(0, 1, (m, n)).astype(np.float32)
    dy = dev(y0)
    dx = dev(x)
    call("h3_cuda_gemm_f32in_f16w_f32out_dd_ex", cuda.h, p(dx), p(wh), m, n, k, p(dy), 0.75, 1.0)
    cuda.check()
    want = 0.75 * (x.astype(np.float64) @ host(wh).astype(np.float64).T) + y0
    assert rel_l2(host(dy), want) < 1e-5
    # the side-stream switch of the reference's LoRA overlap: the f32 GEMMs move to side stream 1 and back
    call("h3_cuda_cublas_use_side", cuda.h, 1)
    from h3c_b200.lib import load
    assert load().h3_cuda_cublas_stream(cuda.h) == load().h3_cuda_stream(cuda.h, 1)
    y3 = cuda.gemm_f32_dd(dx, dw)
    torch.cuda.synchronize()
    call("h3_cuda_cublas_use_side", cuda.h, 0)
    assert load().h3_cuda_cublas_stream(cuda.h) == load().h3_cuda_op_stream(cuda.h)
    assert np.array_equal(host(y3), y)


def test_convrot_f16_and_requantise_helper(cuda, oracle):
    rng = np.random.default_rng(2)
    m, k, gs = 150, 1024, 256
    x = acts(rng, m, k)
    xh = dev(x, torch.float16)
    yh = torch.empty_like(xh)
    call("h3_cuda_convrot_act_f16_dd", cuda.h, p(xh), m, k, gs, p(yh))
    cuda.check()
    want = oracle.convrot(host(xh), gs)
    assert rel_l2(host(yh), want) < 5e-4          # one f16 rounding of the rotated values
    # ConvRot + per-row INT8 into library scratch == the two separate operators of this library
    q_ptr, s_ptr = C.c_void_p(), C.c_void_p()
    dx = dev(x)
    call("h3_cuda_epi_fuse_ink_prep_fc2", cuda.h, p(dx), m, k, gs, C.byref(q_ptr), C.byref(s_ptr))
    cuda.check()
    rot = cuda.convrot_act_f32_dd(dx, gs)
    q2, s2 = cuda.quantize_act_int8(rot)
    m_pad = (m + 127) // 128 * 128
    q = torch.empty((m_pad, k), dtype=torch.int8, device="cuda")
    s = torch.empty(m_pad, dtype=torch.float32, device="cuda")
    C.CDLL("libcudart.so.12").cudaMemcpy(C.c_void_p(q.data_ptr()), q_ptr, C.c_size_t(m_pad * k), 3)
    C.CDLL("libcudart.so.12").cudaMemcpy(C.c_void_p(s.data_ptr()), s_ptr, C.c_size_t(m_pad * 4), 3)
    assert torch.equal(q[:m], q2) and torch.equal(s[:m], s2)
    assert not q[m:].any() and not s[m:].any()     # padded rows read as zero
    # the codes feed the pre-quantised GEMM entry point
    w_i8 = rng.integers(-127, 128, (256, k), dtype=np.int8)
    sc = rng.uniform(1e-3, 1e-2, 256).astype(np.float32)
    w = cuda.weight_from_i8(w_i8, sc)
    y = torch.empty((m, 256), dtype=torch.float32, device="cuda")
    call("h3_cuda_gemm_i8_dequant_f32_dev_pre_q", cuda.h, w.h, q_ptr, s_ptr, m, p(y), None, None, None, 0, None)
    cuda.check()
    assert np.array_equal(host(y), oracle.gemm_i8_dequant(host(q2), w_i8, host(s2), sc))


# ------------------------------------------------------------------ NVFP4 chain

def test_nvfp4_fc1_swiglu_requant_fc2_chain(cuda, oracle):
    rng = np.random.default_rng(3)
    m, dim, ffn, slots = 200, 512, 1024, 6
    x = acts(rng, m, dim)
    w1 = rng.normal(0, 0.05, (2 * ffn, dim)).astype(np.float32)
    w2 = rng.normal(0, 0.05, (dim, ffn)).astype(np.float32)
    w1q, w1sf = oracle.quantize_nvfp4(w1, rule=1)
    w2q, w2sf = oracle.quantize_nvfp4(w2, rule=1)
    x4, sfx = cuda.quantize_act_nvfp4(dev(x))
    # FC1 with f32 accumulators written out
    acc = torch.empty((m, 2 * ffn), dtype=torch.float32, device="cuda")
    dw1, dsf1 = dev(w1q), dev(w1sf)
    call("h3_cutlass_nvfp4_fc1_f32_run", cuda.h, p(dw1), p(dsf1), p(x4), p(sfx), m, 2 * ffn, dim, p(acc), None)
    cuda.check()
    want_acc = oracle.gemm_nvfp4(host(x4), host(sfx), w1q, w1sf, 1.0)
    assert rel_l2(host(acc), want_acc) < 1e-5
    # SwiGLU + requantise: codes and scales of silu(s g) * (s u) under the activation quantiser's rounding rules
    scale2 = 0.6
    m_pad = (m + 127) // 128 * 128
    from h3c_b200.lib import load
    sfb = int(load().h3_cuda_nvfp4_sf_bytes(m_pad, ffn))
    a4 = torch.zeros((m_pad, ffn // 2), dtype=torch.uint8, device="cuda")
    asf = torch.full((sfb,), 0xAA, dtype=torch.uint8, device="cuda")
    call("h3_nvfp4_swiglu_requant_dev", cuda.h, p(acc), scale2, None, m, ffn, p(a4), p(asf))
    cuda.check()
    a = host(acc)
    g, u = np.float32(scale2) * a[:, :ffn], np.float32(scale2) * a[:, ffn:]
    v = ((g / (np.float32(1) + np.exp(-g).astype(np.float32))) * u).astype(np.float32)
    vq, vsf = oracle.quantize_nvfp4(v)
    code_match = np.mean(host(a4)[:m] == vq)
    sf_match = np.mean(host(asf)[: vsf.size] == vsf)
    assert code_match > 0.999 and sf_match > 0.999, (code_match, sf_match)    # expf of the device vs glibc: rare one-step moves
    # ... and the dequantised activation is the same to the quantisation step
    assert rel_l2(oracle.dequant_nvfp4(host(a4), host(asf))[:m], oracle.dequant_nvfp4(vq, vsf)[:m]) < 2e-3
    # FC2 on those codes with the gate + residual epilogue
    wh = cuda.nvfp4_weight(w2q, w2sf, 0.5, dim, ffn)
    res = rng.normal(0, 1, (m, dim)).astype(np.float32)
    mod = rng.normal(0, 0.5, (3, slots, dim)).astype(np.float32)
    rmap = (np.arange(m) % 3).astype(np.uint32)
    y = torch.empty((m, dim), dtype=torch.float32, device="cuda")
    d_res, d_mod, d_map = dev(res), dev(mod), dev(rmap.view(np.int32))
    err = C.create_string_buffer(512)
    assert load().h3_cuda_gemm_fp4_pre_q_dev(cuda.h, wh, p(a4), p(asf), m, p(d_res), p(d_mod), p(d_map), slots, 5, None, p(y),
                                             None, None, err, 512, b"test.fc2") == 1, err.value
    cuda.check()
    base = oracle.gemm_nvfp4(host(a4)[:m], host(asf), w2q, w2sf, 0.5)
    assert rel_l2(host(y), oracle.gate(res, base, mod, rmap, slots, 5)) < 1e-5
    assert int(load().h3_cuda_nvfp4_chain_scratch_bytes(m, dim, ffn)) >= m_pad * (dim // 2 + 2 * ffn * 4 + ffn // 2)
    cuda.nvfp4_weight_free(wh)


# ------------------------------------------------------------------ attention entry points of the reference

def _qkv_case(rng, oracle, seq, heads, grid):
    hd = 128
    qkv = rng.normal(0, 1, (seq, 3 * heads * hd)).astype(np.float32)
    qn, kn = rng.normal(1, 0.1, hd).astype(np.float32), rng.normal(1, 0.1, hd).astype(np.float32)
    inv_freq = (1.0 / (10000.0 ** (np.arange(16) / 16.0))).astype(np.float32)
    pt, ph, pw = oracle.fill_video_pos(8, *grid)
    cos, sin = oracle.rope_tables(inv_freq, pt, ph, pw, 1.0)
    assert len(pt) == seq
    return qkv, qn, kn, cos, sin


def test_reference_rope_sdpa_entry_points_f16(cuda, oracle):
    """f32 QKV and f16 QKV forms; f16 staging like the reference's default path: within 1e-3 of the f32 CPU chain
    (the reference's own CUDA path sits at the same distance: 11-bit operands, f32 accumulation)."""
    rng = np.random.default_rng(4)
    seq, heads, hd = 4 * 6 * 8, 3, 128
    qkv, qn, kn, cos, sin = _qkv_case(rng, oracle, seq, heads, (4, 12, 16))
    q, k, v = oracle.qkv_rope(qkv, qn, kn, cos, sin, heads, hd, 48)
    want = oracle.sdpa(q, k, v)
    out = torch.empty((seq, heads * hd), dtype=torch.float32, device="cuda")
    be = C.create_string_buffer(64)
    d_qkv, d_qn, d_kn, d_cos, d_sin = dev(qkv), dev(qn), dev(kn), dev(cos), dev(sin)    # kept alive across the calls
    args = (p(d_qn), p(d_kn), p(d_cos), p(d_sin), seq, heads, hd, 48, 1e-5, hd ** -0.5, 0)
    call("h3_cuda_qkv_rope_sdpa_f16_dev_layout", cuda.h, p(d_qkv), *args, 0, 1, p(out), None, None, be, 64)
    cuda.check()
    assert be.value == b"tcgen05_flash_f16"
    e32 = rel_l2(host(out), want)
    assert e32 < 1e-3
    qkv_h = dev(qkv, torch.float16)
    out2 = torch.empty_like(out)
    call("h3_cuda_qkv_rope_sdpa_f16_dev_f16qkv", cuda.h, p(qkv_h), *args, p(out2), None, None, None, 0)
    cuda.check()
    q2, k2, v2 = oracle.qkv_rope(host(qkv_h), qn, kn, cos, sin, heads, hd, 48)
    assert rel_l2(host(out2), oracle.sdpa(q2, k2, v2)) < 1e-3
    # windowed attention is refused, not ignored
    import h3c_b200
    with pytest.raises(h3c_b200.H3Error, match="windowed"):
        call("h3_cuda_qkv_rope_sdpa_f16_dev_layout", cuda.h, p(d_qkv), *args[:-1], 24, 0, 1, p(out), None, None, None, 0)


def test_history_keys_and_saved_rows(cuda, oracle):
    """h3_cuda_sdpa_bind_kvcat / _kvsave: queries stay `seq` long, keys and values are [current | history];
    chosen current K / V rows are copied out as f16."""
    rng = np.random.default_rng(5)
    seq, heads, hd, hist = 2 * 6 * 8, 2, 128, 77
    qkv, qn, kn, cos, sin = _qkv_case(rng, oracle, seq, heads, (2, 12, 16))
    q, k, v = oracle.qkv_rope(qkv, qn, kn, cos, sin, heads, hd, 48)
    kh = dev(rng.normal(0, 1, (hist, heads, hd)).astype(np.float32), torch.float16)
    vh = dev(rng.normal(0, 1, (hist, heads, hd)).astype(np.float32), torch.float16)
    idx = np.array([5, 0, seq - 1, 17], np.uint32)
    ks = torch.zeros((len(idx), heads, hd), dtype=torch.float16, device="cuda")
    vs = torch.zeros_like(ks)
    d_idx = dev(idx.view(np.int32))
    from h3c_b200.lib import load
    load().h3_cuda_sdpa_bind_kvcat(p(kh), p(vh), hist)
    load().h3_cuda_sdpa_bind_kvsave(p(ks), p(vs), p(d_idx), len(idx))
    out = torch.empty((seq, heads * hd), dtype=torch.float32, device="cuda")
    d_qkv, d_qn, d_kn, d_cos, d_sin = dev(qkv), dev(qn), dev(kn), dev(cos), dev(sin)    # kept alive across the calls
    call("h3_cuda_qkv_rope_sdpa_f16_dev", cuda.h, p(d_qkv), p(d_qn), p(d_kn), p(d_cos), p(d_sin), seq, heads, hd,
         48, 1e-5, hd ** -0.5, 0, p(out), None, None, None, 0)
    load().h3_cuda_sdpa_clear_kvext()
    cuda.check()
    k_all = np.concatenate([k.reshape(seq, heads, hd), host(kh)])
    v_all = np.concatenate([v.reshape(seq, heads, hd), host(vh)])
    assert rel_l2(host(out), oracle.sdpa(q.reshape(seq, heads, hd), k_all, v_all)) < 1e-3
    assert rel_l2(host(ks), k.reshape(seq, heads, hd)[idx]) < 5e-4 and rel_l2(host(vs), v.reshape(seq, heads, hd)[idx]) < 5e-4
    # cleared: the next call is square again
    call("h3_cuda_qkv_rope_sdpa_f16_dev", cuda.h, p(d_qkv), p(d_qn), p(d_kn), p(d_cos), p(d_sin), seq, heads, hd,
         48, 1e-5, hd ** -0.5, 0, p(out), None, None, None, 0)
    cuda.check()
    assert rel_l2(host(out), oracle.sdpa(q, k, v)) < 1e-3


def test_host_tensor_attention_forms(cuda, oracle):
    rng = np.random.default_rng(6)
    seq, heads, hd = 130, 2, 128
    q, k, v = (rng.normal(0, 1, (seq, heads, hd)).astype(np.float32) for _ in range(3))
    want = oracle.sdpa(q, k, v)
    for name in ("h3_cuda_sdpa_f16", "h3_cuda_sdpa_f32"):
        out = np.empty((seq, heads * hd), np.float32)
        call(name, cuda.h, q.ctypes.data, k.ctypes.data, v.ctypes.data, seq, heads, hd, hd ** -0.5, out.ctypes.data, None)
        # the f32 NAME runs the f16 tensor-core kernel too: 11-bit operands, f32 softmax and accumulation
        assert rel_l2(out, want) < 1e-3, name
    out = np.empty((seq, heads * hd), np.float32)
    be = C.create_string_buffer(64)
    call("h3_cuda_sdpa_f16_ex", cuda.h, q.ctypes.data, k.ctypes.data, v.ctypes.data, seq, heads, hd, hd ** -0.5, 0,
         out.ctypes.data, None, be, 64)
    assert rel_l2(out, want) < 1e-3 and be.value.startswith(b"tcgen05")


# ------------------------------------------------------------------ token reduction

def _pool_expand_reference(x, pairs, bidx, parents, baseline_rows, video_start, video_rows, scale, reduced_update):
    """The reference's two kernels in numpy (h3_gpu_cuda.cu:12927-12981)."""
    first, second = pairs[:, 0], pairs[:, 1]
    pooled = np.where((first != second)[:, None], np.float32(0.5) * (x[first] + x[second]), x[first]).astype(np.float32)
    baseline = np.zeros((baseline_rows, x.shape[1]), np.float32)
    has = bidx != 0xFFFFFFFF
    baseline[bidx[has]] = pooled[has]
    red = reduced_update(pooled)
    out = red[parents].copy()
    rows = np.arange(len(parents))
    in_video = (rows >= video_start) & (rows < video_start + video_rows) & (bidx[parents] != 0xFFFFFFFF)
    b = bidx[parents[in_video]]
    out[in_video] = x[in_video] + np.float32(scale) * (red[parents[in_video]] - baseline[b])
    return pooled, baseline, out


def test_token_pool_and_expand(cuda):
    rng = np.random.default_rng(7)
    width, text, video = 256, 10, 24          # rows: 10 text rows kept, 24 video rows paired horizontally
    full = text + video
    x = rng.normal(0, 1, (full, width)).astype(np.float32)
    pairs = [(i, i) for i in range(text)] + [(text + 2 * j, text + 2 * j + 1) for j in range(video // 2)]
    pairs = np.array(pairs, np.uint32)
    reduced = len(pairs)
    bidx = np.full(reduced, 0xFFFFFFFF, np.uint32)
    bidx[text:] = np.arange(video // 2)
    parents = np.zeros(full, np.uint32)
    for r, (a, b) in enumerate(pairs):
        parents[a] = parents[b] = r
    upd = lambda pooled: (pooled * np.float32(1.25) + np.float32(0.5)).astype(np.float32)   # stand-in for the blocks in between
    want_pool, want_base, want_out = _pool_expand_reference(x, pairs, bidx, parents, video // 2, text, video, 0.8, upd)

    # device-resident form
    d_in = dev(x)
    d_out = torch.empty((reduced, width), device="cuda")
    d_orig = torch.zeros((full, width), device="cuda")
    d_base = torch.zeros((video // 2, width), device="cuda")
    call("h3_cuda_token_pool_f32_dev", cuda.h, p(d_in), full, pairs.ctypes.data, bidx.ctypes.data, reduced, video // 2, width,
         p(d_out), p(d_orig), p(d_base), None)
    cuda.check()
    assert np.array_equal(host(d_out), want_pool) and np.array_equal(host(d_orig), x) and np.array_equal(host(d_base), want_base)
    d_red = dev(upd(want_pool))
    d_y = torch.empty((full, width), device="cuda")
    call("h3_cuda_token_expand_f32_dev", cuda.h, p(d_orig), p(d_red), p(d_base), bidx.ctypes.data, parents.ctypes.data, full,
         reduced, video // 2, width, text, video, 0.8, p(d_y), None)
    cuda.check()
    assert np.array_equal(host(d_y), want_out)

    # host-activation form: the library allocates `original` and `baseline` and hands them to the caller
    out = np.empty((reduced, width), np.float32)
    po, pb = C.c_void_p(), C.c_void_p()
    call("h3_cuda_token_pool_f32", cuda.h, x.ctypes.data, full, pairs.ctypes.data, bidx.ctypes.data, reduced, video // 2, width,
         out.ctypes.data, C.byref(po), C.byref(pb), None)
    assert np.array_equal(out, want_pool) and po.value and pb.value
    y = np.empty((full, width), np.float32)
    red_h = upd(want_pool)
    call("h3_cuda_token_expand_f32", cuda.h, po, red_h.ctypes.data, pb, bidx.ctypes.data, parents.ctypes.data, full, reduced,
         video // 2, width, text, video, 0.8, y.ctypes.data, None)
    assert np.array_equal(y, want_out)
    rt = C.CDLL("libcudart.so.12")
    rt.cudaFree(po)
    rt.cudaFree(pb)


# ------------------------------------------------------------------ housekeeping and absent features

def test_housekeeping_and_absent_features(cuda):
    import h3c_b200
    from h3c_b200.lib import load
    L = load()
    for name in ("h3_cuda_copy_stream_synchronize", "h3_cuda_recreate_blas", "h3_cuda_dit_scratch_check",
                 "h3_cuda_dit_scratch_rehome"):
        call(name, cuda.h)
    buf = np.zeros(1 << 16, np.uint8)
    call("h3_cuda_host_register", buf.ctypes.data, buf.nbytes)
    L.h3_cuda_host_unregister(buf.ctypes.data)
    # distance attention: configuring it off is fine, on is refused with a message that names this library
    call("h3_cuda_dist_attn_configure", cuda.h, 100, 10, 90, 2, 5, 9, 15.0, 3.0, 0)
    with pytest.raises(h3c_b200.H3Error, match="not supported by libh3_b200"):
        call("h3_cuda_dist_attn_configure", cuda.h, 100, 10, 90, 2, 5, 9, 15.0, 3.0, 1)
    assert L.h3_cuda_dist_attn_active() == 0 and L.h3_cuda_sage3_pool_bytes() == 0 and L.h3_nvfp4_cuda_enabled() == 0
    L.h3_cuda_dist_attn_clear()
    L.h3_cuda_sol_cute_set_step(3)
    L.h3_cuda_sol_profile_add_unpack(1.5)
    L.h3_nvfp4_cuda_cache_clear()
    with pytest.raises(h3c_b200.H3Error, match="not supported by libh3_b200"):
        call("h3_nvfp4_cuda_encode_text_layers", None, None, 0, 0)
    assert L.h3_nvfp4_debug_nan_dev() in (0, 1)


# ------------------------------------------------------------------ the attention plugin ABI

def test_sdpa_plugin_through_dlopen(cuda, oracle):
    """libh3_b200_sdpa.so: the four symbols the reference looks up in an attention plugin (h3_sage3_init / _fwd /
    _fwd_ex / _warmup).  Driven the way the reference drives a plugin: init returns four f16 [heads, seq, 128]
    buffers owned by the plugin, the caller fills Q / K / V, calls fwd, reads O."""
    from h3c_b200 import build
    lib = C.CDLL(str(build.SDPA_PLUGIN))
    rng = np.random.default_rng(8)
    seq, heads, hd = 333, 3, 128
    err, be = C.create_string_buffer(512), C.create_string_buffer(64)
    ptrs = [C.c_void_p() for _ in range(4)]
    assert lib.h3_sage3_warmup(b"", seq, heads, hd, C.c_float(hd ** -0.5), 0, 0, err, C.c_size_t(512)) == 1, err.value
    assert lib.h3_sage3_init(b"", seq, heads, hd, C.c_float(hd ** -0.5), 0, 0, *[C.byref(x) for x in ptrs], be, C.c_size_t(64), err,
                             C.c_size_t(512)) == 1, err.value
    assert be.value == b"h3_b200_tcgen05_flash_f16" and all(x.value for x in ptrs)
    q, k, v = (rng.normal(0, 1, (heads, seq, hd)).astype(np.float16) for _ in range(3))     # [heads, seq, 128]
    rt = C.CDLL("libcudart.so.12")
    for dst, a in zip(ptrs[:3], (q, k, v)):
        assert rt.cudaMemcpy(dst, C.c_void_p(a.ctypes.data), C.c_size_t(a.nbytes), 1) == 0
    kern_ms = C.c_double(0)
    assert lib.h3_sage3_fwd_ex(err, C.c_size_t(512), None, C.byref(kern_ms), None, None, None) == 1, err.value
    o = np.empty_like(q)
    assert rt.cudaMemcpy(C.c_void_p(o.ctypes.data), ptrs[3], C.c_size_t(o.nbytes), 2) == 0
    want = oracle.sdpa(*(np.ascontiguousarray(a.astype(np.float32).transpose(1, 0, 2)) for a in (q, k, v)))
    got = o.astype(np.float32).transpose(1, 0, 2).reshape(seq, heads * hd)
    assert rel_l2(got, want) < 1e-3 and kern_ms.value > 0
    assert lib.h3_sage3_fwd(err, C.c_size_t(512)) == 1
    # shapes the kernel does not serve are refused with a message, like the reference's plugin errors
    assert lib.h3_sage3_init(b"", seq, heads, 64, C.c_float(0.125), 0, 0, *[C.byref(x) for x in ptrs], be, C.c_size_t(64), err,
                             C.c_size_t(512)) == 0 and b"head_dim 128" in err.value
