"""Parity of the CUDA operators (called through the C ABI of libh3_b200.so) against the CPU oracle
on the same seeded inputs.  Integer / byte results: bit-exact.  Float results: bit-exact where the
kernel keeps the reference's operation order, otherwise within the tolerance written in the test."""
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
    x[rng.random((m, k)) < 0.001] *= 20  # the benchmark's 0.1 % outliers
    return x


# ------------------------------------------------------------------ weights

def test_w4a8_weight_decode_exact(cuda, oracle):
    rng = np.random.default_rng(10)
    n, k = 96, 512
    packed = rng.integers(-128, 128, (n, k // 2), dtype=np.int8)
    codebook = rng.normal(0, 50, 16).astype(np.float32)
    s_rel = rng.integers(0x20, 0x50, (n, k // 16), dtype=np.uint8)
    s_ch = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    w = cuda.weight_from_w4a8(packed, codebook, s_rel, s_ch)
    assert (w.n, w.k) == (n, k)
    assert np.array_equal(w.download_int8(), oracle.w4a8_dequant_to_int8(packed, codebook, s_rel))
    assert np.array_equal(w.download_scales(), s_ch)


def test_w4g128_weight_decode_exact(cuda, oracle):
    rng = np.random.default_rng(11)
    wf = rng.normal(0, 0.02, (64, 512)).astype(np.float32)
    packed, scales = oracle.w4g128_encode(wf, 128)
    w = cuda.weight_from_w4g(packed, scales, 128)
    w_i8, s = oracle.w4g128_decode_to_int8(packed, scales, 128)
    assert np.array_equal(w.download_int8(), w_i8)
    assert np.array_equal(w.download_scales(), s)
    # the int4 -> int8 re-expression stays within half an int8 step of s*q
    assert rel_l2(w_i8 * s[:, None], wf) < 0.12


# ------------------------------------------------------------- row-wise ops

@pytest.mark.parametrize("m,k", [(1, 64), (37, 3072), (5, 100)])
def test_quantize_act_int8_exact(cuda, oracle, m, k):
    rng = np.random.default_rng(12)
    x = acts(rng, m, k)
    x[0, : k // 2] = 0.0
    if m > 2:
        x[2] = 0.0  # zero row -> scale 1
    q, s = cuda.quantize_act_int8(dev(x))
    qo, so = oracle.quantize_act_int8(x)
    assert np.array_equal(host(q), qo) and np.array_equal(host(s), so)
    # bf16 input: same rule applied to the bf16 values
    xb = dev(x, torch.bfloat16)
    q, s = cuda.quantize_act_int8(xb)
    qo, so = oracle.quantize_act_int8(host(xb))
    assert np.array_equal(host(q), qo) and np.array_equal(host(s), so)


def test_rowwise_f32_ops(cuda, oracle):
    rng = np.random.default_rng(13)
    rows, width, slots = 50, 3072, 6
    x = rng.normal(0, 1.5, (rows, width)).astype(np.float32)
    br = rng.normal(0, 1, (rows, width)).astype(np.float32)
    nw = rng.normal(1, 0.1, width).astype(np.float32)
    mod = rng.normal(0, 0.3, (3, slots, width)).astype(np.float32)
    rmap = (np.arange(rows) % 3).astype(np.uint32)
    dx, dbr, dnw, dmod, drm = dev(x), dev(br), dev(nw), dev(mod), dev(rmap.view(np.int32))
    tol = 2e-6  # only the order of the row sum of squares differs
    assert rel_l2(host(cuda.adaln_f32_dev(dx, dnw, dmod, drm, slots, 0, 1)), oracle.adaln(x, nw, mod, rmap, slots, 0, 1)) < tol
    assert rel_l2(host(cuda.rms_norm_f32_dev(dx, dnw)), oracle.rms_norm(x, nw)) < tol
    assert np.array_equal(host(cuda.gate_f32_dev(dx, dbr, dmod, drm, slots, 2)), oracle.gate(x, br, mod, rmap, slots, 2))
    g, n = cuda.gate_adaln_f32_dev(dx, dbr, dnw, dmod, drm, slots, 2, 3, 4)
    go, no = oracle.gate_adaln(x, br, nw, mod, rmap, slots, 2, 3, 4)
    assert np.array_equal(host(g), go) and rel_l2(host(n), no) < tol
    fused = rng.normal(0, 2, (rows, 2 * width)).astype(np.float32)
    assert rel_l2(host(cuda.swiglu_f32_dev(dev(fused))), oracle.swiglu(fused)) < 1e-6
    # identity row map (NULL): row r uses modulation row r
    mod_id = rng.normal(0, 0.3, (rows, slots, width)).astype(np.float32)
    assert rel_l2(host(cuda.adaln_f32_dev(dx, dnw, dev(mod_id), None, slots, 3, 4)),
                  oracle.adaln(x, nw, mod_id, None, slots, 3, 4)) < tol


def test_fused_adaln_quant_bf16(cuda, oracle):
    """adaLN -> bf16 round -> INT8 codes in one launch.  The codes must be exactly the reference rule
    applied to the kernel's own (bf16) normalised values; against the unfused CPU chain only the
    reduction order differs, which may flip a few codes by one step."""
    rng = np.random.default_rng(14)
    rows, width = 64, 3072
    x = dev(rng.normal(0, 1, (rows, width)).astype(np.float32), torch.bfloat16)
    nw = rng.normal(1, 0.1, width).astype(np.float32)
    mod = rng.normal(0, 0.3, (1, 6, width)).astype(np.float32)
    rmap = np.zeros(rows, np.uint32)
    normed = torch.empty_like(x)
    q = torch.empty((rows, width), dtype=torch.int8, device="cuda")
    s = torch.empty(rows, dtype=torch.float32, device="cuda")
    cuda.norm(x, norm_w=dev(nw), modulation=dev(mod), row_map=dev(rmap.view(np.int32)), slots=6, shift_slot=0,
              scale_slot=1, normed=normed, q=q, scales=s)
    qo, so = oracle.quantize_act_int8(host(normed))
    assert np.array_equal(host(q), qo) and np.array_equal(host(s), so)
    cpu = oracle.bf16_round(oracle.adaln(host(x), nw, mod, rmap, 6, 0, 1))
    qc, sc = oracle.quantize_act_int8(cpu)
    diff = np.abs(host(q).astype(np.int32) - qc.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 5e-3
    assert rel_l2(host(normed), cpu) < 2e-3


@pytest.mark.parametrize("gs", [256, 16])
def test_convrot(cuda, oracle, gs):
    rng = np.random.default_rng(15)
    x = acts(rng, 33, 1024)
    y = host(cuda.convrot_act_f32_dd(dev(x), gs))
    assert rel_l2(y, oracle.convrot(x, gs)) < 1e-6
    # fused rotate + quantise: codes follow the reference rule on the kernel's rotated values
    rot = torch.empty((33, 1024), dtype=torch.float32, device="cuda")
    q = torch.empty((33, 1024), dtype=torch.int8, device="cuda")
    s = torch.empty(33, dtype=torch.float32, device="cuda")
    cuda.norm(dev(x), identity=True, convrot_gs=gs, rot=rot, q=q, scales=s)
    qo, so = oracle.quantize_act_int8(host(rot))
    assert np.array_equal(host(q), qo) and np.array_equal(host(s), so)


@pytest.mark.parametrize("gs", [256, 64, 8, 2])
def test_convrot_sylvester_switch(cuda, oracle, gs, monkeypatch):
    """H3_CONVROT_SYLVESTER=1 (the reference's switch, h3_w4a8_dequant.c:371-375): Walsh-Hadamard groups by radix-2
    butterflies, bit-identical to the reference's in-place transform; group sizes that are not powers of four exist
    only under the switch."""
    rng = np.random.default_rng(17)
    x = acts(rng, 45, 1024)
    monkeypatch.setenv("H3_CONVROT_SYLVESTER", "1")
    y = host(cuda.convrot_act_f32_dd(dev(x), gs))
    assert np.array_equal(y, oracle.fwht(x, gs))
    monkeypatch.delenv("H3_CONVROT_SYLVESTER")
    if gs in (8, 2):
        with pytest.raises(Exception):
            cuda.convrot_act_f32_dd(dev(x), gs)
    else:
        assert rel_l2(host(cuda.convrot_act_f32_dd(dev(x), gs)), oracle.convrot(x, gs)) < 1e-6


def test_qkv_rope(cuda, oracle):
    rng = np.random.default_rng(16)
    heads, hd = 3, 128
    pt, ph, pw = oracle.fill_video_pos(16, 3, 8, 12)
    inv_freq = (1.0 / (10000.0 ** (np.arange(16) / 16.0))).astype(np.float32)
    cos, sin = oracle.rope_tables(inv_freq, pt, ph, pw, 1.0)
    seq = len(pt)
    qkv = rng.normal(0, 1, (seq, 3 * heads * hd)).astype(np.float32)
    qn, kn = rng.normal(1, 0.1, hd).astype(np.float32), rng.normal(1, 0.1, hd).astype(np.float32)
    for grouped, split in ((0, 1), (0, 0), (1, 1)):
        q, k, v = cuda.qkv_rope(dev(qkv), dev(qn), dev(kn), dev(cos), dev(sin), heads, hd, 48, grouped=grouped,
                                split_half=split)
        qo, ko, vo = oracle.qkv_rope(qkv, qn, kn, cos, sin, heads, hd, 48, grouped=grouped, split_half=split)
        assert rel_l2(host(q), qo) < 1e-6 and rel_l2(host(k), ko) < 1e-6 and np.array_equal(host(v), vo)
    q, k, v = cuda.qkv_rope(dev(qkv), dev(qn), dev(kn), None, None, heads, hd, 0)
    qo, ko, vo = oracle.qkv_rope(qkv, qn, kn, None, None, heads, hd, 0)
    assert rel_l2(host(q), qo) < 1e-6 and rel_l2(host(k), ko) < 1e-6


# ---------------------------------------------------------------------- GEMM

def make_weight(cuda, rng, n, k):
    w_i8 = rng.integers(-127, 128, (n, k), dtype=np.int8)
    s = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    return cuda.weight_from_i8(w_i8, s), w_i8, s


@pytest.mark.parametrize("m,n,k", [(1, 128, 128), (127, 256, 256), (129, 384, 512), (300, 640, 3072),
                                   (16, 256, 144), (257, 24, 64), (1000, 1280, 1024)])
def test_gemm_int32_accumulators_exact(cuda, m, n, k):
    """m <= 128 runs the single-CTA tile, larger m the CTA-pair (256 x 256) tile."""
    import h3c_b200
    rng = np.random.default_rng(20 + m)
    w, w_i8, _ = make_weight(cuda, rng, n, k)
    x = rng.integers(-127, 128, (m, k), dtype=np.int8)
    a = torch.ones(m, dtype=torch.float32, device="cuda")
    acc = cuda.gemm_i8(w, dev(x), a, out_dtype=torch.int32)
    cuda.check()
    assert np.array_equal(host(acc), x.astype(np.int32) @ w_i8.astype(np.int32).T)


@pytest.mark.parametrize("m", [200, 96])   # CTA-pair tile, single-CTA tile
def test_gemm_epilogues(cuda, oracle, m):
    import h3c_b200
    rng = np.random.default_rng(30)
    n, k, slots = 512, 256, 6
    w, w_i8, s = make_weight(cuda, rng, n, k)
    x = acts(rng, m, k)
    xq, xs = oracle.quantize_act_int8(x)
    dq, ds = dev(xq), dev(xs)
    acc = oracle.gemm_i8_i32(xq, w_i8)
    # plain, f32: same operation order as the reference -> identical bits
    y = cuda.gemm_i8(w, dq, ds)
    assert np.array_equal(host(y), oracle.gemm_i8_dequant(xq, w_i8, xs, s))
    # gate + residual with a row map, f32
    res = rng.normal(0, 1, (m, n)).astype(np.float32)
    mod = rng.normal(0, 0.5, (3, slots, n)).astype(np.float32)
    rmap = (np.arange(m) % 3).astype(np.uint32)
    y = cuda.gemm_i8(w, dq, ds, kind=h3c_b200.EPI_GATE, residual=dev(res), modulation=dev(mod),
                     row_map=dev(rmap.view(np.int32)), slots=slots, gate_slot=5)
    assert np.array_equal(host(y), oracle.dequant_gate(acc, xs, s, res, mod, rmap, slots, 5))
    # residual only (no modulation)
    y = cuda.gemm_i8(w, dq, ds, kind=h3c_b200.EPI_GATE, residual=dev(res))
    assert np.array_equal(host(y), res + oracle.gemm_i8_dequant(xq, w_i8, xs, s))
    # SwiGLU (expf) and tanh-GELU (tanhf): device libm differs from glibc in the last ulps
    y = cuda.gemm_i8(w, dq, ds, kind=h3c_b200.EPI_SWIGLU)
    assert y.shape == (m, n // 2) and rel_l2(host(y), oracle.dequant_swiglu(acc, xs, s)) < 1e-6
    y = cuda.gemm_i8(w, dq, ds, kind=h3c_b200.EPI_GELU)
    assert rel_l2(host(y), oracle.dequant_gelu(acc, xs, s)) < 1e-6
    # already-scaled LoRA deltas added before the gate / activation (h3_dit_fused_epi.h:85-141)
    lora = rng.normal(0, 0.05, (m, n)).astype(np.float32)
    y = cuda.gemm_i8(w, dq, ds, kind=h3c_b200.EPI_GATE, residual=dev(res), modulation=dev(mod),
                     row_map=dev(rmap.view(np.int32)), slots=slots, gate_slot=5, lora=dev(lora))
    assert np.array_equal(host(y), oracle.dequant_gate(acc, xs, s, res, mod, rmap, slots, 5, lora))
    y = cuda.gemm_i8(w, dq, ds, kind=h3c_b200.EPI_SWIGLU, lora=dev(lora))
    assert rel_l2(host(y), oracle.dequant_swiglu(acc, xs, s, lora)) < 1e-6
    y = cuda.gemm_i8(w, dq, ds, lora=dev(lora))
    assert np.array_equal(host(y), oracle.gemm_i8_dequant(xq, w_i8, xs, s) + lora)
    # bf16 outputs are the f32 results rounded once
    y = cuda.gemm_i8(w, dq, ds, out_dtype=torch.bfloat16)
    assert np.array_equal(host(y), oracle.bf16_round(oracle.gemm_i8_dequant(xq, w_i8, xs, s)))
    resb = dev(res, torch.bfloat16)
    y = cuda.gemm_i8(w, dq, ds, kind=h3c_b200.EPI_GATE, out_dtype=torch.bfloat16, residual=resb, modulation=dev(mod),
                     row_map=dev(rmap.view(np.int32)), slots=slots, gate_slot=2)
    assert np.array_equal(host(y), oracle.bf16_round(oracle.dequant_gate(acc, xs, s, host(resb), mod, rmap, slots, 2)))
    cuda.check()


@pytest.mark.parametrize("m,n,k", [(6280, 3072, 3072), (2560, 2048, 512), (6280, 9216, 512)])
def test_gemm_split_tail_tiles(cuda, oracle, m, n, k, monkeypatch):
    """A last wave that fills at most half of the CTA pairs can be cut along K (on 74 pairs: 300 tiles = 4 waves + 4 tiles;
    80 tiles = 1 wave + 6; 900 tiles = 12 waves + 12).  Int32 sums are exact in any order, so every epilogue gives the
    bits of the whole-tile form, call after call (the slots are left cleared)."""
    import h3c_b200
    rng = np.random.default_rng(m + n)
    w, w_i8, s = make_weight(cuda, rng, n, k)
    x = rng.integers(-127, 128, (m, k), dtype=np.int8)
    xs = rng.uniform(0.005, 0.02, m).astype(np.float32)
    dq, ds = dev(x), dev(xs)
    res = dev(rng.normal(0, 1, (m, n)).astype(np.float32), torch.bfloat16)
    heads = n // 384
    qn = dev(rng.normal(1, 0.1, 128).astype(np.float32))
    cos, sin = dev(rng.random((m, 64)).astype(np.float32)), dev(rng.random((m, 64)).astype(np.float32))

    def run_all():
        out = [cuda.gemm_i8(w, dq, torch.ones_like(ds), out_dtype=torch.int32),
               cuda.gemm_i8(w, dq, ds, out_dtype=torch.bfloat16),
               cuda.gemm_i8(w, dq, ds, kind=h3c_b200.EPI_GATE, residual=res, out_dtype=torch.bfloat16),
               cuda.gemm_i8(w, dq, ds, kind=h3c_b200.EPI_GELU, out_dtype=torch.bfloat16),
               cuda.gemm_i8(w, dq, ds, kind=h3c_b200.EPI_SWIGLU, out_dtype=torch.bfloat16),
               cuda.gemm_i8(w, dq, ds, kind=h3c_b200.EPI_SWIGLU)]
        if n == heads * 384:
            out += list(cuda.gemm_i8_qkv_rope(w, dq, ds, qn, qn, cos, sin, 64))
        cuda.check()
        return out

    monkeypatch.setenv("H3B_GEMM_SPLITK", "0")
    whole = run_all()
    for mode in ("1", "12", "3"):   # the library's own choice, and forced slice counts
        monkeypatch.setenv("H3B_GEMM_SPLITK", mode)
        for _ in range(2):
            for a, b in zip(run_all(), whole):
                assert torch.equal(a, b)
    rows = np.unique(np.concatenate([[0, 127, 128, 255, 256, m - 1, m - 2, (m - 1) // 256 * 256], rng.integers(0, m, 8)]))
    want = x[rows].astype(np.int32) @ w_i8.astype(np.int32).T
    assert np.array_equal(host(whole[0][torch.from_numpy(rows).cuda()]), want)


def test_gemm_qkv_rope_epilogue(cuda, oracle):
    """QKV projection with the QK-norm and split-half RoPE fused into the GEMM epilogue, against the oracle
    chain dequant -> (round to bf16) -> h3_dit_w4a8_qkv_rope_f32."""
    rng = np.random.default_rng(33)
    heads, hd, k = 3, 128, 256
    pt, ph, pw = oracle.fill_video_pos(16, 5, 8, 12)
    inv_freq = (1.0 / (10000.0 ** (np.arange(16) / 16.0))).astype(np.float32)
    cos, sin = oracle.rope_tables(inv_freq, pt, ph, pw, 1.0)
    m = len(pt)   # 120 rows: not a multiple of the row tile
    w, w_i8, s = make_weight(cuda, rng, 3 * heads * hd, k)
    xq, xs = oracle.quantize_act_int8(acts(rng, m, k))
    qn, kn = rng.normal(1, 0.1, hd).astype(np.float32), rng.normal(1, 0.1, hd).astype(np.float32)
    qkv = oracle.gemm_i8_dequant(xq, w_i8, xs, s)
    for rope_half, rnd in ((48, True), (48, False), (0, True), (64, True)):
        c, sn = (cos, sin) if rope_half == 48 else (np.ones((m, 64), np.float32), np.zeros((m, 64), np.float32))
        c, sn = (None, None) if rope_half == 0 else (c, sn)
        q, kk, v = cuda.gemm_i8_qkv_rope(w, dev(xq), dev(xs), dev(qn), dev(kn), None if c is None else dev(c),
                                         None if sn is None else dev(sn), rope_half, round_qkv=rnd)
        cuda.check()
        src = oracle.bf16_round(qkv) if rnd else qkv
        qo, ko, vo = oracle.qkv_rope(src, qn, kn, c, sn, heads, hd, rope_half)
        # only the order of the sum of squares differs from the oracle: outputs agree to bf16 rounding
        assert rel_l2(host(q), qo) < 3e-3 and rel_l2(host(kk), ko) < 3e-3
        assert np.array_equal(host(v), oracle.bf16_round(vo))
        assert np.mean(host(q) != oracle.bf16_round(qo)) < 2e-3
        if rnd and rope_half:
            # the same bits as the two-launch form (GEMM to bf16, then the stand-alone QK-norm + RoPE kernel),
            # which is what the sequence-parallel chain runs on the gathered heads
            y16 = cuda.gemm_i8(w, dev(xq), dev(xs), out_dtype=torch.bfloat16)
            q2, k2, v2 = cuda.qkv_rope(y16, dev(qn), dev(kn), dev(c), dev(sn), heads, hd, rope_half)
            assert torch.equal(q, q2) and torch.equal(kk, k2) and torch.equal(v, v2)


def test_reference_linear_entry_point(cuda, oracle):
    """h3_cuda_gemm_i8_dequant_f32_w_act_dev(_epi): f32 activations in, ConvRot + quant + GEMM inside."""
    from h3c_b200.lib import DitGemmEpi
    rng = np.random.default_rng(31)
    m, n, k = 70, 256, 512
    w, w_i8, s = make_weight(cuda, rng, n, k)
    x = acts(rng, m, k)
    for gs in (0, 256):
        y = cuda.gemm_i8_dequant_f32_w_act_dev(w, dev(x), gs)
        xq, xs = oracle.quantize_act_int8(oracle.convrot(x, gs))
        ref = oracle.gemm_i8_dequant(xq, w_i8, xs, s)
        if gs == 0:
            assert np.array_equal(host(y), ref)
        else:
            assert rel_l2(host(y), ref) < 2e-3  # butterfly vs dense rotation: a few codes move by one step
    epi = DitGemmEpi()
    epi.swiglu = 1
    y = cuda.gemm_i8_dequant_f32_w_act_dev(w, dev(x), 0, epi)
    xq, xs = oracle.quantize_act_int8(x)
    assert rel_l2(host(y), oracle.dequant_swiglu(oracle.gemm_i8_i32(xq, w_i8), xs, s)) < 1e-6
    # the reference's d_lora field through its own entry point
    lora = dev(rng.normal(0, 0.05, (m, n)).astype(np.float32))
    epi.d_lora = lora.data_ptr()
    y = cuda.gemm_i8_dequant_f32_w_act_dev(w, dev(x), 0, epi)
    assert rel_l2(host(y), oracle.dequant_swiglu(oracle.gemm_i8_i32(xq, w_i8), xs, s, host(lora))) < 1e-6


def test_gemm_full_size_sampled(cuda):
    """Benchmark shape (M=6144, K=3072, N=9216): exact accumulators on sampled rows, every column."""
    rng = np.random.default_rng(32)
    m, n, k = 6144, 9216, 3072
    w, w_i8, _ = make_weight(cuda, rng, n, k)
    x = rng.integers(-127, 128, (m, k), dtype=np.int8)
    a = torch.ones(m, dtype=torch.float32, device="cuda")
    acc = cuda.gemm_i8(w, dev(x), a, out_dtype=torch.int32)
    cuda.check()
    rows = np.concatenate([[0, 127, 128, m - 1], rng.integers(0, m, 28)])
    want = x[rows].astype(np.int32) @ w_i8.astype(np.int32).T
    assert np.array_equal(host(acc[torch.from_numpy(rows).cuda()]), want)
    # linearity in the activation scale (size-independent property of the dequant epilogue)
    y1 = cuda.gemm_i8(w, dev(x), a)
    y2 = cuda.gemm_i8(w, dev(x), 2 * a)
    assert torch.equal(y2, 2 * y1)


# ----------------------------------------------------------------- attention

@pytest.mark.parametrize("lq,lk,heads", [(128, 128, 2), (200, 333, 3), (64, 1, 1), (384, 1024, 2)])
def test_sdpa_bf16(cuda, oracle, lq, lk, heads):
    rng = np.random.default_rng(40 + lq)
    hd = 128
    q = dev(rng.normal(0, 1, (lq, heads, hd)).astype(np.float32), torch.bfloat16)
    k = dev(rng.normal(0, 1, (lk, heads, hd)).astype(np.float32), torch.bfloat16)
    v = dev(rng.normal(0, 1, (lk, heads, hd)).astype(np.float32), torch.bfloat16)
    out = cuda.sdpa_bf16(q, k, v)
    cuda.check()
    want = oracle.sdpa(host(q), host(k), host(v))
    # bf16 probabilities and bf16 output: 2e-3 relative L2 against the f32 evaluation of the same inputs
    assert rel_l2(host(out), want) < 4e-3


def test_sdpa_growing_row_maximum(cuda, oracle):
    """Later key tiles carry much larger scores, so the running maximum jumps by more than the lazy-rescale
    threshold several times and the accumulator rescale path runs."""
    rng = np.random.default_rng(44)
    lq, lk, heads, hd = 300, 1024, 2, 128
    q = dev(rng.normal(0, 1, (lq, heads, hd)).astype(np.float32), torch.bfloat16)
    kf = rng.normal(0, 1, (lk, heads, hd)).astype(np.float32) * np.linspace(0.05, 6.0, lk, dtype=np.float32)[:, None, None]
    k = dev(kf, torch.bfloat16)
    v = dev(rng.normal(0, 1, (lk, heads, hd)).astype(np.float32), torch.bfloat16)
    out = cuda.sdpa_bf16(q, k, v)
    cuda.check()
    assert rel_l2(host(out), oracle.sdpa(host(q), host(k), host(v))) < 4e-3


def test_sdpa_cross_strided(cuda, oracle):
    """Cross-attention: K and V are the two halves of one [T, 2*D] projection (row stride 2*D)."""
    rng = np.random.default_rng(45)
    lq, t, heads, hd = 300, 512, 2, 128
    D = heads * hd
    q = dev(rng.normal(0, 1, (lq, heads, hd)).astype(np.float32), torch.bfloat16)
    kv = dev(rng.normal(0, 1, (t, 2 * D)).astype(np.float32), torch.bfloat16)
    k = kv[:, :D].view(t, heads, hd)
    v = kv[:, D:].view(t, heads, hd)
    out = cuda.sdpa_bf16(q, k, v)
    cuda.check()
    want = oracle.sdpa(host(q), host(k.contiguous()), host(v.contiguous()))
    assert rel_l2(host(out), want) < 4e-3


def test_sdpa_full_size_sampled(cuda, oracle):
    """Self-attention at the benchmark's 6,144 tokens (2 of 24 heads): sampled query rows against the oracle."""
    rng = np.random.default_rng(46)
    L, heads, hd = 6144, 2, 128
    q = dev(rng.normal(0, 1, (L, heads, hd)).astype(np.float32), torch.bfloat16)
    k = dev(rng.normal(0, 1, (L, heads, hd)).astype(np.float32), torch.bfloat16)
    v = dev(rng.normal(0, 1, (L, heads, hd)).astype(np.float32), torch.bfloat16)
    out = cuda.sdpa_bf16(q, k, v)
    cuda.check()
    rows = np.concatenate([[0, 127, 128, L - 1], rng.integers(0, L, 12)])
    want = oracle.sdpa(host(q)[rows], host(k), host(v))
    assert rel_l2(host(out)[rows], want) < 4e-3
    # softmax rows sum to one: with V = 1 the output is exactly 1 up to bf16 rounding of P
    ones = torch.ones_like(v)
    o1 = cuda.sdpa_bf16(q, k, ones)
    assert float((o1.float() - 1).abs().max()) < 2e-2


def test_reference_sdpa_entry_point(cuda, oracle):
    rng = np.random.default_rng(47)
    seq, heads, hd = 150, 2, 128
    q, k, v = (rng.normal(0, 1, (seq, heads, hd)).astype(np.float32) for _ in range(3))
    out = cuda.sdpa_f16_dev(dev(q), dev(k), dev(v))
    cuda.check()
    assert rel_l2(host(out), oracle.sdpa(q, k, v)) < 1e-3  # f16 staging like the reference: 11-bit operands, f32 accumulation


# --------------------------------------------------------------------- NVFP4

@pytest.mark.parametrize("m,k", [(5, 64), (130, 256), (128, 3072)])
def test_quantize_act_nvfp4_exact(cuda, oracle, m, k):
    rng = np.random.default_rng(50 + m)
    x = acts(rng, m, k)
    x[0, :16] = 0.0          # all-zero block -> scale byte for 1.0
    x[1 % m, 16:32] = 1e-9   # underflow -> clamped to byte 1
    packed, sf = cuda.quantize_act_nvfp4(dev(x))
    po, so = oracle.quantize_nvfp4(x)
    assert np.array_equal(host(packed), po)
    assert np.array_equal(host(sf), so)


# N >= 256 takes the 128 x 256 tile (N = 384 and 648 end in a tile without a second scale block, 648 also in a
# column group cut by the tensor edge), N = 128 the 128 x 128 tile
@pytest.mark.parametrize("m,n,k", [(128, 128, 256), (200, 384, 512), (130, 256, 3072), (64, 128, 192), (300, 648, 1024)])
def test_gemm_nvfp4(cuda, oracle, m, n, k):
    """Block-scaled FP4 GEMM against the dequantised f32 product of the same codes and scales."""
    rng = np.random.default_rng(60 + m)
    x = acts(rng, m, k)
    w = rng.normal(0, 0.02, (n, k)).astype(np.float32)
    w4, sfw = oracle.quantize_nvfp4(w, rule=1)           # the reference's weight-side quantiser
    x4, sfx = cuda.quantize_act_nvfp4(dev(x))            # its activation-side rule, on the device
    y = cuda.gemm_fp4(dev(w4), dev(sfw), x4, sfx, alpha=0.5)
    cuda.check()
    want = oracle.gemm_nvfp4(host(x4), host(sfx), w4, sfw, 0.5)
    assert rel_l2(host(y), want) < 1e-5
    yb = cuda.gemm_fp4(dev(w4), dev(sfw), x4, sfx, alpha=1.0, out_dtype=torch.bfloat16)
    assert rel_l2(host(yb), oracle.gemm_nvfp4(host(x4), host(sfx), w4, sfw, 1.0)) < 3e-3
    # quantisation itself costs a few percent against the f32 product: a sanity bound on the whole path
    assert rel_l2(host(y), 0.5 * x @ w.T) < 0.2


@pytest.mark.parametrize("m,k,gs,dtype", [(300, 512, 256, "f32"), (128, 3072, 0, "f32"), (77, 1024, 64, "bf16")])
def test_row_kernel_quantises_to_nvfp4_in_its_last_stage(cuda, oracle, m, k, gs, dtype):
    """RMSNorm + modulation + ConvRot + NVFP4 quantisation in one pass over the row: codes and scale bytes equal the
    stand-alone quantiser applied to the values the same launch writes out (bit for bit), pad rows' scale bytes are 0."""
    rng = np.random.default_rng(83)
    td = torch.float32 if dtype == "f32" else torch.bfloat16
    x = dev(acts(rng, m, k)).to(td)
    nw = dev(rng.normal(1, 0.1, k).astype(np.float32))
    mod = dev(rng.normal(0, 0.3, (3, 6, k)).astype(np.float32))
    rmap = dev((np.arange(m) % 3).astype(np.int32))
    fp4 = torch.full((m, k // 2), 0xAB, dtype=torch.uint8, device="cuda")
    sf = torch.full((int(oracle.nvfp4_sf_bytes(m, k)),), 0xCD, dtype=torch.uint8, device="cuda")
    vals = torch.empty((m, k), dtype=torch.float32 if gs else td, device="cuda")
    cuda.norm(x, norm_w=nw, modulation=mod, row_map=rmap, slots=6, shift_slot=3, scale_slot=4, convrot_gs=gs,
              rot=vals if gs else None, normed=None if gs else vals, fp4=fp4, sf=sf)
    cuda.check()
    want4, wantsf = cuda.quantize_act_nvfp4(vals.float().contiguous())
    assert torch.equal(fp4, want4)
    assert torch.equal(sf, wantsf)
    po, so = oracle.quantize_nvfp4(host(vals.float()))      # and the stand-alone quantiser is pinned to the checker
    assert np.array_equal(host(fp4), po) and np.array_equal(host(sf), so)


@pytest.mark.parametrize("m,n,k", [(150, 512, 512), (333, 1024, 256), (128, 256, 1024)])
def test_gemm_nvfp4_swiglu_in_the_epilogue(cuda, oracle, m, n, k):
    """SwiGLU on the f32 accumulators inside the GEMM (gate rows | up rows of the weight): the reference's chain
    h3_cutlass_nvfp4_fc1_f32_run -> SwiGLU (h3_dit_nvfp4_chain.cu:201-277) as one kernel."""
    import h3c_b200
    if not h3c_b200.plugin_enabled("H3B_FP4_WIDE"):
        pytest.skip("the fused SwiGLU epilogue belongs to the 128 x 256 tile form (H3B_FP4_WIDE=0 is set)")
    rng = np.random.default_rng(71)
    x = acts(rng, m, k)
    w = rng.normal(0, 0.05, (n, k)).astype(np.float32)
    w4, sfw = oracle.quantize_nvfp4(w, rule=1)
    x4, sfx = cuda.quantize_act_nvfp4(dev(x))
    want = oracle.swiglu(oracle.gemm_nvfp4(host(x4), host(sfx), w4, sfw, 0.5))
    y = cuda.gemm_fp4(dev(w4), dev(sfw), x4, sfx, alpha=0.5, swiglu=True)
    assert y.shape == (m, n // 2)
    assert rel_l2(host(y), want) < 1e-5
    yb = cuda.gemm_fp4(dev(w4), dev(sfw), x4, sfx, alpha=0.5, swiglu=True, out_dtype=torch.bfloat16)
    assert rel_l2(host(yb), want) < 3e-3
    cuda.check()


@pytest.mark.parametrize("m,heads,k,rope_half", [(200, 2, 256, 48), (130, 3, 512, 64), (300, 2, 256, 0)])
def test_gemm_nvfp4_qkv_rope_in_the_epilogue(cuda, oracle, m, heads, k, rope_half):
    """NVFP4 QKV projection with QK-norm and split-half RoPE in its epilogue: the bits of the two-step route (GEMM to
    f32, then the stand-alone QK-norm + RoPE kernel), which the checker's h3_dit_w4a8_qkv_rope_f32 holds to bf16
    rounding.  Three heads: the last 256-column tile holds one head only."""
    from h3c_b200.lib import call, ptr
    rng = np.random.default_rng(90 + m)
    n, hd = 3 * heads * 128, 128
    w = rng.normal(0, 0.05, (n, k)).astype(np.float32)
    w4, sfw = oracle.quantize_nvfp4(w, rule=1)
    wh = cuda.nvfp4_weight(w4, sfw, 0.75, n, k)
    x4, sfx = cuda.quantize_act_nvfp4(dev(acts(rng, m, k)))
    qn, kn = dev(rng.normal(1, 0.1, hd).astype(np.float32)), dev(rng.normal(1, 0.1, hd).astype(np.float32))
    ang = rng.uniform(0, 6.28, (m, max(rope_half, 1))).astype(np.float32)
    cos, sin = dev(np.cos(ang)), dev(np.sin(ang))
    q, kk, v = (torch.full((m, heads, hd), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(3))
    call("h3b_gemm_fp4_w_preq_qkv_rope_dev", cuda.h, wh, ptr(x4), ptr(sfx), m, 1.0, ptr(qn), ptr(kn),
         ptr(cos) if rope_half else None, ptr(sin) if rope_half else None, rope_half, heads, 1e-5, ptr(q), ptr(kk), ptr(v))
    cuda.check()
    qkv = cuda.gemm_fp4(dev(w4), dev(sfw), x4, sfx, alpha=0.75)
    q2, k2, v2 = cuda.qkv_rope(qkv, qn, kn, cos, sin, heads, hd, rope_half, out_dtype=torch.bfloat16)
    assert torch.equal(q, q2) and torch.equal(kk, k2) and torch.equal(v, v2)
    qo, ko, vo = oracle.qkv_rope(host(qkv), host(qn), host(kn), host(cos) if rope_half else None,
                                 host(sin) if rope_half else None, heads, hd, rope_half)
    assert rel_l2(host(q), qo) < 3e-3 and rel_l2(host(kk), ko) < 3e-3 and np.array_equal(host(v), oracle.bf16_round(vo))
    cuda.nvfp4_weight_free(wh)


@pytest.mark.parametrize("m,n,k", [(150, 256, 512), (300, 640, 1024), (90, 128, 256)])
def test_reference_nvfp4_linear_entry_points(cuda, oracle, m, n, k):
    rng = np.random.default_rng(61)
    slots = 6
    x = acts(rng, m, k)
    w = rng.normal(0, 0.02, (n, k)).astype(np.float32)
    w4, sfw = oracle.quantize_nvfp4(w, rule=1)
    wh = cuda.nvfp4_weight(w4, sfw, 0.75, n, k)
    x4, sfx = oracle.quantize_nvfp4(x)
    base = oracle.gemm_nvfp4(x4, sfx, w4, sfw, 0.75)
    y = cuda.gemm_fp4_w_act_dev(wh, dev(x))
    assert rel_l2(host(y), base) < 1e-5
    res = rng.normal(0, 1, (m, n)).astype(np.float32)
    mod = rng.normal(0, 0.5, (3, slots, n)).astype(np.float32)
    rmap = (np.arange(m) % 3).astype(np.uint32)
    y = cuda.gemm_fp4_w_act_dev(wh, dev(x), kind="gate", residual=dev(res), modulation=dev(mod),
                                row_map=dev(rmap.view(np.int32)), slots=slots, gate_slot=5)
    assert rel_l2(host(y), oracle.gate(res, base, mod, rmap, slots, 5)) < 1e-5
    y = cuda.gemm_fp4_w_act_dev(wh, dev(x), kind="swiglu")
    import h3c_b200
    if n % 256 == 0 and h3c_b200.plugin_enabled("H3B_FP4_WIDE"):   # SwiGLU on the f32 accumulators in the GEMM epilogue
        assert rel_l2(host(y), oracle.swiglu(base)) < 1e-5
    else:              # other widths: bf16 accumulators and a second kernel, as in the reference's fp4 path
        fused = oracle.bf16_round(oracle.gemm_nvfp4(x4, sfx, w4, sfw, 1.0)) * np.float32(0.75)
        assert rel_l2(host(y), oracle.swiglu(fused)) < 2e-3
    cuda.check()
    cuda.nvfp4_weight_free(wh)


def test_host_buffer_adaln(cuda, oracle):
    rng = np.random.default_rng(51)
    x = rng.normal(0, 1, (9, 64)).astype(np.float32)
    nw = rng.normal(1, 0.1, 64).astype(np.float32)
    mod = rng.normal(0, 0.3, (3, 6, 64)).astype(np.float32)
    rmap = (np.arange(9) % 3).astype(np.uint32)
    assert rel_l2(cuda.adaln_f32(x, nw, mod, rmap, 6, 0, 1), oracle.adaln(x, nw, mod, rmap, 6, 0, 1)) < 2e-6


def test_scatter_epilogues_on_one_gpu(cuda, oracle):
    """The sequence-parallel stores of the QKV GEMM epilogue and of the attention epilogue, exercised on one
    GPU: two emulated ranks whose "peer" buffers are all local.  Gathered Q/K/V must be the plain kernel's
    output permuted by the reference's all-to-all map, and the scattered attention rows the plain
    attention's output, bit for bit."""
    from h3c_b200.lib import UlyssesDirect
    rng = np.random.default_rng(41)
    u, heads, hd, k, seq_local = 2, 4, 128, 256, 150          # seq_local not a multiple of the row tile
    hl, seq = heads // u, u * seq_local
    pt, ph, pw = oracle.fill_video_pos(16, 12, 10, 10)
    inv_freq = (1.0 / (10000.0 ** (np.arange(16) / 16.0))).astype(np.float32)
    cos, sin = oracle.rope_tables(inv_freq, pt[:seq], ph[:seq], pw[:seq], 1.0)
    w, w_i8, s = make_weight(cuda, rng, 3 * heads * hd, k)
    xq, xs = oracle.quantize_act_int8(acts(rng, seq, k))
    qn, kn = rng.normal(1, 0.1, hd).astype(np.float32), rng.normal(1, 0.1, hd).astype(np.float32)
    dqn, dkn, dcos, dsin = dev(qn), dev(kn), dev(cos), dev(sin)
    q_ref, k_ref, v_ref = cuda.gemm_i8_qkv_rope(w, dev(xq), dev(xs), dqn, dkn, dcos, dsin, 48)   # [seq, heads, hd]
    # per emulated rank: gathered Q/K/V [seq, hl, hd] and attention rows [seq_local, heads, hd]
    gq, gk, gv = ([torch.zeros((seq, hl, hd), dtype=torch.bfloat16, device="cuda") for _ in range(u)] for _ in range(3))
    att = [torch.zeros((seq_local, heads, hd), dtype=torch.bfloat16, device="cuda") for _ in range(u)]
    directs = []
    for r in range(u):
        d = UlyssesDirect()
        d.ulysses, d.rank, d.seq_local, d.heads, d.head_dim = u, r, seq_local, heads, hd
        d.q, d.k, d.v, d.att = gq[r].data_ptr(), gk[r].data_ptr(), gv[r].data_ptr(), att[r].data_ptr()
        for p_ in range(u):
            d.peer_q[p_], d.peer_k[p_], d.peer_v[p_] = gq[p_].data_ptr(), gk[p_].data_ptr(), gv[p_].data_ptr()
            d.peer_att[p_] = att[p_].data_ptr()
        directs.append(d)
    for r in range(u):
        rows = slice(r * seq_local, (r + 1) * seq_local)
        cuda.gemm_i8_qkv_rope_scatter(w, dev(xq[rows]), dev(xs[rows]), dqn, dkn, dev(cos[rows]), dev(sin[rows]), 48,
                                      directs[r])
    cuda.check()
    for r in range(u):
        for got, ref in ((gq[r], q_ref), (gk[r], k_ref), (gv[r], v_ref)):
            assert torch.equal(got, ref[:, r * hl:(r + 1) * hl])
    seq_real = seq - 7                                            # pad rows stay zero
    o_ref = cuda.sdpa_bf16(q_ref[:seq_real], k_ref[:seq_real], v_ref[:seq_real]).view(seq_real, heads, hd)
    for r in range(u):
        cuda.sdpa_bf16_scatter(directs[r], seq_real)
    cuda.check()
    got = torch.cat(att, 0)
    assert torch.equal(got[:seq_real], o_ref) and not got[seq_real:].any()


def test_empty_and_misaligned_inputs_are_refused(cuda):
    """Zero-sized or misaligned calls return the reference-style error instead of launching anything."""
    import h3c_b200
    rng = np.random.default_rng(42)
    w, _, _ = make_weight(cuda, rng, 128, 128)
    x0 = torch.empty((0, 128), dtype=torch.int8, device="cuda")
    with pytest.raises(h3c_b200.H3Error):
        cuda.gemm_i8(w, x0, torch.empty(0, device="cuda"))
    with pytest.raises(h3c_b200.H3Error):
        cuda.quantize_act_int8(torch.empty((0, 128), device="cuda"))
    q = torch.zeros((8, 2, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(h3c_b200.H3Error):
        cuda.sdpa_bf16(q[:0], q, q)
    with pytest.raises(h3c_b200.H3Error):                       # head_dim 64 is not built
        cuda.sdpa_bf16(q[..., :64].contiguous(), q[..., :64].contiguous(), q[..., :64].contiguous())
    xq = torch.zeros((9, 129), dtype=torch.int8, device="cuda")[:, 1:]   # rows not 16-byte aligned
    with pytest.raises(h3c_b200.H3Error):
        cuda.gemm_i8(w, xq, torch.ones(9, device="cuda"))
    cuda.check()


# ------------------------------------------------- the step on either side of the block chain

@pytest.mark.parametrize("m,n,k", [(70, 256, 96), (300, 96, 3072), (129, 32, 1000), (17, 65, 30)])
def test_dense_f32(cuda, oracle, m, n, k):
    """Patch-embedding / final-head linear: f32 FMA chain in k order against the reference's scalar loop
    (which starts its sum at the bias); 1e-5 relative L2 covers the different rounding of the partial sums."""
    rng = np.random.default_rng(70 + m)
    x = rng.normal(0, 1, (m, k)).astype(np.float32)
    w = rng.normal(0, 0.05, (n, k)).astype(np.float32)
    b = rng.normal(0, 0.1, n).astype(np.float32)
    want = oracle.dense(x, w, b)
    assert rel_l2(host(cuda.dense_f32(dev(x), dev(w), dev(b))), want) < 1e-5
    two_calls = cuda.bias_add_f32(cuda.gemm_f32_dd(dev(x), dev(w)), dev(b))   # the reference's pair of calls
    assert rel_l2(host(two_calls), want) < 1e-5
    assert rel_l2(host(cuda.dense_f32(dev(x), dev(w))), oracle.dense(x, w)) < 1e-5
    if k % 4:   # the scalar-load form is also reached by a misaligned view
        assert rel_l2(host(cuda.gemm_f32_dd(dev(x), dev(w))), oracle.dense(x, w)) < 1e-5


def test_step_sides_against_golden_vectors(cuda, golden):
    """Patch embedding, final head (adaLN with one modulation row + dense) and Euler update on the vectors
    that the reference's own functions produced; the Euler update is bit-exact given the same velocity."""
    import h3c_b200
    g = golden("step_sides")
    emb = cuda.dense_f32(dev(g["latent"]), dev(g["patch_w"]), dev(g["patch_b"]))
    assert rel_l2(host(emb), g["embedded"]) < 1e-5
    vel = cuda.final_head_f32(dev(g["x"]), dev(g["norm_w"]), dev(g["modulation"]), dev(g["final_w"]), dev(g["final_b"]))
    assert rel_l2(host(vel), g["velocity"]) < 1e-5
    s0, s1 = (float(v) for v in g["sigma"])
    stepped = cuda.euler_step_f32(dev(g["latent"]), dev(g["velocity"]), s0, s1)
    assert np.array_equal(host(stepped), g["stepped"])
    for sigma, nxt in ((0.5, 0.5), (0.25, 0.5), (0.5, -0.1), (float("nan"), 0.1)):   # pairs the reference rejects
        with pytest.raises(h3c_b200.H3Error):
            cuda.euler_step_f32(dev(g["latent"]), dev(g["velocity"]), sigma, nxt)


def test_flag_barrier_gives_up_on_an_absent_rank(cuda):
    """The barrier of the exchange-free Ulysses form waits a bounded time: with the peer's word set it passes,
    with a peer that never arrives it returns after the budget with status 6 and the context stays usable."""
    import ctypes as C
    from h3c_b200.lib import call
    arrived, absent = C.c_int(-1), C.c_int(-1)
    call("h3b_ulysses_barrier_selftest", 2_000_000, C.byref(arrived), C.byref(absent))   # about a millisecond
    assert arrived.value == 0 and absent.value == 6
    x = torch.arange(8, device="cuda")
    assert int(x.sum().item()) == 28
    cuda.check()


def test_lora_delta_by_the_reference_call_pair(cuda, oracle):
    """t = x A^T, delta = scale * t B^T + beta * delta with the reference's two calls (h3_dit_w4a8.c:1036-1050),
    against the same products in float64; the delta then rides the INT8 GEMM epilogue as d_lora (tested above)."""
    rng = np.random.default_rng(95)
    m, k, r, n, scale = 200, 512, 16, 384, 0.7
    x = rng.normal(0, 1, (m, k)).astype(np.float32)
    a = rng.normal(0, 0.05, (r, k)).astype(np.float32)
    b = rng.normal(0, 0.05, (n, r)).astype(np.float32)
    d0 = rng.normal(0, 0.1, (m, n)).astype(np.float32)
    t = cuda.gemm_f32_dd(dev(x), dev(a))
    assert rel_l2(host(t), oracle.dense(x, a)) < 1e-5
    for beta, tf32_name in ((0.0, False), (1.0, False), (0.5, True)):
        want = scale * (x.astype(np.float64) @ a.T.astype(np.float64)) @ b.T.astype(np.float64) + beta * d0
        got = cuda.gemm_f32_dd_ex(t, dev(b), dev(d0.copy()), alpha=scale, beta=beta, tf32_name=tf32_name)
        assert rel_l2(host(got), want.astype(np.float32)) < 1e-5
