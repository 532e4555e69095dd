"""The reference's other two checkpoint formats through this library's own reader and block host: the W4A8 checkpoint
(packed 4-bit codes + codebook + E4M3 group scales + per-channel scale, h3_w4a8.c:75-115) and the NVFP4 sidecar
(h3_dit_w4a8.c:3158-3274).  A block loaded from a synthetic file gives the bits of the same block put together by hand
from the same arrays, and malformed files are refused with the tensor's name."""
import ctypes as C
import json
import struct

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

ERR = 512
DIM, HEADS, HD, FFN, MODS, TFEAT, SLOTS = 256, 2, 128, 512, 3, 8, 6
SUFFIX = {"qkv": "attn.qkv_proj", "out": "attn.out_proj", "fc1": "mlp.fc1", "fc2": "mlp.fc2"}
SHAPES = {"qkv": (3 * HEADS * HD, DIM), "out": (DIM, HEADS * HD), "fc1": (2 * FFN, DIM), "fc2": (DIM, FFN)}


def write_safetensors(path, tensors):
    """tensors: name -> (dtype name of the container, array)."""
    header, offset = {}, 0
    for name, (dt, a) in tensors.items():
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [offset, offset + a.nbytes]}
        offset += a.nbytes
    blob = json.dumps(header).encode()
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, a in tensors.values():
            f.write(np.ascontiguousarray(a).tobytes())


@pytest.fixture(scope="module")
def cuda():
    import h3c_b200
    c = h3c_b200.Cuda(0)
    yield c
    c.close()


@pytest.fixture(scope="module")
def oracle():
    from oracle.pyoracle import Oracle
    return Oracle()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def aux_tensors(rng):
    t = {"blocks.0.norm1.weight": rng.normal(1, 0.1, DIM), "blocks.0.norm2.weight": rng.normal(1, 0.1, DIM),
         "blocks.0.attn.q_norm.weight": rng.normal(1, 0.1, HD), "blocks.0.attn.k_norm.weight": rng.normal(1, 0.1, HD)}
    return {k: ("F32", v.astype(np.float32)) for k, v in t.items()}


def block_inputs(rng, seq=200):
    x = rng.normal(0, 1, (seq, DIM)).astype(np.float32)
    ang = rng.uniform(0, 6.28, (seq, 48)).astype(np.float32)
    mod = rng.normal(0, 0.3, (MODS, SLOTS, DIM)).astype(np.float32)
    rmap = (np.arange(seq) % MODS).astype(np.int32)
    return x, np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32), mod, rmap


def new_dit(cuda):
    from h3c_b200 import dit as D
    geo = D.DitGeometry(dim=DIM, heads=HEADS, head_dim=HD, ffn=FFN, n_blocks=1, mod_rows=MODS, t_dim=TFEAT,
                        kind=D.BLOCK_REFERENCE, stream_dtype=D.F32, convrot_gs=256)
    return D.Dit(cuda, geo)


def run(cuda, dit, inputs):
    x, cos, sin, mod, rmap = inputs
    y = dit.block_forward(0, dev(x), dev(cos), dev(sin), modulation=dev(mod), row_map=dev(rmap))
    cuda.check()
    return y


def open_ckpt(path):
    import h3c_b200
    err = C.create_string_buffer(ERR)
    h = h3c_b200.load().h3b_ckpt_open(str(path).encode(), err, ERR)
    assert h, err.value
    return h


def quads(rng):
    out = {}
    for name, (n, k) in SHAPES.items():
        out[name] = dict(packed=rng.integers(-128, 128, (n, k // 2), dtype=np.int8),
                         codebook=np.sort(rng.normal(0, 40, 16)).astype(np.float32),
                         s_rel=rng.integers(0x28, 0x48, (n, k // 16), dtype=np.uint8),
                         s_ch=rng.uniform(2e-4, 8e-4, n).astype(np.float32))
    return out


def test_w4a8_checkpoint_block(cuda, oracle, tmp_path):
    import h3c_b200
    from h3c_b200 import dit as D
    from h3c_b200.lib import call
    rng = np.random.default_rng(5)
    q, aux = quads(rng), aux_tensors(rng)
    tensors = dict(aux)
    for name, w in q.items():
        base = f"blocks.0.{SUFFIX[name]}"
        tensors[base + ".weight"] = ("I8", w["packed"])
        tensors[base + ".weight_codebook"] = ("F32", w["codebook"])
        tensors[base + ".weight_s_rel"] = ("F8_E4M3", w["s_rel"])
        tensors[base + ".weight_s_channel"] = ("F32", w["s_ch"])
    path = tmp_path / "synthetic_w4a8.safetensors"
    write_safetensors(path, tensors)

    loaded = new_dit(cuda)
    ck = open_ckpt(path)
    call("h3b_dit_load_w4a8_block", loaded.h, ck, 0, 0)
    h3c_b200.load().h3b_ckpt_close(ck)          # the weights are resident: the mapping may go

    by_hand = new_dit(cuda)
    for name, w in q.items():
        wt = cuda.weight_from_w4a8(w["packed"], w["codebook"], w["s_rel"], w["s_ch"])
        # the decode is the reference's rule, bit for bit
        assert np.array_equal(wt.download_int8(), oracle.w4a8_dequant_to_int8(w["packed"], w["codebook"], w["s_rel"]))
        by_hand.set_linear(0, D.LIN_NAMES_REF[name], wt)
    by_hand.set_block_aux(0, *(aux[f"blocks.0.{n}.weight"][1] for n in ("norm1", "norm2", "attn.q_norm", "attn.k_norm")))

    inputs = block_inputs(rng)
    y_loaded, y_hand = run(cuda, loaded, inputs), run(cuda, by_hand, inputs)
    assert torch.isfinite(y_loaded).all() and torch.equal(y_loaded, y_hand)
    loaded.close()
    by_hand.close()

    # refused, naming the tensor: a group-scale tensor of the wrong type, a missing codebook
    err = C.create_string_buffer(ERR)
    for breakage, word in (("dtype", b"weight_s_rel"), ("missing", b"weight_codebook")):
        bad = dict(tensors)
        if breakage == "dtype":
            bad["blocks.0.mlp.fc1.weight_s_rel"] = ("U8", q["fc1"]["s_rel"])
        else:
            del bad["blocks.0.attn.out_proj.weight_codebook"]
        bpath = tmp_path / f"bad_{breakage}.safetensors"
        write_safetensors(bpath, bad)
        d = new_dit(cuda)
        ck = open_ckpt(bpath)
        assert h3c_b200.load().h3b_dit_load_w4a8_block(d.h, ck, 0, 0, err, ERR) == 0
        assert word in err.value
        h3c_b200.load().h3b_ckpt_close(ck)
        d.close()


@pytest.mark.parametrize("mask", [0b1111, 0b1100])
def test_nvfp4_sidecar_block(cuda, oracle, tmp_path, mask):
    """INT8-ConvRot checkpoint + NVFP4 sidecar, with the sidecar used for all four linears or for the MLP only (the
    reference's per-linear NVFP4 / INT8 choice, h3_dit_w4a8.c:3519-3590)."""
    import h3c_b200
    from h3c_b200 import dit as D
    from h3c_b200.lib import call
    rng = np.random.default_rng(6)
    aux = aux_tensors(rng)
    base_t, side_t, i8, fp4 = dict(aux), {}, {}, {}
    for idx, (name, (n, k)) in enumerate(SHAPES.items()):
        w_i8 = rng.integers(-127, 128, (n, k), dtype=np.int8)
        s = rng.uniform(2e-4, 8e-4, (n, 1)).astype(np.float32)
        i8[name] = (w_i8, s[:, 0].copy())
        base = f"blocks.0.{SUFFIX[name]}"
        base_t[base + ".weight"] = ("I8", w_i8)
        base_t[base + ".weight_scale"] = ("F32", s)
        w = w_i8.astype(np.float32) * s
        scale2 = np.float32(np.abs(w).max() / (6.0 * 448.0))
        w4, sfw = oracle.quantize_nvfp4(w / scale2, rule=1)
        fp4[name] = (w4, sfw, scale2)
        side_t[base + ".weight_fp4"] = ("U8", w4)
        side_t[base + ".weight_sf"] = ("U8", sfw)
        if idx != 1:   # `weight_scale2` is optional: the out projection goes without it, with its weights scaled to fit
            side_t[base + ".weight_scale2"] = ("F32", np.array([scale2], np.float32))
        else:
            w4, sfw = oracle.quantize_nvfp4(w, rule=1)
            fp4[name] = (w4, sfw, np.float32(1.0))
            side_t[base + ".weight_fp4"], side_t[base + ".weight_sf"] = ("U8", w4), ("U8", sfw)
    path, side = tmp_path / "synthetic.safetensors", tmp_path / "synthetic.nvfp4.safetensors"
    write_safetensors(path, base_t)
    write_safetensors(side, side_t)

    loaded = new_dit(cuda)
    ck, sc = open_ckpt(path), open_ckpt(side)
    call("h3b_dit_load_int8_convrot_block", loaded.h, ck, 0, 0)
    call("h3b_dit_load_nvfp4_block", loaded.h, sc, 0, 0, mask)
    h3c_b200.load().h3b_ckpt_close(ck)
    h3c_b200.load().h3b_ckpt_close(sc)

    by_hand = new_dit(cuda)
    for idx, name in enumerate(SHAPES):
        by_hand.set_linear(0, D.LIN_NAMES_REF[name], cuda.weight_from_i8(*i8[name]))
        if mask & (1 << idx):
            w4, sfw, scale2 = fp4[name]
            by_hand.set_linear_nvfp4(0, D.LIN_NAMES_REF[name], cuda.nvfp4_weight(w4, sfw, float(scale2), *SHAPES[name]), own=True)
    by_hand.set_block_aux(0, *(aux[f"blocks.0.{n}.weight"][1] for n in ("norm1", "norm2", "attn.q_norm", "attn.k_norm")))

    inputs = block_inputs(rng)
    y_loaded, y_hand = run(cuda, loaded, inputs), run(cuda, by_hand, inputs)
    assert torch.isfinite(y_loaded).all() and torch.equal(y_loaded, y_hand)
    loaded.close()
    by_hand.close()

    # a sidecar whose scale tensor has the wrong size is refused, naming it
    bad = dict(side_t)
    bad["blocks.0.mlp.fc2.weight_sf"] = ("U8", side_t["blocks.0.mlp.fc2.weight_sf"][1][:-512])
    bpath = tmp_path / "bad.nvfp4.safetensors"
    write_safetensors(bpath, bad)
    d = new_dit(cuda)
    sc = open_ckpt(bpath)
    err = C.create_string_buffer(ERR)
    assert h3c_b200.load().h3b_dit_load_nvfp4_block(d.h, sc, 0, 0, 0b1000, err, ERR) == 0
    assert b"weight_sf" in err.value
    h3c_b200.load().h3b_ckpt_close(sc)
    d.close()
