"""The drop-in, run: the reference's UNMODIFIED DiT host (oracle/_ref/libh3_refhost.so = its h3_dit_w4a8.c,
weight cache, safetensors and INT8-ConvRot readers, linked against libh3_b200.so in place of its own CUDA
operator library) opens a seeded synthetic INT8-ConvRot checkpoint at the reference's real geometry
(hidden 5376, 56 x 128 heads, FFN 14336, SwiGLU, 256-wide rotation) and runs one block through its own
h3_dit_w4a8_block_forward_f32.  Every GPU operator underneath is this library's.  The result is compared with
the reference's f32 CPU block (the oracle's restatement of it, which the golden tests pin to the reference bit
for bit): relative L2 <= 2e-2, the bound stated for the f32 CPU block."""
import ctypes as C
import json
import struct
from pathlib import Path

import numpy as np
import pytest

from tests.conftest import rel_l2

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

ROOT = Path(__file__).resolve().parent.parent
REFHOST = ROOT / "oracle" / "_ref" / "libh3_refhost.so"

HIDDEN, HEADS, HD, FFN, SLOTS, MODS, TFEAT = 5376, 56, 128, 14336, 6, 3, 8
INNER = HEADS * HD
ERR = 512


def write_safetensors(path, tensors):
    """Minimal writer of the safetensors container: 8-byte little-endian header length, JSON header, raw data."""
    dt = {np.dtype(np.int8): "I8", np.dtype(np.float32): "F32", np.dtype(np.uint8): "U8"}
    header, offset = {}, 0
    for name, a in tensors.items():
        header[name] = {"dtype": dt[a.dtype], "shape": list(a.shape), "data_offsets": [offset, offset + a.nbytes]}
        offset += a.nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for a in tensors.values():
            f.write(np.ascontiguousarray(a).tobytes())


class BlockAux(C.Structure):   # h3_dit_w4a8_block_aux (h3_dit_w4a8.h:94-106)
    _fields_ = [("norm1", C.c_void_p), ("norm2", C.c_void_p), ("q_norm", C.c_void_p), ("k_norm", C.c_void_p),
                ("adaln_w", C.c_void_p), ("adaln_b", C.c_void_p), ("adaln_out", C.c_size_t), ("adaln_in", C.c_size_t),
                ("inv_freq", C.c_void_p), ("t_table", C.c_void_p), ("t_table_rows", C.c_size_t)]


class CacheConfig(C.Structure):   # h3_w4a8_cache_config (h3_w4a8_cache.h:39-45)
    _fields_ = [("n_blocks", C.c_uint), ("policy", C.c_int), ("window_size", C.c_uint), ("vram_budget_bytes", C.c_size_t),
                ("vram_reserve_bytes", C.c_size_t)]


def fptr(a):
    return a.ctypes.data_as(C.c_void_p)


def test_reference_host_runs_a_real_geometry_block_on_this_library(tmp_path, oracle):
    if not REFHOST.exists():
        pytest.skip("oracle/_ref/libh3_refhost.so not built (reference tree absent at build time)")
    rng = np.random.default_rng(2024)
    seq = 96

    def lin(n, k):
        return rng.integers(-127, 128, (n, k), dtype=np.int8), rng.uniform(5e-5, 2e-4, n).astype(np.float32)

    W = {"attn.qkv_proj": lin(3 * INNER, HIDDEN), "attn.out_proj": lin(HIDDEN, INNER), "mlp.fc1": lin(2 * FFN, HIDDEN),
         "mlp.fc2": lin(HIDDEN, FFN)}
    n1, n2 = (rng.normal(1, 0.1, HIDDEN).astype(np.float32) for _ in range(2))
    qn, kn = (rng.normal(1, 0.1, HD).astype(np.float32) for _ in range(2))
    inv_freq = (1.0 / (10000.0 ** (np.arange(16) / 16.0))).astype(np.float32)
    tensors = {"rope.inv_freq": inv_freq, "blocks.0.norm1.weight": n1, "blocks.0.norm2.weight": n2,
               "blocks.0.attn.q_norm.weight": qn, "blocks.0.attn.k_norm.weight": kn,
               "blocks.0.adaln_proj.linear.weight": rng.normal(0, 0.1, (MODS * SLOTS * HIDDEN, TFEAT)).astype(np.float32),
               "blocks.0.adaln_proj.linear.bias": rng.normal(0, 0.1, MODS * SLOTS * HIDDEN).astype(np.float32),
               "adaln_t_table": rng.normal(0, 1, (1025, TFEAT)).astype(np.float32)}
    for name, (w, s) in W.items():
        tensors[f"blocks.0.{name}.weight"] = w
        tensors[f"blocks.0.{name}.weight_scale"] = s
    path = tmp_path / "synthetic_int8_convrot.safetensors"
    write_safetensors(path, tensors)

    L = C.CDLL(str(REFHOST))
    err = C.create_string_buffer(ERR)
    for fn in ("h3_cuda_create", "h3_dit_int8_store_open", "h3_dit_w4a8_open_int8", "h3_dit_int8_store_header"):
        getattr(L, fn).restype = C.c_void_p
    cuda = L.h3_cuda_create(0, err, ERR)
    assert cuda, err.value
    store = L.h3_dit_int8_store_open(str(path).encode(), err, ERR)
    assert store, err.value
    cfg = CacheConfig()
    L.h3_dit_w4a8_config_init(C.byref(cfg))
    cfg.n_blocks = 1
    ctx = L.h3_dit_w4a8_open_int8(C.c_void_p(cuda), C.c_void_p(store), C.byref(cfg), err, ERR)
    assert ctx, err.value
    assert L.h3_dit_w4a8_convrot_groupsize(C.c_void_p(ctx)) == 256
    aux = BlockAux()
    assert L.h3_dit_w4a8_load_block_aux_hdr(C.c_void_p(L.h3_dit_int8_store_header(C.c_void_p(store))), 0, C.byref(aux), err,
                                            ERR) == 1, err.value
    assert aux.adaln_out == MODS * SLOTS * HIDDEN and aux.t_table_rows == 1025

    # inputs: the reference's own host functions build the positions, tables, time feature and modulation
    x = rng.normal(0, 1, (seq, HIDDEN)).astype(np.float32)
    row_map = (np.arange(seq) % MODS).astype(np.uint32)
    pt, ph, pw = (np.empty(seq, np.float32) for _ in range(3))
    assert L.h3_dit_w4a8_fill_metal_video_pos(C.c_size_t(16), 2, 12, 16, fptr(pt), fptr(ph), fptr(pw), err, ERR) == 1
    cos, sin = np.empty((seq, 48), np.float32), np.empty((seq, 48), np.float32)
    assert L.h3_dit_w4a8_rope_tables_f32(fptr(inv_freq), C.c_size_t(seq), fptr(pt), fptr(ph), fptr(pw), C.c_float(1.0),
                                         fptr(cos), fptr(sin), err, ERR) == 1
    L.h3_dit_w4a8_t_row_from_sigma.restype = C.c_size_t
    t_row = L.h3_dit_w4a8_t_row_from_sigma(C.c_float(0.5), C.c_size_t(1025))
    t_feat = np.empty(TFEAT, np.float32)
    assert L.h3_dit_w4a8_time_feat_from_table(C.byref(aux), C.c_size_t(t_row), fptr(t_feat), err, ERR) == 1
    mod = np.empty((MODS, SLOTS, HIDDEN), np.float32)
    assert L.h3_dit_w4a8_adaln_project_f32(C.byref(aux), fptr(t_feat), fptr(mod), err, ERR) == 1

    y = np.empty_like(x)
    ok = L.h3_dit_w4a8_block_forward_f32(C.c_void_p(ctx), 0, C.byref(aux), fptr(x), C.c_size_t(seq), fptr(mod), fptr(row_map),
                                         fptr(cos), fptr(sin), fptr(y), None, err, ERR)
    assert ok == 1, err.value
    L.h3_cuda_sdpa_last_backend_name.restype = C.c_char_p
    assert L.h3_cuda_sdpa_last_backend_name().startswith(b"tcgen05")      # this library's attention ran
    assert np.isfinite(y).all()

    weights = {"qkv": W["attn.qkv_proj"], "out": W["attn.out_proj"], "fc1": W["mlp.fc1"], "fc2": W["mlp.fc2"],
               "norm1": n1, "norm2": n2, "q_norm": qn, "k_norm": kn, "modulation": mod}
    want = oracle.block_r(weights, x, cos, sin, row_map, heads=HEADS, head_dim=HD, ffn=FFN, convrot_gs=256)
    err_l2 = rel_l2(y, want)
    print(f"reference host on libh3_b200, real-geometry block, seq {seq}: rel-L2 vs the f32 CPU block {err_l2:.2e}")
    assert err_l2 < 2e-2

    L.h3_dit_w4a8_block_aux_free(C.byref(aux))
    L.h3_dit_w4a8_free(C.c_void_p(ctx))
    L.h3_dit_int8_store_free(C.c_void_p(store))
    L.h3_cuda_free(C.c_void_p(cuda))

    # ---- the same file through this library's own reader and block host (h3b_ckpt_open +
    # h3b_dit_load_int8_convrot_block): same operators underneath, this library's orchestration
    import h3c_b200
    from h3c_b200 import dit as D
    from h3c_b200.lib import call
    cu = h3c_b200.Cuda(0)
    geo = D.DitGeometry(dim=HIDDEN, heads=HEADS, head_dim=HD, ffn=FFN, n_blocks=1, mod_rows=MODS, t_dim=TFEAT,
                        kind=D.BLOCK_REFERENCE, stream_dtype=D.F32, convrot_gs=256)
    dit = D.Dit(cu, geo)
    ck = h3c_b200.load().h3b_ckpt_open(str(path).encode(), err, ERR)
    assert ck, err.value
    call("h3b_dit_load_int8_convrot_block", dit.h, ck, 0, 0)
    h3c_b200.load().h3b_ckpt_close(ck)          # the weights are resident: the mapping may go
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    y2 = dit.block_forward(0, dev(x), dev(cos), dev(sin), modulation=dev(mod), row_map=dev(row_map.view(np.int32)))
    cu.check()
    y2 = y2.cpu().numpy()
    e_native, e_hosts = rel_l2(y2, want), rel_l2(y2, y)
    print(f"native reader + h3b_dit block: rel-L2 vs the f32 CPU block {e_native:.2e}, vs the reference host's run {e_hosts:.2e}")
    assert e_native < 2e-2 and e_hosts < 5e-3
    dit.close()
    cu.close()
