"""ctypes front-end of the two CPU checker libraries.  TEST INFRASTRUCTURE ONLY.

`Oracle` wraps oracle/_build/libh3_oracle.so (this repository's restatement) and `Ref`
wraps oracle/_ref/libh3_ref.so (the reference's own C functions, when that library was
built).  Only tests/, the smoke check and the benchmark's cpu_baseline / reference arm
may import this module; the product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent

c_f32p = C.POINTER(C.c_float)
c_i8p = C.POINTER(C.c_int8)
c_u8p = C.POINTER(C.c_uint8)
c_u16p = C.POINTER(C.c_uint16)
c_u32p = C.POINTER(C.c_uint32)
c_i32p = C.POINTER(C.c_int32)
sz = C.c_size_t


def _p(a, typ):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "array must be C contiguous"
    return a.ctypes.data_as(typ)


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class HoLinear(C.Structure):
    _fields_ = [("w_f32", c_f32p), ("w_i8", c_i8p), ("s_channel", c_f32p), ("n", sz), ("k", sz)]


class HoBlockCfg(C.Structure):
    _fields_ = [("dim", sz), ("heads", sz), ("head_dim", sz), ("ffn", sz), ("rope_half", sz),
                ("eps", C.c_float), ("quantised", C.c_int), ("bf16_stream", C.c_int),
                ("convrot_gs", C.c_int)]


class HoBlockB(C.Structure):
    _fields_ = [(n, HoLinear) for n in ("qkv", "o", "cq", "ckv", "co", "up", "down")] + \
               [(n, c_f32p) for n in ("norm1", "norm_c", "norm2", "q_norm", "k_norm", "modulation")]


class HoBlockR(C.Structure):
    _fields_ = [(n, HoLinear) for n in ("qkv", "out", "fc1", "fc2")] + \
               [(n, c_f32p) for n in ("norm1", "norm2", "q_norm", "k_norm", "modulation")] + \
               [("row_map", c_u32p)]


class Oracle:
    """Thin numpy wrappers; every method returns fresh arrays."""

    def __init__(self, threads: int | None = None):
        path = HERE / "_build" / "libh3_oracle.so"
        if not path.exists():
            import importlib.util
            spec = importlib.util.spec_from_file_location("_h3_oracle_build", HERE / "build.py")
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.build_oracle()
        self.lib = L = C.CDLL(str(path))
        L.ho_f8e4m3fn_to_f32.restype = C.c_float
        L.ho_f8e4m3fn_to_f32.argtypes = [C.c_uint8]
        L.ho_ue4m3_to_f32.restype = C.c_float
        L.ho_ue4m3_to_f32.argtypes = [C.c_uint8]
        L.ho_f32_to_ue4m3.restype = C.c_uint8
        L.ho_f32_to_ue4m3.argtypes = [C.c_float]
        L.ho_e2m1_nibble.restype = C.c_uint8
        L.ho_e2m1_nibble.argtypes = [C.c_float]
        L.ho_bf16_round.restype = C.c_float
        L.ho_bf16_round.argtypes = [C.c_float]
        L.ho_gelu_tanh.restype = C.c_float
        L.ho_gelu_tanh.argtypes = [C.c_float]
        L.ho_nvfp4_sf_bytes.restype = sz
        L.ho_nvfp4_sf_bytes.argtypes = [sz, sz]
        L.ho_nvfp4_sf_offset.restype = sz
        L.ho_nvfp4_sf_offset.argtypes = [sz, sz, sz]
        L.ho_ulysses_pad_seq.restype = sz
        L.ho_ulysses_pad_seq.argtypes = [sz, C.c_int]
        L.ho_ulysses_local_rows.restype = sz
        L.ho_ulysses_local_rows.argtypes = [sz, C.c_int, C.c_int]
        L.ho_fnv1a64.restype = C.c_uint64
        L.ho_fnv1a64.argtypes = [C.c_void_p, sz]
        L.ho_checksum_f32.restype = C.c_uint64
        L.ho_checksum_f32.argtypes = [c_f32p, sz]
        self.set_threads(threads if threads else 1)

    def set_threads(self, n: int):
        self.lib.ho_set_threads(C.c_int(int(n)))

    # ---- formats
    def bf16_round(self, x):
        x = f32(x)
        u = x.view(np.uint32).astype(np.uint64)
        r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32) << 16
        out = r.astype(np.uint32).view(np.float32).reshape(x.shape)
        return np.where(np.isnan(x), x, out)

    # ---- weights
    def w4a8_dequant_to_int8(self, packed, codebook, s_rel, group_size=16):
        n, kh = packed.shape
        out = np.empty((n, kh * 2), np.int8)
        ok = self.lib.ho_w4a8_dequant_to_int8(_p(packed, c_i8p), sz(n), sz(kh), _p(f32(codebook), c_f32p),
                                              _p(s_rel, c_u8p), C.c_int(group_size), _p(out, c_i8p))
        assert ok == 1
        return out

    def w4g128_encode(self, w, group=128):
        w = f32(w)
        n, k = w.shape
        packed = np.zeros((n, k // 2), np.uint8)
        scales = np.zeros((n, k // group), np.uint16)
        assert self.lib.ho_w4g128_encode(_p(w, c_f32p), sz(n), sz(k), C.c_int(group), _p(packed, c_u8p),
                                         _p(scales, c_u16p)) == 1
        return packed, scales

    def w4g128_decode_to_int8(self, packed, scales, group=128):
        n, kh = packed.shape
        k = kh * 2
        w = np.empty((n, k), np.int8)
        s = np.empty(n, np.float32)
        assert self.lib.ho_w4g128_decode_to_int8(_p(packed, c_u8p), _p(scales, c_u16p), sz(n), sz(k),
                                                 C.c_int(group), _p(w, c_i8p), _p(s, c_f32p)) == 1
        return w, s

    # ---- convrot
    def hadamard(self, size):
        h = np.empty((size, size), np.float32)
        assert self.lib.ho_hadamard_normalized(C.c_int(size), _p(h, c_f32p)) == 1
        return h

    def convrot(self, x, gs):
        x = f32(x)
        y = np.empty_like(x)
        assert self.lib.ho_convrot_act_f32(_p(x, c_f32p), sz(x.shape[0]), sz(x.shape[1]), C.c_int(gs),
                                           _p(y, c_f32p)) == 1
        return y

    def fwht(self, x, gs):
        """Sylvester (Walsh-Hadamard) rotation per group, the H3_CONVROT_SYLVESTER=1 form."""
        x = f32(x)
        y = np.empty_like(x)
        assert self.lib.ho_fwht_act_f32(_p(x, c_f32p), sz(x.shape[0]), sz(x.shape[1]), C.c_int(gs), _p(y, c_f32p)) == 1
        return y

    # ---- act quant + GEMM
    def quantize_act_int8(self, x):
        x = f32(x)
        m, k = x.shape
        q = np.empty((m, k), np.int8)
        s = np.empty(m, np.float32)
        assert self.lib.ho_quantize_act_int8(_p(x, c_f32p), sz(m), sz(k), _p(q, c_i8p), _p(s, c_f32p)) == 1
        return q, s

    def gemm_i8_i32(self, x, w):
        m, k = x.shape
        n = w.shape[0]
        acc = np.empty((m, n), np.int32)
        self.lib.ho_gemm_i8_i32(_p(x, c_i8p), _p(w, c_i8p), sz(m), sz(n), sz(k), _p(acc, c_i32p))
        return acc

    def gemm_i8_dequant(self, x, w, a, s):
        m, k = x.shape
        n = w.shape[0]
        y = np.empty((m, n), np.float32)
        self.lib.ho_gemm_i8_dequant_f32(_p(x, c_i8p), _p(w, c_i8p), _p(f32(a), c_f32p), _p(f32(s), c_f32p),
                                        sz(m), sz(n), sz(k), _p(y, c_f32p))
        return y

    def gemm_f32(self, x, w):
        x, w = f32(x), f32(w)
        y = np.empty((x.shape[0], w.shape[0]), np.float32)
        self.lib.ho_gemm_f32(_p(x, c_f32p), _p(w, c_f32p), sz(x.shape[0]), sz(w.shape[0]), sz(x.shape[1]),
                             _p(y, c_f32p))
        return y

    # ---- epilogues
    def dequant_swiglu(self, acc, a, s, lora=None):
        rows, n = acc.shape
        out = np.empty((rows, n // 2), np.float32)
        self.lib.ho_dequant_swiglu_f32(_p(acc, c_i32p), _p(f32(a), c_f32p), _p(f32(s), c_f32p), sz(rows),
                                       sz(n // 2), _p(None if lora is None else f32(lora), c_f32p),
                                       _p(out, c_f32p))
        return out

    def dequant_gate(self, acc, a, s, residual, modulation, row_map, slots, gate_slot, lora=None):
        rows, n = acc.shape
        out = np.empty((rows, n), np.float32)
        self.lib.ho_dequant_gate_f32(_p(acc, c_i32p), _p(f32(a), c_f32p), _p(f32(s), c_f32p),
                                     _p(f32(residual), c_f32p), _p(f32(modulation), c_f32p),
                                     _p(row_map, c_u32p), sz(rows), sz(n), sz(slots), sz(gate_slot),
                                     _p(None if lora is None else f32(lora), c_f32p), _p(out, c_f32p))
        return out

    def dequant_gelu(self, acc, a, s):
        rows, n = acc.shape
        out = np.empty((rows, n), np.float32)
        self.lib.ho_dequant_gelu_f32(_p(acc, c_i32p), _p(f32(a), c_f32p), _p(f32(s), c_f32p), sz(rows),
                                     sz(n), _p(out, c_f32p))
        return out

    def gelu_tanh(self, x):
        x = f32(x)
        return np.array([self.lib.ho_gelu_tanh(C.c_float(v)) for v in x.ravel()], np.float32).reshape(x.shape)

    # ---- row ops
    def rms_norm(self, x, w, eps=1e-5):
        x = f32(x)
        out = np.empty_like(x)
        self.lib.ho_rms_norm_f32(_p(x, c_f32p), _p(f32(w), c_f32p), sz(x.shape[0]), sz(x.shape[1]),
                                 C.c_float(eps), _p(out, c_f32p))
        return out

    def adaln(self, x, norm_w, modulation, row_map, slots, shift_slot, scale_slot, eps=1e-5):
        x = f32(x)
        out = np.empty_like(x)
        self.lib.ho_adaln_f32(_p(x, c_f32p), _p(f32(norm_w), c_f32p), _p(f32(modulation), c_f32p),
                              _p(row_map, c_u32p), sz(x.shape[0]), sz(x.shape[1]), sz(slots),
                              sz(shift_slot), sz(scale_slot), C.c_float(eps), _p(out, c_f32p))
        return out

    def gate(self, residual, branch, modulation, row_map, slots, gate_slot):
        residual = f32(residual)
        out = np.empty_like(residual)
        self.lib.ho_gate_f32(_p(residual, c_f32p), _p(f32(branch), c_f32p), _p(f32(modulation), c_f32p),
                             _p(row_map, c_u32p), sz(residual.shape[0]), sz(residual.shape[1]), sz(slots),
                             sz(gate_slot), _p(out, c_f32p))
        return out

    def gate_adaln(self, residual, branch, norm_w, modulation, row_map, slots, gate_slot, shift_slot,
                   scale_slot, eps=1e-5):
        residual = f32(residual)
        gated = np.empty_like(residual)
        normed = np.empty_like(residual)
        self.lib.ho_gate_adaln_f32(_p(residual, c_f32p), _p(f32(branch), c_f32p), _p(f32(norm_w), c_f32p),
                                   _p(f32(modulation), c_f32p), _p(row_map, c_u32p), sz(residual.shape[0]),
                                   sz(residual.shape[1]), sz(slots), sz(gate_slot), sz(shift_slot),
                                   sz(scale_slot), C.c_float(eps), _p(gated, c_f32p), _p(normed, c_f32p))
        return gated, normed

    def swiglu(self, fused):
        fused = f32(fused)
        out = np.empty((fused.shape[0], fused.shape[1] // 2), np.float32)
        self.lib.ho_swiglu_f32(_p(fused, c_f32p), sz(fused.shape[0]), sz(fused.shape[1] // 2), _p(out, c_f32p))
        return out

    # ---- rope / attention
    def qkv_rope(self, qkv, q_norm, k_norm, cos, sin, heads, head_dim, rope_half, eps=1e-5, grouped=0,
                 split_half=1):
        qkv = f32(qkv)
        seq = qkv.shape[0]
        q = np.empty((seq, heads, head_dim), np.float32)
        k = np.empty_like(q)
        v = np.empty_like(q)
        ok = self.lib.ho_qkv_rope_f32(_p(qkv, c_f32p), _p(f32(q_norm), c_f32p), _p(f32(k_norm), c_f32p),
                                      _p(None if cos is None else f32(cos), c_f32p),
                                      _p(None if sin is None else f32(sin), c_f32p), sz(seq), sz(heads),
                                      sz(head_dim), sz(rope_half), C.c_float(eps), C.c_int(grouped),
                                      C.c_int(split_half), _p(q, c_f32p), _p(k, c_f32p), _p(v, c_f32p))
        assert ok == 1
        return q, k, v

    def sdpa(self, q, k, v, scale=None):
        """q [lq,H,d], k/v [lk,H,d] (contiguous) -> [lq, H*d]."""
        q, k, v = f32(q), f32(k), f32(v)
        lq, H, d = q.shape
        lk = k.shape[0]
        scale = (1.0 / np.sqrt(d)) if scale is None else scale
        out = np.empty((lq, H * d), np.float32)
        ok = self.lib.ho_sdpa_rect_f32(_p(q, c_f32p), sz(H * d), _p(k, c_f32p), sz(H * d), _p(v, c_f32p),
                                       sz(H * d), sz(lq), sz(lk), sz(H), sz(d), C.c_float(scale),
                                       _p(out, c_f32p))
        assert ok == 1
        return out

    def rope_tables(self, inv_freq, pos_t, pos_h, pos_w, spatial_scale=1.0):
        inv_freq = f32(inv_freq)
        seq = len(pos_t)
        nf = len(inv_freq)
        cos = np.empty((seq, 3 * nf), np.float32)
        sin = np.empty_like(cos)
        ok = self.lib.ho_rope_tables_f32(_p(inv_freq, c_f32p), sz(nf), sz(seq), _p(f32(pos_t), c_f32p),
                                         _p(f32(pos_h), c_f32p), _p(f32(pos_w), c_f32p),
                                         C.c_float(spatial_scale), _p(cos, c_f32p), _p(sin, c_f32p))
        assert ok == 1
        return cos, sin

    def fill_video_pos(self, text_len, latent_t, latent_h, latent_w):
        n = latent_t * (latent_h // 2) * (latent_w // 2)
        pt, ph, pw = (np.empty(n, np.float32) for _ in range(3))
        ok = self.lib.ho_fill_video_pos(sz(text_len), C.c_int(latent_t), C.c_int(latent_h), C.c_int(latent_w),
                                        _p(pt, c_f32p), _p(ph, c_f32p), _p(pw, c_f32p))
        assert ok == 1
        return pt, ph, pw

    def adaln_project(self, w, b, t_feat):
        w = f32(w)
        mod = np.empty(w.shape[0], np.float32)
        self.lib.ho_adaln_project_f32(_p(w, c_f32p), _p(f32(b), c_f32p), sz(w.shape[0]), sz(w.shape[1]),
                                      _p(f32(t_feat), c_f32p), _p(mod, c_f32p))
        return mod

    def dense(self, x, w, bias=None):
        """y = x W^T + b in f32 (patch embeddings, final heads)."""
        x, w = f32(x), f32(w)
        y = np.empty((x.shape[0], w.shape[0]), np.float32)
        b = f32(bias) if bias is not None else None
        self.lib.ho_dense_f32(_p(x, c_f32p), _p(w, c_f32p), _p(b, c_f32p) if b is not None else None, sz(x.shape[0]),
                              sz(w.shape[0]), sz(x.shape[1]), _p(y, c_f32p))
        return y

    def euler_step(self, sample, velocity, sigma, sigma_next):
        """Returns the updated sample, or None where the reference rejects the sigma pair."""
        out = f32(sample).copy()
        self.lib.ho_euler_step_f32.restype = C.c_int
        ok = self.lib.ho_euler_step_f32(_p(out, c_f32p), _p(f32(velocity), c_f32p), sz(out.size), C.c_float(sigma),
                                        C.c_float(sigma_next))
        return out if ok == 1 else None

    def final_head(self, x, norm_w, modulation, w, bias, eps=1e-5):
        """adaLN with shift = modulation[0], scale = modulation[1] for every token, then the dense head."""
        x = f32(x)
        zeros = np.zeros(x.shape[0], np.uint32)
        return self.dense(self.adaln(x, norm_w, f32(modulation).reshape(1, 2, -1), zeros, 2, 0, 1, eps), w, bias)

    # ---- nvfp4
    def nvfp4_sf_bytes(self, rows, k):
        return int(self.lib.ho_nvfp4_sf_bytes(sz(rows), sz(k)))

    def quantize_nvfp4(self, x, rule=0):
        """rule 0: the reference's CUDA activation rule; rule 1: its Python weight-quantiser rule."""
        x = f32(x)
        m, k = x.shape
        packed = np.zeros((m, k // 2), np.uint8)
        sf = np.zeros(self.nvfp4_sf_bytes(m, k), np.uint8)
        assert self.lib.ho_quantize_nvfp4_rule(_p(x, c_f32p), sz(m), sz(k), C.c_int(rule), _p(packed, c_u8p),
                                               _p(sf, c_u8p)) == 1
        return packed, sf

    def dequant_nvfp4(self, packed, sf):
        m, kh = packed.shape
        x = np.empty((m, kh * 2), np.float32)
        assert self.lib.ho_dequant_nvfp4(_p(packed, c_u8p), _p(sf, c_u8p), sz(m), sz(kh * 2), _p(x, c_f32p)) == 1
        return x

    def gemm_nvfp4(self, x_fp4, x_sf, w_fp4, w_sf, scale2):
        m, kh = x_fp4.shape
        n = w_fp4.shape[0]
        y = np.empty((m, n), np.float32)
        assert self.lib.ho_gemm_nvfp4_f32(_p(x_fp4, c_u8p), _p(x_sf, c_u8p), _p(w_fp4, c_u8p), _p(w_sf, c_u8p),
                                          C.c_float(scale2), sz(m), sz(n), sz(kh * 2), _p(y, c_f32p)) == 1
        return y

    # ---- ulysses
    def ulysses_a2a_qkv(self, ins, heads, head_dim):
        """ins: list of U arrays [seq_local, 3, heads, head_dim] -> list of [U*seq_local, 3, heads/U, head_dim]."""
        u = len(ins)
        ins = [np.ascontiguousarray(a) for a in ins]
        sl = ins[0].shape[0]
        outs = [np.empty((u * sl, 3, heads // u, head_dim), ins[0].dtype) for _ in range(u)]
        ip = (C.c_void_p * u)(*[a.ctypes.data for a in ins])
        op = (C.c_void_p * u)(*[a.ctypes.data for a in outs])
        self.lib.ho_ulysses_a2a_qkv_sim(ip, op, sz(sl), sz(heads), sz(head_dim), C.c_int(u),
                                        sz(ins[0].dtype.itemsize))
        return outs

    def ulysses_a2a_attn(self, ins, heads, head_dim):
        """ins: list of U arrays [U*seq_local, heads/U, head_dim] -> list of [seq_local, heads, head_dim]."""
        u = len(ins)
        ins = [np.ascontiguousarray(a) for a in ins]
        sl = ins[0].shape[0] // u
        outs = [np.empty((sl, heads, head_dim), ins[0].dtype) for _ in range(u)]
        ip = (C.c_void_p * u)(*[a.ctypes.data for a in ins])
        op = (C.c_void_p * u)(*[a.ctypes.data for a in outs])
        self.lib.ho_ulysses_a2a_attn_sim(ip, op, sz(sl), sz(heads), sz(head_dim), C.c_int(u),
                                         sz(ins[0].dtype.itemsize))
        return outs

    # ---- blocks
    @staticmethod
    def _linear(keep, w_f32=None, w_i8=None, s=None):
        l = HoLinear()
        if w_f32 is not None:
            w_f32 = f32(w_f32)
            keep.append(w_f32)
            l.w_f32 = _p(w_f32, c_f32p)
            l.n, l.k = w_f32.shape
        if w_i8 is not None:
            w_i8 = np.ascontiguousarray(w_i8, np.int8)
            s = f32(s)
            keep += [w_i8, s]
            l.w_i8 = _p(w_i8, c_i8p)
            l.s_channel = _p(s, c_f32p)
            l.n, l.k = w_i8.shape
        return l

    def block_b(self, weights: dict, x, text, cos, sin, *, heads, head_dim, ffn, rope_half=48, eps=1e-5,
                quantised=False, bf16_stream=False):
        """weights: name -> f32 [n,k] (quantised=False) or (int8 [n,k], s[n]) (quantised=True) for
        qkv,o,cq,ckv,co,up,down; plus norm1,norm_c,norm2,q_norm,k_norm,modulation([6,dim])."""
        keep = []
        x, text = f32(x), f32(text)
        m, dim = x.shape
        cfg = HoBlockCfg(dim, heads, head_dim, ffn, rope_half, eps, int(quantised), int(bf16_stream), 0)
        blk = HoBlockB()
        for name in ("qkv", "o", "cq", "ckv", "co", "up", "down"):
            w = weights[name]
            setattr(blk, name, self._linear(keep, w_i8=w[0], s=w[1]) if quantised else self._linear(keep, w_f32=w))
        for name in ("norm1", "norm_c", "norm2", "q_norm", "k_norm", "modulation"):
            a = f32(weights[name])
            keep.append(a)
            setattr(blk, name, _p(a, c_f32p))
        y = np.empty_like(x)
        cos, sin = f32(cos), f32(sin)
        ok = self.lib.ho_block_b_forward(C.byref(cfg), C.byref(blk), _p(x, c_f32p), sz(m), _p(text, c_f32p),
                                         sz(text.shape[0]), _p(cos, c_f32p), _p(sin, c_f32p), _p(y, c_f32p))
        assert ok == 1
        return y

    def block_r(self, weights: dict, x, cos, sin, row_map, *, heads, head_dim, ffn, rope_half=48, eps=1e-5,
                quantised=True, convrot_gs=0):
        keep = []
        x = f32(x)
        m, dim = x.shape
        cfg = HoBlockCfg(dim, heads, head_dim, ffn, rope_half, eps, int(quantised), 0, convrot_gs)
        blk = HoBlockR()
        for name in ("qkv", "out", "fc1", "fc2"):
            w = weights[name]
            setattr(blk, name, self._linear(keep, w_i8=w[0], s=w[1]) if quantised else self._linear(keep, w_f32=w))
        for name in ("norm1", "norm2", "q_norm", "k_norm", "modulation"):
            a = f32(weights[name])
            keep.append(a)
            setattr(blk, name, _p(a, c_f32p))
        row_map = None if row_map is None else np.ascontiguousarray(row_map, np.uint32)
        blk.row_map = _p(row_map, c_u32p)
        y = np.empty_like(x)
        cos, sin = f32(cos), f32(sin)
        ok = self.lib.ho_block_r_forward(C.byref(cfg), C.byref(blk), _p(x, c_f32p), sz(m), _p(cos, c_f32p),
                                         _p(sin, c_f32p), _p(y, c_f32p))
        assert ok == 1
        return y

    def checksum_f32(self, x):
        x = f32(x)
        return int(self.lib.ho_checksum_f32(_p(x, c_f32p), sz(x.size)))


ERR = 256


class Ref:
    """The reference's own CPU functions (libh3_ref.so), same numpy calling style."""

    @staticmethod
    def available() -> bool:
        return (HERE / "_ref" / "libh3_ref.so").exists()

    def __init__(self):
        self.lib = L = C.CDLL(str(HERE / "_ref" / "libh3_ref.so"))
        L.h3_f8e4m3fn_to_f32.restype = C.c_float
        L.h3_f8e4m3fn_to_f32.argtypes = [C.c_uint8]
        L.h3_ulysses_pad_seq.restype = sz
        L.h3_ulysses_pad_seq.argtypes = [sz, C.c_int]
        L.h3_ulysses_local_rows.restype = sz
        L.h3_ulysses_local_rows.argtypes = [sz, C.c_int, C.c_int]
        L.h3_w4a8_hadamard_normalized.restype = C.c_void_p
        L.h3_dit_w4a8_checksum_f32.restype = C.c_uint64
        L.ref_act_f16_pre_scale.restype = C.c_float
        L.ref_act_f16_pre_scale.argtypes = [C.c_float, C.c_int]
        L.ref_int8_gemm_tile_rows.restype = sz
        L.ref_int8_gemm_tile_rows.argtypes = [sz, sz]
        self._err = C.create_string_buffer(ERR)

    def w4a8_dequant_to_int8(self, packed, codebook, s_rel, group_size=16):
        n, kh = packed.shape
        out = np.empty((n, kh * 2), np.int8)
        ok = self.lib.h3_w4a8_dequant_to_int8(_p(packed, c_i8p), sz(n), sz(kh), _p(f32(codebook), c_f32p),
                                              _p(s_rel, c_u8p), C.c_int(group_size), _p(out, c_i8p),
                                              self._err, sz(ERR))
        assert ok == 1, self._err.value
        return out

    def hadamard(self, size):
        ptr = self.lib.h3_w4a8_hadamard_normalized(C.c_int(size), self._err, sz(ERR))
        assert ptr
        arr = np.ctypeslib.as_array(C.cast(ptr, c_f32p), shape=(size, size)).copy()
        C.CDLL(None).free(C.c_void_p(ptr))
        return arr

    def convrot(self, x, gs):
        x = f32(x)
        y = np.empty_like(x)
        ok = self.lib.h3_w4a8_convrot_act_f32(_p(x, c_f32p), sz(x.shape[0]), sz(x.shape[1]), C.c_int(gs),
                                              _p(y, c_f32p), self._err, sz(ERR))
        assert ok == 1, self._err.value
        return y

    def fwht(self, x, gs):
        x = f32(x)
        y = np.empty_like(x)
        ok = self.lib.h3_w4a8_fwht_act_f32(_p(x, c_f32p), sz(x.shape[0]), sz(x.shape[1]), C.c_int(gs), _p(y, c_f32p),
                                           self._err, sz(ERR))
        assert ok == 1, self._err.value
        return y

    def quantize_act_int8(self, x):
        x = f32(x)
        m, k = x.shape
        q = np.empty((m, k), np.int8)
        s = np.empty(m, np.float32)
        ok = self.lib.h3_w4a8_quantize_act_int8(_p(x, c_f32p), sz(m), sz(k), C.c_int(1), _p(q, c_i8p),
                                                _p(s, c_f32p), self._err, sz(ERR))
        assert ok == 1, self._err.value
        return q, s

    def gemm_i8_dequant(self, x, w, a, s):
        m, k = x.shape
        n = w.shape[0]
        y = np.empty((m, n), np.float32)
        self.lib.h3_w4a8_gemm_i8_dequant_f32(_p(x, c_i8p), _p(w, c_i8p), _p(f32(a), c_f32p), C.c_int(0),
                                             _p(f32(s), c_f32p), sz(m), sz(n), sz(k), _p(y, c_f32p))
        return y

    def gemm_f32(self, x, w):
        x, w = f32(x), f32(w)
        y = np.empty((x.shape[0], w.shape[0]), np.float32)
        self.lib.h3_w4a8_gemm_f32(_p(x, c_f32p), _p(w, c_f32p), sz(x.shape[0]), sz(w.shape[0]), sz(x.shape[1]),
                                  _p(y, c_f32p))
        return y

    def dequant_swiglu(self, acc, a, s, lora=None):
        rows, n = acc.shape
        out = np.empty((rows, n // 2), np.float32)
        self.lib.ref_dequant_swiglu_f32(_p(acc, c_i32p), _p(f32(a), c_f32p), C.c_int(0), _p(f32(s), c_f32p),
                                        sz(rows), sz(n // 2), _p(None if lora is None else f32(lora), c_f32p),
                                        _p(out, c_f32p))
        return out

    def dequant_gate(self, acc, a, s, residual, modulation, row_map, slots, gate_slot, lora=None):
        rows, n = acc.shape
        out = np.empty((rows, n), np.float32)
        self.lib.ref_dequant_gate_f32(_p(acc, c_i32p), _p(f32(a), c_f32p), C.c_int(0), _p(f32(s), c_f32p),
                                      _p(f32(residual), c_f32p), _p(f32(modulation), c_f32p),
                                      _p(row_map, c_u32p), sz(rows), sz(n), sz(slots), sz(gate_slot),
                                      _p(None if lora is None else f32(lora), c_f32p), _p(out, c_f32p))
        return out

    def rms_norm(self, x, w, eps=1e-5):
        x = f32(x)
        out = np.empty_like(x)
        self.lib.h3_dit_w4a8_rms_norm_f32(_p(x, c_f32p), _p(f32(w), c_f32p), sz(x.shape[0]), sz(x.shape[1]),
                                          C.c_float(eps), _p(out, c_f32p))
        return out

    def adaln(self, x, norm_w, modulation, row_map, slots, shift_slot, scale_slot, eps=1e-5):
        x = f32(x)
        out = np.empty_like(x)
        self.lib.h3_dit_w4a8_adaln_f32(_p(x, c_f32p), _p(f32(norm_w), c_f32p), _p(f32(modulation), c_f32p),
                                       _p(row_map, c_u32p), sz(x.shape[0]), sz(x.shape[1]), sz(slots),
                                       sz(shift_slot), sz(scale_slot), C.c_float(eps), _p(out, c_f32p))
        return out

    def dense(self, x, w, bias=None):
        x, w = f32(x), f32(w)
        y = np.empty((x.shape[0], w.shape[0]), np.float32)
        b = f32(bias) if bias is not None else None
        err = C.create_string_buffer(256)
        self.lib.h3_dit_w4a8_dense_f32.restype = C.c_int
        ok = self.lib.h3_dit_w4a8_dense_f32(_p(x, c_f32p), _p(w, c_f32p), _p(b, c_f32p) if b is not None else None,
                                            sz(x.shape[0]), sz(w.shape[0]), sz(x.shape[1]), _p(y, c_f32p), err, sz(256))
        assert ok == 1, err.value
        return y

    def euler_step(self, sample, velocity, sigma, sigma_next):
        out = f32(sample).copy()
        err = C.create_string_buffer(256)
        self.lib.h3_dit_w4a8_euler_step_f32.restype = C.c_int
        ok = self.lib.h3_dit_w4a8_euler_step_f32(_p(out, c_f32p), _p(f32(velocity), c_f32p), sz(out.size),
                                                 C.c_float(sigma), C.c_float(sigma_next), err, sz(256))
        return out if ok == 1 else None

    def gate(self, residual, branch, modulation, row_map, slots, gate_slot):
        residual = f32(residual)
        out = np.empty_like(residual)
        self.lib.h3_dit_w4a8_gate_f32(_p(residual, c_f32p), _p(f32(branch), c_f32p),
                                      _p(f32(modulation), c_f32p), _p(row_map, c_u32p),
                                      sz(residual.shape[0]), sz(residual.shape[1]), sz(slots), sz(gate_slot),
                                      _p(out, c_f32p))
        return out

    def gate_adaln(self, residual, branch, norm_w, modulation, row_map, slots, gate_slot, shift_slot,
                   scale_slot, eps=1e-5):
        residual = f32(residual)
        gated = np.empty_like(residual)
        normed = np.empty_like(residual)
        self.lib.ref_gate_adaln_f32(_p(residual, c_f32p), _p(f32(branch), c_f32p), _p(f32(norm_w), c_f32p),
                                    _p(f32(modulation), c_f32p), _p(row_map, c_u32p), sz(residual.shape[0]),
                                    sz(residual.shape[1]), sz(slots), sz(gate_slot), sz(shift_slot),
                                    sz(scale_slot), C.c_float(eps), _p(gated, c_f32p), _p(normed, c_f32p))
        return gated, normed

    def swiglu(self, fused):
        fused = f32(fused)
        out = np.empty((fused.shape[0], fused.shape[1] // 2), np.float32)
        self.lib.h3_dit_w4a8_swiglu_f32(_p(fused, c_f32p), sz(fused.shape[0]), sz(fused.shape[1] // 2),
                                        _p(out, c_f32p))
        return out

    def qkv_rope(self, qkv, q_norm, k_norm, cos, sin, heads, head_dim, rope_half, eps=1e-5):
        qkv = f32(qkv)
        seq = qkv.shape[0]
        q = np.empty((seq, heads, head_dim), np.float32)
        k = np.empty_like(q)
        v = np.empty_like(q)
        ok = self.lib.h3_dit_w4a8_qkv_rope_f32(_p(qkv, c_f32p), _p(f32(q_norm), c_f32p), _p(f32(k_norm), c_f32p),
                                               _p(None if cos is None else f32(cos), c_f32p),
                                               _p(None if sin is None else f32(sin), c_f32p), sz(seq),
                                               sz(heads), sz(head_dim), sz(rope_half), C.c_float(eps),
                                               _p(q, c_f32p), _p(k, c_f32p), _p(v, c_f32p), self._err, sz(ERR))
        assert ok == 1, self._err.value
        return q, k, v

    def sdpa(self, q, k, v, scale=None):
        q, k, v = f32(q), f32(k), f32(v)
        seq, H, d = q.shape
        scale = (1.0 / np.sqrt(d)) if scale is None else scale
        out = np.empty((seq, H * d), np.float32)
        ok = self.lib.h3_dit_w4a8_sdpa_f32(_p(q, c_f32p), _p(k, c_f32p), _p(v, c_f32p), sz(seq), sz(H), sz(d),
                                           C.c_float(scale), _p(out, c_f32p), self._err, sz(ERR))
        assert ok == 1, self._err.value
        return out

    def rope_tables(self, inv_freq, pos_t, pos_h, pos_w, spatial_scale=1.0):
        inv_freq = f32(inv_freq)
        assert len(inv_freq) == 16
        seq = len(pos_t)
        cos = np.empty((seq, 48), np.float32)
        sin = np.empty_like(cos)
        os.environ["H3_ROPE_MEMO"] = "0"
        ok = self.lib.h3_dit_w4a8_rope_tables_f32(_p(inv_freq, c_f32p), sz(seq), _p(f32(pos_t), c_f32p),
                                                  _p(f32(pos_h), c_f32p), _p(f32(pos_w), c_f32p),
                                                  C.c_float(spatial_scale), _p(cos, c_f32p), _p(sin, c_f32p),
                                                  self._err, sz(ERR))
        assert ok == 1, self._err.value
        return cos, sin

    def fill_video_pos(self, text_len, latent_t, latent_h, latent_w):
        n = latent_t * (latent_h // 2) * (latent_w // 2)
        pt, ph, pw = (np.empty(n, np.float32) for _ in range(3))
        ok = self.lib.h3_dit_w4a8_fill_metal_video_pos(sz(text_len), C.c_int(latent_t), C.c_int(latent_h),
                                                       C.c_int(latent_w), _p(pt, c_f32p), _p(ph, c_f32p),
                                                       _p(pw, c_f32p), self._err, sz(ERR))
        assert ok == 1, self._err.value
        return pt, ph, pw

    def ulysses_validate(self, heads, align, tp, u, ring):
        return int(self.lib.h3_ulysses_validate(C.c_int(heads), C.c_int(align), C.c_int(tp), C.c_int(u),
                                                C.c_int(ring), self._err, sz(ERR)))

    def checksum_f32(self, x):
        x = f32(x)
        return int(self.lib.h3_dit_w4a8_checksum_f32(_p(x, c_f32p), sz(x.size)))
