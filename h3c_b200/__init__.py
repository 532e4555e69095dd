"""h3c_b200: host-side mirror of the reference's operator interface for the DiT denoiser block
path, bound to libh3_b200.so (hand-written sm_100a kernels behind a C ABI).

`Cuda` mirrors the reference's `h3_cuda` handle and its `h3_cuda_*` operators (same names minus
the prefix, same argument meaning, errors raised as `H3Error` carrying the library's message);
`Weight` mirrors `h3_cuda_w4a8_weight`.  torch tensors are used only as device buffers.
"""
from __future__ import annotations

import ctypes as C

from . import lib as _l
from .lib import BF16, EPI_GATE, EPI_GELU, EPI_PLAIN, EPI_SWIGLU, F16, F32, I32, H3Error, call, load, ptr

__all__ = ["Cuda", "Weight", "H3Error", "F32", "BF16", "F16", "I32", "EPI_PLAIN", "EPI_GATE", "EPI_SWIGLU",
           "EPI_GELU", "load"]


def _dt(t):
    import torch
    return {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16, torch.int32: I32}[t.dtype]


class Weight:
    """Resident INT8 [N,K] weight + per-channel scale (h3_cuda_w4a8_weight)."""

    def __init__(self, cuda: "Cuda", handle: int):
        self.cuda, self.h = cuda, handle

    @property
    def n(self):
        return int(load().h3_cuda_w4a8_weight_n(self.h))

    @property
    def k(self):
        return int(load().h3_cuda_w4a8_weight_k(self.h))

    def download_int8(self):
        import numpy as np
        out = np.empty((self.n, self.k), np.int8)
        call("h3_cuda_w4a8_weight_download_int8", self.h, out.ctypes.data)
        return out

    def download_scales(self):
        import numpy as np
        out = np.empty(self.n, np.float32)
        call("h3b_w4a8_weight_download_scales", self.h, out.ctypes.data)
        return out

    def free(self):
        if self.h:
            load().h3_cuda_w4a8_weight_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Cuda:
    """One handle per device (h3_cuda).  Work is enqueued on torch's current stream."""

    def __init__(self, device_index: int = 0):
        import torch
        load()
        err = C.create_string_buffer(_l.ERR_LEN)
        self.h = load().h3_cuda_create(device_index, err, _l.ERR_LEN)
        if not self.h:
            raise H3Error(f"h3_cuda_create: {err.value.decode(errors='replace')}")
        self.device = torch.device("cuda", device_index)
        self.use_stream(torch.cuda.current_stream(self.device))

    def use_stream(self, stream):
        call("h3_cuda_set_op_stream", self.h, stream.cuda_stream)

    def close(self):
        if self.h:
            load().h3_cuda_free(self.h)
            self.h = None

    def check(self):
        """Synchronises and raises if any kernel gave up a bounded wait."""
        st = C.c_int(0)
        call("h3b_cuda_check", self.h, C.byref(st))

    def launch_count(self, reset=False) -> int:
        return int(load().h3b_cuda_launch_count(self.h, int(reset)))

    def set_quiet(self, on: bool):
        load().h3_cuda_set_quiet(self.h, int(on))

    # ---- weights
    def weight_from_w4a8(self, packed, codebook, s_rel, s_channel, group_size=16) -> Weight:
        import numpy as np
        packed = np.ascontiguousarray(packed, np.int8)
        h = C.c_void_p()
        call("h3_cuda_w4a8_weight_create", self.h, packed.ctypes.data, packed.shape[0], packed.shape[1],
             np.ascontiguousarray(codebook, np.float32).ctypes.data, np.ascontiguousarray(s_rel, np.uint8).ctypes.data,
             np.ascontiguousarray(s_channel, np.float32).ctypes.data, group_size, C.byref(h), None, None)
        return Weight(self, h.value)

    def weight_from_i8(self, w_i8, s_channel) -> Weight:
        import numpy as np
        w_i8 = np.ascontiguousarray(w_i8, np.int8)
        s_channel = np.ascontiguousarray(s_channel, np.float32)
        h = C.c_void_p()
        call("h3_cuda_w4a8_weight_create_from_i8", self.h, w_i8.ctypes.data, w_i8.shape[0], w_i8.shape[1],
             s_channel.ctypes.data, C.byref(h), None, 1)
        return Weight(self, h.value)

    def weight_from_w4g(self, packed, scales_f16, group=128) -> Weight:
        import numpy as np
        packed = np.ascontiguousarray(packed, np.uint8)
        scales_f16 = np.ascontiguousarray(scales_f16, np.uint16)
        h = C.c_void_p()
        call("h3b_w4g_weight_create", self.h, packed.ctypes.data, scales_f16.ctypes.data, packed.shape[0],
             packed.shape[1] * 2, group, C.byref(h))
        return Weight(self, h.value)

    # ---- row-wise operators
    def norm(self, x, *, branch=None, norm_w=None, modulation=None, row_map=None, slots=0, gate_slot=0, shift_slot=0,
             scale_slot=0, eps=1e-5, identity=False, convrot_gs=0, gated=None, normed=None, rot=None, q=None,
             scales=None, fp4=None, sf=None):
        a = _l.NormArgs(ptr(x), ptr(branch), ptr(norm_w), ptr(modulation), ptr(row_map), x.shape[0], x.shape[1],
                        slots, gate_slot, shift_slot, scale_slot, eps, _dt(x), int(identity), convrot_gs, ptr(gated),
                        ptr(normed), ptr(rot), ptr(q), ptr(scales), ptr(fp4), ptr(sf))
        call("h3b_norm_dev", self.h, C.byref(a))

    def quantize_act_int8(self, x):
        import torch
        q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
        s = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
        call("h3b_quantize_act_int8_dev", self.h, ptr(x), _dt(x), x.shape[0], x.shape[1], ptr(q), ptr(s))
        return q, s

    def adaln_f32_dev(self, x, norm_w, modulation, row_map, slots, shift_slot, scale_slot, eps=1e-5):
        import torch
        out = torch.empty_like(x)
        call("h3_cuda_adaln_f32_dev", self.h, ptr(x), ptr(norm_w), ptr(modulation), ptr(row_map), x.shape[0],
             x.shape[1], slots, shift_slot, scale_slot, eps, ptr(out), None)
        return out

    def rms_norm_f32_dev(self, x, w, eps=1e-5):
        import torch
        out = torch.empty_like(x)
        call("h3_cuda_rms_norm_f32_dev", self.h, ptr(x), ptr(w), x.shape[0], x.shape[1], eps, ptr(out))
        return out

    def gate_f32_dev(self, residual, branch, modulation, row_map, slots, gate_slot):
        import torch
        out = torch.empty_like(residual)
        call("h3_cuda_gate_f32_dev", self.h, ptr(residual), ptr(branch), ptr(modulation), ptr(row_map),
             residual.shape[0], residual.shape[1], slots, gate_slot, ptr(out), None)
        return out

    def gate_adaln_f32_dev(self, residual, branch, norm_w, modulation, row_map, slots, gate_slot, shift_slot,
                           scale_slot, eps=1e-5):
        import torch
        gated, normed = torch.empty_like(residual), torch.empty_like(residual)
        call("h3_cuda_gate_adaln_f32_dev", self.h, ptr(residual), ptr(branch), ptr(norm_w), ptr(modulation),
             ptr(row_map), residual.shape[0], residual.shape[1], slots, gate_slot, shift_slot, scale_slot, eps,
             ptr(gated), ptr(normed), None)
        return gated, normed

    def swiglu_f32_dev(self, fused):
        import torch
        out = torch.empty((fused.shape[0], fused.shape[1] // 2), dtype=fused.dtype, device=fused.device)
        call("h3_cuda_swiglu_f32_dev", self.h, ptr(fused), fused.shape[0], fused.shape[1] // 2, ptr(out), None)
        return out

    def convrot_act_f32_dd(self, x, gs):
        import torch
        y = torch.empty_like(x)
        call("h3_cuda_convrot_act_f32_dd", self.h, ptr(x), x.shape[0], x.shape[1], gs, ptr(y))
        return y

    def qkv_rope(self, qkv, q_norm, k_norm, cos, sin, heads, head_dim, rope_half, eps=1e-5, grouped=0, split_half=1,
                 out_dtype=None):
        import torch
        out_dtype = out_dtype or qkv.dtype
        seq = qkv.shape[0]
        q, k, v = (torch.empty((seq, heads, head_dim), dtype=out_dtype, device=qkv.device) for _ in range(3))
        call("h3b_qkv_rope_dev", self.h, ptr(qkv), _dt(qkv), ptr(q_norm), ptr(k_norm), ptr(cos), ptr(sin), seq, heads,
             head_dim, rope_half, eps, grouped, split_half, ptr(q), ptr(k), ptr(v), _dt(q))
        return q, k, v

    def cast(self, x, dtype):
        import torch
        out = torch.empty(x.shape, dtype=dtype, device=x.device)
        call("h3b_cast_dev", self.h, ptr(x), _dt(x), ptr(out), _dt(out), x.numel())
        return out

    # ---- linears
    def gemm_i8(self, weight: Weight, x_i8, act_scales, *, kind=EPI_PLAIN, out_dtype=None, residual=None,
                modulation=None, row_map=None, slots=0, gate_slot=0, out=None, lora=None):
        import torch
        out_dtype = out_dtype or torch.float32
        m = x_i8.shape[0]
        n_out = weight.n // 2 if kind == EPI_SWIGLU else weight.n
        if out is None:
            out = torch.empty((m, n_out), dtype=out_dtype, device=x_i8.device)
        e = _l.GemmEpi(kind, _dt(out), ptr(residual), ptr(modulation), ptr(row_map), slots, gate_slot)  # rest zero
        e.d_lora = ptr(lora)   # optional [m, n] f32 delta (h3_dit_fused_epi.h:85-141)
        call("h3b_gemm_i8_dev", self.h, weight.h, ptr(x_i8), ptr(act_scales), m, ptr(out), C.byref(e))
        return out

    def gemm_i8_qkv_rope(self, weight: Weight, x_i8, act_scales, q_norm, k_norm, cos, sin, rope_half, eps=1e-5,
                         round_qkv=True):
        """QKV projection with QK-norm + RoPE in the epilogue -> (q, k, v) bf16 [m, heads, 128]."""
        import torch
        m, heads = x_i8.shape[0], weight.n // 384
        q, k, v = (torch.empty((m, heads, 128), dtype=torch.bfloat16, device=x_i8.device) for _ in range(3))
        e = _l.GemmEpi(_l.EPI_QKV_ROPE, BF16, None, None, None, 0, 0, ptr(k), ptr(v), ptr(q_norm), ptr(k_norm), ptr(cos),
                       ptr(sin), rope_half, eps, int(round_qkv))
        call("h3b_gemm_i8_dev", self.h, weight.h, ptr(x_i8), ptr(act_scales), m, ptr(q), C.byref(e))
        return q, k, v

    def gemm_i8_qkv_rope_scatter(self, weight: Weight, x_i8, act_scales, q_norm, k_norm, cos, sin, rope_half,
                                 direct: "_l.UlyssesDirect", eps=1e-5):
        """The same projection with every (row, head) slice stored into direct.peer_{q,k,v}[head // hl]."""
        e = _l.GemmEpi(_l.EPI_QKV_ROPE, BF16, None, None, None, 0, 0, None, None, ptr(q_norm), ptr(k_norm), ptr(cos),
                       ptr(sin), rope_half, eps, 1, C.addressof(direct))
        call("h3b_gemm_i8_dev", self.h, weight.h, ptr(x_i8), ptr(act_scales), x_i8.shape[0], None, C.byref(e))

    def sdpa_bf16_scatter(self, direct: "_l.UlyssesDirect", seq_real, scale=None):
        """Attention over direct.q/k/v (this rank's heads of the gathered sequence); rows go to direct.peer_att."""
        call("h3b_sdpa_bf16_scatter_dev", self.h, C.addressof(direct), seq_real,
             float(scale if scale is not None else direct.head_dim ** -0.5))

    def gemm_i8_dequant_f32_w_act_dev(self, weight: Weight, x_f32, convrot_gs=0, epi: _l.DitGemmEpi | None = None):
        import torch
        m = x_f32.shape[0]
        n_out = weight.n // 2 if (epi is not None and epi.swiglu) else weight.n
        y = torch.empty((m, n_out), dtype=torch.float32, device=x_f32.device)
        backend = C.create_string_buffer(32)
        call("h3_cuda_gemm_i8_dequant_f32_w_act_dev_epi", self.h, weight.h, ptr(x_f32), convrot_gs, m, ptr(y), None,
             None, backend, 32, C.byref(epi) if epi is not None else None)
        return y

    def gemm_i8_dequant_f32_w_act_dev_noalloc(self, weight: Weight, x_f32, convrot_gs=0, out=None):
        """The linear for hosts that must not allocate device memory: same result as
        gemm_i8_dequant_f32_w_act_dev, scratch taken from a fixed area inside the library."""
        import torch
        m = x_f32.shape[0]
        if out is None:
            out = torch.empty((m, weight.n), dtype=torch.float32, device=x_f32.device)
        call("h3b_gemm_i8_dequant_f32_w_act_dev_noalloc", self.h, weight.h, ptr(x_f32), convrot_gs, m, ptr(out))
        return out

    # ---- the step on either side of the block chain (f32, device tensors)
    def gemm_f32_dd(self, x, w):
        """h3_cuda_gemm_f32_dd: x [m,k] @ w [n,k]^T -> [m,n], all f32."""
        import torch
        y = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32, device=x.device)
        call("h3_cuda_gemm_f32_dd", self.h, ptr(x), ptr(w), x.shape[0], w.shape[0], x.shape[1], ptr(y), None)
        return y

    def gemm_f32_dd_ex(self, x, w, y, alpha=1.0, beta=0.0, tf32_name=False):
        """In place: y = alpha * (x @ w^T) + beta * y (h3_cuda_gemm_f32_dd_ex / _tf32_ex)."""
        if tf32_name:
            call("h3_cuda_gemm_f32_dd_tf32_ex", self.h, ptr(x), ptr(w), x.shape[0], w.shape[0], x.shape[1], ptr(y),
                 float(alpha), float(beta))
        else:
            call("h3_cuda_gemm_f32_dd_ex", self.h, ptr(x), ptr(w), x.shape[0], w.shape[0], x.shape[1], ptr(y),
                 float(alpha), float(beta), None)
        return y

    def bias_add_f32(self, y, bias):
        call("h3_cuda_bias_add_f32_dev", self.h, ptr(y), ptr(bias), y.shape[0], y.shape[1])
        return y

    def dense_f32(self, x, w, bias=None):
        """y = x W^T + b in one launch (patch embedding: k = 96; final heads: n = 96 or 32)."""
        import torch
        y = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32, device=x.device)
        call("h3b_dense_f32_dev", self.h, ptr(x), ptr(w), ptr(bias), x.shape[0], w.shape[0], x.shape[1], ptr(y))
        return y

    def final_head_f32(self, x, norm_w, modulation, w, bias, eps=1e-5):
        """adaLN with shift = modulation[0], scale = modulation[1] for every token, then the dense head."""
        import torch
        seq, hidden = x.shape
        need = int(load().h3b_final_head_scratch_bytes(seq, hidden))
        scratch = torch.empty(need, dtype=torch.uint8, device=x.device)
        y = torch.empty((seq, w.shape[0]), dtype=torch.float32, device=x.device)
        call("h3b_final_head_f32_dev", self.h, ptr(x), ptr(norm_w), ptr(modulation), seq, hidden, ptr(w), ptr(bias),
             w.shape[0], float(eps), ptr(scratch), need, ptr(y))
        return y

    def euler_step_f32(self, sample, velocity, sigma, sigma_next):
        """In place: sample += (sigma - sigma_next) * velocity; raises H3Error for a pair the reference rejects."""
        call("h3b_euler_step_f32_dev", self.h, ptr(sample), ptr(velocity), sample.numel(), float(sigma), float(sigma_next))
        return sample

    # ---- attention
    def sdpa_bf16(self, q, k, v, scale=None, out=None):
        """q [lq,H,128], k/v [lk,H,128] bf16 views whose last two dims are contiguous -> [lq, H*128] bf16."""
        import torch
        lq, heads, hd = q.shape
        lk = k.shape[0]
        scale = float(scale if scale is not None else hd ** -0.5)
        if out is None:
            out = torch.empty((lq, heads * hd), dtype=torch.bfloat16, device=q.device)
        call("h3b_sdpa_bf16_dev", self.h, ptr(q), q.stride(0), ptr(k), k.stride(0), ptr(v), v.stride(0), lq, lk, heads,
             hd, scale, ptr(out), out.stride(0))
        return out

    # ---- int4 group-128 weights multiplied exactly (packed in HBM, expanded in registers)
    def w4g_exact_weight(self, packed, scales_f16_bits):
        """packed uint8 [n, k/2] (low nibble = even k), scales uint16 (f16 bits) [n, k/128] -> handle."""
        import numpy as np
        packed = np.ascontiguousarray(packed, np.uint8)
        scales = np.ascontiguousarray(scales_f16_bits, np.uint16)
        h = C.c_void_p()
        call("h3b_w4g_exact_weight_create", self.h, packed.ctypes.data, scales.ctypes.data, packed.shape[0],
             packed.shape[1] * 2, C.byref(h))
        return h.value

    def w4g_exact_weight_free(self, handle):
        load().h3b_w4g_exact_weight_free(handle)

    def gemm_w4g_exact(self, handle, n, x_i8, act_scales, out_dtype=None):
        import torch
        out_dtype = out_dtype or torch.float32
        y = torch.empty((x_i8.shape[0], n), dtype=out_dtype, device=x_i8.device)
        call("h3b_gemm_w4g_exact_dev", self.h, handle, ptr(x_i8), ptr(act_scales), x_i8.shape[0], ptr(y), _dt(y))
        return y

    def sdpa(self, q, k, v, scale=None, out=None):
        """q [lq,H,128], k/v [lk,H,128], all bf16 or all f16, any row / head strides that are multiples of 8
        elements -> [lq, H*128] of the same type (h3b_sdpa_strided_dev)."""
        import torch
        lq, heads, hd = q.shape
        lk = k.shape[0]
        scale = float(scale if scale is not None else hd ** -0.5)
        if out is None:
            out = torch.empty((lq, heads * hd), dtype=q.dtype, device=q.device)
        dtype = {torch.bfloat16: 1, torch.float16: 2}[q.dtype]
        call("h3b_sdpa_strided_dev", self.h, dtype, ptr(q), q.stride(0), q.stride(1), ptr(k), k.stride(0), k.stride(1),
             ptr(v), v.stride(0), v.stride(1), lq, lk, heads, hd, scale, ptr(out), out.stride(0), hd)
        return out

    def sdpa_f16_dev(self, q, k, v, scale=None):
        import torch
        seq, heads, hd = q.shape
        out = torch.empty((seq, heads * hd), dtype=torch.float32, device=q.device)
        call("h3_cuda_sdpa_f16_dev", self.h, ptr(q), ptr(k), ptr(v), seq, heads, hd,
             float(scale if scale is not None else hd ** -0.5), ptr(out), None)
        return out

    # ---- NVFP4
    def quantize_act_nvfp4(self, x):
        import torch
        m, k = x.shape
        packed = torch.zeros((m, k // 2), dtype=torch.uint8, device=x.device)
        sf = torch.zeros(int(load().h3_cuda_nvfp4_sf_bytes(m, k)), dtype=torch.uint8, device=x.device)
        call("h3_cuda_quantize_act_nvfp4_dev", self.h, ptr(x), m, k, ptr(packed), ptr(sf))
        return packed, sf

    def gemm_fp4(self, w_fp4, sf_w, x_fp4, sf_x, alpha=1.0, out_dtype=None, swiglu=False):
        """Block-scaled NVFP4 GEMM: packed E2M1 [n,k/2] x [m,k/2] with blocked UE4M3 scales -> [m,n]
        (swiglu: weight rows gate | up, -> [m, n/2] with SwiGLU on the f32 accumulators)."""
        import torch
        out_dtype = out_dtype or torch.float32
        n, m, k = w_fp4.shape[0], x_fp4.shape[0], x_fp4.shape[1] * 2
        y = torch.empty((m, n // 2 if swiglu else n), dtype=out_dtype, device=x_fp4.device)
        call("h3b_gemm_fp4_swiglu_dev" if swiglu else "h3b_gemm_fp4_dev", self.h, ptr(w_fp4), ptr(sf_w), ptr(x_fp4),
             ptr(sf_x), m, n, k, float(alpha), ptr(y), _dt(y))
        return y

    def nvfp4_weight(self, packed, sf, scale2, n, k):
        import numpy as np
        packed = np.ascontiguousarray(packed, np.uint8)
        sf = np.ascontiguousarray(sf, np.uint8)
        # The constructor owns its two host buffers once it has succeeded and releases them with free()
        # (h3_gpu_cuda.h:437-444): it gets malloc'ed copies, never numpy's memory.
        libc = C.CDLL(None)
        libc.malloc.restype, libc.malloc.argtypes, libc.free.argtypes = C.c_void_p, [C.c_size_t], [C.c_void_p]
        bufs = []
        for a in (packed, sf):
            ptr = libc.malloc(max(a.nbytes, 1))
            if not ptr:
                for b in bufs:
                    libc.free(b)
                raise MemoryError("nvfp4_weight: host staging")
            C.memmove(ptr, a.ctypes.data, a.nbytes)
            bufs.append(ptr)
        h = C.c_void_p()
        try:
            call("h3_cuda_nvfp4_weight_create", self.h, bufs[0], bufs[1], float(scale2), n, k, C.byref(h), None)
        except Exception:
            for b in bufs:   # on failure the caller keeps them
                libc.free(b)
            raise
        return h.value

    def nvfp4_weight_free(self, handle):
        load().h3_cuda_nvfp4_weight_free(self.h, handle)

    def gemm_fp4_w_act_dev(self, weight_handle, x_f32, act_scale=1.0, kind="plain", residual=None, modulation=None,
                           row_map=None, slots=0, gate_slot=0):
        """h3_cuda_gemm_fp4_w_act_dev / _swiglu / _gate: f32 activations in, f32 out."""
        import torch
        lib = load()
        n = int(lib.h3_cuda_nvfp4_weight_n(weight_handle))
        m = x_f32.shape[0]
        y = torch.empty((m, n // 2 if kind == "swiglu" else n), dtype=torch.float32, device=x_f32.device)
        err = C.create_string_buffer(_l.ERR_LEN)
        if kind == "plain":
            rc = lib.h3_cuda_gemm_fp4_w_act_dev(self.h, weight_handle, ptr(x_f32), act_scale, m, ptr(y), None, None, None,
                                                err, _l.ERR_LEN, None)
        elif kind == "swiglu":
            rc = lib.h3_cuda_gemm_fp4_w_act_dev_swiglu(self.h, weight_handle, ptr(x_f32), act_scale, m, None, ptr(y), None,
                                                       None, None, err, _l.ERR_LEN, None)
        else:
            rc = lib.h3_cuda_gemm_fp4_w_act_dev_gate(self.h, weight_handle, ptr(x_f32), act_scale, m, ptr(residual),
                                                     ptr(modulation), ptr(row_map), slots, gate_slot, None, ptr(y), None,
                                                     None, None, err, _l.ERR_LEN, None)
        if rc != 1:
            raise H3Error(f"gemm_fp4_w_act_dev[{kind}]: {err.value.decode(errors='replace')}")
        return y

    # ---- host-buffer forms (numpy in, numpy out)
    def adaln_f32(self, x, norm_w, modulation, row_map, slots, shift_slot, scale_slot, eps=1e-5):
        import numpy as np
        x = np.ascontiguousarray(x, np.float32)
        modulation = np.ascontiguousarray(modulation, np.float32)
        out = np.empty_like(x)
        call("h3_cuda_adaln_f32", self.h, ptr(x), ptr(np.ascontiguousarray(norm_w, np.float32)), ptr(modulation),
             ptr(row_map), x.shape[0], x.shape[1], slots, modulation.shape[0], shift_slot, scale_slot, eps, ptr(out),
             None)
        return out


def ulysses_validate(heads, packed_align, tp, ulysses, ring):
    """h3_ulysses_validate: returns (ok, message)."""
    err = C.create_string_buffer(_l.ERR_LEN)
    ok = load().h3_ulysses_validate(heads, packed_align, tp, ulysses, ring, err, _l.ERR_LEN)
    return bool(ok), err.value.decode()


def ulysses_pad_seq(seq, align=64):
    return int(load().h3_ulysses_pad_seq(seq, align))


def ulysses_local_rows(seq_pad, ulysses, rank):
    return int(load().h3_ulysses_local_rows(seq_pad, ulysses, rank))


def tensor_pipe_rate(cuda: "Cuda", kind: int, iters: int) -> float:
    """Tera-operations per second this GPU sustains on back-to-back tcgen05.mma from a resident tile (no loads,
    no epilogue): kind 0 int8 128x256x32, 1 bf16 128x256x16, 2 nvfp4 128x256x64, 3 bf16 128x128x16 from shared
    memory, 4 bf16 128x128x16 with A in tensor memory, 5 nvfp4 128x128x64.  About a second of MMAs at
    iters = 1,000,000.  Lives in libh3_b200_probe.so, a helper of the bench."""
    from . import build as _b
    if not _b.PROBE.exists():
        raise H3Error(f"{_b.PROBE} is missing: run `python -m h3c_b200.build`")
    lib = C.CDLL(str(_b.PROBE))
    lib.h3b_umma_peak_dev.restype = C.c_int
    lib.h3b_umma_peak_dev.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_double), C.c_char_p, C.c_size_t]
    v, err = C.c_double(0), C.create_string_buffer(_l.ERR_LEN)
    if lib.h3b_umma_peak_dev(cuda.h, kind, iters, C.byref(v), err, _l.ERR_LEN) != 1:
        raise H3Error(f"h3b_umma_peak_dev: {err.value.decode(errors='replace')}")
    return v.value


def plugin_value(name: str):
    """Value of a registered switch (environment, else its default); raises for an unregistered name."""
    v = load().h3b_plugin_value(name.encode())
    if v is None:
        raise H3Error(f"switch {name} is not in the registry (include/h3b_plugin.h)")
    return v.decode()


def plugin_enabled(name: str) -> bool:
    plugin_value(name)
    return bool(load().h3b_plugin_enabled(name.encode()))


def plugin_catalogue():
    out = []
    n, s, g, d = (C.c_char_p() for _ in range(4))
    for i in range(load().h3b_plugin_count()):
        load().h3b_plugin_get(i, C.byref(n), C.byref(s), C.byref(g), C.byref(d))
        out.append((n.value.decode(), s.value.decode(), g.value.decode(), d.value.decode()))
    return out


def fill_video_pos(text_len, latent_t, latent_h, latent_w):
    """RoPE coordinates (t, h, w) of the video tokens (h3_dit_w4a8_fill_metal_video_pos); host arrays."""
    import numpy as np
    n = latent_t * (latent_h // 2) * (latent_w // 2)
    pt, ph, pw = (np.empty(max(n, 1), np.float32) for _ in range(3))
    call("h3_dit_w4a8_fill_metal_video_pos", text_len, latent_t, latent_h, latent_w, pt.ctypes.data, ph.ctypes.data,
         pw.ctypes.data)
    return pt[:n], ph[:n], pw[:n]


def rope_tables(inv_freq, pos_t, pos_h, pos_w, spatial_scale=1.0):
    """cos / sin [seq, 48] from 16 inverse frequencies and the three coordinates (h3_dit_w4a8_rope_tables_f32)."""
    import numpy as np
    inv_freq, pos_t, pos_h, pos_w = (np.ascontiguousarray(a, np.float32) for a in (inv_freq, pos_t, pos_h, pos_w))
    if inv_freq.size != 16:
        raise H3Error("rope_tables: inv_freq must hold 16 frequencies")
    cos = np.empty((len(pos_t), 48), np.float32)
    sin = np.empty_like(cos)
    call("h3_dit_w4a8_rope_tables_f32", inv_freq.ctypes.data, len(pos_t), pos_t.ctypes.data, pos_h.ctypes.data,
         pos_w.ctypes.data, C.c_float(spatial_scale), cos.ctypes.data, sin.ctypes.data)
    return cos, sin


def video_rope_tables(inv_freq, text_len, grid, spatial_scale=1.0, pad_rows=0):
    """Tables of a whole step for the token grid (t, h, w), with `pad_rows` trailing rows of angle zero."""
    import numpy as np
    inv_freq = np.ascontiguousarray(inv_freq, np.float32)
    if inv_freq.size != 16:
        raise H3Error("video_rope_tables: inv_freq must hold 16 frequencies")
    rows = grid[0] * grid[1] * grid[2] + pad_rows
    cos = np.empty((rows, 48), np.float32)
    sin = np.empty_like(cos)
    call("h3b_dit_video_rope_tables", inv_freq.ctypes.data, text_len, grid[0], grid[1], grid[2],
         C.c_float(spatial_scale), pad_rows, cos.ctypes.data, sin.ctypes.data)
    return cos, sin


def t_row_from_sigma(sigma, t_table_rows):
    return int(load().h3_dit_w4a8_t_row_from_sigma(C.c_float(sigma), t_table_rows))


def ulysses_shard_rows(seq_real, world, rank, align=64):
    """Ulysses row split (h3_dit_w4a8.c:6275-6277): pad to a multiple of 64, equal slices per rank.
    Returns (seq_pad, seq_local, first_row, real_rows_of_this_rank)."""
    seq_pad = ulysses_pad_seq(seq_real, align)
    seq_local = seq_pad // world
    first = rank * seq_local
    return seq_pad, seq_local, first, max(0, min(seq_local, seq_real - first))


class UlyssesComm:
    """Per-rank sequence-parallel communicator (h3_ulysses_cfg + h3b_ulysses_comm_init_rank)."""

    def __init__(self, rank: int, world_size: int, unique_id: bytes, device_index: int):
        self.cfg = _l.UlyssesCfg(1, world_size, 1, rank, world_size, None)
        buf = C.create_string_buffer(unique_id, 128)
        call("h3b_ulysses_comm_init_rank", C.byref(self.cfg), rank, world_size, buf, device_index)
        self.rank, self.world_size = rank, world_size

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        call("h3b_ulysses_unique_id", buf)
        return buf.raw

    def set_compute(self, stream):
        call("h3_ulysses_comm_set_compute", C.byref(self.cfg), self.rank, stream.cuda_stream)

    def a2a_qkv(self, x, out, seq_local, heads, head_dim):
        call("h3_ulysses_a2a_qkv", C.byref(self.cfg), ptr(x), ptr(out), seq_local, heads, head_dim, x.element_size())

    def a2a_attn_out(self, x, out, seq_local, heads, head_dim):
        call("h3_ulysses_a2a_attn_out", C.byref(self.cfg), ptr(x), ptr(out), seq_local, heads, head_dim,
             x.element_size())

    def setup_direct(self, seq_local, heads, head_dim):
        """Maps every rank's gathered Q/K/V and attention-row buffers (collective): the sequence-parallel chain
        then stores into peer memory from the GEMM and attention epilogues instead of exchanging."""
        call("h3b_ulysses_direct_setup", C.byref(self.cfg), seq_local, heads, head_dim)

    def enable_direct(self, on: bool):
        load().h3b_ulysses_direct_enable(C.byref(self.cfg), int(on))

    @property
    def direct(self) -> bool:
        return bool(load().h3b_ulysses_direct_get(C.byref(self.cfg)))

    def barrier(self):
        call("h3b_ulysses_barrier", C.byref(self.cfg))

    def check(self):
        """Synchronises the compute stream; raises H3Error if a barrier between the ranks gave up waiting."""
        call("h3b_ulysses_check", C.byref(self.cfg), None)

    def close(self):
        load().h3_ulysses_comm_destroy(C.byref(self.cfg))
