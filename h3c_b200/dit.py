"""Block / block-chain front-end (h3b_dit_* in the C ABI) and a seeded synthetic model builder.

`Dit` mirrors the reference's `h3_dit_w4a8` context for the denoiser block path: weights are
attached per block and linear slot, `block_forward` / `layers_forward` run on device tensors,
`layers_forward_f32` takes and returns host float32 arrays like `h3_dit_w4a8_layers_forward_f32`.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import lib as _l
from .lib import BF16, F32, H3Error, call, load, ptr

BLOCK_REFERENCE, BLOCK_CROSS_GELU = 0, 1
LIN_QKV, LIN_OUT, LIN_FC1, LIN_FC2, LIN_CROSS_Q, LIN_CROSS_KV, LIN_CROSS_OUT = range(7)
LIN_NAMES_CROSS = {"qkv": LIN_QKV, "o": LIN_OUT, "up": LIN_FC1, "down": LIN_FC2, "cq": LIN_CROSS_Q,
                   "ckv": LIN_CROSS_KV, "co": LIN_CROSS_OUT}
LIN_NAMES_REF = {"qkv": LIN_QKV, "out": LIN_OUT, "fc1": LIN_FC1, "fc2": LIN_FC2}


@dataclass
class DitGeometry:
    dim: int = 3072
    heads: int = 24
    head_dim: int = 128
    ffn: int = 12288
    rope_half: int = 48
    n_blocks: int = 50
    mod_rows: int = 1
    t_dim: int = 256
    kind: int = BLOCK_CROSS_GELU
    stream_dtype: int = BF16
    convrot_gs: int = 0
    eps: float = 1e-5


class Dit:
    def __init__(self, cuda, geo: DitGeometry):
        self.cuda, self.geo = cuda, geo
        cfg = _l.DitConfig(geo.kind, geo.stream_dtype, geo.convrot_gs, geo.dim, geo.heads, geo.head_dim, geo.ffn,
                           geo.rope_half, geo.n_blocks, geo.mod_rows, geo.t_dim, geo.eps)
        err = C.create_string_buffer(_l.ERR_LEN)
        self.h = load().h3b_dit_create(cuda.h, C.byref(cfg), err, _l.ERR_LEN)
        if not self.h:
            raise H3Error(f"h3b_dit_create: {err.value.decode(errors='replace')}")
        self._weights = []  # keep the borrowed weight objects alive
        self._fp4 = []      # NVFP4 weight handles this object owns (set_linear_nvfp4(..., own=True))

    def close(self):
        if self.h:
            load().h3b_dit_free(self.h)
            self.h = None
        for w in self._weights:
            w.free()
        self._weights = []
        for h in self._fp4:
            self.cuda.nvfp4_weight_free(h)
        self._fp4 = []

    def close_keep_weights(self):
        """Frees the context only; for a context whose weight objects belong to another one."""
        if self.h:
            load().h3b_dit_free(self.h)
            self.h = None
        self._weights = []

    def set_linear(self, block, which, weight):
        call("h3b_dit_set_linear", self.h, block, which, weight.h)
        self._weights.append(weight)

    def set_linear_nvfp4(self, block, which, weight_handle, own=False):
        """NVFP4 form of QKV / OUT / FC1 / FC2 (handle from Cuda.nvfp4_weight; None returns the linear to INT8).
        own: the handle is freed by close()."""
        call("h3b_dit_set_linear_nvfp4", self.h, block, which, weight_handle)
        if own and weight_handle:
            self._fp4.append(weight_handle)

    def set_block_aux(self, block, norm1, norm2, q_norm, k_norm, norm_cross=None):
        f = lambda a: None if a is None else np.ascontiguousarray(a, np.float32)
        arrs = [f(a) for a in (norm1, norm2, q_norm, k_norm, norm_cross)]
        call("h3b_dit_set_block_aux", self.h, block, *[ptr(a) for a in arrs])

    def set_adaln(self, block, w, b):
        w, b = np.ascontiguousarray(w, np.float32), np.ascontiguousarray(b, np.float32)
        call("h3b_dit_set_adaln", self.h, block, ptr(w), ptr(b))

    def project_modulation(self, t_feat_dev):
        call("h3b_dit_project_modulation", self.h, ptr(t_feat_dev))

    def modulation(self, block):
        """Device f32 view [mod_rows, 6, dim] of the projected modulation."""
        import torch
        n = self.geo.mod_rows * 6 * self.geo.dim
        p = load().h3b_dit_modulation(self.h, block)
        if not p:
            raise H3Error("modulation not projected")
        class _View:  # zero-copy view of library-owned device memory
            __cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (int(p), False), "version": 2}
        return torch.as_tensor(_View(), device=self.cuda.device).view(self.geo.mod_rows, 6, self.geo.dim)

    def reserve(self, seq, text_seq=0):
        call("h3b_dit_reserve", self.h, seq, text_seq)

    def block_forward(self, block, x, cos, sin, *, modulation=None, row_map=None, text=None, out=None):
        import torch
        out = torch.empty_like(x) if out is None else out
        call("h3b_dit_block_forward_dev", self.h, block, ptr(x), x.shape[0], ptr(modulation), ptr(row_map), ptr(cos),
             ptr(sin), ptr(text), 0 if text is None else text.shape[0], ptr(out))
        return out

    def layers_forward(self, x, cos, sin, *, first=0, n=None, row_map=None, text=None, out=None):
        import torch
        n = self.geo.n_blocks - first if n is None else n
        out = torch.empty_like(x) if out is None else out
        call("h3b_dit_layers_forward_dev", self.h, first, n, ptr(x), x.shape[0], ptr(row_map), ptr(cos), ptr(sin),
             ptr(text), 0 if text is None else text.shape[0], ptr(out))
        return out

    def layers_forward_graph(self, x, cos, sin, *, first=0, n=None, row_map=None, text=None, out=None):
        """The chain as one CUDA graph launch: captured by the C host on the first call for these tensors, replayed
        on the following ones."""
        import torch
        n = self.geo.n_blocks - first if n is None else n
        out = torch.empty_like(x) if out is None else out
        call("h3b_dit_layers_forward_graph_dev", self.h, first, n, ptr(x), x.shape[0], ptr(row_map), ptr(cos), ptr(sin),
             ptr(text), 0 if text is None else text.shape[0], ptr(out))
        return out

    @property
    def graph_nodes(self):
        return int(load().h3b_dit_graph_nodes(self.h))

    def layers_forward_f32(self, t_feat, x, cos, sin, *, first=0, n=None, row_map=None, text=None, out=None):
        """Host arrays in, host array out (pinned torch tensors or numpy arrays)."""
        n = self.geo.n_blocks - first if n is None else n
        if out is None:
            out = np.empty((x.shape[0], x.shape[1]), np.float32)
        call("h3b_dit_layers_forward_f32", self.h, first, n, ptr(t_feat), ptr(x), x.shape[0], ptr(row_map), ptr(cos),
             ptr(sin), ptr(text), 0 if text is None else text.shape[0], ptr(out))
        return out

    def denoise_step(self, latent, patch_w, patch_b, final_norm, final_mod, final_w, final_b, cos, sin, sigma, sigma_next, *,
                     text=None, row_map=None):
        """One sampler step with everything on the device: patch embedding (f32 dense) -> block chain in the
        stream type -> final adaLN head (f32) -> Euler update of `latent` in place.  The modulation of the blocks
        must have been projected for this step's time feature (project_modulation).  Returns the velocity."""
        import torch
        stream_dtype = {1: torch.bfloat16, 2: torch.float16}.get(self.geo.stream_dtype, torch.float32)
        hidden = self.cuda.dense_f32(latent, patch_w, patch_b)
        y = self.layers_forward(hidden.to(stream_dtype), cos, sin, row_map=row_map, text=text)
        velocity = self.cuda.final_head_f32(y.float(), final_norm, final_mod, final_w, final_b)
        self.cuda.euler_step_f32(latent, velocity, sigma, sigma_next)
        return velocity

    def set_ulysses(self, comm):
        """Attaches a per-rank `UlyssesComm` (None detaches)."""
        call("h3b_dit_set_ulysses", self.h, C.byref(comm.cfg) if comm is not None else None)
        self._uly = comm

    def layers_forward_ulysses(self, x_local, seq_real, cos_full, sin_full, *, first=0, n=None, row_map=None, text=None,
                               out=None):
        import torch
        n = self.geo.n_blocks - first if n is None else n
        out = torch.empty_like(x_local) if out is None else out
        call("h3b_dit_layers_forward_ulysses_dev", self.h, first, n, ptr(x_local), x_local.shape[0], seq_real,
             ptr(row_map), ptr(cos_full), ptr(sin_full), ptr(text), 0 if text is None else text.shape[0], ptr(out))
        return out

    def layers_forward_ulysses_f32(self, t_feat, x_local, seq_real, cos_full, sin_full, *, first=0, n=None, row_map=None,
                                   text=None, out=None):
        n = self.geo.n_blocks - first if n is None else n
        if out is None:
            out = np.empty((x_local.shape[0], x_local.shape[1]), np.float32)
        call("h3b_dit_layers_forward_ulysses_f32", self.h, first, n, ptr(t_feat), ptr(x_local), x_local.shape[0],
             seq_real, ptr(row_map), ptr(cos_full), ptr(sin_full), ptr(text), 0 if text is None else text.shape[0],
             ptr(out))
        return out

    @property
    def launches_per_block(self):
        return int(load().h3b_dit_launches_per_block(self.h))


# ---------------------------------------------------------------------------------------------
# Seeded synthetic weights with the benchmark's distributions: weights ~ N(0, 0.02^2), norm
# weights ~ N(1, 0.1), adaLN projection ~ N(0, 0.02^2).  int4 weights are produced on the device
# (quantise -> pack -> the library's own decode) so that 50 blocks build in seconds.

def _rand_w4g_weight(cuda, gen, n, k, group=128, std=0.02):
    """Returns (Weight, packed uint8 [n,k/2] numpy, scales f16-bits [n,k/group] numpy)."""
    import torch
    w = torch.randn((n, k), generator=gen, device=cuda.device, dtype=torch.float32) * std
    g = w.view(n, k // group, group)
    amax = g.abs().amax(dim=2, keepdim=True)
    s = torch.where(amax > 0, amax / 7.0, torch.ones_like(amax)).to(torch.float16)
    s = torch.where(s == 0, torch.full_like(s, 5.960464477539063e-08), s)
    q = torch.clamp(torch.round(g / s.float()), -8, 7).to(torch.int32).view(n, k) & 0xF
    packed = (q[:, 0::2] | (q[:, 1::2] << 4)).to(torch.uint8).cpu().numpy()
    scales = s.view(n, k // group).view(torch.int16).cpu().numpy().view(np.uint16)
    return cuda.weight_from_w4g(packed, scales, group), packed, scales


def _rand_nvfp4_weight(cuda, gen, n, k, std=0.02):
    """Handle of an NVFP4 weight: N(0, std^2) values scaled to the E2M1 range, quantised on the device by the
    library's block quantiser (16-value blocks, UE4M3 scales in the 128 x 4 tile layout), second-level scale
    undoing the range scaling."""
    import torch
    up = 6.0 * 448.0 / (4.0 * std)                      # a 4-sigma weight lands on the largest code x largest scale
    w = torch.randn((n, k), generator=gen, device=cuda.device, dtype=torch.float32) * (std * up)
    packed, sf = cuda.quantize_act_nvfp4(w)
    return cuda.nvfp4_weight(packed.cpu().numpy(), sf.cpu().numpy(), 1.0 / up, n, k)


def build_synthetic(cuda, geo: DitGeometry, seed=0, keep_host=False, nvfp4=False):
    """Builds a `Dit` with seeded random W4 (group 128, f16 scales) weights.  With keep_host the
    packed weights and aux tensors are also returned per block (for oracle comparisons); an integer
    keep_host keeps the aux tensors (not the packed weights) of that many leading blocks only.
    nvfp4: the four linears of the reference block as NVFP4 weights instead (f32 stream)."""
    aux_only = 0 if isinstance(keep_host, bool) else int(keep_host)
    import torch
    gen = torch.Generator(device=cuda.device)
    gen.manual_seed(seed)
    rng = np.random.default_rng(seed)
    dit = Dit(cuda, geo)
    D, I, F = geo.dim, geo.heads * geo.head_dim, geo.ffn
    if geo.kind == BLOCK_CROSS_GELU:
        shapes = {"qkv": (3 * I, D), "o": (D, I), "up": (F, D), "down": (D, F), "cq": (I, D), "ckv": (2 * I, D),
                  "co": (D, I)}
        names = LIN_NAMES_CROSS
    else:
        shapes = {"qkv": (3 * I, D), "out": (D, I), "fc1": (2 * F, D), "fc2": (D, F)}
        names = LIN_NAMES_REF
    host = []
    for b in range(geo.n_blocks):
        rec = {}
        for name, (n, k) in shapes.items():
            if nvfp4:
                dit.set_linear_nvfp4(b, names[name], _rand_nvfp4_weight(cuda, gen, n, k), own=True)
                continue
            w, packed, scales = _rand_w4g_weight(cuda, gen, n, k)
            dit.set_linear(b, names[name], w)
            if keep_host and not aux_only:
                rec[name] = (packed, scales)
        aux = {"norm1": rng.normal(1, 0.1, D), "norm2": rng.normal(1, 0.1, D), "q_norm": rng.normal(1, 0.1, geo.head_dim),
               "k_norm": rng.normal(1, 0.1, geo.head_dim)}
        if geo.kind == BLOCK_CROSS_GELU:
            aux["norm_c"] = rng.normal(1, 0.1, D)
        aux = {k_: v.astype(np.float32) for k_, v in aux.items()}
        dit.set_block_aux(b, aux["norm1"], aux["norm2"], aux["q_norm"], aux["k_norm"], aux.get("norm_c"))
        ada_w = rng.normal(0, 0.02, (geo.mod_rows * 6 * D, geo.t_dim)).astype(np.float32)
        ada_b = rng.normal(0, 0.02, geo.mod_rows * 6 * D).astype(np.float32)
        dit.set_adaln(b, ada_w, ada_b)
        if keep_host and (not aux_only or b < aux_only):
            rec.update(aux)
            rec["adaln_w"], rec["adaln_b"] = ada_w, ada_b
            host.append(rec)
    return (dit, host) if keep_host else dit
