"""Runs the REFERENCE's own CUDA operator library (oracle/_ref/cuda/libh3_refcuda.so: its cuBLASLt int8
linear, its activation quantisers, its in-tree flash attention or its cuDNN attention) on seeded inputs, in a
process of its own: the library exports the same h3_cuda_* names as libh3_b200.so, so the two are never loaded
together.  Test infrastructure only; nothing in the product imports this file.

    python oracle/ref_cuda_worker.py JOB.json OUT.npz

JOB.json: {"env": {...}, "ops": [ {"op": ..., ...}, ... ]}.  Every op draws its inputs from numpy's default_rng
with the seed it names, the same way the calling test does, so only shapes and seeds cross the process boundary.
Device memory comes from the CUDA runtime directly (ctypes); torch is not imported.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "_ref" / "cuda" / "libh3_refcuda.so"
ERR = 512
vp, sz, f32c, i32 = C.c_void_p, C.c_size_t, C.c_float, C.c_int


def seeded_acts(seed, m, k, outliers=True):
    """N(0,1) activations with 0.1 % entries x20 (the benchmark's distribution)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k), dtype=np.float32)
    if outliers:
        x[rng.random((m, k)) < 0.001] *= 20
    return x


def seeded_weight_i8(seed, n, k):
    rng = np.random.default_rng(seed)
    return rng.integers(-127, 128, (n, k), dtype=np.int8), rng.uniform(1e-3, 1e-2, n).astype(np.float32)


def tiled_acts(seed, m, k, block=1024):
    """Cheap large activation matrix for timing: a seeded block of rows repeated."""
    base = seeded_acts(seed, min(block, m), k)
    reps = -(-m // base.shape[0])
    return np.ascontiguousarray(np.tile(base, (reps, 1))[:m])


class Rt:
    """The few CUDA runtime calls the worker needs."""

    def __init__(self):
        self.rt = C.CDLL("libcudart.so.12")
        self.rt.cudaMalloc.argtypes = [C.POINTER(vp), sz]
        self.rt.cudaMemcpy.argtypes = [vp, vp, sz, i32]
        self.rt.cudaMemset.argtypes = [vp, i32, sz]
        self.rt.cudaFree.argtypes = [vp]
        self.rt.cudaEventCreate.argtypes = [C.POINTER(vp)]
        self.rt.cudaEventRecord.argtypes = [vp, vp]
        self.rt.cudaEventSynchronize.argtypes = [vp]
        self.rt.cudaEventElapsedTime.argtypes = [C.POINTER(f32c), vp, vp]
        self.live = []

    def ok(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"{what}: cuda error {rc}")

    def alloc(self, nbytes):
        p = vp()
        self.ok(self.rt.cudaMalloc(C.byref(p), max(int(nbytes), 16)), "cudaMalloc")
        self.live.append(p)
        return p

    def up(self, a):
        a = np.ascontiguousarray(a)
        p = self.alloc(a.nbytes)
        self.ok(self.rt.cudaMemcpy(p, a.ctypes.data, a.nbytes, 1), "cudaMemcpy H2D")
        return p

    def down(self, p, shape, dtype, offset=0):
        out = np.empty(shape, dtype)
        self.ok(self.rt.cudaMemcpy(out.ctypes.data, vp(p.value + offset) if isinstance(p, vp) else vp(p + offset),
                                   out.nbytes, 2), "cudaMemcpy D2H")
        return out

    def free_all(self):
        self.rt.cudaDeviceSynchronize()
        for p in self.live:
            self.rt.cudaFree(p)
        self.live = []

    def sync(self):
        self.ok(self.rt.cudaDeviceSynchronize(), "cudaDeviceSynchronize")

    def time_ms(self, fn, iters, warmup=2):
        """Median device time of fn() on the legacy default stream (the stream the library uses by default)."""
        for _ in range(warmup):
            fn()
        self.sync()
        e0, e1 = vp(), vp()
        self.rt.cudaEventCreate(C.byref(e0))
        self.rt.cudaEventCreate(C.byref(e1))
        out = []
        for _ in range(iters):
            self.rt.cudaEventRecord(e0, None)
            fn()
            self.rt.cudaEventRecord(e1, None)
            self.rt.cudaEventSynchronize(e1)
            ms = f32c()
            self.rt.cudaEventElapsedTime(C.byref(ms), e0, e1)
            out.append(ms.value)
        return float(np.median(out))

    def time_ms_stream(self, fn, iters, warmup=2):
        """Device time per call of `iters` calls queued back to back (one event pair around all of them)."""
        for _ in range(warmup):
            fn()
        self.sync()
        e0, e1 = vp(), vp()
        self.rt.cudaEventCreate(C.byref(e0))
        self.rt.cudaEventCreate(C.byref(e1))
        self.rt.cudaEventRecord(e0, None)
        for _ in range(iters):
            fn()
        self.rt.cudaEventRecord(e1, None)
        self.rt.cudaEventSynchronize(e1)
        ms = f32c()
        self.rt.cudaEventElapsedTime(C.byref(ms), e0, e1)
        return ms.value / iters


class RefCuda:
    def __init__(self):
        self.rt = Rt()
        self.lib = L = C.CDLL(str(LIB))
        self.err = C.create_string_buffer(ERR)
        L.h3_cuda_create.restype = vp
        L.h3_cuda_create.argtypes = [i32, C.c_char_p, sz]
        self.h = L.h3_cuda_create(0, self.err, ERR)
        if not self.h:
            raise RuntimeError(f"h3_cuda_create: {self.err.value.decode()}")
        L.h3_cuda_set_quiet.argtypes = [vp, i32]

    def call(self, name, *args):
        fn = getattr(self.lib, name)
        fn.restype = i32
        rc = fn(*args, self.err, ERR)
        if rc != 1:
            raise RuntimeError(f"{name}: {self.err.value.decode(errors='replace')}")

    def weight(self, w_i8, s):
        h = vp()
        self.call("h3_cuda_w4a8_weight_create_from_i8", vp(self.h), vp(w_i8.ctypes.data), sz(w_i8.shape[0]),
                  sz(w_i8.shape[1]), vp(s.ctypes.data), C.byref(h), None, i32(1))
        self.call("h3_cuda_w4a8_weight_ensure_ready", h)
        return h

    # ---- ops ---------------------------------------------------------------------------------------------
    def op_linear(self, o, out, tag):
        """ConvRot + per-row INT8 quant + cuBLASLt int8 GEMM + dequant, f32 in / f32 out."""
        m, n, k, gs = o["m"], o["n"], o["k"], o.get("gs", 0)
        w_i8, s = seeded_weight_i8(o["seed"] + 1, n, k)
        x = tiled_acts(o["seed"], m, k) if o.get("tiled") else seeded_acts(o["seed"], m, k)
        w = self.weight(w_i8, s)
        dx, dy = self.rt.up(x), self.rt.alloc(m * n * 4)
        prep, gemm = C.c_double(0), C.c_double(0)
        be = C.create_string_buffer(64)

        def run():
            self.call("h3_cuda_gemm_i8_dequant_f32_w_act_dev", vp(self.h), w, dx, i32(gs), sz(m), dy, C.byref(prep),
                      C.byref(gemm), be, sz(64))
        run()
        self.rt.sync()
        rows = np.asarray(o.get("rows", list(range(min(m, 64)))), np.int64)
        y = np.stack([self.rt.down(dy, (n,), np.float32, int(r) * n * 4) for r in rows])
        out[f"{tag}_rows"], out[f"{tag}_y"] = rows, y
        out[f"{tag}_backend"] = np.frombuffer(be.value, np.uint8)
        if o.get("iters", 0):
            preps, gemms = [], []
            for _ in range(o["iters"]):
                run()
                preps.append(prep.value)
                gemms.append(gemm.value)
            self.lib.h3_cuda_set_quiet(vp(self.h), 1)
            total = self.rt.time_ms(run, o["iters"])
            self.lib.h3_cuda_set_quiet(vp(self.h), 0)
            out[f"{tag}_ms"] = np.array([np.median(preps), np.median(gemms), total])
        self.lib.h3_cuda_w4a8_weight_free.argtypes = [vp]
        self.lib.h3_cuda_w4a8_weight_free(w)
        self.rt.free_all()

    def op_act_codes(self, o, out, tag):
        """The reference CUDA path's rotated activations and the INT8 codes / scales it derives from them."""
        m, k, gs = o["m"], o["k"], o["gs"]
        x = seeded_acts(o["seed"], m, k)
        dx, drot = self.rt.up(x), self.rt.alloc(m * k * 4)
        self.call("h3_cuda_convrot_act_f32_dd", vp(self.h), dx, sz(m), sz(k), i32(gs), drot)
        xi8, sc = vp(), vp()
        self.call("h3_cuda_epi_fuse_ink_prep_fc2", vp(self.h), dx, sz(m), sz(k), i32(gs), C.byref(xi8), C.byref(sc))
        self.rt.sync()
        out[f"{tag}_rot"] = self.rt.down(drot, (m, k), np.float32)
        out[f"{tag}_codes"] = self.rt.down(xi8, (m, k), np.int8)
        out[f"{tag}_scales"] = self.rt.down(sc, (m,), np.float32)
        self.rt.free_all()

    def op_quant_nvfp4(self, o, out, tag):
        m, k = o["m"], o["k"]
        x = seeded_acts(o["seed"], m, k)
        if o.get("edge"):
            x[0, :16] = 0.0
            x[1 % m, 16:32] = 1e-9
            x[2 % m, 32:48] = 3000.0
        self.lib.h3_cuda_nvfp4_sf_bytes.restype = sz
        self.lib.h3_cuda_nvfp4_sf_bytes.argtypes = [sz, sz]
        m_pad = (m + 127) // 128 * 128
        sfb = int(self.lib.h3_cuda_nvfp4_sf_bytes(m_pad, k))
        dx, d4, dsf = self.rt.up(x), self.rt.alloc(m_pad * k // 2), self.rt.alloc(sfb)
        self.rt.rt.cudaMemset(d4, 0, m_pad * k // 2)
        self.rt.rt.cudaMemset(dsf, 0, sfb)
        self.call("h3_cuda_quantize_act_nvfp4_dev", vp(self.h), dx, sz(m), sz(k), d4, dsf)
        self.rt.sync()
        out[f"{tag}_fp4"] = self.rt.down(d4, (m, k // 2), np.uint8)
        out[f"{tag}_sf"] = self.rt.down(dsf, (sfb,), np.uint8)
        self.rt.free_all()

    def op_sdpa(self, o, out, tag):
        """Attention through the backend the environment selects (in-tree flash f16 or cuDNN), f32 in/out."""
        seq, heads, hd = o["seq"], o["heads"], 128
        rng = np.random.default_rng(o["seed"])
        q, k, v = (rng.standard_normal((seq, heads, hd), dtype=np.float32) for _ in range(3))
        dq, dk, dv, do = self.rt.up(q), self.rt.up(k), self.rt.up(v), self.rt.alloc(q.nbytes)
        ms = C.c_double(0)
        be = C.create_string_buffer(64)

        def run():
            self.call("h3_cuda_sdpa_f16_dev_ex", vp(self.h), dq, dk, dv, sz(seq), sz(heads), sz(hd),
                      f32c(1.0 / np.sqrt(hd)), i32(0), do, C.byref(ms), be, sz(64))
        run()
        self.rt.sync()
        rows = np.asarray(o.get("rows", list(range(min(seq, 32)))), np.int64)
        out[f"{tag}_rows"] = rows
        out[f"{tag}_o"] = np.stack([self.rt.down(do, (heads * hd,), np.float32, int(r) * heads * hd * 4) for r in rows])
        out[f"{tag}_backend"] = np.frombuffer(be.value, np.uint8)
        if o.get("iters", 0):
            inner = []
            for _ in range(o["iters"]):
                run()
                inner.append(ms.value)
            self.lib.h3_cuda_set_quiet(vp(self.h), 1)
            total = self.rt.time_ms(run, o["iters"])
            self.lib.h3_cuda_set_quiet(vp(self.h), 0)
            out[f"{tag}_ms"] = np.array([np.median(inner), total])
        self.rt.free_all()

    def op_fp4_gemm(self, o, out, tag):
        """cuBLASLt block-scaled FP4 GEMM on operands its own activation quantiser produced."""
        m, n, k = o["m"], o["n"], o["k"]
        self.lib.h3_cuda_nvfp4_sf_bytes.restype = sz
        self.lib.h3_cuda_nvfp4_sf_bytes.argtypes = [sz, sz]
        bufs = []
        for rows, seed in ((n, o["seed"] + 1), (m, o["seed"])):
            x = tiled_acts(seed, rows, k)
            rp = (rows + 127) // 128 * 128
            sfb = int(self.lib.h3_cuda_nvfp4_sf_bytes(rp, k))
            dx, d4, dsf = self.rt.up(x), self.rt.alloc(rp * k // 2), self.rt.alloc(sfb)
            self.rt.rt.cudaMemset(d4, 0, rp * k // 2)
            self.rt.rt.cudaMemset(dsf, 0, sfb)
            self.call("h3_cuda_quantize_act_nvfp4_dev", vp(self.h), dx, sz(rows), sz(k), d4, dsf)
            bufs += [d4, dsf]
        dy = self.rt.alloc(((m + 127) // 128 * 128) * n * 2)
        ms = C.c_double(0)

        def run():
            self.call("h3_cuda_gemm_fp4_bs_dev", vp(self.h), bufs[0], bufs[1], bufs[2], bufs[3], sz(m), sz(n), sz(k), dy,
                      C.byref(ms))
        run()
        self.rt.sync()
        self.lib.h3_cuda_set_quiet(vp(self.h), 1)
        out[f"{tag}_ms"] = np.array([self.rt.time_ms(run, o.get("iters", 5)), self.rt.time_ms_stream(run, 3 * o.get("iters", 5))])
        self.lib.h3_cuda_set_quiet(vp(self.h), 0)
        self.rt.free_all()


def main():
    job = json.loads(Path(sys.argv[1]).read_text())
    for k, v in job.get("env", {}).items():
        os.environ[k] = str(v)
    ref = RefCuda()
    out, failures = {}, {}
    for i, o in enumerate(job["ops"]):
        tag = o.get("tag", f"op{i}")
        try:
            getattr(ref, "op_" + o["op"])(o, out, tag)
        except Exception as exc:   # one unsupported shape must not lose the others' results
            failures[tag] = str(exc)
            try:
                ref.rt.free_all()
            except Exception:
                pass
    out["failures_json"] = np.frombuffer(json.dumps(failures).encode(), np.uint8)
    np.savez(sys.argv[2], **out)
    print(json.dumps({"ops": len(job["ops"]), "failures": failures}))


if __name__ == "__main__":
    main()
