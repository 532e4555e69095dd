"""Benchmark of the DiT denoiser step (milliseconds per 50-block step) on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload at every N: the full 50-block W4A8 step at 50,220 video tokens (31x30x54 patch grid) + 512 text
tokens, D = 3072, 24 x 128 heads, FFN 12288, bf16 residual stream, t = 0.5 (the metric's headline workload).
N = 1 runs it on one GPU; N > 1 (under torchrun, one rank per GPU) shards the rows across the ranks
(Ulysses sequence parallelism), so the per-N values are the same work and compare directly.
`--workload step6144` times the 6,144-token single-GPU step (6x32x32 grid) instead; `--weights nvfp4` the same
token count on the reference's own block with every linear as an NVFP4 weight.
`--impl reference` times the reference's CPU implementation of the same block on the host cores.
`--kernel NAME` times one operator on synthetic data (the commands behind the summaries under profiles/).

Prints ONE JSON line (rank 0).  `value` is ms per step with every input resident in HBM; `e2e` is the
same step through the host-buffer entry point (h3b_dit_layers_forward_f32) with pinned host arrays,
host<->device copies inside the timed region.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "dit_denoiser_ms_per_step_50_blocks"
UNIT = "ms/step"

GEO = dict(dim=3072, heads=24, head_dim=128, ffn=12288, n_blocks=50, text=512)
GRID_1GPU = (6, 32, 32)      # 6,144 tokens
GRID_ULYSSES = (31, 30, 54)  # 50,220 tokens


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"], src="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, src="fallback")


def block_flops(m, text, dim, ffn):
    """Algorithmic work of one block (FLOPs = 2MNK for linears, 4 Lq Lk H d for attention)."""
    lin = 2.0 * m * (dim * (3 * dim + dim + dim + dim + ffn) + ffn * dim) + 2.0 * text * dim * 2 * dim
    attn = 4.0 * m * m * dim + 4.0 * m * text * dim
    return lin, attn


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.file,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.file.read().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.file.name)
        if sm:
            # keep the samples taken under load (upper half), report their median
            load = sorted(sm)[len(sm) // 2:]
            out.update(sm_mhz=float(np.median(load)), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


# ------------------------------------------------------------------------------- CPU baseline

def cpu_block_sample(kind: str, threads: int, budget_s: float = 15.0, grid=None):
    """Times the reference's CPU block path on a bounded row sample of the workload given by `grid`.

    kind "reference": the reference's own C functions (oracle/_ref/libh3_ref.so) driven over row slices
    from `threads` host threads (its loops are serial); attention rows use the rectangular restatement of
    the reference's loop (its own function only handles Lq == Lk).  kind "port": the CPU restatement.
    Returns (ms_per_step_extrapolated, description)."""
    from oracle.pyoracle import Oracle, Ref
    dim, heads, hd, ffn, text_len = GEO["dim"], GEO["heads"], GEO["head_dim"], GEO["ffn"], GEO["text"]
    grid = grid or GRID_1GPU
    m_full = grid[0] * grid[1] * grid[2]
    oracle = Oracle(threads=1)
    impl = Ref() if kind == "reference" else oracle
    rng = np.random.default_rng(0)

    def qweight(n, k):
        w = rng.integers(-127, 128, (n, k), dtype=np.int8)
        return w, rng.uniform(1e-4, 1e-3, n).astype(np.float32)

    W = {k: qweight(*s) for k, s in dict(qkv=(3 * dim, dim), o=(dim, dim), cq=(dim, dim), ckv=(2 * dim, dim),
                                         co=(dim, dim), up=(ffn, dim), down=(dim, ffn)).items()}
    norm = rng.normal(1, 0.1, dim).astype(np.float32)
    qn = rng.normal(1, 0.1, hd).astype(np.float32)
    mod = rng.normal(0, 0.3, (1, 6, dim)).astype(np.float32)
    inv_freq = (1.0 / (10000.0 ** (np.arange(16) / 16.0))).astype(np.float32)
    pt, ph, pw = oracle.fill_video_pos(text_len, grid[0], 2 * grid[1], 2 * grid[2])
    cos, sin = oracle.rope_tables(inv_freq, pt, ph, pw, 1.0)
    k_all = rng.normal(0, 1, (m_full, heads, hd)).astype(np.float32)
    v_all = rng.normal(0, 1, (m_full, heads, hd)).astype(np.float32)
    ckv_all = rng.normal(0, 1, (text_len, 2 * dim)).astype(np.float32)
    ck = np.ascontiguousarray(ckv_all[:, :dim]).reshape(text_len, heads, hd)
    cv = np.ascontiguousarray(ckv_all[:, dim:]).reshape(text_len, heads, hd)

    def linear(x, name):
        q, s = impl.quantize_act_int8(impl.convrot(x, 0))
        return impl.gemm_i8_dequant(q, W[name][0], s, W[name][1])

    def rows_job(r0, r1):
        n = r1 - r0
        x = rng.normal(0, 1, (n, dim)).astype(np.float32)
        rmap = np.zeros(n, np.uint32)
        a = impl.adaln(x, norm, mod, rmap, 6, 0, 1)
        q, _, _ = impl.qkv_rope(linear(a, "qkv"), qn, qn, cos[r0:r1], sin[r0:r1], heads, hd, 48)
        att = oracle.sdpa(q, k_all, v_all)
        x1 = impl.gate(x, linear(att, "o"), mod, rmap, 6, 2)
        cq = linear(impl.rms_norm(x1, norm), "cq").reshape(n, heads, hd)
        x2 = x1 + linear(oracle.sdpa(cq, ck, cv), "co")
        up = linear(impl.adaln(x2, norm, mod, rmap, 6, 3, 4), "up")
        h = (0.5 * up * (1.0 + np.tanh(0.7978845608028654 * (up + 0.044715 * up ** 3)))).astype(np.float32)
        return impl.gate(x2, linear(h, "down"), mod, rmap, 6, 5)

    def text_job(r0, r1):
        return linear(rng.normal(0, 1, (r1 - r0, dim)).astype(np.float32), "ckv")

    def run(rows_per_thread):
        t0 = time.perf_counter()
        with ThreadPoolExecutor(threads) as ex:
            list(ex.map(lambda i: rows_job(i * rows_per_thread, (i + 1) * rows_per_thread), range(threads)))
            list(ex.map(lambda i: text_job(i, i + 1), range(threads)))
        return time.perf_counter() - t0

    t1 = run(1)                                    # calibration: one row per thread
    rpt = int(max(1, min(128, budget_s / max(t1, 1e-3))))
    t = run(rpt) if rpt > 1 else t1
    rows, trow = threads * rpt, threads
    # the sample covered `rows` of m_full query rows and `trow` of text_len text rows of ONE block
    frac = t / (rows / m_full + 0.0)               # crude: text rows are <1 % of the work, scale by query rows
    ms_step = frac * GEO["n_blocks"] * 1e3
    desc = (f"{rows} of {m_full} query rows (all linears, QK-norm+RoPE, self-attention against all {m_full} keys, "
            f"cross-attention, FFN) + {trow} of {text_len} text rows of one block, {t:.1f} s on {threads} threads, "
            f"scaled by rows x 50 blocks; attention rows via the rectangular form of the reference loop")
    return ms_step, desc


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle.pyoracle import Ref
    kind = "reference" if Ref.available() else "port"
    cores = os.cpu_count() or 1
    vals = []
    desc = ""
    # a whole step would take about a day of CPU time: every "step" here is one bounded row sample of one block,
    # scaled to 50 blocks; two samples are taken whatever --steps asks for, and the line says so
    samples = max(1, min(args.steps, 2))
    for _ in range(samples):
        v, desc = cpu_block_sample(kind, cores, budget_s=20.0, grid=GRID_ULYSSES if big_workload(args) else GRID_1GPU)
        vals.append(v)
    value = float(np.median(vals))
    cfg = workload_config(1, big_workload(args))
    cfg["parallelism"] = f"{cores} host threads (the CPU path does not shard over GPUs; the same figure is reported at every N)"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": samples, "warmup": 0, "steps_asked": args.steps, "ms_per_step": value, "higher_is_better": False,
            "extrapolated": True,
            "extrapolation": "median of the samples, each scaled from its sampled query rows of ONE block to all rows x 50 blocks",
            "scaling": "strong" if big_workload(args) else "weak", "vs_baseline": None,
            "dtype": "int8 linears + f32 attention (CPU)", "data": "synthetic",
            "config": cfg,
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": desc},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    OUT.emit(json.dumps(line))


def big_workload(args):
    """The metric's workload is the 50,220-token step at every N (the same work on 1, 2, 4 or 8 GPUs, so that
    per-N values compare); `--workload step6144` selects the 6,144-token single-GPU step instead."""
    return args.workload != "step6144"


def workload_config(n_gpus, big):
    grid = GRID_ULYSSES if big else GRID_1GPU
    tokens = grid[0] * grid[1] * grid[2]
    return {"workload": ("50-block W4A8 DiT denoiser step, 864x480x121 frames (Ulysses sequence-parallel for N > 1)"
                         if big else "50-block W4A8 DiT denoiser step, 512x512x22 frames"),
            "tokens": tokens, "patch_grid": list(grid), "text_tokens": GEO["text"], "dim": GEO["dim"],
            "heads": GEO["heads"], "head_dim": GEO["head_dim"], "ffn": GEO["ffn"], "blocks": GEO["n_blocks"],
            "weights": "int4 group-128 f16 scales, decoded once to resident int8 + per-channel scale",
            "activations": "per-token absmax int8, bf16 residual stream", "timestep": 0.5,
            "parallelism": "single GPU" if n_gpus == 1 else f"ulysses{n_gpus}",
            "l2": "each step streams 3.4 GB of weights and >1 GB of activations, far above the 126 MB L2",
            "other_workload": "--workload step6144 times the 6,144-token single-GPU step" if big else
                              "default (no --workload) times the 50,220-token step"}


# -------------------------------------------------------------------------------------- GPU arm

def gpu_arm(args):
    import torch
    import h3c_b200
    from h3c_b200 import dit as D

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cuda = h3c_b200.Cuda(local)
    cuda.set_quiet(True)
    geo = D.DitGeometry(dim=GEO["dim"], heads=GEO["heads"], head_dim=GEO["head_dim"], ffn=GEO["ffn"],
                        n_blocks=GEO["n_blocks"], mod_rows=1, t_dim=256, kind=D.BLOCK_CROSS_GELU, stream_dtype=D.BF16)
    # same seed on every rank: replicated weights; host copies of the first two blocks' small tensors are kept for
    # the checks that follow the timed region
    dit, host_blocks = D.build_synthetic(cuda, geo, seed=0, keep_host=2)
    ulysses = big_workload(args)
    if world > 1 and not ulysses:
        raise SystemExit("--workload step6144 is a single-GPU workload")
    grid = GRID_ULYSSES if ulysses else GRID_1GPU
    seq_real, text_len = grid[0] * grid[1] * grid[2], GEO["text"]
    seq_pad, seq_local, first_row, real_rows = h3c_b200.ulysses_shard_rows(seq_real, world, rank)
    comm = None
    if world > 1:
        uid = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            uid.copy_(torch.frombuffer(bytearray(h3c_b200.UlyssesComm.unique_id()), dtype=torch.uint8))
        dist.broadcast(uid, 0)
        comm = h3c_b200.UlyssesComm(rank, world, bytes(uid.cpu().numpy().tobytes()), local)
        comm.set_compute(torch.cuda.current_stream())
        if h3c_b200.plugin_enabled("H3B_ULYSSES_DIRECT"):
            # peers' Q/K/V and attention-row buffers mapped into this rank: the epilogues store across NVLink.
            # If the mapping fails on any rank (no peer access), every rank falls back to the NCCL exchange.
            ok = torch.ones(1, dtype=torch.int32, device="cuda")
            try:
                comm.setup_direct(seq_local, geo.heads, geo.head_dim)
            except h3c_b200.H3Error as exc:
                print(f"rank {rank}: direct stores unavailable ({exc}); using the exchange", file=sys.stderr)
                ok.zero_()
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            comm.enable_direct(bool(ok.item()))
        dit.set_ulysses(comm)
    rows = seq_local if world > 1 else seq_real
    inv_freq = (1.0 / (10000.0 ** (np.arange(16) / 16.0))).astype(np.float32)
    # positions and RoPE tables come from the library's own host code; under sequence parallelism they
    # cover the padded gathered sequence (pad rows get angle 0)
    cos_h, sin_h = h3c_b200.video_rope_tables(inv_freq, text_len, grid, 1.0,
                                              pad_rows=(seq_pad - seq_real) if world > 1 else 0)
    rng = np.random.default_rng(1000 + rank)
    x_np = rng.normal(0, 1, (rows, geo.dim)).astype(np.float32)
    if world > 1:
        x_np[real_rows:] = 0.0   # pad rows of the last rank
    text_np = np.random.default_rng(7).normal(0, 1, (text_len, geo.dim)).astype(np.float32)   # replicated
    x_h = torch.from_numpy(x_np).pin_memory()
    text_h = torch.from_numpy(text_np).pin_memory()
    cos_p, sin_p = torch.from_numpy(cos_h).pin_memory(), torch.from_numpy(sin_h).pin_memory()
    # timestep t = 0.5: sinusoidal feature of width t_dim (synthetic stand-in for the embedding table)
    half = geo.t_dim // 2
    freqs = np.exp(-np.log(10000.0) * np.arange(half) / half)
    t_feat_h = torch.from_numpy(np.concatenate([np.cos(500.0 * freqs), np.sin(500.0 * freqs)]).astype(np.float32)).pin_memory()
    y_h = torch.empty((rows, geo.dim), dtype=torch.float32).pin_memory()
    x_d = x_h.cuda().to(torch.bfloat16)
    text_d = text_h.cuda().to(torch.bfloat16)
    cos_d, sin_d, t_d = cos_p.cuda(), sin_p.cuda(), t_feat_h.cuda()
    rmap_d = torch.zeros(rows, dtype=torch.int32, device="cuda")
    y_d = torch.empty_like(x_d)
    dit.reserve(rows, text_len)

    def step_resident():
        dit.project_modulation(t_d)
        if world > 1:
            dit.layers_forward_ulysses(x_d, seq_real, cos_d, sin_d, row_map=rmap_d, text=text_d, out=y_d)
        else:
            dit.layers_forward(x_d, cos_d, sin_d, row_map=rmap_d, text=text_d, out=y_d)

    if args.graph and world == 1:
        # The resident step with its block chain as one CUDA graph, captured and replayed by the C host
        # (h3b_dit_layers_forward_graph_dev): removes the host launch gaps of the ~800 launches of a step.
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        torch.cuda.set_stream(side)
        cuda.use_stream(side)            # capture needs a real stream
        eager_step = step_resident

        def step_resident():
            dit.project_modulation(t_d)
            dit.layers_forward_graph(x_d, cos_d, sin_d, row_map=rmap_d, text=text_d, out=y_d)

        step_resident()                  # eager pass + capture
        side.synchronize()
        graph_launches = dit.graph_nodes + geo.n_blocks   # nodes of one replay + the projection launches

    def step_e2e():
        if world > 1:
            dit.layers_forward_ulysses_f32(t_feat_h, x_h, seq_real, cos_p, sin_p, text=text_h, out=y_h)
        else:
            dit.layers_forward_f32(t_feat_h, x_h, cos_p, sin_p, text=text_h, out=y_h)

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(args.warmup):
        step_resident()
    sync_all()
    cuda.check()

    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    cuda.launch_count(reset=True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    e0.record()
    for _ in range(args.steps):
        step_resident()
    e1.record()
    sync_all()
    launches = cuda.launch_count(reset=True)
    if args.graph and world == 1:
        launches = graph_launches * args.steps
    ms_step = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    clocks = sampler.stop()
    cuda.check()
    if comm is not None:
        comm.check()

    prof = profile_classes(cuda, dit, eager_step if (args.graph and world == 1) else step_resident)
    sync_all()

    checks = {}
    if not args.skip_checks:
        if world > 1:
            checks["ulysses_check"] = ulysses_check(cuda, dit, geo, host_blocks, world, rank, seq_real, seq_pad, seq_local,
                                                    cos_d, sin_d, text_d, t_d, dist)
        if rank == 0:
            checks["parity_check"] = parity_check(cuda, dit, geo, host_blocks[0], grid, text_np, t_d)
        sync_all()

    e2e_ms = None
    if not args.skip_e2e:
        for _ in range(max(1, min(args.warmup, 2))):
            step_e2e()
        sync_all()
        t0 = time.perf_counter()
        e0.record()
        for _ in range(args.steps):
            step_e2e()
        e1.record()
        torch.cuda.synchronize()
        e2e_ms = max_over_ranks(max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3) / args.steps)
    tables = cos_p.numel() * 8
    h2d = x_h.numel() * 4 + text_h.numel() * 4 + tables + t_feat_h.numel() * 4
    d2h = y_h.numel() * 4

    if rank == 0:
        pk = peaks()
        # algorithmic work of this rank: its rows through every linear, heads/U heads of the full attention
        lin_f, _ = block_flops(rows, text_len, geo.dim, geo.ffn)
        attn_f = (4.0 * seq_real * seq_real * geo.dim) / world + 4.0 * rows * text_len * geo.dim
        # the rate this GPU sustains on about a second of back-to-back MMAs from a resident tile, measured now:
        # the int8 denominator (the measured-peaks file has none) and a second opinion on the bf16 one
        probe = {"int8": h3c_b200.tensor_pipe_rate(cuda, 0, 1000000), "bf16": h3c_b200.tensor_pipe_rate(cuda, 3, 1000000)}
        roof = roofline(prof, lin_f, attn_f, geo.n_blocks, pk, probe)
        if roof and roof.get("bound") == "tensor":
            traffic = traffic_per_launch(roof["kernel"], seq_real if world == 1 else None)
            if traffic:
                roof["traffic"], roof["traffic_note"] = traffic
        lin_all, attn_all = block_flops(seq_real, text_len, geo.dim, geo.ffn)
        if args.skip_cpu_baseline or world > 1:
            cpu = None
        else:
            kind = "reference" if ref_available() else "port"
            cpu_ms, cpu_desc = cpu_block_sample(kind, os.cpu_count() or 1, grid=grid)
            cpu = {"value": cpu_ms, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": kind, "sample": cpu_desc}
        cfg = workload_config(world, ulysses)
        if args.graph and world == 1:
            cfg["launch"] = "one CUDA graph replay per step"
        if comm is not None:
            cfg["exchange"] = ("direct stores into peer memory from the QKV and attention epilogues + 2 barriers per block"
                               if comm.direct else "NCCL send/recv all-to-all around self-attention")
        line = {"metric": METRIC, "value": ms_step, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": False,
                "scaling": "strong" if ulysses else "weak", "vs_baseline": None,
                "dtype": "int8 (linears, int32 accumulate) + bf16 (attention, f32 accumulate)", "data": "synthetic",
                "config": cfg,
                "e2e": {"value": e2e_ms, "unit": UNIT, "h2d_bytes_per_step": int(h2d) * world,
                        "d2h_bytes_per_step": int(d2h) * world},
                "gpu_launches": int(launches) * world, "clocks": clocks, "roofline": roof, "cpu_baseline": cpu,
                "step_tflops": (lin_all + attn_all) * geo.n_blocks / (ms_step * 1e-3) / 1e12, "kernel_classes": prof}
        line.update(checks)
        OUT.emit(json.dumps(line))
    sync_all()
    dit.close()
    if comm is not None:
        comm.close()
    cuda.close()
    if dist is not None:
        dist.destroy_process_group()


def nvfp4_arm(args):
    """`--weights nvfp4`: the 6,144-token step on the reference's own block (SwiGLU FFN, no cross-attention, f32
    residual stream, 256-wide ConvRot) with all four linears per block as NVFP4 weights, the path the reference
    takes through nvfp4_gemm_dispatch.  One GPU.  Roofline on the block-scaled GEMM."""
    import torch
    import h3c_b200
    from h3c_b200 import dit as D
    if int(os.environ.get("WORLD_SIZE", "1")) != 1 or args.gpus != 1:
        raise SystemExit("--weights nvfp4 is a single-GPU workload")
    torch.cuda.set_device(0)
    cuda = h3c_b200.Cuda(0)
    cuda.set_quiet(True)
    geo = D.DitGeometry(dim=GEO["dim"], heads=GEO["heads"], head_dim=GEO["head_dim"], ffn=GEO["ffn"],
                        n_blocks=GEO["n_blocks"], mod_rows=1, t_dim=256, kind=D.BLOCK_REFERENCE, stream_dtype=D.F32,
                        convrot_gs=256)
    dit = D.build_synthetic(cuda, geo, seed=0, nvfp4=True)
    grid = GRID_1GPU
    seq = grid[0] * grid[1] * grid[2]
    inv_freq = (1.0 / (10000.0 ** (np.arange(16) / 16.0))).astype(np.float32)
    cos_h, sin_h = h3c_b200.video_rope_tables(inv_freq, GEO["text"], grid, 1.0)
    x_h = torch.from_numpy(np.random.default_rng(1000).normal(0, 1, (seq, geo.dim)).astype(np.float32)).pin_memory()
    cos_p, sin_p = torch.from_numpy(cos_h).pin_memory(), torch.from_numpy(sin_h).pin_memory()
    half = geo.t_dim // 2
    freqs = np.exp(-np.log(10000.0) * np.arange(half) / half)
    t_feat_h = torch.from_numpy(np.concatenate([np.cos(500.0 * freqs), np.sin(500.0 * freqs)]).astype(np.float32)).pin_memory()
    y_h = torch.empty((seq, geo.dim), dtype=torch.float32).pin_memory()
    x_d, cos_d, sin_d, t_d = x_h.cuda(), cos_p.cuda(), sin_p.cuda(), t_feat_h.cuda()
    rmap_d = torch.zeros(seq, dtype=torch.int32, device="cuda")
    y_d = torch.empty_like(x_d)
    dit.reserve(seq, 0)

    def step_resident():
        dit.project_modulation(t_d)
        dit.layers_forward(x_d, cos_d, sin_d, row_map=rmap_d, out=y_d)

    def step_e2e():
        dit.layers_forward_f32(t_feat_h, x_h, cos_p, sin_p, out=y_h)

    for _ in range(args.warmup):
        step_resident()
    torch.cuda.synchronize()
    cuda.check()
    sampler = ClockSampler(0)
    sampler.start()
    time.sleep(0.3)
    cuda.launch_count(reset=True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step_resident()
    e1.record()
    torch.cuda.synchronize()
    launches = cuda.launch_count(reset=True)
    ms_step = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop()
    cuda.check()
    finite = bool(torch.isfinite(y_d).all().item())
    prof = profile_classes(cuda, dit, step_resident)
    if "gemm_i8" in prof:
        prof["gemm_fp4"] = prof.pop("gemm_i8")   # the GEMM class of this workload is the block-scaled NVFP4 kernel
    e2e_ms = None
    if not args.skip_e2e:
        step_e2e()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step_e2e()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    D_, F_ = geo.dim, geo.ffn
    lin_f = 2.0 * seq * (D_ * 3 * D_ + D_ * D_ + D_ * 2 * F_ + F_ * D_)
    attn_f = 4.0 * seq * seq * D_
    g = prof.get("gemm_fp4")
    roof = None
    if g:
        probe = h3c_b200.tensor_pipe_rate(cuda, 2, 1000000)
        achieved = lin_f * geo.n_blocks / (g["ms"] * 1e-3) / 1e12
        roof = {"bound": "tensor", "kernel": "gemm_fp4", "achieved": achieved, "peak": probe, "unit": "TFLOP/s",
                "frac": achieved / probe, "traffic": None,
                "peak_note": "NVFP4 block-scaled tcgen05.mma rate of this GPU over about a second of back-to-back MMAs from "
                             "a resident tile, measured in this run",
                "share_of_step": g["ms"] / sum(v["ms"] for v in prof.values())}
    line = {"metric": METRIC, "value": ms_step, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
            "dtype": "nvfp4 (linears, f32 accumulate) + bf16 (attention, f32 accumulate)", "data": "synthetic",
            "config": {"workload": "50 reference blocks (SwiGLU, no cross-attention), 6,144 tokens, every linear NVFP4",
                       "tokens": seq, "patch_grid": list(grid), "dim": D_, "heads": geo.heads, "head_dim": geo.head_dim,
                       "ffn": F_, "blocks": geo.n_blocks, "convrot": 256,
                       "weights": "NVFP4 (E2M1, UE4M3 scale per 16, f32 second-level scale)",
                       "activations": "ConvRot + NVFP4 per linear, f32 residual stream",
                       "l2": "each step streams 3.8 GB of weights and >1 GB of activations, far above the 126 MB L2"},
            "e2e": {"value": e2e_ms, "unit": UNIT, "h2d_bytes_per_step": int(x_h.numel() * 4 + cos_p.numel() * 8 + t_feat_h.numel() * 4),
                    "d2h_bytes_per_step": int(y_h.numel() * 4)},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roof, "cpu_baseline": None,
            "step_tflops": (lin_f + attn_f) * geo.n_blocks / (ms_step * 1e-3) / 1e12, "kernel_classes": prof,
            "output_finite": finite}
    OUT.emit(json.dumps(line))
    dit.close()
    cuda.close()


def full_input_rows(world, seq_real, seq_pad, dim):
    """The activations of the whole (padded) sequence as the ranks generate them: rank r seeds its own slice."""
    seq_local = seq_pad // world
    rows = seq_local if world > 1 else seq_real
    parts = []
    for r in range(world):
        x = np.random.default_rng(1000 + r).normal(0, 1, (rows, dim)).astype(np.float32)
        if world > 1:
            x[max(0, min(seq_local, seq_real - r * seq_local)):] = 0.0
        parts.append(x)
    return np.concatenate(parts)


def second_context(cuda, dit, geo, host_blocks, n_blocks):
    """A context over the first `n_blocks` blocks of `dit` (same weight objects, borrowed) with no communicator
    attached: the unsharded chain the sharded one is compared with."""
    from dataclasses import replace
    from h3c_b200 import dit as D
    geo2 = replace(geo, n_blocks=n_blocks)
    ctx = D.Dit(cuda, geo2)
    per_block = 7 if geo.kind == D.BLOCK_CROSS_GELU else 4
    for b in range(n_blocks):
        for which, w in enumerate(dit._weights[b * per_block:(b + 1) * per_block]):
            from h3c_b200.lib import call
            call("h3b_dit_set_linear", ctx.h, b, which, w.h)      # borrowed: `dit` keeps ownership
        h = host_blocks[b]
        ctx.set_block_aux(b, h["norm1"], h["norm2"], h["q_norm"], h["k_norm"], h.get("norm_c"))
        ctx.set_adaln(b, h["adaln_w"], h["adaln_b"])
    return ctx


def ulysses_check(cuda, dit, geo, host_blocks, world, rank, seq_real, seq_pad, seq_local, cos_d, sin_d, text_d, t_d, dist):
    """Sharding self-check at the real size: the first two blocks run sequence-parallel (the exchange the timed
    step used) and, on every rank, unsharded over the whole sequence; this rank's rows of both must agree bit for
    bit.  Returns the largest absolute difference over all ranks (0.0 when the sharded path is exact)."""
    import torch
    x_full = torch.from_numpy(full_input_rows(world, seq_real, seq_pad, geo.dim)).cuda().to(torch.bfloat16)
    mine = slice(rank * seq_local, (rank + 1) * seq_local)
    rmap = torch.zeros(seq_pad, dtype=torch.int32, device="cuda")
    dit.project_modulation(t_d)
    y_sharded = dit.layers_forward_ulysses(x_full[mine].contiguous(), seq_real, cos_d, sin_d, n=2, row_map=rmap[:seq_local],
                                           text=text_d)
    solo = second_context(cuda, dit, geo, host_blocks, 2)
    solo.project_modulation(t_d)
    y_full = solo.layers_forward(x_full[:seq_real].contiguous(), cos_d[:seq_real].contiguous(), sin_d[:seq_real].contiguous(),
                                 row_map=rmap[:seq_real], text=text_d)
    cuda.check()
    real = max(0, min(seq_local, seq_real - rank * seq_local))
    diff = (y_sharded[:real].float() - y_full[mine][:real].float()).abs().max() if real else torch.zeros((), device="cuda")
    d = diff.reshape(1).double()
    dist.all_reduce(d, op=dist.ReduceOp.MAX)
    solo.close_keep_weights()
    return float(d.item())


def parity_check(cuda, dit, geo, blk, grid, text_np, t_d, n_rows=8):
    """Output rows of block 0 of the REAL workload (whole sequence on this GPU) against the CPU checker.  The GPU
    runs the block; the checker recomputes `n_rows` of its output rows in f32 from the block's input: every
    linear (the resident int8 weights are downloaded), QK-norm + RoPE, self-attention of those rows against the
    keys and values of ALL tokens (taken from the GPU's own QKV projection, 16-bit), cross-attention, the FFN.
    Bound: 2e-2 relative L2, the figure stated for the f32 CPU block (the GPU path keeps a bf16 residual stream)."""
    import torch
    import h3c_b200
    from oracle.pyoracle import Oracle, Ref
    impl = Ref() if Ref.available() else Oracle()
    oracle = Oracle()
    seq = grid[0] * grid[1] * grid[2]
    heads, hd, dim = geo.heads, geo.head_dim, geo.dim
    x = torch.from_numpy(full_input_rows(1, seq, seq, dim)).cuda().to(torch.bfloat16)
    inv_freq = (1.0 / (10000.0 ** (np.arange(16) / 16.0))).astype(np.float32)
    cos_h, sin_h = h3c_b200.video_rope_tables(inv_freq, GEO["text"], grid)
    cos, sin = torch.from_numpy(cos_h).cuda(), torch.from_numpy(sin_h).cuda()
    text = torch.from_numpy(text_np).cuda().to(torch.bfloat16)
    rmap = torch.zeros(seq, dtype=torch.int32, device="cuda")
    solo = second_context(cuda, dit, geo, [blk], 1)
    solo.project_modulation(t_d)
    y = solo.block_forward(0, x, cos, sin, row_map=rmap, text=text)
    mod = solo.modulation(0).cpu().numpy()
    # keys and values of all tokens: the block's own first two launches, repeated through the operator interface
    w = {name: dit._weights[i] for i, name in enumerate(("qkv", "o", "up", "down", "cq", "ckv", "co"))}
    q8 = torch.empty((seq, dim), dtype=torch.int8, device="cuda")
    s8 = torch.empty(seq, dtype=torch.float32, device="cuda")
    cuda.norm(x, norm_w=torch.from_numpy(blk["norm1"]).cuda(), modulation=solo.modulation(0), row_map=rmap, slots=6,
              shift_slot=0, scale_slot=1, q=q8, scales=s8)
    _, k_all, v_all = cuda.gemm_i8_qkv_rope(w["qkv"], q8, s8, torch.from_numpy(blk["q_norm"]).cuda(),
                                            torch.from_numpy(blk["k_norm"]).cuda(), cos, sin, 48)
    cuda.check()
    rows = np.unique(np.concatenate([[0, 255, 256, seq - 1, (seq - 1) // 256 * 256],
                                     np.random.default_rng(5).integers(0, seq, n_rows)]))[:max(n_rows, 8)]
    idx = torch.from_numpy(rows).cuda()
    k_h, v_h = k_all.float().cpu().numpy(), v_all.float().cpu().numpy()
    W = {n_: (w_.download_int8(), w_.download_scales()) for n_, w_ in w.items()}
    zero = np.zeros(len(rows), np.uint32)

    def linear(a, name):
        q, s = impl.quantize_act_int8(a)
        return impl.gemm_i8_dequant(q, W[name][0], s, W[name][1])

    xr = x[idx].float().cpu().numpy()
    a = impl.adaln(xr, blk["norm1"], mod, zero, 6, 0, 1)
    q_r, _, _ = impl.qkv_rope(linear(a, "qkv"), blk["q_norm"], blk["k_norm"], cos_h[rows], sin_h[rows], heads, hd, 48)
    x1 = impl.gate(xr, linear(oracle.sdpa(q_r, k_h, v_h), "o"), mod, zero, 6, 2)
    cq = linear(impl.rms_norm(x1, blk["norm_c"]), "cq").reshape(len(rows), heads, hd)
    ckv = linear(text.float().cpu().numpy(), "ckv")
    ck = np.ascontiguousarray(ckv[:, :dim]).reshape(-1, heads, hd)
    cv = np.ascontiguousarray(ckv[:, dim:]).reshape(-1, heads, hd)
    x2 = x1 + linear(oracle.sdpa(cq, ck, cv), "co")
    up = linear(impl.adaln(x2, blk["norm2"], mod, zero, 6, 3, 4), "up")
    h = (0.5 * up * (1.0 + np.tanh(0.7978845608028654 * (up + 0.044715 * up ** 3)))).astype(np.float32)
    want = impl.gate(x2, linear(h, "down"), mod, zero, 6, 5)
    got = y[idx].float().cpu().numpy()
    rel = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    solo.close_keep_weights()
    return {"rows": int(len(rows)), "of_rows": int(seq), "rel_l2": rel, "bound": 2e-2, "ok": bool(rel < 2e-2),
            "checker": "reference CPU functions" if Ref.available() else "CPU restatement"}


def ref_available():
    from oracle.pyoracle import Ref
    return Ref.available()


def profile_classes(cuda, dit, step):
    """Runs one extra step with event pairs around every kernel launch (a library facility) and returns
    {class: {"launches": n, "ms": total}} for the classes gemm_i8 / attention / rows / other."""
    import ctypes as C
    from h3c_b200.lib import load
    lib = load()
    lib.h3b_cuda_profile_begin(cuda.h)
    step()
    ms = (C.c_double * 8)()
    cnt = (C.c_int * 8)()
    n = lib.h3b_cuda_profile_end(cuda.h, ms, cnt, 8)
    names = ["gemm_i8", "attention", "rows", "rope", "other"]
    return {names[i]: {"launches": int(cnt[i]), "ms": float(ms[i])} for i in range(min(n, len(names))) if cnt[i]}


def traffic_per_launch(kernel, tokens):
    """DRAM bytes per launch of the dominant kernel class, read from the table of ncu captures committed under
    profiles/ (rows `| class | tokens | MB per launch | ... |`); None when no capture covers this workload."""
    table = ROOT / "profiles" / "dram_traffic_per_launch.md"
    if tokens is None or not table.exists():
        return None
    for line in table.read_text().splitlines():
        cells = [c.strip() for c in line.strip().strip("|").split("|")]
        if len(cells) >= 4 and cells[0] == kernel and cells[1].replace(",", "") == str(tokens):
            try:
                return float(cells[2]) * 1e6, f"{cells[3]} (profiles/dram_traffic_per_launch.md)"
            except ValueError:
                return None
    return None


def roofline(prof, lin_flops_block, attn_flops_block, n_blocks, pk, probe):
    """Roofline entry for the kernel class with the largest share of the step."""
    if not prof:
        return None
    top = max(prof, key=lambda k: prof[k]["ms"])
    p = prof[top]
    per_launch_ms = p["ms"] / p["launches"]
    extra = {}
    if top == "gemm_i8":
        flops = lin_flops_block * n_blocks / p["launches"]
        # no int8 figure exists among the measured peaks: the denominator is the int8 MMA rate measured live
        peak = probe["int8"]
        note = "int8 tcgen05.mma rate of this GPU over about a second of back-to-back MMAs from a resident tile, measured in this run"
    elif top == "attention":
        flops = attn_flops_block * n_blocks / p["launches"]
        peak = pk["bf16_sustained"]
        note = f"{pk['src']} sustained bf16"
        extra = {"probe_peak": probe["bf16"], "probe_note": "bf16 128x128x16 tcgen05.mma rate measured in this run"}
    else:
        return {"bound": "hbm", "kernel": top, "achieved": None, "peak": pk["hbm"], "unit": "GB/s", "frac": None,
                "traffic": None, "share_of_step": p["ms"] / sum(v["ms"] for v in prof.values())}
    achieved = flops / (per_launch_ms * 1e-3) / 1e12
    out = {"bound": "tensor", "kernel": top, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
           "frac": achieved / peak, "traffic": None, "peak_note": note,
           "share_of_step": p["ms"] / sum(v["ms"] for v in prof.values())}
    if extra:
        out.update(extra, frac_of_probe=achieved / extra["probe_peak"])
    return out


# ------------------------------------------------------------------------- single kernels

def _time_kernel(fn, iters, warmup=3):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def kernel_arm(a):
    """One operator of the library on synthetic data, timed with CUDA events on the launching stream; prints
    achieved TFLOP/s or GB/s.  These are also the small, self-contained commands behind the ncu summaries
    under profiles/."""
    import torch
    import h3c_b200
    cuda = h3c_b200.Cuda(0)
    g = torch.Generator(device="cuda")
    g.manual_seed(0)
    out = {"kernel": a.kernel}
    if a.kernel == "gemm":
        w_i8 = np.random.default_rng(0).integers(-127, 128, (a.n, a.k), dtype=np.int8)
        w = cuda.weight_from_i8(w_i8, np.full(a.n, 1e-3, np.float32))
        x = torch.randint(-127, 128, (a.m, a.k), generator=g, device="cuda", dtype=torch.int8)
        s = torch.full((a.m,), 0.01, device="cuda")
        if a.epi == "qkv":   # QKV projection with QK-norm and RoPE in the epilogue (N = 3 * heads * 128)
            qn = torch.ones(128, device="cuda")
            cos = torch.rand((a.m, 64), generator=g, device="cuda")
            sin = torch.rand((a.m, 64), generator=g, device="cuda")
            ms = _time_kernel(lambda: cuda.gemm_i8_qkv_rope(w, x, s, qn, qn, cos, sin, 64), a.iters)
            out.update(m=a.m, n=a.n, k=a.k, epi=a.epi, ms=ms, tops=2.0 * a.m * a.n * a.k / ms / 1e9)
            OUT.emit(json.dumps(out))
            return
        kind = {"plain": h3c_b200.EPI_PLAIN, "gate": h3c_b200.EPI_GATE, "gelu": h3c_b200.EPI_GELU,
                "swiglu": h3c_b200.EPI_SWIGLU}[a.epi]
        n_out = a.n // 2 if a.epi == "swiglu" else a.n
        y = torch.empty((a.m, n_out), dtype=torch.bfloat16, device="cuda")
        res = torch.zeros_like(y) if a.epi == "gate" else None
        ms = _time_kernel(lambda: cuda.gemm_i8(w, x, s, kind=kind, residual=res, out=y), a.iters)
        out.update(m=a.m, n=a.n, k=a.k, epi=a.epi, ms=ms, tops=2.0 * a.m * a.n * a.k / ms / 1e9)
    elif a.kernel == "gemm_w4g":   # exact int4 group-128 product next to the resident-int8 form of the same weight
        rng = np.random.default_rng(0)
        packed = rng.integers(0, 256, (a.n, a.k // 2), dtype=np.uint8)
        scales = np.full((a.n, a.k // 128), np.float16(0.003)).view(np.uint16)
        x = torch.randint(-127, 128, (a.m, a.k), generator=g, device="cuda", dtype=torch.int8)
        s = torch.full((a.m,), 0.01, device="cuda")
        h = cuda.w4g_exact_weight(packed, scales)
        y = torch.empty((a.m, a.n), dtype=torch.bfloat16, device="cuda")
        from h3c_b200.lib import call as call_, ptr as ptr_
        ms = _time_kernel(lambda: call_("h3b_gemm_w4g_exact_dev", cuda.h, h, ptr_(x), ptr_(s), a.m, ptr_(y), 1), a.iters)
        w8 = cuda.weight_from_w4g(packed, scales, 128)
        ms8 = _time_kernel(lambda: cuda.gemm_i8(w8, x, s, kind=h3c_b200.EPI_PLAIN, out=y), a.iters)
        out.update(m=a.m, n=a.n, k=a.k, exact_ms=ms, exact_tops=2.0 * a.m * a.n * a.k / ms / 1e9, resident_int8_ms=ms8,
                   resident_int8_tops=2.0 * a.m * a.n * a.k / ms8 / 1e9)
        cuda.w4g_exact_weight_free(h)
    elif a.kernel == "peak":
        for kind, name in ((0, "int8"), (1, "bf16"), (2, "nvfp4"), (3, "bf16_n128_ss"), (4, "bf16_n128_ts"), (5, "nvfp4_n128")):
            out[name + "_burst_tops"] = h3c_b200.tensor_pipe_rate(cuda, kind, 20000)         # ~10 ms of MMAs: burst clocks
            out[name + "_sustained_tops"] = h3c_b200.tensor_pipe_rate(cuda, kind, 2000000)   # ~1 s: under the power limit
    elif a.kernel == "sides":   # patch embedding, final head and Euler update of a.m tokens (f32, hidden = a.n)
        lat = torch.randn((a.m, 96), generator=g, device="cuda")
        pw, pb = torch.randn((a.n, 96), generator=g, device="cuda"), torch.randn(a.n, generator=g, device="cuda")
        x = torch.randn((a.m, a.n), generator=g, device="cuda")
        nw, mod = torch.ones(a.n, device="cuda"), torch.zeros((2, a.n), device="cuda")
        fw, fb = torch.randn((96, a.n), generator=g, device="cuda"), torch.randn(96, generator=g, device="cuda")
        vel = torch.randn((a.m, 96), generator=g, device="cuda")
        out.update(m=a.m, hidden=a.n,
                   patch_embed_ms=_time_kernel(lambda: cuda.dense_f32(lat, pw, pb), a.iters),
                   final_head_ms=_time_kernel(lambda: cuda.final_head_f32(x, nw, mod, fw, fb), a.iters),
                   euler_ms=_time_kernel(lambda: cuda.euler_step_f32(lat, vel, 0.8, 0.7), a.iters))
    elif a.kernel == "gemm_fp4":
        x4 = torch.randint(0, 256, (a.m, a.k // 2), generator=g, device="cuda", dtype=torch.uint8)
        w4 = torch.randint(0, 256, (a.n, a.k // 2), generator=g, device="cuda", dtype=torch.uint8)
        sfb = lambda rows: int(h3c_b200.load().h3_cuda_nvfp4_sf_bytes(rows, a.k))
        sfx = torch.full((sfb(a.m),), 0x38, device="cuda", dtype=torch.uint8)
        sfw = torch.full((sfb(a.n),), 0x38, device="cuda", dtype=torch.uint8)
        ms = _time_kernel(lambda: cuda.gemm_fp4(w4, sfw, x4, sfx, out_dtype=torch.bfloat16, swiglu=a.epi == "swiglu"), a.iters)
        out.update(m=a.m, n=a.n, k=a.k, epi=a.epi, ms=ms, tflops=2.0 * a.m * a.n * a.k / ms / 1e9)
    elif a.kernel == "attn":
        lk = a.lk or a.lq
        dt = torch.float16 if a.f16 else torch.bfloat16
        q = torch.randn((a.lq, a.heads, 128), generator=g, device="cuda").to(dt)
        k = torch.randn((lk, a.heads, 128), generator=g, device="cuda").to(dt)
        v = torch.randn((lk, a.heads, 128), generator=g, device="cuda").to(dt)
        o = torch.empty((a.lq, a.heads * 128), dtype=dt, device="cuda")
        ms = _time_kernel(lambda: cuda.sdpa(q, k, v, out=o), a.iters)
        if a.check:   # relative L2 of the first rows against f64 softmax attention computed by torch on the GPU
            rows = min(a.lq, 512)
            s_ = torch.einsum("qhd,khd->hqk", q[:rows].double(), k.double()) * 128 ** -0.5
            want = torch.einsum("hqk,khd->qhd", torch.softmax(s_, dim=-1), v.double()).reshape(rows, -1)
            out["rel_l2"] = float((o[:rows].double() - want).norm() / want.norm())
        out.update(lq=a.lq, lk=lk, heads=a.heads, dtype="f16" if a.f16 else "bf16", ms=ms, tflops=4.0 * a.lq * lk * a.heads * 128 / ms / 1e9)
    elif a.kernel == "norm":
        x = torch.randn((a.m, a.k), generator=g, device="cuda").to(torch.bfloat16)
        q = torch.empty((a.m, a.k), dtype=torch.int8, device="cuda")
        s = torch.empty(a.m, dtype=torch.float32, device="cuda")
        if a.plain_quant:
            ms = _time_kernel(lambda: cuda.norm(x, identity=True, q=q, scales=s), a.iters)
        else:
            nw = torch.ones(a.k, device="cuda")
            mod = torch.zeros((1, 6, a.k), device="cuda")
            rm = torch.zeros(a.m, dtype=torch.int32, device="cuda")
            ms = _time_kernel(lambda: cuda.norm(x, norm_w=nw, modulation=mod, row_map=rm, slots=6, shift_slot=0, scale_slot=1,
                                         q=q, scales=s), a.iters)
        out.update(m=a.m, k=a.k, ms=ms, gbs=(a.m * a.k * 3 + a.m * 4) / ms / 1e6)
    else:
        qkv = torch.randn((a.m, 3 * a.heads * 128), generator=g, device="cuda").to(torch.bfloat16)
        qn = torch.ones(128, device="cuda")
        cos = torch.ones((a.m, 48), device="cuda")
        sin = torch.zeros((a.m, 48), device="cuda")
        ms = _time_kernel(lambda: cuda.qkv_rope(qkv, qn, qn, cos, sin, a.heads, 128, 48), a.iters)
        out.update(m=a.m, heads=a.heads, ms=ms, gbs=a.m * a.heads * 128 * 3 * 4 / ms / 1e6)
    cuda.check()
    OUT.emit(json.dumps(out))


class QuietStdout:
    """Keeps file descriptor 1 free of library chatter (NCCL prints its version banner there): everything
    written to stdout is sent to stderr until `emit` writes the one JSON line to the real stdout."""

    def __init__(self):
        sys.stdout.flush()
        self.real = os.dup(1)
        os.dup2(2, 1)

    def emit(self, text):
        sys.stdout.flush()
        os.write(self.real, (text + "\n").encode())


OUT = None


def main():
    global OUT
    OUT = QuietStdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="auto", choices=["auto", "ulysses", "step6144"],
                    help="auto / ulysses: the 50,220-token step at any N; step6144: the 6,144-token single-GPU step")
    ap.add_argument("--weights", default="w4a8", choices=["w4a8", "nvfp4"],
                    help="nvfp4: the 6,144-token step on the reference block with every linear NVFP4 (N = 1)")
    ap.add_argument("--graph", action="store_true", help="replay the resident step as one CUDA graph (N = 1)")
    ap.add_argument("--skip-cpu-baseline", action="store_true", help="omit the CPU sample (profiling runs)")
    ap.add_argument("--skip-e2e", action="store_true", help="omit the host-buffer measurement (profiling runs)")
    ap.add_argument("--skip-checks", action="store_true", help="omit the parity / sharding self-checks (profiling runs)")
    ap.add_argument("--kernel", default=None,
                    choices=["gemm", "gemm_fp4", "gemm_w4g", "attn", "norm", "rope", "peak", "sides"],
                    help="time ONE operator on synthetic data instead of the step (also the ncu capture commands)")
    ap.add_argument("--m", type=int, default=6144)
    ap.add_argument("--n", type=int, default=9216)
    ap.add_argument("--k", type=int, default=3072)
    ap.add_argument("--lq", type=int, default=6144)
    ap.add_argument("--lk", type=int, default=0)
    ap.add_argument("--heads", type=int, default=24)
    ap.add_argument("--epi", default="plain", choices=["plain", "gate", "gelu", "swiglu", "qkv"])
    ap.add_argument("--plain-quant", action="store_true")
    ap.add_argument("--f16", action="store_true", help="--kernel attn: f16 tensors instead of bf16")
    ap.add_argument("--check", action="store_true", help="--kernel attn: also report the error against f64 attention")
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    if args.kernel:
        kernel_arm(args)
    elif args.impl == "reference":
        reference_arm(args)
    elif args.weights == "nvfp4":
        nvfp4_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
