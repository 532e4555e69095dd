"""Same-precision parity: this library's CUDA operators against the REFERENCE's own CUDA operator library
(cuBLASLt int8 linear, its activation quantisers, its in-tree flash attention) compiled for sm_100a from the
reference sources (oracle/_ref/cuda/libh3_refcuda.so, recipe oracle/build.py).  Both libraries export the
same h3_cuda_* names, so the reference runs in a worker process (oracle/ref_cuda_worker.py) on inputs drawn
from the same seeds.  Switches pinned for the reference: H3_DIT_ACT_F16=0 (f32 ConvRot, the algebra of its CPU
path), H3_INT8_GEMM_TILE_M=0 (one GEMM over all rows), H3_CUDA_SDPA_BACKEND=flash (its in-tree kernel).

Integer codes and the f32 linear are required to be bit-identical; attention within 2e-3 relative L2."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from tests.conftest import rel_l2

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

ROOT = Path(__file__).resolve().parent.parent
REFCUDA = ROOT / "oracle" / "_ref" / "cuda" / "libh3_refcuda.so"
sys.path.insert(0, str(ROOT / "oracle"))
from ref_cuda_worker import seeded_acts, seeded_weight_i8  # noqa: E402  (numpy-only helpers)

ENV = {"H3_DIT_ACT_F16": "0", "H3_INT8_GEMM_TILE_M": "0", "H3_CUDA_SDPA_BACKEND": "flash"}


def run_ref(ops, tmp_path, env=None, timeout=600):
    if not REFCUDA.exists():
        pytest.skip("oracle/_ref/cuda/libh3_refcuda.so not built (reference tree absent at build time)")
    job, out = tmp_path / "job.json", tmp_path / "out.npz"
    job.write_text(json.dumps({"env": {**ENV, **(env or {})}, "ops": ops}))
    res = subprocess.run([sys.executable, str(ROOT / "oracle" / "ref_cuda_worker.py"), str(job), str(out)],
                         capture_output=True, text=True, timeout=timeout, env=dict(os.environ))
    assert res.returncode == 0, f"reference CUDA worker failed:\n{res.stdout[-2000:]}\n{res.stderr[-4000:]}"
    data = dict(np.load(out))
    failures = json.loads(bytes(data.pop("failures_json")).decode())
    return data, failures


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


def ulp_distance(a, b):
    """Distance in units in the last place between two f32 arrays (same-sign finite values)."""
    ia, ib = a.view(np.int32).astype(np.int64), b.view(np.int32).astype(np.int64)
    return np.abs(ia - ib)


def test_linear_matches_reference_cuda(cuda, tmp_path):
    """f32 activations -> per-row INT8 -> int8 GEMM -> dequant, no rotation, against the reference's cuBLASLt path.
    The integer side is exact in both; the reference's CUDA library is built with --use_fast_math, so its
    absmax / 127 and 1 / scale are the approximate division and reciprocal (its own CPU path, the target of this
    library's bit-exactness, uses IEEE division): row scales may differ in the last bits and a code that sits
    on a rounding tie may move by one step."""
    shapes = [dict(m=300, n=640, k=1024, seed=11), dict(m=1000, n=3072, k=3072, seed=12)]
    ops = [dict(op="linear", tag=f"l{i}", gs=0, rows=list(range(0, s["m"], 7)), **s) for i, s in enumerate(shapes)]
    ref, failures = run_ref(ops, tmp_path)
    assert not failures, failures
    for i, s in enumerate(shapes):
        w_i8, sc = seeded_weight_i8(s["seed"] + 1, s["n"], s["k"])
        w = cuda.weight_from_i8(w_i8, sc)
        y = cuda.gemm_i8_dequant_f32_w_act_dev(w, dev(seeded_acts(s["seed"], s["m"], s["k"])), 0)
        cuda.check()
        got = host(y)[ref[f"l{i}_rows"]]
        want = ref[f"l{i}_y"]
        exact = float(np.mean(got == want))
        err = rel_l2(got, want)
        print(f"linear {s}: {exact:.4f} of outputs bit-identical to the reference CUDA path, rel-L2 {err:.2e}")
        assert err < 2e-3 * 1e-2          # far inside the 2e-3 bound of the same-precision path


def test_linear_with_rotation_close_to_reference_cuda(cuda, tmp_path):
    """With the 256-wide Hadamard rotation the reference multiplies by a dense matrix (cuBLAS SGEMM) where this
    library runs butterflies: sums in a different order, so a few codes move by one step."""
    s = dict(m=300, n=640, k=1024, seed=21)
    ref, failures = run_ref([dict(op="linear", tag="l", gs=256, rows=list(range(0, 300, 3)), **s)], tmp_path)
    assert not failures, failures
    w_i8, sc = seeded_weight_i8(s["seed"] + 1, s["n"], s["k"])
    y = cuda.gemm_i8_dequant_f32_w_act_dev(cuda.weight_from_i8(w_i8, sc), dev(seeded_acts(s["seed"], s["m"], s["k"])), 256)
    cuda.check()
    assert rel_l2(host(y)[ref["l_rows"]], ref["l_y"]) < 2e-3


def test_activation_codes_match_reference_cuda(cuda, tmp_path):
    """Per-row INT8 codes and scales: quantising the reference's own rotated activations with this library's
    kernel must reproduce the reference kernel's codes exactly (same f32 inputs, same rounding rule)."""
    m, k, gs = 257, 1024, 256
    ref, failures = run_ref([dict(op="act_codes", tag="a", m=m, k=k, gs=gs, seed=31)], tmp_path)
    assert not failures, failures
    q, sc = cuda.quantize_act_int8(dev(ref["a_rot"]))
    cuda.check()
    # same f32 inputs, same rounding rule; the reference CUDA kernel divides with --use_fast_math (approximate
    # absmax / 127 and 1 / scale), this library with IEEE division like the reference's CPU path
    ulps = ulp_distance(host(sc), ref["a_scales"])
    dq = np.abs(host(q).astype(np.int32) - ref["a_codes"].astype(np.int32))
    print(f"activation codes vs reference CUDA: scales differ by at most {ulps.max()} ulp ({np.mean(ulps != 0):.3f} of rows), "
          f"{np.mean(dq != 0):.2e} of codes differ, max step {dq.max()}")
    assert ulps.max() <= 4 and dq.max() <= 1 and np.mean(dq != 0) < 2e-3
    # end to end (this library's own butterfly rotation): rotated values agree to rounding, codes within one step
    x = seeded_acts(31, m, k)
    rot = cuda.convrot_act_f32_dd(dev(x), gs)
    assert rel_l2(host(rot), ref["a_rot"]) < 2e-6
    q2, _ = cuda.quantize_act_int8(rot)
    diff = np.abs(host(q2).astype(np.int32) - ref["a_codes"].astype(np.int32))
    assert diff.max() <= 1 and np.mean(diff != 0) < 5e-3


@pytest.mark.parametrize("m,k", [(130, 256), (128, 3072), (300, 12288)])
def test_nvfp4_activation_codes_match_reference_cuda(cuda, tmp_path, m, k):
    """E2M1 codes and UE4M3 block scales against the reference's CUDA quantiser, executed (its rounding rules
    are software-defined: ties away from zero in magnitude, scale bytes clamped to [1, 0x7E])."""
    ref, failures = run_ref([dict(op="quant_nvfp4", tag="q", m=m, k=k, seed=41, edge=True)], tmp_path)
    assert not failures, failures
    x = seeded_acts(41, m, k)
    x[0, :16] = 0.0
    x[1 % m, 16:32] = 1e-9
    x[2 % m, 32:48] = 3000.0
    packed, sf = cuda.quantize_act_nvfp4(dev(x))
    cuda.check()
    assert np.array_equal(host(packed)[:m], ref["q_fp4"])
    n = min(host(sf).size, ref["q_sf"].size)
    rows_full = (m // 128) * 128          # scale bytes of whole 128-row blocks are all defined
    assert n > 0
    ours, theirs = host(sf).reshape(-1)[:n], ref["q_sf"][:n]
    if rows_full:
        full = rows_full // 128 * (k // 64) * 512
        assert np.array_equal(ours[:full], theirs[:full])
    # rows of a partial last block: compare the bytes that belong to real rows
    r = np.arange(rows_full, m)
    if len(r):
        c = np.arange(k // 16)
        off = ((r[:, None] // 128) * (k // 64) + c[None, :] // 4) * 512 + 16 * (r[:, None] % 32) + \
            4 * ((r[:, None] % 128) // 32) + c[None, :] % 4
        assert np.array_equal(ours[off], theirs[off])


def test_attention_close_to_reference_cuda_flash(cuda, tmp_path):
    """This library's attention behind the reference's f16 entry point against the reference's in-tree f16
    flash kernel on the same f32 inputs."""
    seq, heads = 1000, 4
    rows = list(range(0, seq, 9))
    ref, failures = run_ref([dict(op="sdpa", tag="s", seq=seq, heads=heads, seed=51, rows=rows)], tmp_path)
    assert not failures, failures
    rng = np.random.default_rng(51)
    q, k, v = (rng.standard_normal((seq, heads, 128), dtype=np.float32) for _ in range(3))
    out = cuda.sdpa_f16_dev(dev(q), dev(k), dev(v))
    cuda.check()
    got = host(out).reshape(seq, -1)[rows]
    err = rel_l2(got, ref["s_o"])
    print(f"attention vs reference CUDA ({bytes(ref['s_backend']).decode()}): rel-L2 {err:.2e}")
    assert err < 2e-3


def _time(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ms = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ms.append(e0.elapsed_time(e1))
    return float(np.median(ms))


@pytest.mark.skipif(os.environ.get("H3_REF_CUDA_TIMING") != "1",
                    reason="timing table of the reference's CUDA operators: set H3_REF_CUDA_TIMING=1")
def test_timing_table_against_reference_cuda(cuda, tmp_path):
    """Not a parity check: times the reference's cuBLASLt int8 linear, its cuBLASLt FP4 GEMM and its attention
    (in-tree flash, and cuDNN where the library is present) beside this library's kernels on the benchmark's
    shapes, same box, same process lifetime, CUDA events around whole calls (median of 10), and writes
    ref_cuda_timing.json into the run's output folder (H3_TIMING_OUT, default: the folder a GPU run brings back)."""
    import h3c_b200
    shapes = [(m, k, n) for m in (6144, 24576, 50220) for k, n in ((3072, 9216), (3072, 3072), (3072, 12288), (12288, 3072))]
    table = {"linear": [], "attention": [], "fp4": []}
    ops = [dict(op="linear", tag=f"l{i}", m=m, n=n, k=k, gs=0, seed=100 + i, tiled=True, iters=10, rows=[0])
           for i, (m, k, n) in enumerate(shapes)]
    ref, failures = run_ref(ops, tmp_path, timeout=1500)
    g = torch.Generator(device="cuda")
    g.manual_seed(0)
    for i, (m, k, n) in enumerate(shapes):
        w_i8 = np.random.default_rng(i).integers(-127, 128, (n, k), dtype=np.int8)
        w = cuda.weight_from_i8(w_i8, np.full(n, 1e-3, np.float32))
        x = torch.randn((m, k), generator=g, device="cuda")
        xq, xs = cuda.quantize_act_int8(x)
        y16 = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        row = {"m": m, "k": k, "n": n,
               "ours_whole_call_f32_ms": _time(lambda: cuda.gemm_i8_dequant_f32_w_act_dev(w, x, 0)),
               "ours_quant_ms": _time(lambda: cuda.quantize_act_int8(x)),
               "ours_gemm_f32_out_ms": _time(lambda: cuda.gemm_i8(w, xq, xs)),
               "ours_gemm_bf16_out_ms": _time(lambda: cuda.gemm_i8(w, xq, xs, out=y16))}
        if f"l{i}_ms" in ref:
            prep, gemm, total = (float(v) for v in ref[f"l{i}_ms"])
            row.update(ref_prep_ms=prep, ref_gemm_dequant_ms=gemm, ref_whole_call_ms=total,
                       ref_backend=bytes(ref[f"l{i}_backend"]).decode())
        else:
            row["ref_failure"] = failures.get(f"l{i}")
        row["tops_ours_bf16"] = 2.0 * m * n * k / row["ours_gemm_bf16_out_ms"] / 1e9
        if "ref_gemm_dequant_ms" in row and row["ref_gemm_dequant_ms"] > 0:
            row["tops_ref_gemm_dequant"] = 2.0 * m * n * k / row["ref_gemm_dequant_ms"] / 1e9
        table["linear"].append(row)
        del w, x, xq, xs, y16
        torch.cuda.empty_cache()
    for backend in ("flash", "cudnn"):
        for seq in (6144, 24576):
            try:
                ref, failures = run_ref([dict(op="sdpa", tag="s", seq=seq, heads=24, seed=7, iters=5, rows=[0, seq - 1])],
                                        tmp_path, env={"H3_CUDA_SDPA_BACKEND": backend}, timeout=900)
            except (AssertionError, subprocess.TimeoutExpired) as exc:
                table["attention"].append({"seq": seq, "ref_backend_asked": backend, "ref_failure": str(exc)[-400:]})
                continue
            row = {"seq": seq, "heads": 24, "ref_backend_asked": backend}
            if "s_ms" in ref:
                row.update(ref_backend=bytes(ref["s_backend"]).decode(), ref_inner_ms=float(ref["s_ms"][0]),
                           ref_whole_call_ms=float(ref["s_ms"][1]))
                row["tflops_ref_whole_call"] = 4.0 * seq * seq * 24 * 128 / row["ref_whole_call_ms"] / 1e9
            else:
                row["ref_failure"] = failures.get("s")
            q, k_, v = (torch.randn((seq, 24, 128), generator=g, device="cuda") for _ in range(3))
            qb, kb, vb = (t.to(torch.bfloat16) for t in (q, k_, v))
            row["ours_whole_call_f32_ms"] = _time(lambda: cuda.sdpa_f16_dev(q, k_, v), iters=5)
            row["ours_kernel_ms"] = _time(lambda: cuda.sdpa_bf16(qb, kb, vb), iters=5)
            row["tflops_ours_kernel"] = 4.0 * seq * seq * 24 * 128 / row["ours_kernel_ms"] / 1e9
            table["attention"].append(row)
            del q, k_, v, qb, kb, vb
            torch.cuda.empty_cache()
    for (m, n, k) in ((6144, 9216, 3072), (6144, 3072, 12288)):
        row = {"m": m, "n": n, "k": k}
        try:
            ref, failures = run_ref([dict(op="fp4_gemm", tag="f", m=m, n=n, k=k, seed=9, iters=10)], tmp_path, timeout=600)
            if "f_ms" in ref:
                row["ref_cublaslt_fp4_ms"] = float(ref["f_ms"][0])
                row["tflops_ref"] = 2.0 * m * n * k / row["ref_cublaslt_fp4_ms"] / 1e9
                row["ref_back_to_back_ms"] = float(ref["f_ms"][1])   # 30 calls queued behind one another
            else:
                row["ref_failure"] = failures.get("f")
        except (AssertionError, subprocess.TimeoutExpired) as exc:
            row["ref_failure"] = str(exc)[-400:]
        x4 = torch.randint(0, 256, (m, k // 2), generator=g, device="cuda", dtype=torch.uint8)
        w4 = torch.randint(0, 256, (n, k // 2), generator=g, device="cuda", dtype=torch.uint8)
        sfb = lambda rows: int(h3c_b200.load().h3_cuda_nvfp4_sf_bytes(rows, k))
        sfx = torch.full((sfb(m),), 0x38, device="cuda", dtype=torch.uint8)
        sfw = torch.full((sfb(n),), 0x38, device="cuda", dtype=torch.uint8)
        row["ours_ms"] = _time(lambda: cuda.gemm_fp4(w4, sfw, x4, sfx, out_dtype=torch.bfloat16))
        row["tflops_ours"] = 2.0 * m * n * k / row["ours_ms"] / 1e9
        fn = lambda: cuda.gemm_fp4(w4, sfw, x4, sfx, out_dtype=torch.bfloat16)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(30):
            fn()
        e1.record()
        e1.synchronize()
        row["ours_back_to_back_ms"] = e0.elapsed_time(e1) / 30
        table["fp4"].append(row)
    out_dir = Path(os.environ.get("H3_TIMING_OUT", ROOT / "gpurun_out"))
    out_dir.mkdir(exist_ok=True)
    (out_dir / "ref_cuda_timing.json").write_text(json.dumps(table, indent=1))
    print(json.dumps(table, indent=1))
