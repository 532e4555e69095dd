"""The linear that allocates nothing (h3b_gemm_i8_dequant_f32_w_act_dev_noalloc), for hosts that
cannot call cudaMalloc while they run -- device memory fully handed to resident weights, or no room
in the step loop for the device-wide synchronisation an allocation brings.  It must give exactly what
the allocating entry point gives, call after call: its scratch is one fixed area inside the library
that keeps the previous call's contents.  This file sorts last on purpose, so a run that stops at the
first failure has already exercised everything else."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def test_noalloc_linear_matches_allocating_linear_twice_in_a_row():
    import h3c_b200
    cuda = h3c_b200.Cuda(0)
    rng = np.random.default_rng(77)
    n, k = 384, 512
    w_i8 = rng.integers(-127, 128, (n, k), dtype=np.int8)
    s = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    w = cuda.weight_from_i8(w_i8, s)
    # second call is smaller and uses the rotation: stale codes of the first call stay in the area
    for call_no, (m, gs) in enumerate(((300, 0), (70, 256))):
        x = torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).cuda()
        want = cuda.gemm_i8_dequant_f32_w_act_dev(w, x, gs)
        # outputs preallocated: nothing below allocates on the device
        got = torch.empty((m, n), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        cuda.gemm_i8_dequant_f32_w_act_dev_noalloc(w, x, gs, out=got)
        cuda.check()
        if call_no > 0:  # the first call on a device maps the library's built-in area (documented set-up)
            assert torch.cuda.mem_get_info()[0] == free_before, "the no-allocation linear changed free device memory"
        assert torch.equal(got, want), f"m={m} gs={gs}: differs from the allocating entry point"
    # beyond the built-in area: a clear refusal, no fallback
    lib = h3c_b200.load()
    rows = int(lib.h3b_linear_noalloc_max_rows())
    big = torch.zeros((rows + 1, k), dtype=torch.float32, device="cuda")
    with pytest.raises(h3c_b200.H3Error, match="exceeds the built-in scratch"):
        cuda.gemm_i8_dequant_f32_w_act_dev_noalloc(w, big, 0)
    w.free()
    cuda.close()
