"""Two-GPU checks of the sequence-parallel path (skipped with fewer than two GPUs): the NCCL exchange is an
exact permutation (the reference's own 2-GPU test, tests/test_h3_ulysses_a2a.cu, uses integer fills and
max-abs == 0), and the Ulysses chain reproduces the single-GPU chain bit for bit on the real rows, both
through the NCCL exchange and through direct stores into the peers' memory."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    import h3c_b200
    from h3c_b200 import dit as D
    from h3c_b200 import ulysses_shard_rows as shard_rows
    from oracle.pyoracle import Oracle
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)   # plumbing only: distributes the NCCL id
    ids = [h3c_b200.UlyssesComm.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, 0)
    cuda = h3c_b200.Cuda(rank)
    comm = h3c_b200.UlyssesComm(rank, world, ids[0], rank)
    comm.set_compute(torch.cuda.current_stream())
    # ---- exact permutation, bf16 and f32 payloads
    seq_local, heads, hd = 32, 8, 128
    hl = heads // world
    result = {}
    for dtype in (torch.float32, torch.bfloat16):
        base = (torch.arange(seq_local * 3 * heads * hd, device="cuda") % 251 + rank * 256).to(dtype)
        local = base.view(seq_local, 3, heads, hd)
        out = torch.empty((world * seq_local, 3, hl, hd), dtype=dtype, device="cuda")
        comm.a2a_qkv(local, out, seq_local, heads, hd)
        att_in = out[:, 0].contiguous()
        back = torch.empty((seq_local, heads, hd), dtype=dtype, device="cuda")
        comm.a2a_attn_out(att_in, back, seq_local, heads, hd)
        torch.cuda.synchronize()
        result[f"local_{dtype}"] = local.float().cpu().numpy()
        result[f"gathered_{dtype}"] = out.float().cpu().numpy()
        result[f"back_{dtype}"] = back.float().cpu().numpy()
    # ---- chain: 2 blocks, 100 real tokens padded to 128, split over the two ranks
    geo = D.DitGeometry(dim=512, heads=4, head_dim=128, ffn=1024, n_blocks=2, mod_rows=1, t_dim=32,
                        kind=D.BLOCK_CROSS_GELU, stream_dtype=D.BF16)
    dit = D.build_synthetic(cuda, geo, seed=3)
    oracle = Oracle()
    grid, text_len = (4, 5, 5), 16
    seq_real = 100
    inv_freq = (1.0 / (10000.0 ** (np.arange(16) / 16.0))).astype(np.float32)
    pt, ph, pw = oracle.fill_video_pos(text_len, grid[0], 2 * grid[1], 2 * grid[2])
    cos, sin = oracle.rope_tables(inv_freq, pt[:seq_real], ph[:seq_real], pw[:seq_real], 1.0)
    seq_pad, sl, first, real = shard_rows(seq_real, world, rank)
    cos_full = np.concatenate([cos, np.ones((seq_pad - seq_real, 48), np.float32)])
    sin_full = np.concatenate([sin, np.zeros((seq_pad - seq_real, 48), np.float32)])
    rng = np.random.default_rng(5)
    x = rng.normal(0, 1, (seq_pad, geo.dim)).astype(np.float32)
    x[seq_real:] = 0
    text = rng.normal(0, 1, (text_len, geo.dim)).astype(np.float32)
    t_feat = torch.from_numpy(rng.normal(0, 1, geo.t_dim).astype(np.float32)).cuda()
    dev = lambda a, dt=None: (torch.from_numpy(np.ascontiguousarray(a)).cuda() if dt is None
                              else torch.from_numpy(np.ascontiguousarray(a)).cuda().to(dt))
    dit.project_modulation(t_feat)
    # single-GPU chain over the real rows (every rank computes it, identical weights)
    y_single = dit.layers_forward(dev(x[:seq_real], torch.bfloat16), dev(cos), dev(sin), text=dev(text, torch.bfloat16),
                                  row_map=torch.zeros(seq_real, dtype=torch.int32, device="cuda"))
    dit.set_ulysses(comm)
    dit.project_modulation(t_feat)
    y_local = dit.layers_forward_ulysses(dev(x[first:first + sl], torch.bfloat16), seq_real, dev(cos_full), dev(sin_full),
                                         text=dev(text, torch.bfloat16),
                                         row_map=torch.zeros(sl, dtype=torch.int32, device="cuda"))
    cuda.check()
    # the same chain with direct stores into peer memory instead of the NCCL exchange (collective set-up)
    comm.setup_direct(sl, geo.heads, geo.head_dim)
    y_direct = dit.layers_forward_ulysses(dev(x[first:first + sl], torch.bfloat16), seq_real, dev(cos_full), dev(sin_full),
                                          text=dev(text, torch.bfloat16),
                                          row_map=torch.zeros(sl, dtype=torch.int32, device="cuda"))
    cuda.check()
    y_direct2 = dit.layers_forward_ulysses(dev(x[first:first + sl], torch.bfloat16), seq_real, dev(cos_full), dev(sin_full),
                                           text=dev(text, torch.bfloat16),
                                           row_map=torch.zeros(sl, dtype=torch.int32, device="cuda"))
    cuda.check()
    comm.check()   # no barrier between the ranks gave up waiting
    result["y_single"] = y_single.float().cpu().numpy()
    result["y_local"] = y_local.float().cpu().numpy()
    result["y_direct"] = y_direct.float().cpu().numpy()
    result["y_direct2"] = y_direct2.float().cpu().numpy()
    result["first"], result["real"] = first, real
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), **result)
    dist.barrier()
    dit.close()
    comm.close()
    cuda.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_exchange_and_chain(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    res = [np.load(tmp_path / f"r{r}.npz") for r in range(world)]
    seq_local, heads = 32, 8
    hl = heads // world
    for dtype in ("torch.float32", "torch.bfloat16"):
        for r in range(world):
            for src in range(world):
                want = res[src][f"local_{dtype}"][:, :, r * hl:(r + 1) * hl]
                assert np.array_equal(res[r][f"gathered_{dtype}"][src * seq_local:(src + 1) * seq_local], want)
            assert np.array_equal(res[r][f"back_{dtype}"], res[r][f"local_{dtype}"][:, 0])
    for r in range(world):
        first, real = int(res[r]["first"]), int(res[r]["real"])
        assert np.array_equal(res[r]["y_local"][:real], res[r]["y_single"][first:first + real])
        assert np.array_equal(res[r]["y_direct"][:real], res[r]["y_single"][first:first + real])
        assert np.array_equal(res[r]["y_direct2"], res[r]["y_direct"])
