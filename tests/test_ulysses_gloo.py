"""Multi-rank host logic on CPU: two gloo ranks exchange packed QKV / attention chunks with
all_to_all and must reproduce the oracle's model of the reference exchange
(h3_ulysses_comm.cu:256-434); plus the row split the benchmark uses."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, seq_local, heads, hd, out_dir):
    import torch.distributed as dist
    from oracle.pyoracle import Oracle
    import ctypes as C
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    o = Oracle()
    hl = heads // world
    local = (np.arange(seq_local * 3 * heads * hd, dtype=np.float32) + 1 + rank * 100000).reshape(seq_local, 3, heads, hd)
    pack = np.empty_like(local)
    o.lib.ho_ulysses_pack_qkv(local.ctypes.data_as(C.c_void_p), pack.ctypes.data_as(C.c_void_p), C.c_size_t(seq_local),
                              C.c_size_t(heads), C.c_size_t(hd), C.c_int(world), C.c_size_t(4))
    send = torch.from_numpy(pack.reshape(-1))
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send)          # equal chunks: chunk p goes to rank p, lands as chunk `rank` there
    gathered = recv.numpy().reshape(world * seq_local, 3, hl, hd)   # received chunks already are the output layout
    # reverse direction with the Q slice
    att_in = np.ascontiguousarray(gathered[:, 0])
    send2 = torch.from_numpy(att_in.reshape(-1))
    recv2 = torch.empty_like(send2)
    dist.all_to_all_single(recv2, send2)
    back = np.empty((seq_local, heads, hd), np.float32)
    o.lib.ho_ulysses_unpack_attn(recv2.numpy().ctypes.data_as(C.c_void_p), back.ctypes.data_as(C.c_void_p),
                                 C.c_size_t(seq_local), C.c_size_t(heads), C.c_size_t(hd), C.c_int(world), C.c_size_t(4))
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), local=local, gathered=gathered, back=back)
    dist.destroy_process_group()


def test_two_rank_exchange_matches_oracle(tmp_path, oracle):
    import torch.multiprocessing as mp
    world, seq_local, heads, hd = 2, 6, 8, 4
    mp.spawn(_worker, args=(world, _free_port(), seq_local, heads, hd, str(tmp_path)), nprocs=world, join=True)
    res = [np.load(tmp_path / f"r{r}.npz") for r in range(world)]
    want = oracle.ulysses_a2a_qkv([r["local"] for r in res], heads, hd)
    for r in range(world):
        assert np.array_equal(res[r]["gathered"], want[r])
        assert np.array_equal(res[r]["back"], res[r]["local"][:, 0])   # every rank gets its own Q rows back, all heads


def test_row_split():
    from bench import shard_rows
    assert shard_rows(50220, 8, 0) == (50240, 6280, 0, 6280)
    assert shard_rows(50220, 8, 7) == (50240, 6280, 43960, 6260)     # the last rank holds the 20 pad rows
    assert shard_rows(50220, 2, 1) == (50240, 25120, 25120, 25100)
    assert shard_rows(15973, 2, 0)[0] == 16000                        # tests/test_h3_ulysses.c "cafe pad"
    assert shard_rows(6144, 1, 0) == (6144, 6144, 0, 6144)
    assert sum(shard_rows(50220, 4, r)[3] for r in range(4)) == 50220
