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
    from h3c_b200 import ulysses_shard_rows as shard_rows
    assert shard_rows(50220, 8, 0) == (50240, 6280, 0, 6280)
    assert shard_rows(50220, 8, 7) == (50240, 6280, 43960, 6260)     # the last rank holds the 20 pad rows
    assert shard_rows(50220, 2, 1) == (50240, 25120, 25120, 25100)
    assert shard_rows(15973, 2, 0)[0] == 16000                        # tests/test_h3_ulysses.c "cafe pad"
    assert shard_rows(6144, 1, 0) == (6144, 6144, 0, 6144)
    assert sum(shard_rows(50220, 4, r)[3] for r in range(4)) == 50220


# ---- set-up protocol of the exchange-free form: every rank must reach both collectives and take the same
# decision, whichever local step failed on whichever rank (stand-in steps over gloo; the library's own steps do
# the same with CUDA allocations, IPC handles and NCCL)

def _protocol_worker(rank, world, port, fail_rank, fail_step, out_dir):
    import ctypes as C
    import torch.distributed as dist
    import h3c_b200
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    log = []
    PREP = C.CFUNCTYPE(C.c_int, C.c_void_p)
    GATHER = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int)
    AGREE = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.POINTER(C.c_int))
    ROLLBACK = C.CFUNCTYPE(None, C.c_void_p)

    def prepare(_):
        log.append("prepare")
        return 0 if (rank == fail_rank and fail_step == "prepare") else 1

    def gather(_, have):
        log.append(f"gather:{have}")
        mine = torch.tensor([have], dtype=torch.int32)
        got = [torch.zeros(1, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(got, mine)                      # a rank without a handle still takes part
        return 0 if (rank == fail_rank and fail_step == "gather") else 1

    def map_peers(_):
        log.append("map")
        return 0 if (rank == fail_rank and fail_step == "map") else 1

    def agree(_, ok, all_ok):
        log.append(f"agree:{ok}")
        t = torch.tensor([ok], dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        all_ok[0] = int(t.item())
        return 1

    def rollback(_):
        log.append("rollback")

    class Steps(C.Structure):
        _fields_ = [("ctx", C.c_void_p), ("prepare", PREP), ("gather", GATHER), ("map_peers", PREP), ("agree", AGREE),
                    ("rollback", ROLLBACK)]

    steps = Steps(None, PREP(prepare), GATHER(gather), PREP(map_peers), AGREE(agree), ROLLBACK(rollback))
    rc = h3c_b200.load().h3b_ulysses_setup_protocol(C.addressof(steps))
    np.savez(os.path.join(out_dir, f"p{rank}.npz"), rc=rc, log=np.array(log))
    dist.destroy_process_group()


@pytest.mark.parametrize("fail_step", [None, "prepare", "gather", "map"])
def test_setup_protocol_is_collective_under_local_failures(tmp_path, fail_step):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_protocol_worker, args=(world, _free_port(), 1, fail_step, str(tmp_path)), nprocs=world, join=True)   # no hang
    res = [np.load(tmp_path / f"p{r}.npz") for r in range(world)]
    logs = [list(r["log"]) for r in res]
    assert [int(r["rc"]) for r in res] == ([1, 1] if fail_step is None else [0, 0])        # the same decision everywhere
    for log in logs:
        assert sum(x.startswith("gather") for x in log) == 1 and sum(x.startswith("agree") for x in log) == 1
        assert ("rollback" in log) == (fail_step is not None)                                 # everyone rolls back, or nobody
    if fail_step in ("prepare", "gather"):
        assert "map" not in logs[1] and "map" in logs[0]     # the failing rank skips the mapping, its peer finds out at `agree`
    if fail_step == "prepare":
        assert logs[1][1] == "gather:0"
