"""The native reader of the safetensors container (h3b_ckpt_*): header parsing, tensor views, and the malformed files
it must refuse.  No GPU: the C-ABI library is loaded, no compute call is made."""
import ctypes as C
import json
import struct

import numpy as np
import pytest

ERR = 512


class Tensor(C.Structure):   # h3b_ckpt_tensor (include/h3_b200.h)
    _fields_ = [("name", C.c_char_p), ("dtype", C.c_char * 8), ("rank", C.c_int), ("shape", C.c_size_t * 4),
                ("data", C.c_void_p), ("bytes", C.c_size_t)]


def write_safetensors(path, tensors, metadata=None, pad_to=8):
    dt = {np.dtype(np.int8): "I8", np.dtype(np.float32): "F32", np.dtype(np.uint8): "U8", np.dtype(np.float16): "F16"}
    header, offset = {}, 0
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, a in tensors.items():
        header[name] = {"dtype": dt[a.dtype], "shape": list(a.shape), "data_offsets": [offset, offset + a.nbytes]}
        offset += a.nbytes
    blob = json.dumps(header).encode()            # default separators: spaces after ':' and ','
    blob += b" " * (-len(blob) % pad_to)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for a in tensors.values():
            f.write(np.ascontiguousarray(a).tobytes())


@pytest.fixture(scope="module")
def lib():
    import h3c_b200
    return h3c_b200.load()


def open_ckpt(lib, path):
    err = C.create_string_buffer(ERR)
    h = lib.h3b_ckpt_open(str(path).encode(), err, ERR)
    return h, err.value.decode()


def test_reads_back_every_tensor(lib, tmp_path):
    rng = np.random.default_rng(0)
    tensors = {"blocks.0.attn.qkv_proj.weight": rng.integers(-127, 128, (24, 16), dtype=np.int8),
               "blocks.0.attn.qkv_proj.weight_scale": rng.uniform(1e-4, 1e-3, (24, 1)).astype(np.float32),
               'odd "name" \\ with escapes': rng.normal(0, 1, 7).astype(np.float32),
               "scalar": np.float32(3.5).reshape(()),
               "half": rng.normal(0, 1, (2, 3, 4, 5)).astype(np.float16),
               "empty": np.zeros((0, 4), np.float32)}
    path = tmp_path / "t.safetensors"
    write_safetensors(path, tensors, metadata={"format": "pt", "note": "nested {braces} [and] \"quotes\""})
    h, err = open_ckpt(lib, path)
    assert h, err
    assert lib.h3b_ckpt_count(h) == len(tensors)
    seen = set()
    for i in range(len(tensors)):
        t = Tensor()
        assert lib.h3b_ckpt_get(h, i, C.byref(t)) == 1
        name = t.name.decode()
        a = tensors[name]
        seen.add(name)
        assert t.rank == a.ndim and tuple(t.shape[:t.rank]) == a.shape and t.bytes == a.nbytes
        assert C.string_at(t.data, t.bytes) == a.tobytes()
    assert seen == set(tensors)
    t = Tensor()
    assert lib.h3b_ckpt_find(h, b"half", C.byref(t)) == 1 and t.dtype == b"F16" and t.rank == 4
    assert lib.h3b_ckpt_find(h, b"no such tensor", C.byref(t)) == 0
    assert lib.h3b_ckpt_get(h, len(tensors), C.byref(t)) == 0
    lib.h3b_ckpt_close(h)


def test_empty_header_and_compact_separators(lib, tmp_path):
    path = tmp_path / "e.safetensors"
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", 2) + b"{}")
    h, err = open_ckpt(lib, path)
    assert h, err
    assert lib.h3b_ckpt_count(h) == 0
    lib.h3b_ckpt_close(h)
    a = np.arange(6, dtype=np.float32).reshape(2, 3)
    blob = json.dumps({"a": {"dtype": "F32", "shape": [2, 3], "data_offsets": [0, 24]}}, separators=(",", ":")).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)) + blob + a.tobytes())
    h, err = open_ckpt(lib, path)
    assert h, err
    t = Tensor()
    assert lib.h3b_ckpt_find(h, b"a", C.byref(t)) == 1 and C.string_at(t.data, 24) == a.tobytes()
    lib.h3b_ckpt_close(h)


@pytest.mark.parametrize("case", ["missing", "short", "header_too_long", "offsets_past_end", "size_mismatch", "truncated_json",
                                  "rank5", "no_offsets"])
def test_refuses_malformed_files(lib, tmp_path, case):
    path = tmp_path / "bad.safetensors"
    a = np.arange(8, dtype=np.float32)

    def put(header_bytes, data=b"", claim=None):
        with open(path, "wb") as f:
            f.write(struct.pack("<Q", len(header_bytes) if claim is None else claim) + header_bytes + data)

    entry = lambda **kw: json.dumps({"a": dict({"dtype": "F32", "shape": [8], "data_offsets": [0, 32]}, **kw)}).encode()
    if case == "missing":
        pass
    elif case == "short":
        path.write_bytes(b"\x01\x02\x03")
    elif case == "header_too_long":
        put(entry(), a.tobytes(), claim=10 ** 9)
    elif case == "offsets_past_end":
        put(entry(data_offsets=[0, 64], shape=[16]), a.tobytes())
    elif case == "size_mismatch":
        put(entry(shape=[7]), a.tobytes())
    elif case == "truncated_json":
        put(entry()[:-5], a.tobytes())
    elif case == "rank5":
        put(entry(shape=[1, 1, 1, 1, 8]), a.tobytes())
    elif case == "no_offsets":
        put(json.dumps({"a": {"dtype": "F32", "shape": [8]}}).encode(), a.tobytes())
    h, err = open_ckpt(lib, path)
    assert not h and err, case
