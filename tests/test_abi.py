"""CPU-only checks of the C-ABI library: it loads, and it exports every symbol include/h3_b200.h
declares and the Python binding uses (no compute calls here)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib_path():
    from h3c_b200 import build
    return build.build()


def declared_in_header():
    text = (ROOT / "include" / "h3_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(h3_cuda_\w+|h3b_\w+|h3_ulysses_\w+|h3_dit_\w+|h3_nvfp4_\w+|h3_cutlass_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib_path):
    lib = ctypes.CDLL(str(lib_path))
    names = declared_in_header()
    assert len(names) > 40
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in include/h3_b200.h but not exported: {missing}"


def test_python_binding_matches_header(lib_path):
    from h3c_b200 import lib as l
    hdr = set(declared_in_header())
    unknown = [n for n in l.declared_symbols() if n not in hdr]
    assert not unknown, f"bound in h3c_b200/lib.py but not declared in the header: {unknown}"


def test_create_fails_loudly_without_gpu(lib_path):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import h3c_b200
    with pytest.raises(h3c_b200.H3Error):
        h3c_b200.Cuda(0)


def test_ulysses_geometry_helpers_match_reference_vectors(lib_path):
    """Host arithmetic of the library itself (no GPU needed) against the vectors the reference produced."""
    import numpy as np
    import h3c_b200
    g = np.load(ROOT / "tests" / "golden" / "ulysses_helpers.npz")
    got = [int(h3c_b200.ulysses_validate(*map(int, c))[0]) for c in g["cases"]]
    assert got == list(g["valid"])
    assert [h3c_b200.ulysses_pad_seq(int(s), 64) for s in g["seqs"]] == list(g["pads"])
    local = [[h3c_b200.ulysses_local_rows(int(p), u, r) for r in range(-1, 9)]
             for p in (16000, 50240, 10) for u in (1, 2, 4, 8)]
    assert np.array_equal(np.array(local, np.uint64), g["local"])
    ok, msg = h3c_b200.ulysses_validate(56, 64, 1, 3, 1)
    assert not ok and "illegal" in msg
    # tests/test_h3_nvfp4_sf_bytes.c
    sfb = h3c_b200.load().h3_cuda_nvfp4_sf_bytes
    assert sfb(21504, 5376) == 168 * 84 * 512 and sfb(5376, 14336) == 42 * 224 * 512
    assert sfb(1, 64) == 512 and sfb(256, 512) == 2 * 8 * 512 and sfb(1, 63) == 0 and sfb(0, 64) == 0
