"""The selectable variants of the attention kernel (H3B_ATTN_EMU, read once per process, hence one child process per
variant): every variant must reproduce f64 attention of the same inputs within the bound of the default kernel, on
square, ragged and rectangular shapes.  212 / 213 are the CTA-pair form (cta_group::2, K and V tiles split over two
SMs), 13 / 10 / 0 the other exponent shares and the per-instruction election."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
SHAPES = [(512, 512, 2), (300, 300, 3), (1000, 777, 4), (1536, 512, 4), (2048, 2048, 2)]


@pytest.mark.parametrize("variant", ["212", "213", "13", "10", "0"])
@pytest.mark.parametrize("f16", [False, True])
def test_variant_matches_f64_attention(variant, f16):
    if f16 and variant in ("213", "13", "10"):
        pytest.skip("the f16 form has the default, the plain and the pair variant only")
    env = dict(os.environ, H3B_ATTN_EMU=variant)
    cmd = [sys.executable, str(ROOT / "tests" / "attn_variant_worker.py"), "f16" if f16 else "bf16"] + \
          [f"{lq},{lk},{heads}" for lq, lk, heads in SHAPES]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    errors = json.loads(out.stdout.strip().splitlines()[-1])
    assert len(errors) == len(SHAPES)
    for spec, err in errors.items():
        assert err < (1e-3 if f16 else 4e-3), (variant, f16, spec, err)
