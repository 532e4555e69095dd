"""The switch registry (include/h3b_plugin.h): record type and functions of the reference's registry, and the
reference's lint (tools/check_plugin_registry.sh) restated over this repository: every H3_* / H3B_* switch that a
source file reads must be registered, and nothing reads such a switch with a bare getenv / os.environ."""
import re
from pathlib import Path

import h3c_b200

ROOT = Path(__file__).resolve().parent.parent
SOURCES = sorted((ROOT / "h3c_b200" / "csrc").glob("*.c*")) + sorted((ROOT / "h3c_b200" / "csrc").glob("*.h")) + \
    sorted((ROOT / "h3c_b200").glob("*.py")) + [ROOT / "bench.py", ROOT / "__graft_entry__.py"]
NAME = r"\"(H3B?_[A-Z0-9_]+)\""
EXEMPT = {"H3_REFERENCE_ROOT"}     # where the build looks for the h3.c tree: not a switch of the library


def registered():
    text = (ROOT / "include" / "h3b_plugin.h").read_text()
    return set(re.findall(r"^\s*X\(\"(H3B?_[A-Z0-9_]+)\"", text, flags=re.M))


def test_catalogue_is_exported_as_written():
    cat = h3c_b200.plugin_catalogue()
    assert {c[0] for c in cat} == registered() and len(cat) >= 8
    assert all(c[1] in ("STABLE", "EXPERIMENTAL", "DEAD_END_VERIFIED") for c in cat)
    assert all(c[2] in ("DIT", "SP", "MISC") for c in cat)


def test_every_switch_read_is_registered_and_read_through_the_registry():
    reg, read, bare = registered(), {}, []
    for path in SOURCES:
        text = path.read_text()
        for m in re.finditer(r"(h3_plugin_value|h3_plugin_enabled|h3b_plugin_value|h3b_plugin_enabled|plugin_value|"
                             r"plugin_enabled)\s*\(\s*" + NAME, text):
            read.setdefault(m.group(2), path.name)
        for m in re.finditer(r"(getenv\s*\(\s*|environ\.get\s*\(\s*|environ\s*\[\s*)" + NAME, text):
            if m.group(2) not in EXEMPT:
                bare.append((path.name, m.group(2)))
    assert not bare, f"switches read outside the registry: {bare}"
    unregistered = {k: v for k, v in read.items() if k not in reg}
    assert not unregistered, f"read but not registered: {unregistered}"
    assert len(read) >= 6


def test_value_and_enabled_semantics(monkeypatch):
    # reference semantics (tools/h3_plugin.h:232-239): environment wins when not empty, else the default;
    # "0", "false", "off", "no" and "" mean off
    monkeypatch.delenv("H3B_GEMM_PAIRS", raising=False)
    assert h3c_b200.plugin_value("H3B_GEMM_PAIRS") == "1" and h3c_b200.plugin_enabled("H3B_GEMM_PAIRS")
    for off in ("0", "false", "off", "no"):
        monkeypatch.setenv("H3B_GEMM_PAIRS", off)
        assert not h3c_b200.plugin_enabled("H3B_GEMM_PAIRS")
    monkeypatch.setenv("H3B_GEMM_PAIRS", "")
    assert h3c_b200.plugin_enabled("H3B_GEMM_PAIRS")          # empty falls back to the default
    monkeypatch.setenv("H3B_ULYSSES_BARRIER", "nccl")
    assert h3c_b200.plugin_value("H3B_ULYSSES_BARRIER") == "nccl"
    import pytest
    with pytest.raises(h3c_b200.H3Error):
        h3c_b200.plugin_value("H3B_NOT_A_SWITCH")
