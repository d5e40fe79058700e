"""The C-ABI library loads without a GPU and exports exactly what include/promoe_b200.h declares."""
import re
import subprocess
from pathlib import Path

from promoe_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]


def declared_functions():
    text = (ROOT / "include" / "promoe_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pm_[a-z0-9_]+)\s*\(", text)))


def test_header_and_library_agree(lib):
    names = declared_functions()
    assert len(names) >= 35
    out = subprocess.run(["nm", "-D", "--defined-only", str(_lib.LIB_PATH)], capture_output=True, text=True, check=True).stdout
    exported = sorted(ln.split()[-1] for ln in out.splitlines() if " T " in ln and ln.split()[-1].startswith("pm_"))
    assert exported == names, "header and library disagree"
    assert sorted(_lib.SIGNATURES) == names, "the ctypes binding must cover every declared entry point"
    for n in names:
        assert getattr(lib, n) is not None


def test_version_and_error_channel(lib):
    assert lib.pm_version() >= 100
    import ctypes as C
    import pytest
    with pytest.raises(_lib.PromoeError) as e:
        _lib.call("pm_ctx_create", C.byref(C.c_void_p()), 0, 4, b"num_expert_per_token=2")
    assert "num_layer" in str(e.value)
    # device-only calls fail with a message instead of crashing when no slab exists
    ctx = C.c_void_p()
    _lib.call("pm_ctx_create", C.byref(ctx), 2, 4, b"num_expert_per_token=2")
    with pytest.raises(_lib.PromoeError):
        _lib.call("pm_moe_forward", ctx, 0, 8, 1, 8, None)
    _lib.call("pm_ctx_destroy", ctx)


def test_product_never_imports_the_oracle():
    """oracle/ is test infrastructure: nothing under promoe_b200/ may import it."""
    for p in (ROOT / "promoe_b200").rglob("*.py"):
        assert not re.search(r"^\s*(from|import)\s+oracle\b", p.read_text(), flags=re.M), p
    for p in (ROOT / "promoe_b200" / "csrc").glob("*"):
        assert "oracle/" not in p.read_text(), p


def test_numa_helpers():
    from promoe_b200 import numa
    assert numa._cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert numa._cpulist("") == set()
    assert numa.gpu_numa_node(0) is None or isinstance(numa.gpu_numa_node(0), int)  # no GPU here: None
