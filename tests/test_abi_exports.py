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


def test_numa_binding_with_a_fake_sysfs(tmp_path, monkeypatch):
    """numa_node present -> that node's CPUs; numa_node -1 -> the device's local_cpulist when it is
    a proper subset of the usable CPUs; otherwise nothing is bound and the reason is reported."""
    import os
    from promoe_b200 import numa
    allowed = sorted(os.sched_getaffinity(0))
    if len(allowed) < 2:
        import pytest
        pytest.skip("needs two usable CPUs")
    bdf = "0000:1b:00.0"
    monkeypatch.setattr(numa, "_gpu_bdf", lambda i: bdf)
    dev = tmp_path / "bus/pci/devices" / bdf
    dev.mkdir(parents=True)
    node = tmp_path / "devices/system/node/node1"
    node.mkdir(parents=True)
    try:
        (dev / "numa_node").write_text("1\n")
        (node / "cpulist").write_text(f"{allowed[0]}\n")
        r = numa.bind_to_gpu_numa_node(0, sysfs=str(tmp_path))
        assert r == {"numa_node": 1, "bound": True, "cpus": 1, "source": "numa_node"}
        assert os.sched_getaffinity(0) == {allowed[0]}
        os.sched_setaffinity(0, allowed)
        (dev / "numa_node").write_text("-1\n")
        (dev / "local_cpulist").write_text(f"{allowed[1]}\n")
        r = numa.bind_to_gpu_numa_node(0, sysfs=str(tmp_path))
        assert r["bound"] and r["source"] == "local_cpulist" and os.sched_getaffinity(0) == {allowed[1]}
        os.sched_setaffinity(0, allowed)
        (dev / "local_cpulist").write_text(f"{allowed[0]}-{allowed[-1]}\n")
        r = numa.bind_to_gpu_numa_node(0, sysfs=str(tmp_path))
        assert not r["bound"] and "reason" in r and os.sched_getaffinity(0) == set(allowed)
    finally:
        os.sched_setaffinity(0, allowed)
