"""bench.py's JSON contract, checked without a GPU: the reference arm (CPU code path) on the smallest
configuration, and the helpers that shape the roofline and config objects of the GPU arm."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_reference_arm_prints_one_json_line():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--config", "c1", "--steps", "2",
                        "--warmup", "1", "--cpu-sample-layers", "1"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "tokens/s" and d["higher_is_better"] is True
    assert d["value"] > 0 and d["e2e"]["value"] == d["value"]
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["sample"]
    assert "workload" in d["config"] and "model" not in d["config"]


def test_roofline_and_config_helpers():
    sys.path.insert(0, str(ROOT))
    import bench
    from promoe_b200 import synth
    prof = dict(ffn_launches=0, gateup_ms=0.0, down_ms=0.0, gateup_bytes=0, down_bytes=0, fused_launches=10,
                fused_ms=0.5, fused_bytes=2_000_000_000)
    r = bench.roofline_entry(prof, 0.0, 0.0, 4000.0, 6553.6, "measured")
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and abs(r["frac"] - 4000.0 / 6553.6) < 1e-12
    assert r["traffic"] > r["bytes_per_launch"] and r["launches"] == 10 and abs(r["avg_launch_us"] - 50.0) < 1e-9
    # launch pairs only: weight bytes of both launches over the time of both
    prof2 = dict(prof, fused_launches=0, fused_ms=0.0, ffn_launches=4, gateup_ms=0.2, down_ms=0.1,
                 gateup_bytes=600_000_000, down_bytes=300_000_000)
    r2 = bench.roofline_entry(prof2, 3000.0, 3000.0, 0.0, 6553.6, "measured")
    assert abs(r2["achieved"] - 3000.0) < 1e-6 and r2["gateup_gbs"] == 3000.0 and r2["traffic"] is None
    # both kinds: the one with more device time is reported, the other rides along
    prof3 = dict(prof2, fused_launches=2, fused_ms=0.1, fused_bytes=400_000_000)
    r3 = bench.roofline_entry(prof3, 3000.0, 3000.0, 4000.0, 6553.6, "measured")
    assert "launch pair" in r3["kernel"] and abs(r3["share_of_ffn_time"] - 0.75) < 1e-9
    assert r3["other_kernel"]["achieved"] == 4000.0
    c = bench.workload_config(synth.CONFIGS["c2"], 4, False)
    assert c["batch_per_gpu"] == 2 and c["global_batch"] == 8 and "expert parallel" in c["parallelism"]
    peak, src = bench.measured_peak_gbs()
    assert peak > 1000 and ("measured" in src or "fallback" in src)
