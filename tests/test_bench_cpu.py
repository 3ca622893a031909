"""bench.py pieces that need no GPU: workload tables, algorithmic bytes, the reference arm's line."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_workload_tables():
    sys.path.insert(0, ROOT)
    import bench
    full = bench.workload_linears("llama3.1-8b-linears")
    assert len(full) == 32 * 7 + 1
    params = sum(V * H for _, V, H, _ in full)
    assert params == 32 * (2 * 4096 * 4096 + 2 * 1024 * 4096 + 3 * 14336 * 4096) + 128256 * 4096
    # bytes of the q projection at BT=512 with bf16 W/m/v: 209.7 MB
    assert abs(bench.algorithmic_bytes(4096, 4096) - 209.7e6) < 0.1e6
    assert abs(bench.algorithmic_bytes(14336, 4096) - 723.5e6) < 0.1e6
    total = sum(bench.algorithmic_bytes(V, H) for _, V, H, _ in full)
    assert abs(total - 92.9e9) < 0.2e9


def test_reference_arm_line():
    env = dict(os.environ, OMP_NUM_THREADS=str(os.cpu_count() or 1))
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "1"], capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stderr
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "ms/step" and line["higher_is_better"] is False
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["value"] > 0
    assert line["metric"] == "fused_wgrad_adamw_ms_per_step"
    # no GPU here: the reference's GPU kernel is either reported as unavailable or left out
    assert "layer_ms" not in line.get("reference_gpu_kernel", {})
