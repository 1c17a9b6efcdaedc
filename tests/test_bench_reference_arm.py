"""The CPU arm of bench.py (`--impl reference`): one JSON line with the contract's keys, and a run time bounded by its time
budget whatever the step count asked for."""
import json
import os
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_is_bounded_and_prints_the_contract_line():
    env = dict(os.environ, B200MOE_REFERENCE_BUDGET_S="3")
    t0 = time.time()
    p = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "4", "--warmup", "1"], cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=600)
    took = time.time() - t0
    assert p.returncode == 0, p.stderr[-2000:]
    line = json.loads([ln for ln in p.stdout.splitlines() if ln.startswith("{")][-1])
    assert line["impl"] == "reference" and line["unit"] == "GB/s" and line["value"] > 0 and line["higher_is_better"] is True
    assert line["metric"] == "moe_decode_layer_hbm_gbs_on_touched_expert_bytes" and line["steps"] == 4
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["value"] == line["value"] and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "of the ten cases" in line["cpu_baseline"]["sample"]          # the budget forced a subset per step, and the line says so
    assert took < 300, f"the bounded run took {took:.0f} s"
