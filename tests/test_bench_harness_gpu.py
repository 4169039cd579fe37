"""The model-shaped step harness of bench.py (BASELINE configs[4]: B=64, S=512, the attention module of this library
between torch stand-ins of the reference model's other layers) runs, times the attention module inside the step and
reports a clean device status."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
def test_model_step_harness_runs_and_reports_the_attention_share():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--model-step", "--profile"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert lines, out.stdout[-2000:]
    rec = json.loads(lines[-1])
    assert rec["device_status"] == 0
    assert rec["recurrent_positions"] == 512 and rec["ode_unfolds"] == 6
    assert 0.0 < rec["attention_ms"] < rec["step_one_recurrent_position_ms"] < rec["step_ms"]
    assert 0.0 < rec["attention_share"] < rec["attention_share_there"] < 1.0
