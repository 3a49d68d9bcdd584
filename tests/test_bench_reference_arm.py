"""
The reference arm of bench.py (the CPU computation the reference's tests compare against, timed on the
host cores) runs without a GPU and prints the one JSON line the measurement contract asks for.
"""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, str(ROOT / 'bench.py'), '--impl', 'reference', '--steps', '1',
                          '--warmup', '1', '--tokens', '256'], capture_output=True, text=True, timeout=600,
                         cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [line for line in out.stdout.splitlines() if line.startswith('{')]
    assert len(lines) == 1
    record = json.loads(lines[0])
    assert record['impl'] == 'reference'
    assert record['metric'] == 'linear_fwd_bwd_tflops' and record['unit'] == 'TFLOP/s'
    assert record['higher_is_better'] is True and record['n_gpus'] == 1
    assert record['value'] > 0 and record['steps'] == 1
    assert record['config']['workload'] == 'c2'
    baseline = record['cpu_baseline']
    assert baseline['kind'] == 'port' and baseline['cores'] >= 1 and baseline['value'] == record['value']
    e2e = record['e2e']
    assert e2e['value'] == record['value'] and e2e['h2d_bytes_per_step'] == 0 and e2e['d2h_bytes_per_step'] == 0
