"""bench.py's contract as far as it can be checked without a GPU: the profile file it reads the ncu traffic
from, and the reference arm (the CPU restatement timed on the host cores), which needs no device at all."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_traffic_is_read_from_the_committed_profile():
    sys.path.insert(0, ROOT)
    import bench
    t = bench.profiled_traffic()
    # six sibling matrices of 12 896 rows x 4096: 29.78 MB of weights; the capture may add a few KB
    assert isinstance(t, int) and 29_700_000 < t < 30_200_000, t


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, 'bench.py'), '--impl', 'reference', '--steps', '2', '--warmup', '1'],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith('{')]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d['impl'] == 'reference'
    for k in ('metric', 'value', 'unit', 'n_gpus', 'steps', 'warmup', 'ms_per_step', 'higher_is_better', 'config', 'cpu_baseline', 'e2e'):
        assert k in d, k
    assert d['value'] > 0 and d['cpu_baseline']['cores'] >= 1
    assert d['e2e']['h2d_bytes_per_step'] == 0 and d['e2e']['d2h_bytes_per_step'] == 0
