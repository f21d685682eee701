"""Runs the C++ gate that is written against include/gemv.h and include/moe.h (the reference's own
entry points, namespace glm5) and linked with libb200nvfp4.so."""
import os
import subprocess
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def test_cpp_gate_passes():
    exe = os.path.join(ROOT, 'tests', 'cpp', 'gate_dropin')
    if not os.path.exists(exe):
        subprocess.check_call(['make', '-C', os.path.join(ROOT, 'glm-5.3-flash-cuda-server_b200'), 'gate'])
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    print(r.stdout[-3000:], r.stderr[-2000:])
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert 'gate_dropin: PASS' in r.stdout
