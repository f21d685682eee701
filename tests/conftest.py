"""Shared test plumbing: marker registration, repo paths on sys.path, golden-file loader."""
import os, sys
import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, 'oracle')):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run on the B200 box)')


@pytest.fixture(scope='session')
def golden():
    def load(name):
        return np.load(os.path.join(ROOT, 'tests', 'golden', name + '.npz'))
    return load
