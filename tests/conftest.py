"""Shared pytest configuration: the ``gpu`` marker, repo-root import path and
fixture loading."""
import glob
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def golden_layer_names():
    return sorted(os.path.basename(p)[len("layer_"):-len(".npz")]
                  for p in glob.glob(os.path.join(GOLDEN, "layer_*.npz")))


def load_golden(name):
    with np.load(os.path.join(GOLDEN, name + ".npz"), allow_pickle=False) as z:
        return {k: z[k] for k in z.files}


@pytest.fixture(params=golden_layer_names())
def golden_layer(request):
    data = load_golden("layer_" + request.param)
    data["name"] = request.param
    return data
