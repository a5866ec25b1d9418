import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU")


def _has_gpu() -> bool:
    try:
        from fastface_b200 import load_library
        return load_library().ffcu_device_count() > 0
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(scope="session")
def built_lib():
    from fastface_b200 import build
    return build.build()


@pytest.fixture(scope="session")
def model_root(tmp_path_factory):
    """Directory holding models/{synth_seed0_ffw4.bin, op_scales.bin, op_scales_v2.bin}."""
    from fastface_b200 import synth
    root = os.environ.get("FF_TEST_MODEL_ROOT") or str(tmp_path_factory.mktemp("ffmodel"))
    synth.materialize(root, 0)
    return root


@pytest.fixture(scope="session")
def ffw4(model_root):
    return os.path.join(model_root, "models", "synth_seed0_ffw4.bin")


@pytest.fixture(scope="session")
def oracle(model_root, ffw4):
    from oracle import ffo
    return ffo.Oracle(ffw4, os.path.join(model_root, "models", "op_scales.bin"),
                      os.path.join(model_root, "models", "op_scales_v2.bin"))


@pytest.fixture(scope="session")
def oracle_per_tensor(model_root, ffw4):
    from oracle import ffo
    return ffo.Oracle(ffw4, os.path.join(model_root, "models", "op_scales.bin"), None)


GOLDEN = os.path.join(ROOT, "tests", "golden")


def read_trace(path):
    recs = []
    with open(path) as f:
        for line in f:
            if line.startswith("#") or not line.strip():
                continue
            k, i, n, crc = line.split()
            recs.append((k, int(i), int(n), int(crc, 16)))
    return recs
