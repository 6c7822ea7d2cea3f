import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Random-weight model folders of the tiny configurations, made once per session in a
    temporary place: {"a": dir, "b": dir, "c": dir, "d": dir}."""
    from tiny_configs import TINY_A, TINY_B, TINY_C, TINY_D
    from nanoinfer_b200.weights import write_random_model
    root = tmp_path_factory.mktemp("models")
    out = {}
    for key, raw, seed in (("a", TINY_A, 0), ("b", TINY_B, 1), ("c", TINY_C, 2), ("d", TINY_D, 3)):
        d = str(root / key)
        write_random_model(d, raw, seed)
        out[key] = d
    return out
