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
    temporary place: {"a": dir, "b": dir, ...}.  "bs", "ds", "e": query and key projections
    scaled so that the attention is peaked (tiny_configs.sharp); "ds" is D with an untied output."""
    from tiny_configs import TINY_A, TINY_B, TINY_C, TINY_D, TINY_D_UNTIED, TINY_E, TINY_F, sharp
    from nanoinfer_b200.weights import write_random_model
    root = tmp_path_factory.mktemp("models")
    out = {}
    for key, raw, seed, slot_std in (("a", TINY_A, 0, None), ("b", TINY_B, 1, None), ("c", TINY_C, 2, None),
                                     ("d", TINY_D, 3, None), ("bs", TINY_B, 1, sharp(TINY_B)),
                                     ("ds", TINY_D_UNTIED, 3, sharp(TINY_D)), ("e", TINY_E, 4, sharp(TINY_E)),
                                     ("f", TINY_F, 5, None)):
        d = str(root / key)
        write_random_model(d, raw, seed, slot_std=slot_std)
        out[key] = d
    return out
