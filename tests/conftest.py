import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (HERE, ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    """GPU tests fail loudly where a GPU was asked for; without one they are deselected by -m 'not gpu'."""
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Random-weight model folders of the tiny configurations, made once per session in a temp folder."""
    from tiny_configs import ALL
    from nanoinfer_b200.registry import config_from_json_dict
    from nanoinfer_b200.weights import write_random_model
    out = {}
    for name, (cfg_json, page) in ALL.items():
        d = str(tmp_path_factory.mktemp(f"model_{name}"))
        write_random_model(config_from_json_dict(cfg_json), d, seed=1234, dtype="bfloat16")
        out[name] = (d, page)
    return out
