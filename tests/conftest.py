import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (ROOT, HERE):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def tiny_folders(tmp_path_factory):
    """name -> folder of each tiny model with float32 random weights (made once per session)."""
    import torch
    from tiny_configs import OPTIONAL_TENSORS, TINY
    from dynalm_b200.weights import write_model_folder

    out = {}
    for name, (cfg, seed) in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        write_model_folder(str(d), cfg, seed, dtype=torch.float32, optional=OPTIONAL_TENSORS.get(name))
        out[name] = str(d)
    return out


@pytest.fixture(scope="session")
def tiny_folders_bf16(tmp_path_factory):
    import torch
    from tiny_configs import OPTIONAL_TENSORS, TINY
    from dynalm_b200.weights import write_model_folder

    out = {}
    for name, (cfg, seed) in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny_{name}_bf16")
        write_model_folder(str(d), cfg, seed, dtype=torch.bfloat16, optional=OPTIONAL_TENSORS.get(name))
        out[name] = str(d)
    return out
