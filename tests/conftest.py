"""Shared fixtures: tiny model folders with random weights, made in a temporary folder."""
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
    """name → folder with config.json and model.safetensors (bfloat16 weights)."""
    import tiny
    from cretif_b200.weights.random_model import write_random_model
    out = {}
    for name, cfg in tiny.CONFIGS.items():
        d = str(tmp_path_factory.mktemp(f"model_{name}"))
        write_random_model(d, cfg, seed=tiny.SEEDS[name])
        out[name] = d
    return out


@pytest.fixture(scope="session")
def plain_models(model_dirs):
    """name → (config dict, float64 weights) as the plain implementation reads them."""
    import plain_llama
    return {name: plain_llama.read_model_folder(d) for name, d in model_dirs.items()}
