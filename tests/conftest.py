"""Shared fixtures: the `gpu` marker, the tiny configurations and their model folders."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu on a B200")


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name -> folder with config.json + model.safetensors of every tiny configuration."""
    import helpers

    root = tmp_path_factory.mktemp("tiny_models")
    return {name: helpers.make_model_folder(root / name, name) for name in helpers.TINY}
