import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "multigpu: needs more than one CUDA device")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords or "multigpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def tiny_llama_dir(tmp_path_factory):
    """BASELINE config 1: tiny Llama, fp32, random-init N(0, 0.02) from seed 0."""
    import copy
    from onnxruntime_genai_b200.models.arch import PRESETS
    from onnxruntime_genai_b200.models.builder import export_model
    d = str(tmp_path_factory.mktemp("tiny_llama"))
    export_model(copy.deepcopy(PRESETS["tiny-llama"]), d, precision="fp32", execution_provider="cpu", seed=0)
    return d
