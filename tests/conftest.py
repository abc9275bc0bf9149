import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def tiny_llama_path(tmp_path_factory):
    from ollama_b200.models.synth import write_synthetic_gguf
    p = tmp_path_factory.mktemp("models") / "tiny-llama-f32.gguf"
    write_synthetic_gguf(str(p), "tiny-llama", "F32")
    return str(p)


@pytest.fixture(scope="session")
def tiny_llama_q8_path(tmp_path_factory):
    from ollama_b200.models.synth import write_synthetic_gguf
    p = tmp_path_factory.mktemp("models") / "tiny-llama-q8.gguf"
    write_synthetic_gguf(str(p), "tiny-llama", "Q8_0")
    return str(p)
