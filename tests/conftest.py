import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


@pytest.fixture(scope="session")
def small_config():
    """Llama-3.2-1B layer shape with 2 layers and a 4096-token vocabulary: the CUDA kernel's compiled
    shape, but small enough for the CPU oracle to run in milliseconds."""
    from qimeng_megakernel_b200.model_config import LLAMA_3_2_1B
    return dict(LLAMA_3_2_1B, num_hidden_layers=2, vocab_size=4096, max_position_embeddings=4096)


@pytest.fixture(scope="session")
def small_weights(small_config):
    from qimeng_megakernel_b200 import synthetic
    return synthetic.make_weights(small_config, seed=1234, device="cpu")
