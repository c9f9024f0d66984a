import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU (run with -m gpu)")
    config.addinivalue_line("markers", "multigpu: needs 2 or more GPUs")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no GPU on this machine")
    for item in items:
        if "gpu" in item.keywords or "multigpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _reset_state():
    from vllm_torchtpu_b200 import envs
    from vllm_torchtpu_b200.parallel import state, communicator
    yield
    envs.reset()
    if state.get_state().world_size == 1:
        communicator.reset()
