import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
os.environ.setdefault("BMT_QUIET", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def bmt_cpu():
    """In-process world-size-1 runtime on the CPU (gloo)."""
    import bmtrain_b200 as bmt
    from dist_utils import free_port

    if not bmt.is_initialized():
        os.environ.update(RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", LOCAL_WORLD_SIZE="1",
                          MASTER_ADDR="127.0.0.1", MASTER_PORT=str(free_port()))
        bmt.init_distributed(seed=0, device="cpu")
    return bmt


@pytest.fixture(scope="session")
def bmt_gpu():
    """In-process world-size-1 runtime on cuda:0."""
    import torch
    import bmtrain_b200 as bmt
    from dist_utils import free_port

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if not bmt.is_initialized():
        os.environ.update(RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", LOCAL_WORLD_SIZE="1",
                          MASTER_ADDR="127.0.0.1", MASTER_PORT=str(free_port()))
        bmt.init_distributed(seed=0)
    return bmt
