import os
import sys

import pytest

# inherited by the worker processes of the multi-GPU tests, which select their device (and so initialise CUDA)
# before they import the package: kernels that wait for a peer must not meet lazy kernel loading
os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")
# the tests run with the host-side check of every segment-copy descriptor table switched on (bounds of every run,
# no overlapping destinations): the stand-in for a device sanitizer, which this pool does not offer
os.environ.setdefault("FSB200_CHECK_SEGMENTS", "1")

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="module", autouse=True)
def _fresh_rank_processes_per_module():
    """The gloo rank processes of ``tests.common.run_ranks`` are reused within a test module and ended after it."""
    yield
    from tests import common

    common.shutdown_pools()
