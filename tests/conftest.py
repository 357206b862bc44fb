import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "liger-kernel_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


# Collection order of the test files.  The hot path comes first and the sibling operators last, so that under
# `pytest -x` a failure in one operator cannot hide the tests of another that matters more; files not listed keep
# their alphabetical place in the middle, and the entry point for callers that cannot allocate is always last.
_FIRST = ["test_gemm_gpu", "test_flce_gpu", "test_flce_full_size_gpu", "test_flce_skip_ignored_gpu", "test_sharded_gpu",
          "test_model_gpu", "test_device_wait_gpu"]
_LAST = ["test_cross_entropy_gpu", "test_head_losses_gpu", "test_zz_no_alloc"]


def pytest_collection_modifyitems(session, config, items):
    def key(item):
        name = os.path.splitext(os.path.basename(str(item.fspath)))[0]
        if name in _FIRST:
            return (0, _FIRST.index(name))
        if name in _LAST:
            return (2, _LAST.index(name))
        return (1, 0)

    items.sort(key=key)   # stable: the order inside a file and among unlisted files is kept


@pytest.fixture(autouse=True)
def _seed():
    import torch

    torch.manual_seed(42)
    yield
