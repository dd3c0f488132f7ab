import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.build()
    return O


@pytest.fixture(scope="session")
def gpu_ctx():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from shady_thinker_b200.gpu import GpuContext
    torch.cuda.set_device(0)
    # 0x1 is cudaStreamLegacy: the context launches on the same (default) stream torch uses for
    # the test tensors, so uploads, kernels and read-backs are ordered without extra syncs.
    ctx = GpuContext(0, stream=0x1)
    yield ctx
    ctx.synchronize()
    ctx.close()
