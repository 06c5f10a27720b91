import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `pytest -m gpu`)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def fp8_w8a16():
    """Run quantised-weight layers with 16-bit activations (the in-shared-memory dequant kernels) for the duration of a test."""
    from fastllm_b200.ops import quant_gemm as QG

    old, old_i = QG.FP8_NATIVE, QG.INT_A8
    QG.FP8_NATIVE = False
    QG.INT_A8 = False
    yield
    QG.FP8_NATIVE, QG.INT_A8 = old, old_i
