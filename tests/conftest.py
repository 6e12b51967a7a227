import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def ref_ops():
    """torch.ops._C_gguf_ref: the reference's own extension built by oracle/build_ref.py (skip if absent)."""
    import torch

    path = os.path.join(ROOT, "oracle", "_ref", "_C_gguf_ref.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/_C_gguf_ref.so not built")
    if not hasattr(torch.ops, "_C_gguf_ref") or not hasattr(torch.ops._C_gguf_ref, "ggml_dequantize"):
        torch.ops.load_library(path)
    return torch.ops._C_gguf_ref
