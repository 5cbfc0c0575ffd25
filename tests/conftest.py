import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (built on demand with oracle/Makefile)."""
    from oracle import attn_oracle
    if not os.path.exists(os.path.join(ROOT, "oracle", "libattn_oracle.so")):
        attn_oracle.build()
    return attn_oracle


@pytest.fixture(scope="session")
def native_lib():
    """libdecoding_attn_b200.so, built in-tree if it is missing (nvcc cross-compiles without a GPU)."""
    from decoding_attention_b200 import build, cabi
    if not os.path.exists(cabi.LIB_PATH):
        build.build_library()
    return cabi
