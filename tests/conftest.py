import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def load_pkg():
    """The package directory name carries a hyphen, so it is imported by name."""
    return importlib.import_module("gpt-oss_b200")


@pytest.fixture(scope="session")
def pkg():
    return load_pkg()


@pytest.fixture(scope="session")
def synth():
    return importlib.import_module("gpt-oss_b200.synth")


@pytest.fixture(scope="session")
def port():
    import oracle
    return oracle.Port()


GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def golden_cases():
    return sorted(f[:-4] for f in os.listdir(GOLDEN_DIR)
                  if f.endswith(".npz") and not f.startswith(("block_", "quant_")))


def golden_block_cases():
    """Fixtures of the block with its RMSNorm and residual add (reference forward(), run.cpp:657-747)."""
    return sorted(f[:-4] for f in os.listdir(GOLDEN_DIR) if f.endswith(".npz") and f.startswith("block_"))
