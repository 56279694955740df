import importlib
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CACHE = os.environ.get("LG_B200_CACHE", "/tmp/lg_b200_cache")
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def lg_module():
    return importlib.import_module("little-gemma_b200")


def synth_module():
    return importlib.import_module("little-gemma_b200.synth")


def model_files(name: str):
    """(target_path, head_path) of a named seeded test model, generated on first use."""
    from tests.models import build
    return build(name, CACHE)


@pytest.fixture(scope="session")
def synth():
    return synth_module()


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(GOLDEN, "tiny_golden.npz"))


@pytest.fixture(scope="session")
def port_built():
    """Compile the CPU restatement (gcc only)."""
    import subprocess
    subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle"), "port"])
    return True


@pytest.fixture(scope="session")
def lg():
    mod = lg_module()
    if not os.path.exists(mod.LIB_PATH):
        import subprocess
        subprocess.check_call([sys.executable, os.path.join(ROOT, "little-gemma_b200", "build.py")])
    mod.load()
    return mod


def has_ref(n=4):
    from oracle.pyref import ref_lib_path
    return os.path.exists(ref_lib_path(n))
