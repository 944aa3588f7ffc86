"""Shared fixtures.  GPU tests are marked `gpu` and call the CUDA library through
its C-ABI; everything else runs on a CPU-only machine."""
import importlib.util
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) device")


def _load(name: str, path: Path):
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, path, submodule_search_locations=[str(path.parent)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="session")
def b200():
    """The ctypes binding of libggml-b200.so (package directory `llama.cpp_b200`)."""
    return _load("llama_cpp_b200", ROOT / "llama.cpp_b200" / "__init__.py")


@pytest.fixture(scope="session")
def oracle():
    return _load("ggml_oracle", ROOT / "oracle" / "oracle.py")


@pytest.fixture(scope="session")
def golden(oracle):
    return oracle.load_golden()
