"""Shared fixtures. GPU tests are marked `gpu`; everything else runs on a machine without one."""
import importlib.util
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def load_package():
    """Import the hyphen-named package directory as module `swlm_b200`."""
    if "swlm_b200" in sys.modules:
        return sys.modules["swlm_b200"]
    path = os.path.join(ROOT, "swift-mlx-lm_b200", "__init__.py")
    spec = importlib.util.spec_from_file_location("swlm_b200", path, submodule_search_locations=[os.path.dirname(path)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["swlm_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def oracle():
    import oracle_binding

    so = os.path.join(ROOT, "oracle", "liboracle.so")
    if not os.path.exists(so):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle")], check=True)
    return oracle_binding.Oracle(so)


@pytest.fixture(scope="session")
def golden():
    import json

    with open(os.path.join(ROOT, "tests", "golden", "reference_kat.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def lib(pkg):
    return pkg.load_library()
