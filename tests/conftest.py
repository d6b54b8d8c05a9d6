"""pytest configuration: the `gpu` marker, and loaders for the package and the oracle.

The package directory is named `tylo.jl_b200`; a dot cannot appear in a Python module
name, so it is loaded by path under the module name `tylo_b200`."""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
PKG_DIR = ROOT / "tylo.jl_b200"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def load_package():
    if "tylo_b200" in sys.modules:
        return sys.modules["tylo_b200"]
    spec = importlib.util.spec_from_file_location("tylo_b200", PKG_DIR / "__init__.py",
                                                  submodule_search_locations=[str(PKG_DIR)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["tylo_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def load_oracle():
    if "tylo_oracle" in sys.modules:
        return sys.modules["tylo_oracle"]
    spec = importlib.util.spec_from_file_location("tylo_oracle", ROOT / "oracle" / "tylo_oracle.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules["tylo_oracle"] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="session")
def tylo():
    return load_package()


@pytest.fixture(scope="session")
def oracle():
    return load_oracle()


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
