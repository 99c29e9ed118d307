"""pytest configuration: import paths, the `gpu` marker, shared fixtures."""
import os
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(REPO, "deepgemm-das_b200"), os.path.join(REPO, "oracle"), REPO,
          os.path.join(REPO, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def _build():
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "dg_build", os.path.join(REPO, "deepgemm-das_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device of compute capability 10.x (B200)")
    # Before any test module imports the package: libdeepgemm_b200.so and the host glue are
    # looked up at import time (a no-op when the stamps match the sources).
    if not hasattr(config, "workerinput"):      # once, not in every xdist worker
        _build()


def pytest_collection_modifyitems(config, items):
    # GPU tests fail (not skip) on a GPU box whose device is missing; on a CPU-only box they
    # are normally deselected with -m "not gpu", and skipped if collected anyway.
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """The library was built in pytest_configure; kept so that tests can depend on it by name."""
    yield
