"""Shared fixtures: loads the package (its directory name has a dot) and the CPU oracle."""
import importlib.util
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def _load(name: str, path: Path):
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def load_package():
    return _load("worldmodel_cu_b200", ROOT / "worldmodel.cu_b200" / "__init__.py")


def load_oracle():
    return _load("w8a8_ref", ROOT / "oracle" / "w8a8_ref.py")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def ref():
    return load_oracle()


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(ROOT / "tests" / "golden" / "w8a8_reference_golden.npz")


@pytest.fixture(scope="session")
def parity_log():
    """record(name, mismatches, positions): prints a measured mismatch count and, when the environment variable
    W8A8_PARITY_LOG names a file, appends it there as a JSON line, so the numbers quoted in the design notes can
    be refreshed from a test run."""
    import json
    import os

    def record(name, mismatches, positions, **extra):
        row = dict(name=name, mismatches=int(mismatches), positions=int(positions),
                   rate=float(mismatches) / max(int(positions), 1), **extra)
        print("PARITY", json.dumps(row))
        path = os.environ.get("W8A8_PARITY_LOG")
        if path:
            try:
                with open(path, "a") as f:
                    f.write(json.dumps(row) + "\n")
            except OSError:
                pass
        return row

    return record
