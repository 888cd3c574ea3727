import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    _build_if_missing()


def _build_if_missing():
    """The native artefacts are not part of the history: a fresh checkout builds them once (nvcc cross-compiles
    without a GPU, gcc builds the oracle) before the first test imports the package."""
    import glob
    import importlib.util
    import subprocess
    pkg = os.path.join(ROOT, "mor_b200")
    if not (os.path.exists(os.path.join(pkg, "libmor_b200.so")) and glob.glob(os.path.join(pkg, "_C*.so"))):
        spec = importlib.util.spec_from_file_location("_mor_b200_build", os.path.join(pkg, "build.py"))
        b = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(b)
        b.build_all()
    if not os.path.exists(os.path.join(ROOT, "oracle", "libmor_oracle.so")):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "all"], check=True)


def pytest_collection_modifyitems(config, items):
    # GPU tests are selected with -m gpu; without a device they are skipped, not failed
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
