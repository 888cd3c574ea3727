"""The reference's own unittest suites run against this repository's ``mor`` package.

The suites need nothing but ``import mor`` and a GPU.  They are not part of this repository: point
MOR_REFERENCE_TESTS at a directory holding the reference's ``test/test_*.py`` files and this test copies
them to a scratch directory and runs each with ``python -m unittest`` (one process per suite), with the
repository root first on the module path.  Without the variable the test is skipped.

Known differences, by test name (each is a deliberate deviation from the shipped reference, not a
numerical one):
  none are expected in the four suites below; a failure here is a defect of the drop-in surface.
"""
import os
import shutil
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SUITES = ["test_fake_quantize", "test_fake_quantize_block_scaling", "test_fake_quantize_channel_scaling", "test_e8mx"]


@pytest.mark.parametrize("suite", SUITES)
def test_reference_suite_passes_against_this_package(suite, tmp_path):
    src_dir = os.environ.get("MOR_REFERENCE_TESTS")
    if not src_dir or not os.path.exists(os.path.join(src_dir, suite + ".py")):
        pytest.skip("MOR_REFERENCE_TESTS does not point at the reference's test files")
    shutil.copy(os.path.join(src_dir, suite + ".py"), tmp_path / (suite + ".py"))
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-m", "unittest", "-v", suite], cwd=tmp_path, env=env, capture_output=True,
                       text=True, timeout=1800)
    tail = (r.stdout + r.stderr)[-4000:]
    assert r.returncode == 0, f"{suite} failed against this package:\n{tail}"
