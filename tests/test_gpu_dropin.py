"""GPU: the drop-in boundary.  (1) tests/compat_check.cu uses the replacement header exactly as
the reference's harnesses do (kernel template with the harness-derived launch geometry, and
linear_v21_launch) and compares with a CPU loop.  (2) Where it was built, the reference's own
test/test_correctness.cu -- unchanged, linked against this library -- must run to completion."""
import os
import subprocess

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def test_compat_header_and_launcher(cuda):
    from int4linear_b200 import build
    exe = build.build_compat_check()
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "PASS" in r.stdout


def test_reference_correctness_program_runs_unchanged(cuda):
    exe = os.path.join(ROOT, "oracle", "_ref", "test_correctness_dropin")
    if not os.path.exists(exe):
        pytest.skip("built only where the reference checkout is available")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "CUDA FAILED" not in r.stdout + r.stderr
