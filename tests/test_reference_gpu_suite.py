"""The reference's own GPU test file (tests/test_gpu.py of the reference), unmodified, against this
backend: every backend-agnostic test must pass; the three that assert on Triton source text or
Triton tile keys are declared expected failures in tests/reference_suite_plugin.py.

The file is not part of this repository: baseline/install_reference.py copies it beside the
installed reference (baseline/_ref/kiln_tests/, git-ignored).  It runs in a process of its own
because it imports ``kiln.gpu`` at module level."""

import os
import re
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"
SUITE = REF / "kiln_tests"


def test_reference_gpu_tests_pass_on_this_backend(tmp_path):
    if not (SUITE / "test_gpu.py").exists() or not (REF / "kiln" / "api.py").exists():
        pytest.skip("the reference and its tests are not installed under baseline/_ref (baseline/install_reference.py)")
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([str(ROOT / "kiln-compiler_b200"), str(ROOT / "tests"), str(REF), str(SUITE),
                                         env.get("PYTHONPATH", "")])
    env["KILN_CACHE_DIR"] = str(tmp_path)
    proc = subprocess.run([sys.executable, "-m", "pytest", "-p", "reference_suite_plugin", "-q", "--no-header",
                           "-p", "no:cacheprovider", "--rootdir", str(SUITE), str(SUITE / "test_gpu.py")],
                          capture_output=True, text=True, env=env, cwd=str(SUITE), timeout=1200)
    tail = proc.stdout[-3000:] + proc.stderr[-1500:]
    assert proc.returncode == 0, tail
    summary = proc.stdout.strip().splitlines()[-1]
    passed = int(re.search(r"(\d+) passed", summary).group(1))
    assert not re.search(r"\b\d+ (failed|errors?)\b", summary), tail
    assert passed >= 30, summary          # 14 eager cases, 12 random graphs, fusion, views, weights, memory check, autotune, graph replay
