"""Install the unmodified reference into baseline/_ref (git-ignored; it travels to the GPU box).

    python baseline/install_reference.py [--reference /path/to/kiln-compiler]

Two steps, both offline:
  1. pip --target install of the reference package from a scratch copy of the checkout (the
     checkout itself may be read-only and pip builds in the source tree):
        pip install --no-index --no-build-isolation --no-deps --target baseline/_ref <copy>
  2. the reference's own GPU test file and the three test-support files it imports
     (tests/test_gpu.py, tests/test_memory_plan.py, tests/conftest.py, tests/models/) are copied
     beside the installed package, into baseline/_ref/kiln_tests/, so that
     tests/test_reference_gpu_suite.py can run that file, as it is, against this backend on a
     machine that has no checkout of the reference.

Nothing under baseline/_ref is part of this repository's history.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"
TEST_FILES = ["test_gpu.py", "test_memory_plan.py", "conftest.py", "__init__.py"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("KILN_REFERENCE", str(HERE.parent.parent / "reference")))
    ap.add_argument("--tests-only", action="store_true", help="skip the pip step (the package is already installed)")
    args = ap.parse_args()
    ref = Path(args.reference)
    if not (ref / "kiln" / "api.py").exists():
        raise SystemExit(f"no reference checkout at {ref}")
    if not args.tests_only:
        with tempfile.TemporaryDirectory() as tmp:
            copy = Path(tmp) / "kiln-compiler"
            shutil.copytree(ref, copy, ignore=shutil.ignore_patterns(".git", "__pycache__"))
            subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
                            "--find-links", "/opt/wheelhouse", "--upgrade", "--target", str(TARGET), str(copy)], check=True)
    dest = TARGET / "kiln_tests"
    if dest.exists():
        shutil.rmtree(dest)
    (dest / "models").mkdir(parents=True)
    for name in TEST_FILES:
        if (ref / "tests" / name).exists():
            shutil.copy2(ref / "tests" / name, dest / name)
    for f in (ref / "tests" / "models").glob("*.py"):
        shutil.copy2(f, dest / "models" / f.name)
    print(f"reference installed under {TARGET}; its GPU tests under {dest}")


if __name__ == "__main__":
    main()
