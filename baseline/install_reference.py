#!/usr/bin/env python
"""Installs the unmodified reference (PithTrain) under baseline/_ref, where the GPU tests and the benchmark's
`gpu_reference` record import its own Triton MLA kernels and attention modules from.

    python baseline/install_reference.py /path/to/PithTrain

The checkout is copied to a temporary directory first (the build writes into the source tree), then installed with
pip from the offline wheelhouse, without dependencies: deep-gemm, wandb and zstandard are not available here and the
attention path does not import them. baseline/_ref is git-ignored.
"""

import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent


def main() -> int:
    if len(sys.argv) != 2:
        print(__doc__)
        return 2
    src = Path(sys.argv[1]).resolve()
    if not (src / "pyproject.toml").exists() or not (src / "pithtrain").is_dir():
        print(f"{src} does not look like a PithTrain checkout")
        return 2
    target = HERE / "_ref"
    if target.exists():
        shutil.rmtree(target)
    with tempfile.TemporaryDirectory() as tmp:
        copy = Path(tmp) / "src"
        shutil.copytree(src, copy)
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
               "--find-links", "/opt/wheelhouse", "--target", str(target), str(copy)]
        print("$", " ".join(cmd))
        rc = subprocess.call(cmd)
    if rc == 0:
        print(f"installed into {target}")
    return rc


if __name__ == "__main__":
    sys.exit(main())
