"""Install the unmodified reference (loreloc/triturus) into baseline/_ref for side-by-side runs on the GPU box.

    python baseline/install_reference.py [path to a checkout of the reference]

baseline/_ref is git-ignored: nothing of the reference enters this repository's history.  Two things land
there:

* baseline/_ref/triturus/ - the reference package, installed by pip from a scratch copy of the checkout
  (pip builds in the source tree, and the checkout may be read-only).  `--no-deps` because the reference
  pins torch==2.7.1 / triton==3.3.1 and the image carries newer ones.
* baseline/_ref/suite/{baselines,tests}/ - the reference's torch baselines and its two hot-path test files
  with their conftest, which its wheel does not package (`packages.find` includes only `triturus`).

Users: tests/test_reference_triton_gpu.py (parity with the reference's Triton kernels, and the reference's
own tests run unmodified against this repository's drop-in package) and `bench.py`'s `triton_ref` timings.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"
# a checkout of the reference next to this repository, unless the environment names another place
DEFAULT_CHECKOUT = Path(os.environ.get("TRITURUS_REFERENCE_DIR", str(HERE.parent.parent / "reference")))


def install(checkout: Path = DEFAULT_CHECKOUT, force: bool = False) -> bool:
    """Returns True when baseline/_ref holds the reference afterwards."""
    marker = REF_DIR / "triturus" / "lm2exp.py"
    suite = REF_DIR / "suite"
    if marker.exists() and (suite / "tests" / "lm2exp.py").exists() and not force:
        return True
    if not (checkout / "pyproject.toml").exists():
        return marker.exists()
    with tempfile.TemporaryDirectory() as tmp:
        src = Path(tmp) / "reference"
        shutil.copytree(checkout, src)
        cmd = [sys.executable, "-m", "pip", "install", "--quiet", "--no-index", "--no-build-isolation", "--no-deps",
               "--find-links", "/opt/wheelhouse", "--upgrade", "--target", str(REF_DIR), str(src)]  # fmt: skip
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"pip install of the reference failed:\n{proc.stdout}\n{proc.stderr}")
    suite.mkdir(parents=True, exist_ok=True)
    for sub, names in (("baselines", ("__init__.py", "lm2exp.py", "lt2exp.py")),
                       ("tests", ("conftest.py", "lm2exp.py", "lt2exp.py"))):  # fmt: skip
        (suite / sub).mkdir(exist_ok=True)
        for name in names:
            shutil.copyfile(checkout / sub / name, suite / sub / name)
    return marker.exists()


if __name__ == "__main__":
    args = [x for x in sys.argv[1:] if not x.startswith("--")]
    ok = install(Path(args[0]) if args else DEFAULT_CHECKOUT, force="--force" in sys.argv)
    print("reference installed in", REF_DIR if ok else "(nothing: no checkout found)")
