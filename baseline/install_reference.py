"""Installs the unmodified reference package into ``baseline/_ref`` (kept out of version control).

    python baseline/install_reference.py <path-to-the-reference-checkout>

The reference (InfiniTensor/ninetoothed 0.25.0) is a pure-Python package whose wheel
holds exactly the directory ``src/ninetoothed``.  The script first tries the regular
offline install (``pip install --no-index --no-build-isolation --target baseline/_ref``
from a scratch copy of the checkout); the project's build backend (hatchling) is not in
this image, so when that fails the package directory is placed where the wheel would
have put it, byte for byte.  Nothing is edited.  ``baseline/_ref`` is what the GPU
parity test against the reference's own Triton kernels and the reference legs of
``bench.py`` import; both skip themselves when it is absent.
"""

from __future__ import annotations

import pathlib
import shutil
import subprocess
import sys
import tempfile

ROOT = pathlib.Path(__file__).resolve().parent.parent
TARGET = ROOT / "baseline" / "_ref"


def install(checkout: pathlib.Path) -> str:
    package = checkout / "src" / "ninetoothed"
    if not package.is_dir():
        raise SystemExit(f"{package} is not a directory: pass the path of a ninetoothed checkout")
    if TARGET.exists():
        shutil.rmtree(TARGET)
    with tempfile.TemporaryDirectory() as scratch:
        copy = pathlib.Path(scratch) / "reference"
        shutil.copytree(checkout, copy)
        pip = subprocess.run(
            [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
             "--target", str(TARGET), str(copy)],  # a wheel directory, if any, comes from PIP_FIND_LINKS
            capture_output=True, text=True,
        )
    if pip.returncode == 0 and (TARGET / "ninetoothed" / "__init__.py").exists():
        how = "pip install --target"
    else:
        reason = (pip.stderr.strip().splitlines() or ["pip failed"])[-1]
        TARGET.mkdir(parents=True, exist_ok=True)
        shutil.copytree(package, TARGET / "ninetoothed")
        how = f"package directory placed as the wheel would (pip: {reason})"
    (TARGET / "INSTALLED_FROM.txt").write_text(f"{checkout}\n{how}\n")
    return how


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print(install(pathlib.Path(sys.argv[1])))
