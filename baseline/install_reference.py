"""Place an unmodified copy of the reference package under ``baseline/_ref`` (git-ignored).

The prescribed ``pip install --no-index --no-build-isolation --find-links /opt/wheelhouse --target baseline/_ref
<reference>`` fails because the reference ships neither ``setup.py`` nor ``pyproject.toml`` ("Directory is not
installable"); its own instructions put ``gt3d/`` on ``PYTHONPATH`` instead, which is what this script reproduces by
copying the package directory byte for byte."""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def reference_source():
    """Where the reference checkout lives: ``GT_REFERENCE_SRC`` or the ``reference_path`` recorded in ``BASELINE.json``."""
    if os.environ.get("GT_REFERENCE_SRC"):
        return os.environ["GT_REFERENCE_SRC"]
    import json
    with open(os.path.join(os.path.dirname(HERE), "BASELINE.json")) as f:
        return json.load(f)["reference_path"]


def install(src=None):
    src = src or reference_source()
    dst = os.path.join(HERE, "_ref")
    pkg = os.path.join(src, "gt3d", "gt3d")
    if not os.path.isdir(pkg):
        raise SystemExit(f"reference package not found at {pkg}")
    os.makedirs(dst, exist_ok=True)
    target = os.path.join(dst, "gt3d")
    if os.path.isdir(target):
        shutil.rmtree(target)
    shutil.copytree(pkg, target, ignore=shutil.ignore_patterns("__pycache__", "*.so", "pullcomm"))
    print("copied", pkg, "->", target)


if __name__ == "__main__":
    install(*sys.argv[1:])
