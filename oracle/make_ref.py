"""Puts an unmodified copy of the reference's Python package where the benchmark's reference arm can
import it. TEST / MEASUREMENT INFRASTRUCTURE ONLY.

    python oracle/make_ref.py [path of the reference checkout]

Copies `<checkout>/xma` to `oracle/_ref/xma`. `oracle/_ref/` is listed in `.gitignore`: the copy never
enters this repository's history, it only travels with the working tree to the machine that runs
`bench.py --impl reference`, where the reference checkout itself does not exist. No file is edited.
The one documented workaround the reference needs (it forgets to forward `kernel_backend` to
`continuous_count` at xma/layers/moe/__init__.py:219) is applied by the caller at run time, by
rebinding that name (see `oracle/ref_runner.py`).
"""

from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
DEFAULT_SOURCE = "/root/reference"


def make_ref(source: str = DEFAULT_SOURCE) -> str | None:
    """Returns the directory that holds the copied `xma` package, or None when there is no checkout."""
    package = os.path.join(source, "xma")
    if not os.path.isdir(package):
        return None
    target = os.path.join(DEST, "xma")
    if os.path.isdir(target):
        shutil.rmtree(target)
    os.makedirs(DEST, exist_ok=True)
    shutil.copytree(package, target, ignore=shutil.ignore_patterns("__pycache__", "*.pyc", "build"))
    with open(os.path.join(DEST, "SOURCE.txt"), "w") as fh:
        fh.write(f"unmodified copy of {package}\n")
    return DEST


def ref_path() -> str | None:
    """Where the copy lives, if it has been made."""
    return DEST if os.path.isdir(os.path.join(DEST, "xma")) else None


if __name__ == "__main__":
    out = make_ref(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_SOURCE)
    print(out if out else "no reference checkout found; nothing copied")
