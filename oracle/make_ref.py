"""Build ``oracle/_ref/``: an importable copy of the reference's own model code.

    python oracle/make_ref.py [--src /path/to/reference/src]

TEST INFRASTRUCTURE, not product code.  The reference is pure Python / PyTorch, so "building" it
means collecting the modules its policy needs.  This script imports
``boost_and_broadside.models.yemong.{attention,griffin,encoder,policy}`` from the reference's
source tree, lists every ``boost_and_broadside.*`` module that import pulled in (its import
closure) and copies exactly those files, unmodified, into ``oracle/_ref/boost_and_broadside/``.
The folder is git-ignored (nothing of the reference enters the history) but it travels to a GPU
machine with the working tree, where the reference's tree itself does not exist; there it is

* the CPU baseline ``bench.py --impl reference`` times (the reference's modules, chained as
  models/yemong/policy.py:327-340 does),
* the same-box GPU comparator of ``bench.py`` (eager and torch.compile), and
* the unmodified policy the swapped-block parity tests compare against.

``ref_path()`` returns the folder to put on ``sys.path`` (or None when it has not been built).
"""

from __future__ import annotations

import argparse
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
DEFAULT_SRC = os.environ.get("BNB_REFERENCE_SRC", "/root/reference/src")
ROOT_MODULES = (
    "boost_and_broadside.models.yemong.attention",
    "boost_and_broadside.models.yemong.griffin",
    "boost_and_broadside.models.yemong.encoder",
    "boost_and_broadside.models.yemong.policy",
    "boost_and_broadside.config",
)


def ref_path() -> str | None:
    """Folder holding the copied ``boost_and_broadside`` package, or None if absent."""
    return DEST if os.path.isfile(os.path.join(DEST, "boost_and_broadside", "__init__.py")) else None


def make(src: str = DEFAULT_SRC, quiet: bool = False) -> str | None:
    """Copy the import closure; returns DEST, or None when the reference tree is not there."""
    if not os.path.isdir(os.path.join(src, "boost_and_broadside")):
        return None
    import importlib
    import subprocess

    # list the closure in a child interpreter so this process keeps a clean sys.modules
    code = (
        "import sys, importlib, json\n"
        f"sys.path.insert(0, {src!r})\n"
        f"[importlib.import_module(m) for m in {ROOT_MODULES!r}]\n"
        "print(json.dumps(sorted(m.__file__ for n, m in sys.modules.items() "
        "if n.split('.')[0] == 'boost_and_broadside' and getattr(m, '__file__', None))))\n"
    )
    import json

    out = subprocess.run([sys.executable, "-c", code], check=True, capture_output=True, text=True).stdout
    files = json.loads(out.strip().splitlines()[-1])
    if os.path.isdir(DEST):
        shutil.rmtree(DEST)
    n = 0
    for f in files:
        rel = os.path.relpath(f, src)
        if rel.startswith(".."):
            continue
        dst = os.path.join(DEST, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(f, dst)
        n += 1
    if not quiet:
        print(f"copied {n} modules of the reference's import closure into {DEST}")
    importlib.invalidate_caches()
    return DEST


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", default=DEFAULT_SRC)
    a = ap.parse_args()
    if make(a.src) is None:
        raise SystemExit(f"no reference tree at {a.src}")
