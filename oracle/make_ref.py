"""Stage the reference's own CPU implementation of the path for the timed baseline (BENCH
INFRASTRUCTURE, like the rest of this package).

The reference is pure Python on this path: its quantiser, page writer and page reader live in
one module, ``quant/beyond_cute.py``.  There is nothing to compile; "building" it means placing
that one file, unmodified, under ``oracle/_ref/`` - a directory that is git-ignored, so the
reference source never enters this repository's history, but that travels with a working copy
to the machine the benchmark runs on, where no reference checkout exists.

    python oracle/make_ref.py [/path/to/Beyond-KV-Cache]

Without an argument the checkout is looked for in $BEYOND_REFERENCE and in a directory
``reference`` beside this repository.  When there is none the script says so and leaves
``oracle/_ref`` alone; the benchmark then times the numpy restatement instead (kind "port").
"""

from __future__ import annotations

import hashlib
import importlib.util
import json
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
MODULE_RELATIVE = os.path.join("quant", "beyond_cute.py")
STAGED = os.path.join(REF_DIR, "beyond_cute_reference.py")
STAMP = os.path.join(REF_DIR, "STAMP.json")


def find_checkout(explicit: str | None = None) -> str | None:
    repo = os.path.dirname(HERE)
    for cand in (explicit, os.environ.get("BEYOND_REFERENCE"), os.path.join(os.path.dirname(repo), "reference")):
        if cand and os.path.isfile(os.path.join(cand, MODULE_RELATIVE)):
            return os.path.abspath(cand)
    return None


def make_ref(checkout: str | None = None) -> str | None:
    """Place the reference module under ``oracle/_ref``; returns its path, or None without a checkout."""
    root = find_checkout(checkout)
    if root is None:
        return STAGED if os.path.isfile(STAGED) else None
    os.makedirs(REF_DIR, exist_ok=True)
    src = os.path.join(root, MODULE_RELATIVE)
    shutil.copyfile(src, STAGED)
    with open(src, "rb") as f:
        digest = hashlib.sha256(f.read()).hexdigest()
    with open(STAMP, "w") as f:
        json.dump({"module": MODULE_RELATIVE.replace(os.sep, "/"), "sha256": digest, "modified": False}, f)
    return STAGED


def load_ref():
    """The staged reference module, imported under a private name; None when it is not staged."""
    if not os.path.isfile(STAGED):
        return None
    name = "bkv_reference_beyond_cute"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, STAGED)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod  # the module defines dataclasses, which look their module up by name
    try:
        spec.loader.exec_module(mod)
    except Exception:
        sys.modules.pop(name, None)
        raise
    return mod


if __name__ == "__main__":
    path = make_ref(sys.argv[1] if len(sys.argv) > 1 else None)
    print(f"staged {path}" if path else "no reference checkout found: oracle/_ref left as it is")
