"""Byte-compile the reference's front-end modules for machines that have no checkout of it.

    python -m rexsc_b200.frontend.build [reference_root] [--force]

Like the reference's C++/CUDA extensions that the test-suite compiles into ``oracle/_ref``, this is a BUILD OUTPUT
of the unchanged reference sources, compiled from where they lie: one ``<module>.pycode`` per module (the
``py_compile`` output under another extension, because snapshot tools commonly drop ``*.pyc``) under
``baseline/_ref/frontend/`` (a git-ignored directory; no source text is copied anywhere).  ``frontend.load()``
imports from there when no checkout is reachable.  Does nothing when the checkout is absent.
"""
from __future__ import annotations

import os
import py_compile
import sys

from . import COMPILED, COMPILED_EXT, MODULES, reference_root


def build(root: str | None = None, force: bool = False) -> bool:
    """Return True when every module is available under baseline/_ref/frontend after the call."""
    src_root = reference_root(root)
    os.makedirs(COMPILED, exist_ok=True)
    ok = True
    for name in MODULES:
        out = os.path.join(COMPILED, name + COMPILED_EXT)
        if src_root is None:
            ok = ok and os.path.exists(out)
            continue
        src = os.path.join(src_root, name + ".py")
        if force or not os.path.exists(out) or os.path.getmtime(out) < os.path.getmtime(src):
            # unchecked-hash pyc: valid wherever the same interpreter version runs, whatever the source's mtime
            py_compile.compile(src, cfile=out, dfile=name + ".py", doraise=True,
                               invalidation_mode=py_compile.PycInvalidationMode.UNCHECKED_HASH)
    return ok


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    good = build(args[0] if args else None, force="--force" in sys.argv)
    print("baseline/_ref/frontend:", "ready" if good else "reference checkout not available; nothing built")
