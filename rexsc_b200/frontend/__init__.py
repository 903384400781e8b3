"""Run the reference's UNCHANGED Python front end on top of this library.

The front end of nanocad-lab/rex-sc (``utils_functional.py``, ``utils_class.py``, ``resnet_sc.py``, ``network.py``,
``utils_own.py``, ``utils.py``, ``config.py``) is not part of this package and is never edited or re-implemented.
:func:`load` only arranges ``sys.path`` so that those modules import here and now:

* ``sc_extension_cuda`` / ``fixed_extension_cuda`` / ``sc_extension`` / ``fixed_extension``
  (utils_functional.py:17-20) resolve to ``rexsc_b200/dropin``;
* ``bokeh``, ``nvidia.dali`` and ``nvidia_smi`` (utils.py:7-17, utils_own.py:28), which only the reference's plotting
  and data-loading code touches, resolve to the import stand-ins under ``stubs/`` when the real packages are absent;
* the reference's own modules come from a checkout (``reference_root`` argument or ``REXSC_REFERENCE_ROOT``) or,
  on a machine without a checkout, from the byte-compiled copy that ``python -m rexsc_b200.frontend.build`` writes
  (``baseline/_ref/frontend/<module>.pycode``: a code object per module, imported through a small finder because
  snapshot tools commonly drop ``*.pyc``).  TorchScript needs source text, so for the byte-compiled copy
  ``torch.jit.script`` is switched off while the modules are imported: the 27 small scripted helpers of
  utils_functional.py:286-459 then run as the plain Python functions they decorate (same ATen calls).
"""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import marshal
import os
import sys
import types
from typing import Optional

HERE = os.path.dirname(os.path.abspath(__file__))
STUBS = os.path.join(HERE, "stubs")
REPO = os.path.dirname(os.path.dirname(HERE))
COMPILED = os.path.join(REPO, "baseline", "_ref", "frontend")

# modules of the reference that the SC path uses, in import order
MODULES = ("config", "utils_functional", "utils_class", "network", "utils", "utils_own", "resnet_sc")

COMPILED_EXT = ".pycode"      # py_compile output (16-byte header + marshalled code object) under another extension

_loaded: Optional[types.SimpleNamespace] = None


class _CompiledFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    """Imports the reference's top-level modules from their byte-compiled copies under ``COMPILED``."""

    def find_spec(self, name, path=None, target=None):
        if path is not None or name not in MODULES:
            return None
        f = os.path.join(COMPILED, name + COMPILED_EXT)
        if not os.path.exists(f):
            return None
        return importlib.util.spec_from_loader(name, self, origin=f)

    def create_module(self, spec):
        return None

    def exec_module(self, module):
        with open(module.__spec__.origin, "rb") as fh:
            data = fh.read()
        if data[:4] != importlib.util.MAGIC_NUMBER:
            raise ImportError(f"{module.__spec__.origin} was compiled by another Python version; rebuild it with "
                              "`python -m rexsc_b200.frontend.build --force`")
        module.__file__ = module.__spec__.origin
        exec(marshal.loads(data[16:]), module.__dict__)


def have_compiled() -> bool:
    return all(os.path.exists(os.path.join(COMPILED, m + COMPILED_EXT)) for m in MODULES)


def reference_root(explicit: Optional[str] = None) -> Optional[str]:
    """Directory of a reference checkout, or None.  Order: argument, ``REXSC_REFERENCE_ROOT``, the
    ``reference_path`` entry of a ``BASELINE.json`` next to the package."""
    cands = [explicit, os.environ.get("REXSC_REFERENCE_ROOT")]
    meta = os.path.join(REPO, "BASELINE.json")
    if os.path.exists(meta):
        try:
            import json

            with open(meta) as fh:
                cands.append(json.load(fh).get("reference_path"))
        except Exception:
            pass
    for c in cands:
        if c and os.path.exists(os.path.join(c, "utils_functional.py")):
            return c
    return None


def _install_stubs() -> None:
    """Make ``bokeh``, ``nvidia.dali`` and ``nvidia_smi`` importable without shadowing real installations."""
    if STUBS not in sys.path:
        sys.path.append(STUBS)  # at the end: an installed package of the same name is found first
    try:
        importlib.import_module("nvidia.dali")
    except ImportError:
        # ``nvidia`` exists (the CUDA wheels install a regular package of that name) but has no ``dali``:
        # let the stand-in directory extend its search path
        nv = sys.modules.get("nvidia")
        if nv is None:
            nv = importlib.import_module("nvidia")
        stub_nv = os.path.join(STUBS, "nvidia")
        if stub_nv not in list(nv.__path__):
            nv.__path__.append(stub_nv)
        importlib.import_module("nvidia.dali")


def load(reference_root_dir: Optional[str] = None) -> types.SimpleNamespace:
    """Import the reference's front-end modules on top of the drop-in ops and return them as a namespace
    (``fe.utils_functional``, ``fe.utils_class``, ``fe.resnet_sc``, ``fe.network``, ``fe.utils_own``, ``fe.utils``,
    ``fe.config``; ``fe.root`` is where they came from, ``fe.sourceless`` whether that is the byte-compiled copy)."""
    global _loaded
    if _loaded is not None:
        return _loaded
    import torch

    from .. import install_dropin

    install_dropin()
    _install_stubs()
    # REXSC_FRONTEND_COMPILED=1 forces the byte-compiled copy even where a checkout is reachable (used to test it)
    forced = os.environ.get("REXSC_FRONTEND_COMPILED", "0") == "1"
    root = None if forced else reference_root(reference_root_dir)
    sourceless = False
    if root is None:
        if not have_compiled():
            raise ImportError(
                "the reference front end is not available: set REXSC_REFERENCE_ROOT to a checkout of "
                "nanocad-lab/rex-sc, or run `python -m rexsc_b200.frontend.build` where one is present")
        root, sourceless = COMPILED, True
        if not any(isinstance(f, _CompiledFinder) for f in sys.meta_path):
            sys.meta_path.insert(0, _CompiledFinder())
    elif root not in sys.path:
        sys.path.insert(0, root)
    jit_was_on = bool(torch.jit._state._enabled)
    if sourceless and jit_was_on:
        torch.jit._state.disable()
    try:
        mods = {name: importlib.import_module(name) for name in MODULES}
    finally:
        if sourceless and jit_was_on:
            torch.jit._state.enable()
    _loaded = types.SimpleNamespace(root=root, sourceless=sourceless, **mods)
    return _loaded
