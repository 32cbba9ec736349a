"""Test / measurement infrastructure (not product code): a runnable copy of the reference's own fp32 layer file.

The reference is a plain Python tree without packaging, so "installing" it means copying
``modules/base.py`` -- pure PyTorch, it runs on CPU and on CUDA as it is -- into ``oracle/_ref/``, a
directory that is kept out of version control.  ``install()`` does that wherever a checkout of the
reference is present (it is called by the repository's build step); ``load()`` imports the copy under
a private module name and returns it, or ``None`` when there is no copy.  Only the benchmark's
reference arm and the tests use this; nothing in the product package does.
"""
import importlib.util
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
REF_BASE = os.path.join(REF_DIR, "modules", "base.py")
DEFAULT_ROOT = os.environ.get("NES_REFERENCE_ROOT", "/root/reference")


def install(reference_root=DEFAULT_ROOT):
    """Copy ``<reference_root>/modules/base.py`` to ``oracle/_ref/modules/base.py``.  Returns the path of
    the copy, or None when no reference checkout exists at ``reference_root`` (an existing copy is kept)."""
    src = os.path.join(reference_root, "modules", "base.py")
    if not os.path.isfile(src):
        return REF_BASE if os.path.isfile(REF_BASE) else None
    os.makedirs(os.path.dirname(REF_BASE), exist_ok=True)
    if not os.path.isfile(REF_BASE) or os.path.getmtime(REF_BASE) < os.path.getmtime(src):
        shutil.copyfile(src, REF_BASE)
    return REF_BASE


def available():
    return os.path.isfile(REF_BASE)


def load():
    """The reference's ``modules/base.py`` as a module object (imported once), or None."""
    name = "nes_reference_base"
    if name in sys.modules:
        return sys.modules[name]
    if not available():
        return None
    spec = importlib.util.spec_from_file_location(name, REF_BASE)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod
