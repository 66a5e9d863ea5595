"""The reference implementation itself as the timed CPU baseline and as a second checker.

TEST INFRASTRUCTURE ONLY (see oracle/ref.py): imported by ``bench.py``'s CPU legs and by ``__graft_entry__.build()``.

The reference is a pure-Python package.  ``install(checkout)`` puts its package directory under the
git-ignored ``oracle/_ref/`` (what ``pip install --target`` would do; pip itself fails here because the
project's setup.py imports setuptools_scm, which this image lacks) together with the ``version`` module
its build normally generates.  Nothing under ``oracle/_ref/`` is tracked; it only travels with the
working tree to the machine that runs the benchmark.  ``load()`` imports it from there, ahead of any other
``compressed_tensors`` that may be installed in site-packages, in eager mode.
"""
import importlib
import os
import shutil
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(_HERE, "_ref")
PKG = "compressed_tensors"

_VERSION_STUB = '__all__ = ["__version__", "version"]\n__version__ = version = "0.0.0+checkout"\n'


def available() -> bool:
    return os.path.isfile(os.path.join(REF_DIR, PKG, "__init__.py"))


def install(checkout: str, force: bool = False) -> str:
    """Install the package of the reference checkout at `checkout` into oracle/_ref/."""
    src = os.path.join(checkout, "src", PKG)
    if not os.path.isdir(src):
        raise FileNotFoundError(src)
    dst = os.path.join(REF_DIR, PKG)
    if available() and not force:
        return dst
    os.makedirs(REF_DIR, exist_ok=True)
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    with open(os.path.join(dst, "version.py"), "w") as f:
        f.write(_VERSION_STUB)
    return dst


def load():
    """Import the installed reference (eager mode) and return the package."""
    if not available():
        raise ImportError("the reference is not installed under oracle/_ref/ (oracle.reference.install(checkout))")
    os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    stale = [m for m in sys.modules if m == PKG or m.startswith(PKG + ".")]
    if stale and not getattr(sys.modules.get(PKG), "__file__", "").startswith(REF_DIR):
        for m in stale:
            del sys.modules[m]
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    pkg = importlib.import_module(PKG)
    if not pkg.__file__.startswith(REF_DIR):
        raise ImportError(f"imported {pkg.__file__}, not the reference under {REF_DIR}")
    return pkg
