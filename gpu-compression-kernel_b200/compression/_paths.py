"""Makes the `s24` package importable from the drop-in modules, which (like the reference's
files) are meant to be imported flat from this directory or loaded by path."""
import sys
from pathlib import Path

_PKG_ROOT = str(Path(__file__).resolve().parent.parent)
if _PKG_ROOT not in sys.path:
    sys.path.insert(0, _PKG_ROOT)
