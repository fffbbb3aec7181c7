"""Locates and imports the product package for the stand-in extension modules."""
import importlib
import sys
from pathlib import Path

_ROOT = Path(__file__).resolve().parents[2]


def package():
    if str(_ROOT) not in sys.path:
        sys.path.insert(0, str(_ROOT))
    return importlib.import_module(Path(__file__).resolve().parents[1].name)
