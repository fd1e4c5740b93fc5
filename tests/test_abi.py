"""CPU: the shared library builds, loads and exports every symbol that include/*.h declares."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
  names = []
  for header in sorted((ROOT / "include").glob("*.h")):
    text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
    names += re.findall(r"\b(inf(?:dev|eng)_[a-z0-9_]+)\s*\(", text)
  return sorted(set(names))


def test_library_exports_every_declared_entry_point():
  from mtlqwen_b200 import build
  lib = ctypes.CDLL(str(build.build()))
  symbols = declared_symbols()
  assert len(symbols) >= 20
  missing = [name for name in symbols if not hasattr(lib, name)]
  assert not missing, missing


def test_python_binding_declares_the_same_device_symbols():
  from mtlqwen_b200 import device
  lib = device.library()
  declared = {name for name in declared_symbols() if name.startswith("infdev_")}
  assert declared == set(lib._infdev_symbols), declared ^ set(lib._infdev_symbols)
