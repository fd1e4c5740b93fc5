import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def pytest_configure(config):
  config.addinivalue_line("markers", "gpu: needs a B200; runs the CUDA kernels through the C ABI")


@pytest.fixture(scope="session")
def dev():
  """One infdev context for the whole GPU session (creation fails loudly without a B200)."""
  from mtlqwen_b200 import device
  d = device.Device(0)
  yield d
  d.close()
