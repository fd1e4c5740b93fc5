"""GPU: activation images - the quantised operand of the integer Q4_K decode kernel - written by the standalone
kernel and by the producers that fuse it, and read back through infdev_image_supply."""
import numpy as np
import pytest

import oracle
from mtlqwen_b200 import device as D
from mtlqwen_b200.testing import images, synth

pytestmark = pytest.mark.gpu


def image_buffer(dev, rows, k):
  return dev.empty(dev.image_bytes(rows, k), np.uint8)


def same_image(got, want, rows, k):
  for a, b in zip(images.decode(got, rows, k), images.decode(want, rows, k)):
    if a.tobytes() != b.tobytes():
      return False
  return True


@pytest.mark.parametrize("rows", [1, 8, 11])
def test_quantize_matches_numpy(dev, rows):
  k = 4096
  x = synth.activations(rows, k, 5)
  x[0, 256:512] = 0.0          # an all-zero block
  x[-1, 7] = 1000.0            # an outlier
  image = image_buffer(dev, rows, k)
  dev.quantize(dev.array(x), rows, k, image)
  x_int, xs, sums = images.decode(image.download(), rows, k)
  want_int, want_xs, want_sums = images.quantize(x)
  assert np.array_equal(x_int, want_int)
  assert xs.tobytes() == want_xs.tobytes()
  assert np.array_equal(sums, want_sums)
  assert np.abs(x_int * np.repeat(xs, 256, axis=1) - x).max() <= 0.5001 * xs.max()


def test_rms_norm_writes_the_image_of_its_result(dev):
  rows, k = 8, 4096
  x, w = synth.activations(rows, k, 6), (1 + 0.01 * synth.activations(1, k, 7)[0]).astype(np.float32)
  y, plain = dev.empty((rows, k)), dev.empty((rows, k))
  image, want = image_buffer(dev, rows, k), image_buffer(dev, rows, k)
  dev.rms_norm(dev.array(x), dev.array(w), rows, k, plain)
  dev.image_capture(image)
  dev.rms_norm(dev.array(x), dev.array(w), rows, k, y)
  dev.quantize(y, rows, k, want)
  assert y.download().tobytes() == plain.download().tobytes()
  assert same_image(image.download(), want.download(), rows, k)


@pytest.mark.parametrize("m", [3, 8])
def test_supplied_image_gives_the_same_linear_result(dev, m):
  n, k = 1024, 4096
  w, x = dev.array(synth.weight(D.Q4_K, n, k, 8)), dev.array(synth.activations(m, k, 9))
  image = image_buffer(dev, m, k)
  dev.quantize(x, m, k, image)
  a, b = dev.empty((m, n)), dev.empty((m, n))
  dev.linear(D.Q4_K, w, n, k, x, m, a)
  before = dev.launch_count
  dev.image_supply(image)
  dev.linear(D.Q4_K, w, n, k, x, m, b)
  assert dev.launch_count - before == 1  # no quantisation launch
  assert a.download().tobytes() == b.download().tobytes()


@pytest.mark.parametrize("m", [1, 5, 8])
def test_gate_up_writes_the_image_of_its_result(dev, m):
  n, k = 12288, 4096
  wg, wu, x = synth.weight(D.Q4_K, n, k, 70), synth.weight(D.Q4_K, n, k, 71), synth.activations(m, k, 72)
  y, image, want = dev.empty((m, n)), image_buffer(dev, m, n), image_buffer(dev, m, n)
  dev.image_capture(image)
  dev.gate_up(D.Q4_K, dev.array(wg), dev.array(wu), n, k, dev.array(x), m, y)
  dev.quantize(y, m, n, want)
  assert same_image(image.download(), want.download(), m, n)
  got = y.download()
  assert np.abs(got - oracle.gate_up(wg, wu, D.Q4_K, n, k, x)).max() < 1e-3 * np.abs(got).max()


def test_linear_capture_outside_the_integer_kernel(dev):
  """More than 8 rows take another kernel; the image then comes from a quantisation launch on the result."""
  n, k, m = 1024, 4096, 11
  w, x = dev.array(synth.weight(D.Q4_K, n, k, 12)), dev.array(synth.activations(m, k, 13))
  y, image, want = dev.empty((m, n)), image_buffer(dev, m, n), image_buffer(dev, m, n)
  dev.image_capture(image)
  dev.linear(D.Q4_K, w, n, k, x, m, y)
  dev.quantize(y, m, n, want)
  assert same_image(image.download(), want.download(), m, n)


def test_capture_needs_whole_blocks(dev):
  n, k, m = 16, 256, 1
  w, x, y = dev.empty(144 * n, np.uint8), dev.empty((m, k)), dev.empty((m, n))
  dev.image_capture(image_buffer(dev, 8, 256))
  with pytest.raises(RuntimeError, match="multiple of 256"):
    dev.linear(D.Q4_K, w, n, k, x, m, y)
