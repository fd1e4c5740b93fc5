"""GPU: the failure paths of the device layer, exercised without faulting or hanging anything: a commit deadline that
passes while legitimate work is still queued, and a kernel whose bounded wait gives up."""
import numpy as np
import pytest

from mtlqwen_b200 import device as D
from mtlqwen_b200.testing import synth

pytestmark = pytest.mark.gpu
E_TIMEOUT, E_DEVICE = -3, -4


def test_commit_deadline_passes_behind_queued_work_and_the_context_survives():
  """Some hundred large GEMV launches take tens of milliseconds; a commit with a 1 ms deadline reports
  INFDEV_E_TIMEOUT while they run, an untimed commit afterwards succeeds, and the results are right."""
  dev = D.Device(0)
  try:
    n, k, m = 32768, 4096, 8
    w, x, y = dev.array(synth.weight(D.Q6_K, n, k, 1)), dev.array(synth.activations(m, k, 2)), dev.empty((m, n))
    dev.linear(D.Q6_K, w, n, k, x, m, y)
    dev.commit()
    first = y.download()
    for _ in range(400):
      dev.linear(D.Q6_K, w, n, k, x, m, y)
    assert dev.lib.infdev_commit(dev.ctx, 1) == E_TIMEOUT
    assert "deadline" in dev.error()
    assert dev.lib.infdev_commit(dev.ctx, 0) == 0
    assert y.download().tobytes() == first.tobytes()
  finally:
    dev.close()


def test_a_bounded_wait_that_gives_up_is_reported_once_and_the_context_survives():
  dev = D.Device(0)
  try:
    n, k, m = 512, 1024, 4
    w, x, y = dev.array(synth.weight(D.Q4_K, n, k, 3)), dev.array(synth.activations(m, k, 4)), dev.empty((m, n))
    dev.linear(D.Q4_K, w, n, k, x, m, y)
    dev.commit()
    before = y.download()
    dev.check(dev.lib.infdev_check_abort_path(dev.ctx, 2000))
    assert dev.lib.infdev_commit(dev.ctx, 10000) == E_DEVICE
    assert "bounded wait" in dev.error()
    assert dev.lib.infdev_commit(dev.ctx, 10000) == 0  # the status word was cleared
    dev.linear(D.Q4_K, w, n, k, x, m, y)
    dev.commit()
    assert y.download().tobytes() == before.tobytes()
    assert dev.lib.infdev_check_abort_path(dev.ctx, 0) == -2  # argument check
  finally:
    dev.close()


def test_two_contexts_on_one_device_run_every_large_shared_memory_kernel():
  """The opt-in to large dynamic shared memory is recorded per device, not per context or per process."""
  results = []
  for _ in range(2):
    dev = D.Device(0)
    try:
      n, k = 256, 4096
      w4, w6 = dev.array(synth.weight(D.Q4_K, n, k, 5)), dev.array(synth.weight(D.Q6_K, n, k, 6))
      x8, x40 = dev.array(synth.activations(8, k, 7)), dev.array(synth.activations(40, k, 8))
      y8, y6, y40 = dev.empty((8, n)), dev.empty((8, n)), dev.empty((40, n))
      dev.linear(D.Q4_K, w4, n, k, x8, 8, y8)    # integer decode kernel
      dev.linear(D.Q6_K, w6, n, k, x8, 8, y6)    # fp16-MMA kernel
      dev.linear(D.Q4_K, w4, n, k, x40, 40, y40)  # tcgen05 GEMM
      dev.commit()
      results.append((y8.download().tobytes(), y6.download().tobytes(), y40.download().tobytes()))
    finally:
      dev.close()
  assert results[0] == results[1]
