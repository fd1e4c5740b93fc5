"""GPU: the tcgen05 / TMEM Q4_K prefill GEMM (umma.cu: 9 to 128 activation rows per launch, fp16-dequantised weights
in tensor memory, residual and SiLU*mul epilogues, K slices) against the CPU oracle."""
import numpy as np
import pytest

import oracle
from mtlqwen_b200 import device as D
from mtlqwen_b200.testing import synth

pytestmark = pytest.mark.gpu
TOL = 1e-3  # BASELINE: GEMV / GEMM within 1e-3 relative error, fp32 accumulation


def rel_err(got, want):
  want64 = want.astype(np.float64)
  rows = np.linalg.norm(got - want64, axis=-1) / np.maximum(np.linalg.norm(want64, axis=-1), 1e-30)
  return max(float(rows.max()), float(np.abs(got - want64).max() / np.abs(want64).max()))


@pytest.fixture()
def umma(dev):
  dev.set_umma(1)
  return dev


def run(dev, n, k, m, seed, residual=False, pair=False):
  w, x = synth.weight(D.Q4_K, n, k, seed), synth.activations(m, k, seed + 1)
  y = dev.empty((m, n))
  if pair:
    w2 = synth.weight(D.Q4_K, n, k, seed + 2)
    dev.gate_up(D.Q4_K, dev.array(w), dev.array(w2), n, k, dev.array(x), m, y)
    want = oracle.gate_up(w, w2, D.Q4_K, n, k, x)
  else:
    res = synth.activations(m, n, seed + 3) if residual else None
    dev.linear(D.Q4_K, dev.array(w), n, k, dev.array(x), m, y, dev.array(res) if residual else None)
    want = oracle.linear(w, D.Q4_K, n, k, x, res)
  dev.commit()
  return rel_err(y.download(), want)


@pytest.mark.parametrize("n,k,m", [(128, 2048, 128), (256, 4096, 21), (12288, 4096, 128), (4096, 12288, 100), (1024, 4096, 300), (128, 2048, 9),
                                   (19072, 4096, 40)])  # 149 tiles: one more than the SM count
def test_prefill_mode_within_tolerance(umma, n, k, m):
  assert run(umma, n, k, m, 500 + n + k + m, residual=(m % 2 == 0)) < TOL


def test_prefill_mode_gate_up_epilogue(umma):
  assert run(umma, 12288, 4096, 128, 610, pair=True) < TOL


def test_group_launch_on_tcgen05_path(umma):
  k, m, ns = 4096, 24, [8192, 1024, 1024]
  ws = [synth.weight(D.Q4_K, n, k, 700 + i) for i, n in enumerate(ns)]
  x = synth.activations(m, k, 710)
  ys = [umma.empty((m, n)) for n in ns]
  umma.linear_group(D.Q4_K, [umma.array(w) for w in ws], ns, k, umma.array(x), m, ys)
  for w, n, y in zip(ws, ns, ys):
    assert rel_err(y.download(), oracle.linear(w, D.Q4_K, n, k, x)) < TOL


def test_up_to_eight_rows_stay_on_the_gemv(umma):
  """Launches of at most 8 rows never take the GEMM: they keep the accuracy of the decode kernels."""
  assert run(umma, 12288, 4096, 8, 1300) < 1e-4


def test_prefill_k_slices(umma):
  """A matrix of few 128-row tiles is cut along K (three launches: layout, GEMM over (tile, slice) items, fixed-order
  sum of the slices plus residual); the result is reproducible bit for bit."""
  n, k, m = 4096, 12288, 128
  w, x, res = umma.array(synth.weight(D.Q4_K, n, k, 900)), umma.array(synth.activations(m, k, 901)), umma.array(synth.activations(m, n, 902))
  a, b = umma.empty((m, n)), umma.empty((m, n))
  before = umma.launch_count
  umma.linear(D.Q4_K, w, n, k, x, m, a, res)
  assert umma.launch_count - before == 3
  umma.linear(D.Q4_K, w, n, k, x, m, b, res)
  assert a.download().tobytes() == b.download().tobytes()
