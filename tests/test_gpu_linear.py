"""GPU: dequantisation (bit-exact) and the Q4_K / Q6_K linear kernels against the CPU oracle."""
from pathlib import Path

import numpy as np
import pytest

import oracle
from mtlqwen_b200 import device as D
from mtlqwen_b200.testing import synth

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden" / "kquant_dequant.npz"
# BASELINE tolerance for GEMV / GEMM: 1e-3 relative error with fp32 accumulation (normwise per output row
# plus the same bound on the largest element error relative to the largest output).
TOL = 1e-3


def rel_err(got, want):
  want64 = want.astype(np.float64)
  rows = np.linalg.norm(got - want64, axis=-1) / np.maximum(np.linalg.norm(want64, axis=-1), 1e-30)
  return max(float(rows.max()), float(np.abs(got - want64).max() / np.abs(want64).max()))


@pytest.mark.parametrize("name,qtype", [("q4k", D.Q4_K), ("q6k", D.Q6_K)])
def test_dequant_bit_exact_against_golden(dev, name, qtype):
  golden = np.load(GOLDEN)
  blocks, want = golden[name + "_blocks"], golden[name + "_values"]
  out = dev.empty(want.shape)
  dev.dequant(qtype, dev.array(blocks), blocks.shape[0], out)
  assert out.download().tobytes() == want.tobytes()


@pytest.mark.parametrize("qtype", [D.Q4_K, D.Q6_K])
def test_dequant_bit_exact_against_oracle_large(dev, qtype):
  blocks = synth.weight(qtype, 64, 4096, 11)
  out = dev.empty((blocks.shape[0], 256))
  dev.dequant(qtype, dev.array(blocks), blocks.shape[0], out)
  assert out.download().tobytes() == oracle.dequant(blocks, qtype).tobytes()


def run_linear(dev, qtype, n, k, m, seed, residual=False, xsplit=2, integer=True, x=None, w=None):
  """integer: the integer-MMA Q4_K kernel (the default path) or the fp16-MMA kernel."""
  w = synth.weight(qtype, n, k, seed) if w is None else w
  x = synth.activations(m, k, seed + 1) if x is None else x
  res = synth.activations(m, n, seed + 2) if residual else None
  dev.set_xsplit(xsplit)
  dev.set_integer_decode(integer)
  try:
    y = dev.empty((m, n))
    dres = dev.array(res) if residual else None
    dev.linear(qtype, dev.array(w), n, k, dev.array(x), m, y, dres)
    dev.commit()
  finally:
    dev.set_xsplit(2)
    dev.set_integer_decode(True)
  return y.download(), oracle.linear(w, qtype, n, k, x, res)


@pytest.mark.parametrize("integer", [True, False])
@pytest.mark.parametrize("m", [1, 8])
def test_q4k_linear_config1_shape(dev, m, integer):
  """BASELINE config 1: weight 12288 x 4096 Q4_K, fp32 activations ~N(0,1), M in {1, 8}."""
  got, want = run_linear(dev, D.Q4_K, 12288, 4096, m, 1234, integer=integer)
  assert rel_err(got, want) < TOL


def test_integer_kernel_error_level(dev):
  """16-bit activations per 256-value block: the error sits near 3e-5, far inside the contract."""
  got, want = run_linear(dev, D.Q4_K, 4096, 4096, 8, 41)
  assert 1e-7 < rel_err(got, want) < 2e-4


def test_integer_kernel_cannot_overflow(dev):
  """Every quant 15, every scale 63 and constant activations drive the int32 partial sums to their bound."""
  n, k, m = 64, 4096, 8
  blocks = np.zeros((n * k // 256, 144), np.uint8)
  blocks[:, 0:2] = np.frombuffer(np.float16(0.01).tobytes(), np.uint8)
  blocks[:, 2:4] = np.frombuffer(np.float16(0.02).tobytes(), np.uint8)
  blocks[:, 4:16] = 0xFF  # scales and mins 63
  blocks[:, 16:] = 0xFF   # quants 15
  x = np.full((m, k), -3.0, np.float32)
  x[1::2] = 5.0
  got, want = run_linear(dev, D.Q4_K, n, k, m, 0, x=x, w=blocks)
  assert rel_err(got, want) < 1e-5


def test_integer_kernel_with_outliers_and_zero_blocks(dev):
  n, k, m = 256, 4096, 6
  x = synth.activations(m, k, 77)
  x[:, 5::97] *= 200.0   # outlier channels
  x[2, 512:1024] = 0.0   # all-zero blocks
  x[4] = 0.0
  got, want = run_linear(dev, D.Q4_K, n, k, m, 78, x=x)
  assert rel_err(got, want) < TOL


def test_integer_kernel_with_one_large_outlier_per_block(dev):
  """The worst case of the 16-bit activation grid: every 256-value block holds one value of 1e4 among values of
  order one, as the residual stream of a real model does, so the grid step of the block is 1e4 / 32767 = 0.31 and
  the small values keep about two bits. The outlier's own contribution is exact; what the grid costs is judged on
  its own: against the oracle run on the activations without the outliers, the error the kernel adds must stay
  within the rounding bound of the grid, sqrt(k) * step / sqrt(12) * |w|, and this is recorded here as the limit
  of the scheme: such a block is represented to 0.3 absolute, not to 1e-3 of its small values."""
  n, k, m = 256, 4096, 4
  rng = np.random.default_rng(5)
  w = synth.weight(D.Q4_K, n, k, 91)
  small = synth.activations(m, k, 92)
  x = small.copy()
  spots = np.arange(0, k, 256) + rng.integers(0, 256, k // 256)
  x[:, spots] = 1.0e4
  got, want = run_linear(dev, D.Q4_K, n, k, m, 0, x=x, w=w)
  assert rel_err(got, want) < TOL  # dominated by the outliers, as the norm-wise metric is
  # the part of the result that the small values contribute
  only_outliers = np.zeros_like(x)
  only_outliers[:, spots] = 1.0e4
  contribution = got - oracle.linear(w, D.Q4_K, n, k, only_outliers)
  want_small = oracle.linear(w, D.Q4_K, n, k, small - np.where(only_outliers > 0, small, 0).astype(np.float32))
  dense = oracle.dequant(w, D.Q4_K).reshape(n, k)
  step = 1.0e4 / 32767.0
  bound = 5.0 * np.sqrt(k / 12.0) * step * np.sqrt((dense**2).mean())  # five standard deviations of the rounding noise
  error = np.abs(contribution - want_small)
  assert error.max() <= bound, (float(error.max()), float(bound))
  assert error.max() > 1e-3 * np.abs(want_small).max()  # and it is not small: the grid, not the arithmetic, sets it


@pytest.mark.parametrize("qtype,n,k,m", [
  (D.Q4_K, 16, 256, 1),  # one tile, one super-block: most consumer warps idle
  (D.Q4_K, 48, 768, 3),  # partial stage (3 super-blocks)
  (D.Q4_K, 1024, 4096, 5),  # attn_k / attn_v shape, speculative row count
  (D.Q4_K, 4096, 12288, 8),  # ffn_down: three K chunks
  (D.Q4_K, 4096, 8192, 2),  # eh_proj shape
  (D.Q4_K, 2384, 2304, 7),  # ragged: 149 tiles (one more than the SM count), partial chunk
  (D.Q6_K, 16, 2048, 1),
  (D.Q6_K, 4096, 4096, 8),
  (D.Q6_K, 8192, 4096, 3),
  (D.Q6_K, 1024, 12288, 4),
])
def test_linear_shapes(dev, qtype, n, k, m):
  got, want = run_linear(dev, qtype, n, k, m, 77 + n + k + m)
  assert rel_err(got, want) < TOL


def test_linear_residual_in_place(dev):
  n, k, m = 4096, 4096, 8
  w, x, res = synth.weight(D.Q4_K, n, k, 5), synth.activations(m, k, 6), synth.activations(m, n, 7)
  y = dev.array(res)
  dev.linear(D.Q4_K, dev.array(w), n, k, dev.array(x), m, y, y)  # hidden += x.W^T, as Ops::decoder does
  assert rel_err(y.download(), oracle.linear(w, D.Q4_K, n, k, x, res)) < TOL


def test_linear_more_than_eight_rows(dev):
  got, want = run_linear(dev, D.Q4_K, 1024, 4096, 21, 31, residual=True)
  assert rel_err(got, want) < TOL


def test_hi_only_activation_split_stays_inside_tolerance(dev):
  got, want = run_linear(dev, D.Q4_K, 4096, 4096, 8, 41, xsplit=1, integer=False)
  err = rel_err(got, want)
  assert 1e-6 < err < TOL


def test_hi_lo_split_is_fp32_accurate(dev):
  got, want = run_linear(dev, D.Q4_K, 4096, 4096, 8, 41, integer=False)
  assert rel_err(got, want) < 2e-5


def test_subnormal_superblock_scale(dev):
  n, k, m = 64, 1024, 4
  w = synth.q4k_blocks(n * k // 256, np.random.default_rng(9), subnormal=True)
  x = synth.activations(m, k, 10)
  y = dev.empty((m, n))
  dev.linear(D.Q4_K, dev.array(w), n, k, dev.array(x), m, y)
  assert rel_err(y.download(), oracle.linear(w, D.Q4_K, n, k, x)) < TOL


def test_linear_group_shares_activations(dev):
  k, m, ns = 4096, 8, [8192, 1024, 1024]
  ws = [synth.weight(D.Q4_K, n, k, 50 + i) for i, n in enumerate(ns)]
  x = synth.activations(m, k, 60)
  ys = [dev.empty((m, n)) for n in ns]
  dev.linear_group(D.Q4_K, [dev.array(w) for w in ws], ns, k, dev.array(x), m, ys)
  for w, n, y in zip(ws, ns, ys):
    assert rel_err(y.download(), oracle.linear(w, D.Q4_K, n, k, x)) < TOL


@pytest.mark.parametrize("m", [1, 8, 11])
def test_gate_up(dev, m):
  n, k = 12288, 4096
  wg, wu, x = synth.weight(D.Q4_K, n, k, 70), synth.weight(D.Q4_K, n, k, 71), synth.activations(m, k, 72)
  y = dev.empty((m, n))
  dev.gate_up(D.Q4_K, dev.array(wg), dev.array(wu), n, k, dev.array(x), m, y)
  assert rel_err(y.download(), oracle.gate_up(wg, wu, D.Q4_K, n, k, x)) < TOL


def test_bad_arguments_are_refused(dev):
  w, x, y = dev.empty(144 * 16, np.uint8), dev.empty((1, 256)), dev.empty((1, 16))
  assert dev.lib.infdev_linear(dev.ctx, D.Q4_K, w.ptr, 15, 256, x.ptr, 1, y.ptr, None) == -2
  assert dev.lib.infdev_linear(dev.ctx, D.Q4_K, w.ptr, 16, 200, x.ptr, 1, y.ptr, None) == -2
  assert dev.lib.infdev_linear(dev.ctx, 2, w.ptr, 16, 256, x.ptr, 1, y.ptr, None) == -2  # Q4_0: not a type of these files
  assert "linear" in dev.error()


def test_embedding_and_rms_norm(dev):
  rows, k = 5, 4096
  for qtype in (D.Q4_K, D.Q6_K):
    table = synth.weight(qtype, 64, k, 80)
    ids = np.array([3, 0, 63, 17, 3], np.int32)
    out = dev.empty((rows, k))
    dev.embedding(qtype, dev.array(table), k, dev.array(ids), rows, out)
    assert out.download().tobytes() == oracle.embedding(table, qtype, k, ids).tobytes()
  x = synth.activations(rows, k, 81) * 3
  w = (1 + 0.01 * synth.activations(1, k, 82)).reshape(-1)
  y = dev.empty((rows, k))
  dev.rms_norm(dev.array(x), dev.array(w), rows, k, y)
  assert rel_err(y.download(), oracle.rms_norm(x, w)) < 1e-5
