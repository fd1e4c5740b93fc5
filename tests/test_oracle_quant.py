"""CPU: the oracle's K-quant dequantisers against the gguf-py golden vectors, and oracle self-consistency."""
from pathlib import Path

import numpy as np

import oracle
from mtlqwen_b200.testing import synth

GOLDEN = Path(__file__).resolve().parent / "golden" / "kquant_dequant.npz"


def test_q4k_dequant_matches_gguf_py_bit_exact():
  golden = np.load(GOLDEN)
  got = oracle.dequant(golden["q4k_blocks"], oracle.Q4_K)
  assert got.tobytes() == golden["q4k_values"].tobytes()


def test_q6k_dequant_matches_gguf_py_bit_exact():
  golden = np.load(GOLDEN)
  got = oracle.dequant(golden["q6k_blocks"], oracle.Q6_K)
  assert got.tobytes() == golden["q6k_values"].tobytes()


def test_synthetic_weights_have_the_configured_distribution():
  w = oracle.dequant(synth.weight(synth.Q4_K, 64, 4096, 1), oracle.Q4_K)
  assert abs(w.mean()) < 2e-3 and 0.015 < w.std() < 0.025
  w = oracle.dequant(synth.weight(synth.Q6_K, 64, 4096, 2), oracle.Q6_K)
  assert abs(w.mean()) < 2e-3 and 0.015 < w.std() < 0.025


def test_linear_matches_dense_matmul():
  n, k, m = 48, 512, 3
  for qtype in (oracle.Q4_K, oracle.Q6_K):
    w = synth.weight(qtype, n, k, 3)
    x = synth.activations(m, k, 4)
    dense = oracle.dequant(w, qtype).reshape(n, k).astype(np.float64)
    want = x.astype(np.float64) @ dense.T
    got = oracle.linear(w, qtype, n, k, x)
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
    res = synth.activations(m, n, 5)
    assert np.allclose(oracle.linear(w, qtype, n, k, x, res), got + res, atol=1e-6)


def test_gate_up_is_silu_times_up():
  n, k, m = 32, 256, 2
  wg, wu = synth.weight(oracle.Q4_K, n, k, 6), synth.weight(oracle.Q4_K, n, k, 7)
  x = synth.activations(m, k, 8)
  g, u = oracle.linear(wg, oracle.Q4_K, n, k, x), oracle.linear(wu, oracle.Q4_K, n, k, x)
  want = g / (1 + np.exp(-g)) * u
  assert np.allclose(oracle.gate_up(wg, wu, oracle.Q4_K, n, k, x), want, rtol=1e-5, atol=1e-7)


def test_philox_known_answer():
  """Philox4x32-10 with zero key and counter: the first known-answer vector of the Random123 distribution."""
  assert oracle.philox(0, 0) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
  assert 0.0 <= oracle.uniform(5, 9) < 1.0 and oracle.uniform(5, 9) == oracle.uniform(5, 9) != oracle.uniform(5, 10)
