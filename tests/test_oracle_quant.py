"""CPU: the oracle's K-quant dequantisers against the gguf-py golden vectors, and oracle self-consistency."""
from pathlib import Path

import numpy as np
import pytest

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


@pytest.mark.parametrize("name,qtype", [("q5k", oracle.Q5_K), ("q8_0", oracle.Q8_0), ("iq4xs", oracle.IQ4_XS)])
def test_other_gguf_types_dequant_match_gguf_py_bit_exact(name, qtype):
  """The block formats of the real Qwen3.5 GGUF files beyond Q4_K / Q6_K (quant_linear.metal:50-67, 87-115)."""
  golden = np.load(GOLDEN)
  got = oracle.dequant(golden[name + "_blocks"], qtype)
  assert got.tobytes() == golden[name + "_values"].tobytes()


def test_synthetic_weights_have_the_configured_distribution():
  w = oracle.dequant(synth.weight(synth.Q4_K, 64, 4096, 1), oracle.Q4_K)
  assert abs(w.mean()) < 2e-3 and 0.015 < w.std() < 0.025
  w = oracle.dequant(synth.weight(synth.Q6_K, 64, 4096, 2), oracle.Q6_K)
  assert abs(w.mean()) < 2e-3 and 0.015 < w.std() < 0.025


def gguf_py_matrix(w, qtype, n, k):
  """The dense matrix as gguf-py (the third-party implementation of the K-quant formats) dequantises it."""
  gguf = pytest.importorskip("gguf")
  kind = gguf.GGMLQuantizationType.Q4_K if qtype == oracle.Q4_K else gguf.GGMLQuantizationType.Q6_K
  return np.asarray(gguf.quants.dequantize(np.ascontiguousarray(w).reshape(n, -1), kind), dtype=np.float64).reshape(n, k)


def test_linear_matches_a_dense_matmul_of_the_gguf_py_matrix():
  """End to end through the oracle's linear (block walk, row stride, accumulation, residual), pinned on a matrix
  dequantised by gguf-py rather than by the oracle itself."""
  n, k, m = 48, 1024, 3
  for qtype in (oracle.Q4_K, oracle.Q6_K):
    w = synth.weight(qtype, n, k, 3)
    x = synth.activations(m, k, 4)
    want = x.astype(np.float64) @ gguf_py_matrix(w, qtype, n, k).T
    got = oracle.linear(w, qtype, n, k, x)
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
    res = synth.activations(m, n, 5)
    assert np.allclose(oracle.linear(w, qtype, n, k, x, res), got + res, atol=1e-6)
    # more rows than one cache block of the oracle's row loop
    tall = synth.activations(70, k, 6)
    assert np.abs(oracle.linear(w, qtype, n, k, tall) - tall.astype(np.float64) @ gguf_py_matrix(w, qtype, n, k).T).max() <= 1e-5 * np.abs(want).max()


def test_embedding_rows_are_the_gguf_py_rows():
  n, k = 64, 512
  ids = [0, 63, 5, 5, 17]
  for qtype in (oracle.Q4_K, oracle.Q6_K):
    w = synth.weight(qtype, n, k, 9)
    assert np.array_equal(oracle.embedding(w, qtype, k, ids), gguf_py_matrix(w, qtype, n, k)[ids].astype(np.float32))


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
