"""GPU: the block formats of the real Qwen3.5 GGUF files beyond Q4_K / Q6_K - Q5_K, Q8_0, IQ4_XS, F16 - through
dequantisation (bit-exact against the gguf-py golden vectors), the linear and gate / up kernels, the embedding gather,
and a whole reduced model that mixes all of them, against the CPU oracle."""
from pathlib import Path

import numpy as np
import pytest

import oracle
from mtlqwen_b200 import device as D
from mtlqwen_b200.inference import InferenceEngine
from mtlqwen_b200.testing import synth

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden" / "kquant_dequant.npz"
TYPES = [("q5k", D.Q5_K), ("q8_0", D.Q8_0), ("iq4xs", D.IQ4_XS)]
TOL = 1e-3  # BASELINE tolerance for GEMV / GEMM; these kernels accumulate in fp32 and measure about 1e-6


def rel_err(got, want):
  want64 = want.astype(np.float64)
  return float(np.abs(got - want64).max() / np.abs(want64).max())


@pytest.mark.parametrize("name,qtype", TYPES)
def test_dequant_bit_exact_against_golden(dev, name, qtype):
  golden = np.load(GOLDEN)
  blocks, want = golden[name + "_blocks"], golden[name + "_values"]
  out = dev.empty(want.shape)
  dev.dequant(qtype, dev.array(blocks), blocks.shape[0], out)
  assert out.download().tobytes() == want.tobytes()


def test_f16_rows_widen_exactly(dev):
  values = (np.random.default_rng(0).standard_normal(32 * 4096) / 64).astype(np.float16)
  out = dev.empty(values.size)
  dev.dequant(D.F16, dev.array(values.view(np.uint8)), values.size // 256, out)
  assert out.download().tobytes() == values.astype(np.float32).tobytes()


@pytest.mark.parametrize("name,qtype", TYPES)
@pytest.mark.parametrize("n,k,m", [(1024, 4096, 1), (520, 8192, 8), (256, 12288, 21)])
def test_linear_matches_oracle(dev, name, qtype, n, k, m):
  w, x, res = synth.weight(qtype, n, k, 60), synth.activations(m, k, 61), synth.activations(m, n, 62)
  y = dev.array(res)
  dev.linear(qtype, dev.array(w), n, k, dev.array(x), m, y, y)  # residual aliases the result, as in the decoder
  assert rel_err(y.download(), oracle.linear(w, qtype, n, k, x, res)) < 1e-5


@pytest.mark.parametrize("name,qtype", TYPES)
def test_gate_up_matches_oracle(dev, name, qtype):
  n, k, m = 768, 4096, 5
  wg, wu, x = synth.weight(qtype, n, k, 70), synth.weight(qtype, n, k, 71), synth.activations(m, k, 72)
  y = dev.empty((m, n))
  dev.gate_up(qtype, dev.array(wg), dev.array(wu), n, k, dev.array(x), m, y)
  assert rel_err(y.download(), oracle.gate_up(wg, wu, qtype, n, k, x)) < 1e-5


@pytest.mark.parametrize("name,qtype", TYPES)
def test_embedding_rows_are_the_oracle_rows(dev, name, qtype):
  n, k, ids = 96, 4096, np.array([0, 95, 7, 7, 41], np.int32)
  table = synth.weight(qtype, n, k, 80)
  out = dev.empty((ids.size, k))
  dev.embedding(qtype, dev.array(table), k, dev.array(ids), ids.size, out)
  assert out.download().tobytes() == oracle.embedding(table, qtype, k, ids).tobytes()


def test_model_with_the_type_mix_of_the_real_files_matches_the_oracle(tmp_path):
  """A reduced model (4 layers + MTP block) whose projections cycle through Q4_K, Q5_K, IQ4_XS, Q6_K and Q8_0, with a
  Q4_K embedding table, F16 ssm_beta / ssm_alpha and a Q8_0 eh_proj: greedy tokens teacher-forced against the oracle
  (margin rule), through a prefill of more than 8 rows and decode steps, with the MTP tail running."""
  layers, vocab = 4, 4096
  path = tmp_path / "mixed.gguf"
  synth.write_gguf(path, layers=layers, vocab=vocab, mtp=True, seed=17, mixed=True)
  tensors = synth.read_gguf(path)
  kinds = {kind for _, kind in tensors.values()}
  assert {D.Q4_K, D.Q5_K, D.Q6_K, D.Q8_0, D.IQ4_XS, D.F16, D.F32} <= kinds
  engine = InferenceEngine(path, draft_weights=path, max_context=256)
  try:
    prompt = [int(t) for t in np.random.default_rng(2).integers(0, vocab, 45)]
    sequence = engine.sequence()
    cursor, generated = sequence.append(prompt), []
    while len(generated) < 14:
      generated.append(sequence.read(cursor))
      cursor += 1
    sequence.cancel()
    sequence.close()
    reference = oracle.Model(tensors, layers, vocab, 256)
    _, logits = reference.forward(prompt, 1)
    checked = 0
    for index, token in enumerate(generated):
      expected, margin = oracle.sample(logits[-1] if logits.ndim == 2 else logits)
      if margin > 1e-2:
        assert token == expected, (index, margin)
        checked += 1
      _, logits = reference.step(token)
    assert checked >= 10
  finally:
    engine.close()
