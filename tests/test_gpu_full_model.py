"""GPU: the model the benchmark times - 32 layers, vocabulary 248,320, Q4_K projections, Q6_K embedding and lm_head -
checked against the CPU oracle at its real shape: greedy tokens teacher-forced under the margin rule, the recurrent
state and the final hidden state by relative error.

Tolerances. Every kernel on its own is held to 1e-3 by its unit tests (the Q4_K decode GEMV measures 3e-5). Through 32
layers and some hundred positions the per-kernel errors add up: measured on this model, the relative error of the
recurrent state grows by about 4e-5 per layer, from 3e-5 in the first GDN layer to 1.2e-3 in the last, and the final
hidden state ends at 0.7e-3 to 1.0e-3. Nearly all of it is the 16-bit activation grid of the integer GEMV (with the
fp16 hi+lo GEMV in its place the same run ends at 5e-5), so the end-to-end bound asserted here is 2e-3, twice the
per-kernel tolerance, while the tokens are held to the benchmark's own rule without any allowance."""
END_TO_END_TOLERANCE = 2e-3
import os
import threading

import numpy as np
import pytest

import oracle
from mtlqwen_b200.inference import InferenceEngine
from mtlqwen_b200.testing import synth

pytestmark = pytest.mark.gpu
LAYERS, VOCAB = synth.FULL_LAYERS, synth.FULL_VOCAB
GDN_LAYER_FLOATS = 8192 * 4 + 32 * 128 * 128


def tokens_of(seed, length):
  return [int(t) for t in np.random.default_rng(seed).integers(0, VOCAB, length)]


def generate(sequence, prompt, count, started=None):
  cursor, output = sequence.append(prompt), []
  while len(output) < count:
    output.append(sequence.read(cursor))
    cursor += 1
    if started is not None:
      started.set()
  sequence.cancel()
  while (token := sequence.read(cursor)) is not None:
    output.append(token)
    cursor += 1
  return output


def check_against_oracle(tensors, prompt, generated, sequence, minimum):
  """Feeds the oracle the prompt in one pass and then the engine's own tokens one by one; wherever the oracle's
  top-1 margin exceeds 1e-2 the engine's token must be the oracle's argmax. Then compares the state record."""
  reference = oracle.Model(tensors, LAYERS, VOCAB, 1024)
  _, logits = reference.forward(prompt, 1)
  checked, hidden = 0, None
  for index, token in enumerate(generated):
    expected, margin = oracle.sample(logits[-1] if logits.ndim == 2 else logits)
    if margin > 1e-2:
      assert token == expected, (index, margin)
      checked += 1
    if index + 1 < len(generated):
      hidden, logits = reference.step(token)
  assert checked >= minimum, checked
  # The engine holds len(prompt) + len(generated) - 1 positions (the last token has not been fed back), as the oracle.
  assert sequence.length == reference.length == len(prompt) + len(generated) - 1
  record = sequence.state()
  gdn = LAYERS - LAYERS // 4
  worst = 0.0
  for layer in (0, gdn // 2, gdn - 1):
    base = layer * GDN_LAYER_FLOATS
    conv, state = record[base:base + 8192 * 4], record[base + 8192 * 4:base + GDN_LAYER_FLOATS]
    want_conv, want_state = reference._conv[layer].ravel(), reference._S[layer].ravel()
    assert np.abs(conv - want_conv).max() <= END_TO_END_TOLERANCE * np.abs(want_conv).max(), layer
    worst = max(worst, float(np.linalg.norm(state - want_state) / np.linalg.norm(want_state)))
  assert worst <= END_TO_END_TOLERANCE, worst
  seed = record[gdn * GDN_LAYER_FLOATS:]
  assert seed.size == 4096
  assert np.linalg.norm(seed - hidden) <= END_TO_END_TOLERANCE * np.linalg.norm(hidden)  # final hidden state of the last position fed
  return checked


def test_full_shape_tokens_state_and_hidden_match_the_oracle():
  """Two sequences on the 32-layer model. The first starts alone and keeps decoding; the second brings a 530-token
  prompt, so its prefill chunks (the tcgen05 GEMM and the chunked delta rule, more than 128 rows in all) share
  passes with the first one's decode rows, cross the 512-token checkpoint boundary and are followed by decode steps
  at positions past it. The MTP block is loaded so that every pass also leaves the final hidden state in the state
  record."""
  path = synth.ensure_full_model()
  os.environ["INFENG_SEED"] = "1"
  engine = InferenceEngine(path, draft_weights=path, max_context=1024)
  try:
    assert engine.vocab_size == VOCAB and engine.drafter == "mtp"
    first, second = engine.sequence(), engine.sequence()
    prompt_a, prompt_b = tokens_of(41, 40), tokens_of(42, 530)
    started, results = threading.Event(), {}
    worker = threading.Thread(target=lambda: results.update(a=generate(first, prompt_a, 40, started)))
    worker.start()
    started.wait()
    rows_before = engine.step_counters()["rows"]
    results["b"] = generate(second, prompt_b, 20)
    worker.join()
    assert engine.step_counters()["rows"] - rows_before >= 530
    tensors = synth.read_gguf(path)
    checked = check_against_oracle(tensors, prompt_b, results["b"], second, 14)
    checked += check_against_oracle(tensors, prompt_a, results["a"], first, 18)
    assert checked >= 32
    first.close()
    second.close()
  finally:
    engine.close()
