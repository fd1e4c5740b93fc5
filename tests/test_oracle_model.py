"""CPU: the whole-model oracle is consistent with itself - a pass of T tokens equals T one-token steps, a batched
decode step equals the sequences stepped alone - and its MTP block composes from the pinned pieces. These are the
forms the GPU tests and the CPU baseline rely on (multi-row prefill, 8-sequence decode, drafting)."""
import numpy as np
import pytest

import oracle
from mtlqwen_b200.testing import synth

LAYERS, VOCAB = 4, 512


@pytest.fixture(scope="module")
def tensors(tmp_path_factory):
  path = tmp_path_factory.mktemp("gguf") / "tiny-mtp.gguf"
  synth.write_gguf(path, layers=LAYERS, vocab=VOCAB, mtp=True, seed=21)
  return synth.read_gguf(path)


def test_multi_token_pass_equals_single_steps(tensors):
  stepped, passed = oracle.Model(tensors, LAYERS, VOCAB, 32), oracle.Model(tensors, LAYERS, VOCAB, 32)
  tokens = [5, 17, 300, 400, 12, 9, 77]
  singles = [stepped.step(token) for token in tokens]
  hidden, logits = passed.forward(tokens[:4], 2)
  hidden_b, logits_b = passed.forward(tokens[4:], 1)
  for i in range(4):
    assert np.array_equal(singles[i][0], hidden[i])
  for i in range(3):
    assert np.array_equal(singles[4 + i][0], hidden_b[i])
  assert np.array_equal(singles[2][1], logits[0]) and np.array_equal(singles[3][1], logits[1]) and np.array_equal(singles[6][1], logits_b[0])
  assert stepped.length == passed.length == 7


def test_results_do_not_depend_on_the_thread_count(tensors):
  """The oracle's loops are parallel over weight rows, heads and sequences, never over a summation index: one thread and
  all threads give the same bits (the one-thread and all-core timings of the bench time the same arithmetic)."""
  import os
  tokens = [5, 17, 300, 400, 12, 9, 77, 1, 2, 3]
  results = []
  for threads in (1, max(2, os.cpu_count() or 2)):
    oracle.set_threads(threads)
    model = oracle.Model(tensors, LAYERS, VOCAB, 32)
    hidden, logits = model.forward(tokens, 2)
    results.append((hidden.copy(), logits.copy(), model.step(44)[1].copy()))
  oracle.set_threads(max(1, os.cpu_count() or 1))
  for one, many in zip(*results):
    assert one.tobytes() == many.tobytes()


def test_batched_decode_equals_solo_steps(tensors):
  batch = [oracle.Model(tensors, LAYERS, VOCAB, 32) for _ in range(3)]
  solo = [oracle.Model(tensors, LAYERS, VOCAB, 32) for _ in range(3)]
  for models in (batch, solo):  # ragged contexts: fresh, 3 and 7 tokens
    models[1].forward([3, 4, 5], 0)
    models[2].forward([9] * 7, 0)
  for step in range(3):
    tokens = [11 + step, 22 + step, 33 + step]
    hidden, logits = oracle.decode_batch(batch, tokens)
    for i in range(3):
      want_hidden, want_logits = solo[i].step(tokens[i])
      assert np.array_equal(want_hidden, hidden[i]) and np.array_equal(want_logits, logits[i])
  assert [m.length for m in batch] == [3, 6, 10]


def test_mtp_block_composes_from_its_parts(tensors):
  """orc_mtp_step = embedding -> mtp_fuse -> eh_proj -> attention layer blk.<LAYERS> on its own cache -> MLP -> head.
  The tail form stores exactly the K/V the drafting form appends, and a fresh sequence fuses with zeros."""
  model = oracle.Model(tensors, LAYERS, VOCAB, 32)
  assert model.has_mtp
  hidden, _ = model.forward([7, 8, 9], 0)
  nextn = f"blk.{LAYERS}.nextn."
  embedding = oracle.embedding(tensors["token_embd.weight"][0], tensors["token_embd.weight"][1], 4096, [21])[0]
  fused = oracle.mtp_fuse(embedding, hidden[-1], tensors[nextn + "enorm.weight"][0], tensors[nextn + "hnorm.weight"][0])
  assert np.array_equal(fused[:4096], oracle.rms_norm(embedding, tensors[nextn + "enorm.weight"][0]))
  assert np.array_equal(fused[4096:], oracle.rms_norm(hidden[-1], tensors[nextn + "hnorm.weight"][0]))
  assert not oracle.mtp_fuse(embedding, None, tensors[nextn + "enorm.weight"][0], tensors[nextn + "hnorm.weight"][0])[4096:].any()
  model.mtp_step(21, hidden[-1], 3, store_only=True)
  stored = model._mtp_keys[3].copy(), model._mtp_values[3].copy()
  model._mtp_keys[3] = model._mtp_values[3] = 0
  block, logits = model.mtp_step(21, hidden[-1], 3)
  assert np.array_equal(model._mtp_keys[3], stored[0]) and np.array_equal(model._mtp_values[3], stored[1])
  assert block.shape == (4096, ) and logits.shape == (VOCAB, ) and np.isfinite(logits).all()
