"""GPU: the engine through its Python boundary (infeng_* C ABI) on a reduced random-init model (4 decoder
layers = 3 GDN + 1 attention, vocabulary 4096, MTP block), checked against the CPU oracle and against the
self-consistency contracts of the reference's test/test_qwen35.py."""
import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import pytest

import oracle
from mtlqwen_b200.testing import synth
from mtlqwen_b200.inference import InferenceEngine

pytestmark = pytest.mark.gpu
LAYERS, VOCAB = 4, 4096


@pytest.fixture(scope="module")
def weights(tmp_path_factory):
  path = tmp_path_factory.mktemp("gguf") / "tiny-mtp.gguf"
  synth.write_gguf(path, layers=LAYERS, vocab=VOCAB, mtp=True, seed=99)
  return path


@pytest.fixture(scope="module")
def plain_weights(tmp_path_factory):
  path = tmp_path_factory.mktemp("gguf") / "tiny.gguf"
  synth.write_gguf(path, layers=LAYERS, vocab=VOCAB, mtp=False, seed=99)
  return path


@pytest.fixture(scope="module")
def model(plain_weights):
  os.environ["INFENG_SEED"] = "4242"
  engine = InferenceEngine(plain_weights, max_context=2048)
  yield engine
  engine.close()


def complete(sequence, prompt=(), limit=None):  # test/test_qwen35.py:31-44
  cursor, output = sequence.append(prompt), []
  while limit is None or len(output) < limit:
    token = sequence.read(cursor)
    if token is None: break
    cursor += 1
    if token in sequence.stop_token_ids: return output
    output.append(token)
  if limit is not None:
    sequence.cancel()
    while sequence.read(cursor) is not None:
      cursor += 1
  return output


def one(sequence, prompt=()):
  return complete(sequence, prompt, 1)[0]


def parallel(calls):
  with ThreadPoolExecutor(max_workers=len(calls)) as pool:
    return list(pool.map(lambda call: call(), calls))


def prompt_tokens(seed, length):
  return [int(t) for t in np.random.default_rng(seed).integers(0, VOCAB, length)]


def test_engine_reports_model_shape(model):
  assert model.drafter == "none" and model.draft_width == 0 and model.vocab_size == VOCAB
  assert model.weight_bytes > 500e6 and model.parameter_count > 800e6


def test_greedy_tokens_match_oracle_teacher_forced(model, plain_weights):
  """Prefill (one ragged chunk) + 12 greedy decode steps. The oracle is fed the engine's tokens; wherever its
  top-1 margin exceeds 1e-2 the engine must have produced the oracle's argmax (BASELINE parity rule)."""
  prompt = prompt_tokens(1, 37)
  sequence = model.sequence()
  generated = complete(sequence, prompt, 12)
  assert sequence.length >= len(prompt) + 11
  sequence.close()
  reference = oracle.Model(synth.read_gguf(plain_weights), LAYERS, VOCAB, 256)
  checked = 0
  for position, token in enumerate(prompt + generated[:-1]):
    _, logits = reference.step(token, want_logits=position >= len(prompt) - 1)
    if position >= len(prompt) - 1:
      expected, margin = oracle.sample(logits)
      if margin > 1e-2:
        assert generated[position - len(prompt) + 1] == expected, (position, margin)
        checked += 1
  assert checked >= 8


def test_continuous_mixed_batch_matches_solo(model):
  """Batched (prefill + decodes in one pass) == each sequence alone (test_qwen35.py:78-104)."""
  reference = [model.sequence(), model.sequence(), model.sequence()]
  actual = [model.sequence(), model.sequence(), model.sequence()]
  try:
    prompt = prompt_tokens(2, 200)
    expected_pp = complete(reference[0], prompt, 1)
    one(reference[1], [10, 11, 12])
    expected_tg = complete(reference[1], limit=3)
    one(reference[2], [20, 21, 22])
    expected_tg2 = complete(reference[2], limit=3)
    one(actual[1], [10, 11, 12])
    one(actual[2], [20, 21, 22])
    observed = parallel([lambda: complete(actual[0], prompt, 1), lambda: complete(actual[1], limit=3), lambda: complete(actual[2], limit=3)])
    assert observed == [expected_pp, expected_tg, expected_tg2]
    assert actual[0].length == 200
  finally:
    for sequence in reference + actual:
      sequence.close()


def test_prefix_restore_reproduces_the_token(model):
  """A 520-token prompt twice: the second run restores the 512-token checkpoint (test_qwen35.py:106-116)."""
  first, second = model.sequence(), model.sequence()
  try:
    prompt = prompt_tokens(3, 520)
    passes_before = model.step_counters()["rows"]
    expected = one(first, prompt)
    rows_first = model.step_counters()["rows"] - passes_before
    assert first.length == 520
    assert one(second, prompt) == expected and second.length == 520
    rows_second = model.step_counters()["rows"] - passes_before - rows_first
    assert rows_first >= 520 and rows_second <= 16, (rows_first, rows_second)  # only the 8 tokens after the checkpoint are recomputed
    assert complete(first, limit=4) == complete(second, limit=4)
  finally:
    first.close()
    second.close()


def test_evicted_checkpoints_hand_their_state_records_on(model):
  """Eleven different 520-token prompts publish eleven checkpoints into a cache of eight: the evicted ones' state
  records are reused by later sequences, and neither a restored nor a recomputed prefix changes the token."""
  tokens = []
  for seed in range(11):
    sequence = model.sequence()
    try:
      tokens.append(one(sequence, prompt_tokens(100 + seed, 520)))
    finally:
      sequence.close()
  for seed in (10, 0, 5):  # still cached; evicted long ago; in between
    sequence = model.sequence()
    try:
      rows_before = model.step_counters()["rows"]
      assert one(sequence, prompt_tokens(100 + seed, 520)) == tokens[seed]
      rows = model.step_counters()["rows"] - rows_before
      assert rows <= 16 if seed == 10 else rows >= 520, (seed, rows)
    finally:
      sequence.close()


def test_mixed_batch_sampling_matches_greedy(model):
  """temperature 1 with top_k 1 is greedy (test_qwen35.py:207-230)."""
  greedy = [model.sequence() for _ in range(4)]
  sampled = [model.sequence(temperature=1.0, top_k=1) for _ in range(4)]
  try:
    prompts = [prompt_tokens(10 + i, 5 + 30 * i) for i in range(4)]
    want = parallel([lambda s=s, p=p: complete(s, p, 4) for s, p in zip(greedy, prompts)])
    got = parallel([lambda s=s, p=p: complete(s, p, 4) for s, p in zip(sampled, prompts)])
    assert got == want
  finally:
    for sequence in greedy + sampled:
      sequence.close()


def test_seeded_sampling_is_reproducible_and_batching_invariant(plain_weights):
  """The i-th emitted token of a sequence uses the i-th variate of its own Philox stream whatever else is batched, the
  key of that stream depends only on the engine's base seed and on how many sequences were created before it, and
  the next sequence in the same slot draws from a new key (the reference keeps advancing rng[slot] across
  sequences, runtime/engine.cpp:210-211, so a repeated request does not repeat its completion)."""
  prompt = prompt_tokens(20, 24)

  def run(batched):
    os.environ["INFENG_SEED"] = "4242"
    engine = InferenceEngine(plain_weights, max_context=512)
    try:
      sampled = engine.sequence(temperature=0.7, top_p=0.9, top_k=40)
      calls = [lambda: complete(sampled, prompt, 8)]
      if batched:
        other = engine.sequence()
        calls.append(lambda: complete(other, prompt_tokens(21, 90), 8))
      first = parallel(calls)[0]
      slot_length = sampled.length
      sampled.close()
      again = engine.sequence(temperature=0.7, top_p=0.9, top_k=40)  # takes the slot that was just freed
      second = complete(again, prompt, 8)
      again.close()
      assert slot_length >= len(prompt)
      return first, second
    finally:
      engine.close()

  alone, regenerated = run(False)
  together, _ = run(True)
  assert together == alone
  assert regenerated != alone


def test_out_of_range_token_ids_are_refused(model):
  """The embedding gather indexes the table with the appended ids: ids outside the vocabulary never reach the device."""
  sequence = model.sequence()
  try:
    passes = model.step_counters()["passes"]
    for bad in ([VOCAB], [5, -1, 7], [2**31 - 1]):
      with pytest.raises(RuntimeError, match="no available model context"):
        sequence.append(bad)
    assert sequence.length == 0 and model.step_counters()["passes"] == passes
    assert one(sequence, [VOCAB - 1, 0]) is not None
  finally:
    sequence.close()


def test_all_slots_and_ninth_sequence(model):
  """8 slots in parallel == serial; a 9th sequence is refused (test_qwen35.py:275-292)."""
  prompts = [prompt_tokens(30 + i, 12 + 7 * i) for i in range(8)]
  serial = []
  for prompt in prompts:
    sequence = model.sequence()
    serial.append(complete(sequence, prompt, 3))
    sequence.close()
  sequences = [model.sequence() for _ in range(8)]
  try:
    with pytest.raises(RuntimeError, match="maximum live sequence count"):
      model.sequence()
    assert parallel([lambda s=s, p=p: complete(s, p, 3) for s, p in zip(sequences, prompts)]) == serial
  finally:
    for sequence in sequences:
      sequence.close()


def test_append_while_generating_and_empty_append(model):
  sequence = model.sequence()
  try:
    with pytest.raises(RuntimeError, match="no available model context"):
      sequence.append([])
    cursor = sequence.append(prompt_tokens(40, 6))
    assert cursor == 6
    assert sequence.read(cursor) is not None
    sequence.cancel()
    while sequence.read(cursor) is not None:
      cursor += 1
  finally:
    sequence.close()


def test_allocator_failure_is_atomic(plain_weights):
  """max_context 16 gives a one-block pool: a second sequence fails without side effects and succeeds after the
  owner closes (test_qwen35.py:233-246)."""
  engine = InferenceEngine(plain_weights, max_context=16)
  try:
    assert engine.mapped_bytes == 0
    owner, blocked = engine.sequence(), engine.sequence()
    one(owner, [1, 2, 3])
    # one 128-token block: K and V tiles of 256 KiB for the single attention layer
    assert engine.mapped_bytes == 2 * 256 * 1024
    length = owner.length
    with pytest.raises(RuntimeError, match="no evictable capacity"):
      one(blocked, [4, 5, 6])
    assert owner.length == length and blocked.length == 0
    owner.close()
    assert one(blocked, []) is not None
    blocked.close()
  finally:
    engine.close()


def test_context_limit_stops_generation(plain_weights):
  engine = InferenceEngine(plain_weights, max_context=16)
  try:
    sequence = engine.sequence()
    output = complete(sequence, [1, 2, 3, 4])
    assert sequence.length == 16 and len(output) == 13
    with pytest.raises(RuntimeError, match="no available model context"):
      sequence.append([5])
    sequence.close()
  finally:
    engine.close()


def test_engine_outlives_close_while_sequences_live(plain_weights):
  """test_qwen35.py:179-188."""
  engine = InferenceEngine(plain_weights, max_context=256)
  sequence = engine.sequence()
  engine.close()
  assert len(complete(sequence, [7, 8, 9], 2)) == 2
  sequence.close()


def test_invalid_weights_raise(tmp_path, plain_weights):
  bogus = tmp_path / "bogus.gguf"
  bogus.write_bytes(b"not a gguf file at all")
  with pytest.raises(RuntimeError, match="GGUF"):
    InferenceEngine(bogus, max_context=64)
  with pytest.raises(RuntimeError, match="MTP"):
    InferenceEngine(plain_weights, draft_weights=plain_weights, max_context=64)
  with pytest.raises(ValueError):
    InferenceEngine(plain_weights, max_context=0)


def test_speculative_greedy_equals_plain_greedy(weights):
  """Speculative decoding only changes how many target rows a step verifies, never the tokens
  (test_qwen35.py:150-176). Width 4 as BASELINE config 5."""
  os.environ["INFENG_DRAFT_WIDTH"] = "4"
  engine = InferenceEngine(weights, draft_weights=weights, max_context=1024)
  os.environ.pop("INFENG_DRAFT_WIDTH")
  try:
    assert engine.drafter == "mtp" and engine.draft_width == 4
    prompt = prompt_tokens(50, 45)
    plain, speculative = engine.sequence(), engine.sequence(speculative=True)
    want = complete(plain, prompt, 24)
    got = complete(speculative, prompt, 24)
    assert got == want
    counters = speculative.speculative_counters()
    assert counters["drafted_tokens"] > 0 and 0 <= counters["accepted_tokens"] <= counters["drafted_tokens"]
    # stop token inside a step truncates the output there (test_qwen35.py:118-128)
    stopper = engine.sequence(stop_token_ids=[want[2]], speculative=True)
    assert complete(stopper, prompt) == want[:2]
    for sequence in (plain, speculative, stopper):
      sequence.close()
    # mixed pass: prefill + plain decode + speculative decode together equals each alone
    a, b, c = engine.sequence(), engine.sequence(), engine.sequence(speculative=True)
    solo_a = complete(a, prompt_tokens(51, 150), 1)
    one(b, [10, 11, 12]); solo_b = complete(b, limit=2)
    one(c, [20, 21, 22]); solo_c = complete(c, limit=6)
    for sequence in (a, b, c):
      sequence.close()
    a, b, c = engine.sequence(), engine.sequence(), engine.sequence(speculative=True)
    one(b, [10, 11, 12]); one(c, [20, 21, 22])
    observed = parallel([lambda: complete(a, prompt_tokens(51, 150), 1), lambda: complete(b, limit=2), lambda: complete(c, limit=6)])
    assert observed == [solo_a, solo_b, solo_c]
    for sequence in (a, b, c):
      sequence.close()
  finally:
    engine.close()
