"""GPU: the MTP drafter against the CPU oracle. First the input fusion kernel alone in its three modes, then the
proposals of the whole drafter (fuse -> eh_proj -> attention layer over its own K/V cache -> shared head) read back
from a running engine and compared, teacher-forced, with the oracle's drafting chain."""
import os

import numpy as np
import pytest

import oracle
from mtlqwen_b200 import device as D
from mtlqwen_b200.inference import InferenceEngine
from mtlqwen_b200.testing import synth

pytestmark = pytest.mark.gpu
LAYERS, VOCAB, WIDTH = 4, 4096, 4


def test_mtp_fuse_three_modes_match_the_oracle(dev):
  """native_ops.metal:43-87. One pass with a fresh prefill chunk (no predecessor: the hidden half is zero), a
  decode row with a stored seed, and a speculative query of three candidate rows. Mode 1 (the tail of a target
  pass) also stores the next seed: per candidate row for the speculative query, after the last row otherwise."""
  rng = np.random.default_rng(11)
  seed_offset, state_bytes = 1024, 1024 + 4096 * 4  # a small record: some bytes of "state", then the fp32 seed
  counts, previous_set, speculative = [4, 1, 3], [False, True, True], [False, False, True]
  rows = sum(counts)
  embedding = rng.standard_normal((rows, 4096)).astype(np.float32)
  hidden = (2.0 * rng.standard_normal((rows, 4096))).astype(np.float32)
  enorm = (1 + 0.01 * rng.standard_normal(4096)).astype(np.float32)
  hnorm = (1 + 0.01 * rng.standard_normal(4096)).astype(np.float32)
  records = np.zeros((3, state_bytes // 4), np.float32)
  records[:, seed_offset // 4:] = rng.standard_normal((3, 4096))
  previous, following, candidates = dev.array(records), dev.empty((3, state_bytes // 4)), dev.empty((3, state_bytes // 4))
  queries, start = [], 0
  for i, count in enumerate(counts):
    q = D.Query()
    q.start, q.count, q.position, q.slot = start, count, 9 if previous_set[i] else 0, i
    q.previous = previous.ptr + i * state_bytes if previous_set[i] else 0
    q.state = 0 if speculative[i] else D.UNBOUND
    q.next = candidates.ptr if speculative[i] else following.ptr + i * state_bytes
    queries.append(q)
    start += count
  device_queries = dev.queries(queries)
  y = dev.empty((rows, 8192))
  seeds = records[:, seed_offset // 4:]
  for mode in (0, 1, 2):
    dev.mtp_fuse(dev.array(embedding), dev.array(hidden), device_queries, len(queries), dev.array(enorm), dev.array(hnorm), rows, mode, seed_offset,
                 state_bytes, y)
    dev.commit()
    got = y.download()
    for i, q in enumerate(queries):
      for token in range(q.count):
        row = q.start + token
        if mode == 2:  # drafting, step 0: the stored seed (a record without predecessor has none)
          h = seeds[i] if q.previous else None
        elif mode == 1:
          h = (seeds[i] if q.previous else None) if token == 0 else hidden[row - 1]
        else:
          h = hidden[row]
        if not q.previous and token == 0:
          h = None  # `initial` (native_ops.metal:57) holds in every mode
        want = oracle.mtp_fuse(embedding[row], h, enorm, hnorm)
        assert np.abs(got[row] - want).max() <= 1e-5 * np.abs(want).max(), (mode, i, token)
    if mode == 1:
      stored, stored_candidates = following.download()[:, seed_offset // 4:], candidates.download()[:, seed_offset // 4:]
      assert np.array_equal(stored[0], hidden[3]) and np.array_equal(stored[1], hidden[4])  # the last row of each plain query
      for token in range(3):
        assert np.array_equal(stored_candidates[token], hidden[5 + token])  # one seed per candidate row


@pytest.fixture(scope="module")
def weights(tmp_path_factory):
  path = tmp_path_factory.mktemp("gguf") / "tiny-mtp.gguf"
  synth.write_gguf(path, layers=LAYERS, vocab=VOCAB, mtp=True, seed=77)
  return path


def test_drafter_proposals_match_the_oracle_teacher_forced(weights):
  """Every speculative step leaves its anchor position and its proposals in infeng_sequence_info (fields 3, 4..).
  The oracle replays the committed tokens through the target (which yields the seeds and, through the tail of each
  pass, the drafter's K/V cache) and then drafts from the same anchor, fed the engine's own earlier proposals.
  Wherever the oracle's top-1 margin over the drafter's logits exceeds 1e-2 the proposal must be its argmax."""
  os.environ["INFENG_DRAFT_WIDTH"], os.environ["INFENG_SEED"] = str(WIDTH), "7"
  engine = InferenceEngine(weights, draft_weights=weights, max_context=512)
  os.environ.pop("INFENG_DRAFT_WIDTH")
  reference = oracle.Model(synth.read_gguf(weights), LAYERS, VOCAB, 512)
  try:
    sequence = engine.sequence(speculative=True)
    prompt = [int(t) for t in np.random.default_rng(5).integers(0, VOCAB, 150)]  # two prefill passes, then speculative steps
    tokens, steps, drafted = list(prompt), [], 0
    cursor = sequence.append(prompt)
    for _ in range(12):
      # one token, then stop the sequence and collect whatever the passes in flight still emitted
      token = sequence.read(cursor)
      assert token is not None
      tokens.append(token)
      cursor += 1
      sequence.cancel()
      while (token := sequence.read(cursor)) is not None:
        tokens.append(token)
        cursor += 1
      if sequence.speculative_counters()["drafted_tokens"] > drafted:  # a speculative step ran since the last look
        drafted = sequence.speculative_counters()["drafted_tokens"]
        steps.append(sequence.draft_step())
      assert sequence.append([]) == cursor
    sequence.cancel()
    counters = sequence.speculative_counters()
    sequence.close()
    assert len(steps) >= 6 and counters["drafted_tokens"] >= WIDTH * len(steps)

    fed, last_hidden, checked = 0, None, 0
    for anchor, proposals in steps:
      assert fed <= anchor < len(tokens)
      if anchor > fed:
        hidden, _ = reference.forward(tokens[fed:anchor], 0)
        for offset in range(anchor - fed):  # the tail of the target passes: the drafter's K/V of every committed position
          previous = last_hidden if offset == 0 else hidden[offset - 1]
          reference.mtp_step(tokens[fed + offset], previous, fed + offset, store_only=True)
        last_hidden, fed = hidden[-1], anchor
      token, previous = tokens[anchor], last_hidden  # step 0: the anchor token fused with the stored seed
      for s in range(WIDTH):
        block, logits = reference.mtp_step(token, previous, anchor + s)
        expected, margin = oracle.sample(logits)
        if margin > 1e-2:
          assert proposals[s] == expected, (anchor, s, margin)
          checked += 1
        token, previous = proposals[s], block  # later steps: the previous proposal fused with the block's own output
    assert checked >= 16
  finally:
    engine.close()
