"""GPU: on-device sampling against the CPU oracle (greedy, top-k/top-p/temperature, plain temperature)."""
import numpy as np
import pytest

import oracle
from mtlqwen_b200 import device as D

pytestmark = pytest.mark.gpu
VOCAB = 248320


def make_queries(params, seed=1234, position=41):
  queries, logit = [], 0
  for slot, (temperature, top_p, top_k, samples) in enumerate(params):
    q = D.Query()
    q.start, q.count, q.position, q.slot, q.state = logit, samples, position, slot, D.UNBOUND
    q.logit, q.samples, q.temperature, q.topP, q.topK, q.seed = logit, samples, temperature, top_p, top_k, seed + slot
    queries.append(q)
    logit += samples
  return queries, logit


def expected(logits, queries):
  out = []
  for q in queries:
    for s in range(q.samples):
      u = oracle.uniform(q.seed, q.position + q.count - q.samples + s + 1)
      out.append(oracle.sample(logits[q.logit + s], q.temperature, q.topP, q.topK, u)[0])
  return out


def test_greedy_matches_first_index_argmax(dev):
  rng = np.random.default_rng(0)
  logits = (1.3 * rng.standard_normal((8, VOCAB))).astype(np.float32)
  logits[3, 1000] = logits[3, 2000] = 9.5  # a tie: the first index wins
  queries, count = make_queries([(0.0, 1.0, 0, 1)] * 8)
  tokens = dev.empty(count, np.int32)
  dev.sample(dev.array(logits), VOCAB, dev.queries(queries), len(queries), count, 0, tokens)
  got = tokens.download().tolist()
  assert got == expected(logits, queries)
  assert got[3] == 1000


def test_top_k_top_p_temperature_config5(dev):
  """BASELINE config 5 sampling: temperature 0.7, top-p 0.9, top-k 40, seeded per-slot RNG."""
  rng = np.random.default_rng(1)
  logits = (1.3 * rng.standard_normal((40, VOCAB))).astype(np.float32)
  queries, count = make_queries([(0.7, 0.9, 40, 5)] * 8)
  tokens = dev.empty(count, np.int32)
  dev.sample(dev.array(logits), VOCAB, dev.queries(queries), len(queries), count, 0, tokens)
  assert tokens.download().tolist() == expected(logits, queries)


def test_mixed_sampling_parameters(dev):
  rng = np.random.default_rng(2)
  logits = (2.0 * rng.standard_normal((8, VOCAB))).astype(np.float32)
  params = [(1.0, 1.0, 1, 1), (0.0, 1.0, 0, 1), (1.5, 0.5, 64, 1), (0.3, 0.95, 200, 1), (1.0, 1.0, 0, 1), (0.7, 0.0, 40, 1), (2.0, 1.0, 8, 1),
            (1.0, 0.9, 0, 1)]
  queries, count = make_queries(params)
  tokens = dev.empty(count, np.int32)
  dev.sample(dev.array(logits), VOCAB, dev.queries(queries), len(queries), count, 0, tokens)
  got, want = tokens.download().tolist(), expected(logits, queries)
  # top_k = 1 is greedy whatever the temperature (test_mixed_batch_sampling_matches_greedy of the reference)
  assert got[0] == int(np.argmax(logits[0]))
  for i, (g, w) in enumerate(zip(got, want)):
    if params[i][2] == 0 and params[i][0] > 0:
      # full-vocabulary sampling sums 248k terms in a different order than the serial oracle: accept the
      # neighbour when the target falls within rounding of a boundary
      assert abs(g - w) <= 1, (i, g, w)
    else:
      assert g == w, (i, g, w)


def test_ties_at_the_top_k_cut_keep_the_earliest_indices(dev):
  logits = np.full((1, VOCAB), -5.0, np.float32)
  logits[0, [10, 20, 30]] = [3.0, 2.0, 1.0]
  queries, count = make_queries([(1.0, 1.0, 8, 1)])
  tokens = dev.empty(count, np.int32)
  dev.sample(dev.array(logits), VOCAB, dev.queries(queries), 1, count, 0, tokens)
  assert tokens.download().tolist() == expected(logits, queries)


# ---- draft verification on the device against the host loop of the reference ----
def host_acceptance(samples, speculative, sampled, proposals, draft_width, stops):
  """runtime/engine.cpp:205-216 for one query: returns (accepted, emitted, stopped)."""
  accepted, emitted, stopped = 0, 0, False
  for i in range(samples):
    if stopped:
      break
    token = sampled[i]
    emitted += 1
    stopped = token in stops
    if not speculative or i == draft_width or token != proposals[i]:
      break
    accepted += 1
  return accepted, emitted, int(stopped)


def test_verify_drafts_and_commit_states_follow_the_reference_loop(dev):
  """Six queries in one pass, draft width 4: full acceptance (stops at s == width), mismatch at proposal 0, a stop
  token inside an accepted draft (it is emitted, counted when it matches, and ends the query), a plain decode
  row, a prefill chunk without a sample, and a mismatch in the middle. The accepted candidate state row of each
  speculative query must land in the slot's next state record."""
  width, stride = 4, 64
  cases = [  # (speculative, sampled rows, proposals, stop tokens)
    (True, [11, 12, 13, 14, 15], [11, 12, 13, 14], []),
    (True, [21, 22, 23, 24, 25], [99, 22, 23, 24], []),
    (True, [31, 32, 33, 34, 35], [31, 32, 33, 34], [32]),
    (False, [41], [0, 0, 0, 0], [41]),
    (False, [], [0, 0, 0, 0], []),
    (True, [51, 52, 53, 54, 55], [51, 52, 77, 54], [7, 8, 9]),
  ]
  state_bytes = 4096
  queries, sampled, logit, candidate = [], [], 0, 0
  proposed = np.zeros((width + 1, 8), np.int32)
  stops, counts = np.zeros((8, stride), np.int32), np.zeros(8, np.uint32)
  for slot, (speculative, rows, proposals, stop) in enumerate(cases):
    q = D.Query()
    q.slot, q.position, q.count, q.samples, q.logit = slot, 100 + slot, max(len(rows), 1) if rows else 7, len(rows), logit
    q.state = candidate if speculative else D.UNBOUND
    if speculative:
      proposed[1:, candidate // q.count] = proposals  # column = first candidate row / rows per query, as the engine packs them
      candidate += q.count
    stops[slot, :len(stop)], counts[slot] = stop, len(stop)
    sampled += rows
    logit += len(rows)
    queries.append(q)
  rng = np.random.default_rng(3)
  candidates = rng.integers(0, 2**31, (candidate, state_bytes // 4), dtype=np.int64).astype(np.uint32)
  following = dev.empty((8, state_bytes // 4), np.uint32)
  next_addresses = np.array([following.ptr + slot * state_bytes for slot in range(8)], np.uint64)
  candidate_buffer = dev.array(candidates)
  device_queries, verdict = dev.queries(queries), dev.empty(3 * len(queries), np.uint32)
  dev.verify_drafts(device_queries, len(queries), dev.array(np.array(sampled, np.int32)), dev.array(proposed), width, dev.array(stops), stride,
                    dev.array(counts), verdict)
  dev.commit_states(device_queries, len(queries), verdict, dev.array(next_addresses), candidate_buffer.ptr, state_bytes)
  dev.commit()
  got = verdict.download().reshape(-1, 3).tolist()
  want = [list(host_acceptance(len(rows), speculative, rows, proposals, width, stop)) for speculative, rows, proposals, stop in cases]
  assert got == want
  assert want[0] == [4, 5, 0] and want[1] == [0, 1, 0] and want[2] == [2, 2, 1] and want[3] == [0, 1, 1] and want[4] == [0, 0, 0]
  states = following.download()
  for q, (accepted, _, _) in zip(queries, want):
    if q.state != D.UNBOUND:
      assert np.array_equal(states[q.slot], candidates[q.state + accepted]), q.slot
