"""GPU: the allocation-free attention entry point (infdev_attention_static) against the regular one.

Collected last on purpose (pytest orders files by name), so a run that stops at the first failure has already run
every other test. The call is made through the C ABI twice in a row on different inputs: the second call finds the
first call's partials still in the built-in scratch array and must not be affected by them.
"""
import numpy as np
import pytest

from mtlqwen_b200 import device as D

pytestmark = pytest.mark.gpu
BLOCK_TOKENS, SPLITS = 16, 16  # the static variant always uses 16 splits per row


def build_case(dev, seed, contexts):
  rng = np.random.default_rng(seed)
  nq = len(contexts)
  blocks_per_seq = [-(-c // BLOCK_TOKENS) for c in contexts]
  stride, physical = max(blocks_per_seq), int(sum(blocks_per_seq))
  permutation = rng.permutation(physical).astype(np.int32)
  table = np.zeros((nq, stride), np.int32)
  at = 0
  for i, n in enumerate(blocks_per_seq):
    table[i, :n] = permutation[at:at + n]
    at += n
  shape = (physical, 4, BLOCK_TOKENS, 256)
  keys = rng.standard_normal(shape, dtype=np.float32).astype(np.float16).view(np.uint16)
  values = rng.standard_normal(shape, dtype=np.float32).astype(np.float16).view(np.uint16)
  queries = []
  for i, context in enumerate(contexts):
    q = D.Query()
    q.start, q.count, q.position, q.slot, q.state = i, 1, context - 1, i, D.UNBOUND
    queries.append(q)
  return dict(nq=nq, stride=stride, table=dev.array(table), keys=dev.array(keys), values=dev.array(values), queries=dev.queries(queries),
              q=dev.array(rng.standard_normal((nq, 16, 256)).astype(np.float32)), qg=dev.array(rng.standard_normal((nq, 16, 512)).astype(np.float32)))


def run_both(dev, case):
  rows = case["nq"]
  regular, static = dev.empty((rows, 16, 256)), dev.empty((rows, 16, 256))
  partials = dev.empty(dev.attention_scratch_bytes(rows, SPLITS) // 4)
  dev.attention(case["q"], case["qg"], case["keys"], case["values"], case["queries"], rows, rows, case["table"], case["stride"], BLOCK_TOKENS, SPLITS,
                partials, regular)
  code = dev.lib.infdev_attention_static(dev.ctx, case["q"].ptr, case["qg"].ptr, case["keys"].ptr, case["values"].ptr, case["queries"].ptr, rows, rows,
                                         case["table"].ptr, case["stride"], BLOCK_TOKENS, static.ptr)
  assert code == 0, dev.error()
  dev.commit()
  return regular.download(), static.download()


def test_static_scratch_attention_matches_regular_twice_in_a_row(dev):
  # same kernels, same split partition: the results must be identical, which is tighter than the 1e-3 bound
  # the attention tests use against the oracle
  first = build_case(dev, 101, [4000, 17, 1, 2500, 900, 16, 3333, 257])
  regular, static = run_both(dev, first)
  assert np.isfinite(static).all() and np.array_equal(regular, static)
  second = build_case(dev, 202, [35, 1200, 4096])  # fewer rows and shorter contexts: stale partials of call one remain in the array
  regular, static = run_both(dev, second)
  assert np.isfinite(static).all() and np.array_equal(regular, static)


def test_static_scratch_attention_refuses_more_than_eight_rows(dev):
  case = build_case(dev, 303, [20] * 9)
  out = dev.empty((9, 16, 256))
  code = dev.lib.infdev_attention_static(dev.ctx, case["q"].ptr, case["qg"].ptr, case["keys"].ptr, case["values"].ptr, case["queries"].ptr, 9, 9,
                                         case["table"].ptr, case["stride"], BLOCK_TOKENS, out.ptr)
  assert code == -2 and "at most 8" in dev.error()
