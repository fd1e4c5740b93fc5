"""GPU: sparse paged-KV gated GQA attention (BASELINE config 3) against the CPU oracle."""
import numpy as np
import pytest

import oracle
from mtlqwen_b200 import device as D
from mtlqwen_b200.testing import images

pytestmark = pytest.mark.gpu
TOL = 1e-3  # BASELINE: attention outputs within 1e-3 relative error in fp32 accumulation


def rel_err(got, want):
  want = want.astype(np.float64)
  return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


def run_attention(dev, rng, contexts, counts, block_tokens, max_splits=32):
  """Each sequence i holds contexts[i] tokens after this pass, the last counts[i] of which are the rows of the
  pass (counts[i] = 1 is a decode step). The earlier tokens are preloaded into a pool whose blocks are bound
  through a random permutation."""
  nq = len(contexts)
  blocks_per_seq = [-(-c // block_tokens) for c in contexts]
  stride = max(blocks_per_seq)
  physical = int(sum(blocks_per_seq))
  permutation = rng.permutation(physical).astype(np.int32)
  table = np.zeros((nq, stride), np.int32)
  at = 0
  for i, n in enumerate(blocks_per_seq):
    table[i, :n] = permutation[at:at + n]
    at += n
  pool_shape = (physical, 4, block_tokens, 256)
  keys = rng.standard_normal(pool_shape, dtype=np.float32).astype(np.float16)
  values = rng.standard_normal(pool_shape, dtype=np.float32).astype(np.float16)
  rows = int(sum(counts))
  qg = rng.standard_normal((rows, 16, 512)).astype(np.float32)
  k = rng.standard_normal((rows, 4, 256)).astype(np.float32)
  v = rng.standard_normal((rows, 4, 256)).astype(np.float32)
  q_norm = (1 + 0.01 * rng.standard_normal(256)).astype(np.float32)
  k_norm = (1 + 0.01 * rng.standard_normal(256)).astype(np.float32)
  max_context = max(contexts)
  queries, positions, attended, row_table, start = [], [], [], [], 0
  for i, (context, count) in enumerate(zip(contexts, counts)):
    q = D.Query()
    q.start, q.count, q.position, q.slot, q.state = start, count, context - count, i, D.UNBOUND
    queries.append(q)
    for p in range(count):
      positions.append(context - count + p)
      attended.append(context - count + p + 1)
      row_table.append(table[i])
    start += count
  rope = dev.rope_table(max_context)
  dq, dtable = dev.queries(queries), dev.array(table)
  dkeys, dvalues = dev.array(keys.view(np.uint16)), dev.array(values.view(np.uint16))
  q_out, out = dev.empty((rows, 16, 256)), dev.empty((rows, 16, 256))
  dqg = dev.array(qg)
  partials = dev.empty(dev.attention_scratch_bytes(rows, max_splits) // 4)
  dev.attention_prepare(dqg, dev.array(k), dev.array(v), dev.array(q_norm), dev.array(k_norm), rope, dq, nq, rows, dtable, stride, block_tokens,
                        q_out, dkeys, dvalues)
  # The reduce kernel also writes the quantised image of its output when asked; it must equal the quantisation of `out`.
  image, want_image = dev.empty(dev.image_bytes(rows, 4096), np.uint8), dev.empty(dev.image_bytes(rows, 4096), np.uint8)
  dev.image_capture(image)
  dev.attention(q_out, dqg, dkeys, dvalues, dq, nq, rows, dtable, stride, block_tokens, max_splits, partials, out)
  dev.quantize(out, rows, 4096, want_image)
  dev.commit()
  for a, b in zip(images.decode(image.download(), rows, 4096), images.decode(want_image.download(), rows, 4096)):
    assert a.tobytes() == b.tobytes()
  # oracle: same prepare, fp16 rounding at the cache, exact softmax
  rope_host = oracle.rope_table(max_context)
  assert rope.download().tobytes() == rope_host.tobytes()
  q_ref, k_ref = oracle.attention_prepare(qg, k, q_norm, k_norm, rope_host, positions)
  assert rel_err(q_out.download(), q_ref) < 1e-5
  kbits, vbits = oracle.f32_to_f16_bits(k_ref), oracle.f32_to_f16_bits(v)
  keys_u, values_u = keys.view(np.uint16).copy(), values.view(np.uint16).copy()
  row = 0
  for i, (context, count) in enumerate(zip(contexts, counts)):
    for p in range(count):
      pos = context - count + p
      block = table[i, pos // block_tokens]
      keys_u[block, :, pos % block_tokens, :] = kbits[row]
      values_u[block, :, pos % block_tokens, :] = vbits[row]
      row += 1
  # The appended K/V rows match the oracle's to one fp16 ulp (rsqrtf vs sqrt can flip the last rounding);
  # everything that was preloaded must be untouched. The softmax below then runs on the device's cache.
  got_keys, got_values = dkeys.download(), dvalues.download()
  assert np.array_equal(got_values, values_u)
  diff = np.abs(got_keys.view(np.float16).astype(np.float32) - keys_u.view(np.float16).astype(np.float32))
  assert np.all(diff <= 2.0**-10 * np.maximum(np.abs(keys_u.view(np.float16).astype(np.float32)), 2.0**-14))
  assert np.count_nonzero(got_keys != keys_u) <= rows * 1024 // 20
  keys_u = got_keys
  want = oracle.attention(q_ref, qg, keys_u, values_u, np.stack(row_table), attended, block_tokens)
  return rel_err(out.download(), want)


def test_attention_config3_decode(dev):
  """8 sequences, contexts uniform in [1, 32768], 16-token blocks bound through a seeded permutation."""
  rng = np.random.default_rng(7)
  contexts = [int(c) for c in rng.integers(1, 32769, 8)]
  assert run_attention(dev, rng, contexts, [1] * 8, 16) < TOL


@pytest.mark.parametrize("contexts,counts,block_tokens", [
  ([1], [1], 16),  # a single token attends to itself
  ([16, 17, 15], [1, 1, 1], 16),  # tile boundaries
  ([255, 256, 257, 513], [1, 1, 1, 1], 16),  # split boundaries
  ([300], [40], 128),  # prefill chunk: causal inside the chunk, 128-token blocks as the reference
  ([640, 12, 2000], [128, 12, 5], 128),  # mixed pass: long chunk, fresh sequence, speculative rows
  ([8192], [1], 512),
])
def test_attention_shapes(dev, contexts, counts, block_tokens):
  rng = np.random.default_rng(sum(contexts) + len(counts))
  assert run_attention(dev, rng, contexts, counts, block_tokens) < TOL


def test_attention_result_does_not_depend_on_batching(dev):
  """A row's split partition depends only on its own context: the output of a sequence's decode row inside an
  8-row pass equals, byte for byte, the output of the same row run alone on the same cache."""
  rng = np.random.default_rng(11)
  block_tokens, contexts = 16, [5000, 1, 17, 3333, 64, 12001, 700, 2049]
  blocks_per_seq = [-(-c // block_tokens) for c in contexts]
  stride, physical = max(blocks_per_seq), int(sum(blocks_per_seq))
  permutation = rng.permutation(physical).astype(np.int32)
  table, at = np.zeros((8, stride), np.int32), 0
  for i, n in enumerate(blocks_per_seq):
    table[i, :n] = permutation[at:at + n]
    at += n
  keys = rng.standard_normal((physical, 4, block_tokens, 256), dtype=np.float32).astype(np.float16).view(np.uint16)
  values = rng.standard_normal((physical, 4, block_tokens, 256), dtype=np.float32).astype(np.float16).view(np.uint16)
  qg = rng.standard_normal((8, 16, 512)).astype(np.float32)
  k, v = rng.standard_normal((8, 4, 256)).astype(np.float32), rng.standard_normal((8, 4, 256)).astype(np.float32)
  q_norm, k_norm = np.ones(256, np.float32), np.ones(256, np.float32)
  rope, dtable = dev.rope_table(max(contexts)), dev.array(table)

  def run(members):
    """One pass whose rows are the decode rows of the sequences in `members`, on a fresh copy of the cache."""
    rows, queries = len(members), []
    for row, i in enumerate(members):
      q = D.Query()
      q.start, q.count, q.position, q.slot, q.state = row, 1, contexts[i] - 1, i, D.UNBOUND
      queries.append(q)
    dq, dkeys, dvalues = dev.queries(queries), dev.array(keys), dev.array(values)
    dqg, q_out, out = dev.array(qg[members]), dev.empty((rows, 16, 256)), dev.empty((rows, 16, 256))
    partials = dev.empty(dev.attention_scratch_bytes(rows, 32) // 4)
    dev.attention_prepare(dqg, dev.array(k[members]), dev.array(v[members]), dev.array(q_norm), dev.array(k_norm), rope, dq, rows, rows, dtable, stride,
                          block_tokens, q_out, dkeys, dvalues)
    dev.attention(q_out, dqg, dkeys, dvalues, dq, rows, rows, dtable, stride, block_tokens, 32, partials, out)
    dev.commit()
    return out.download()

  together = run(list(range(8)))
  for i in (0, 1, 3, 5, 7):
    assert run([i])[0].tobytes() == together[i].tobytes(), i
  assert run([5, 2])[0].tobytes() == together[5].tobytes()  # another batch composition and row order
