"""GPU: the request-stream workload of the multi-replica benchmark configuration on a reduced model (4 layers,
vocabulary 4096, MTP block): more streams than slots, a shared 2048-token prefix served from the prefix-checkpoint
cache, MTP drafting of width 4, temperature / top-p / top-k sampling with a per-request key."""
import os
import queue
import threading

import numpy as np
import pytest

from mtlqwen_b200.inference import InferenceEngine
from mtlqwen_b200.testing import synth

pytestmark = pytest.mark.gpu
LAYERS, VOCAB, WIDTH, PREFIX, STREAMS, GENERATED = 4, 4096, 4, 2048, 16, 24


@pytest.fixture(scope="module")
def weights(tmp_path_factory):
  path = tmp_path_factory.mktemp("gguf") / "tiny-mtp.gguf"
  synth.write_gguf(path, layers=LAYERS, vocab=VOCAB, mtp=True, seed=31)
  return path


def make_engine(weights):
  """INFENG_BATCH_INVARIANT=1 keeps every projection on the GEMV kernels and the delta rule on its token-by-token form,
  which compute each row on its own: a row's logits are then the same bits in a 40-row speculative pass and in a
  single-row pass, and however the scheduler cut the prompt into pieces, so sampled streams can be compared token for
  token. (By default the tensor-core GEMM takes the passes of more than 8 rows and prompt pieces go through the
  delta rule in 16-token chunks counted from where a piece starts; both differ from the row-wise kernels by some 1e-4,
  which a top-p boundary turns into a different token every few dozen samples.)"""
  os.environ.update(INFENG_DRAFT_WIDTH=str(WIDTH), INFENG_SEED="9", INFENG_KV_BLOCKS="256", INFENG_BATCH_INVARIANT="1")
  try:
    return InferenceEngine(weights, draft_weights=weights, max_context=4096)
  finally:
    os.environ.pop("INFENG_DRAFT_WIDTH"), os.environ.pop("INFENG_KV_BLOCKS"), os.environ.pop("INFENG_BATCH_INVARIANT")


def generate(engine, prompt, seed, speculative=True):
  sequence = engine.sequence(temperature=0.7, top_p=0.9, top_k=40, speculative=speculative, seed=seed)
  try:
    cursor, output = sequence.append(prompt), []
    while len(output) < GENERATED:
      output.append(sequence.read(cursor))
      cursor += 1
    sequence.cancel()
    while sequence.read(cursor) is not None:
      cursor += 1
    return output, sequence.speculative_counters()
  finally:
    sequence.close()


def test_sixteen_streams_over_eight_slots_share_the_prefix_and_sample_reproducibly(weights):
  rng = np.random.default_rng(3)
  prefix = [int(t) for t in rng.integers(0, VOCAB, PREFIX)]
  streams = [prefix + [int(t) for t in rng.integers(0, VOCAB, int(rng.integers(64, 200)))] for _ in range(STREAMS)]
  engine = make_engine(weights)
  try:
    assert engine.draft_width == WIDTH
    # the first stream computes the prefix and publishes its four 512-token checkpoints
    before = engine.step_counters()["prefill_rows"]
    results = {0: generate(engine, streams[0], 100)}
    first_rows = engine.step_counters()["prefill_rows"] - before
    assert first_rows == len(streams[0])
    # the other fifteen run eight at a time behind slot release; each restores the 2048-token prefix
    pending = queue.Queue()
    for index in range(1, STREAMS):
      pending.put(index)

    def worker():
      while True:
        try:
          index = pending.get_nowait()
        except queue.Empty:
          return
        results[index] = generate(engine, streams[index], 100 + index)

    before = engine.step_counters()["prefill_rows"]
    threads = [threading.Thread(target=worker) for _ in range(8)]
    for thread in threads:
      thread.start()
    for thread in threads:
      thread.join()
    computed = engine.step_counters()["prefill_rows"] - before
    suffixes = sum(len(streams[i]) - PREFIX for i in range(1, STREAMS))
    # (a suffix whose last chunk comes out as a single row is decoded, not prefilled, so a few rows may be missing)
    assert suffixes - STREAMS <= computed <= suffixes + 16 * (STREAMS - 1), (computed, suffixes)
    drafted = sum(counters["drafted_tokens"] for _, counters in results.values())
    accepted = sum(counters["accepted_tokens"] for _, counters in results.values())
    assert drafted >= WIDTH * STREAMS and 0 <= accepted <= drafted
  finally:
    engine.close()

  # The same streams alone, in other slots, on a fresh engine, without speculation: the same tokens. The variate of
  # a sequence's i-th token depends only on its key and i, and speculation never changes what is emitted.
  engine = make_engine(weights)
  try:
    for index in (0, 5, 15):
      alone, _ = generate(engine, streams[index], 100 + index, speculative=False)
      assert alone == results[index][0][:len(alone)], index
    other_key, _ = generate(engine, streams[5], 999, speculative=False)
    assert other_key != results[5][0][:len(other_key)]
  finally:
    engine.close()
