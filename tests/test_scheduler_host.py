"""CPU: the engine's host side - scheduler thread, K/V reservation with LRU eviction, prefix-checkpoint cache,
acceptance bookkeeping, error codes - running over a host-only stand-in for the device layer
(tests/fake_device/fake_infdev.cpp, linked with csrc/scheduler.cpp and csrc/forward_pass.cpp into a library of its
own). The stand-in's toy model keeps a running hash of the fed tokens where the real kernels keep the recurrent state
and samples from it, so restoring the wrong checkpoint, committing the wrong candidate row or miscounting rows shows
up in the tokens and counters. These are the behavioural contracts of the reference's test/test_qwen35.py that do
not depend on the arithmetic; the GPU suite repeats the central ones on the real kernels."""
import ctypes
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np
import pytest

from mtlqwen_b200 import inference
from mtlqwen_b200.testing import synth

ROOT = Path(__file__).resolve().parents[1]
LAYERS, VOCAB, WIDTH = 4, 512, 4
BLOCK_BYTES = 2 * 256 * 1024  # K and V tile of one 128-token block of one attention layer (device.hpp:109-111)


@pytest.fixture(scope="module")
def library():
  target = ROOT / "tests" / "_build" / "libinfeng_fake.so"
  target.parent.mkdir(exist_ok=True)
  csrc = ROOT / "mtlqwen_b200" / "csrc"
  sources = [csrc / "scheduler.cpp", csrc / "forward_pass.cpp", ROOT / "tests" / "fake_device" / "fake_infdev.cpp"]
  inputs = sources + list(csrc.glob("*.hpp")) + list((ROOT / "include").glob("*.h"))
  if not target.exists() or any(p.stat().st_mtime > target.stat().st_mtime for p in inputs):
    subprocess.run(["g++", "-O1", "-std=c++17", "-shared", "-fPIC", "-pthread", "-I", str(ROOT / "include"), *map(str, sources), "-o", str(target)],
                   check=True, capture_output=True, text=True)
  lib = inference.bind(target)
  lib.fake_infdev_fail_commits.argtypes = (ctypes.c_int, )
  return lib


@pytest.fixture(scope="module")
def weights(tmp_path_factory):
  path = tmp_path_factory.mktemp("gguf") / "tiny-mtp.gguf"
  synth.write_gguf(path, layers=LAYERS, vocab=VOCAB, mtp=True, seed=5)
  return path


def engine_of(library, weights, context=2048, drafter=False, **environment):
  saved = {key: os.environ.get(key) for key in environment}
  os.environ.update({key: str(value) for key, value in environment.items()})
  try:
    return inference.InferenceEngine(weights, draft_weights=weights if drafter else None, max_context=context, library=library)
  finally:
    for key, value in saved.items():
      os.environ.pop(key) if value is None else os.environ.__setitem__(key, value)


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


def tokens_of(seed, length):
  return [int(t) for t in np.random.default_rng(seed).integers(0, VOCAB, length)]


def test_mixed_batch_equals_solo_and_prefix_restore(library, weights):
  """test_qwen35.py:78-116 on the host logic: a pass that mixes a prefill chunk with decodes gives each sequence what
  it gets alone; a 520-token prompt leaves length 520; the same prompt again restores the 512-token checkpoint and
  recomputes only the 8 tokens after it."""
  model = engine_of(library, weights)
  try:
    assert model.drafter == "none" and model.vocab_size == VOCAB
    reference = [model.sequence() for _ in range(3)]
    prompt = tokens_of(2, 200)
    expected = [complete(reference[0], prompt, 1)]
    for sequence, start in ((reference[1], [10, 11, 12]), (reference[2], [20, 21, 22])):
      one(sequence, start)
      expected.append(complete(sequence, limit=3))
    for sequence in reference:
      sequence.close()
    actual = [model.sequence() for _ in range(3)]
    one(actual[1], [10, 11, 12]), one(actual[2], [20, 21, 22])
    observed = parallel([lambda: complete(actual[0], prompt, 1), lambda: complete(actual[1], limit=3), lambda: complete(actual[2], limit=3)])
    assert observed == expected and actual[0].length >= 200
    for sequence in actual:
      sequence.close()

    first, second = model.sequence(), model.sequence()
    long_prompt = tokens_of(3, 520)
    rows = model.step_counters()["rows"]
    token = one(first, long_prompt)
    computed = model.step_counters()["rows"] - rows
    assert first.length >= 520 and computed >= 520
    computed = model.step_counters()["rows"] - rows  # with the decode rows that ran before the cancel arrived
    assert one(second, long_prompt) == token and second.length >= 520
    assert model.step_counters()["rows"] - rows - computed <= 16  # the 8 tokens after the checkpoint, and decode rows until the cancel
    assert complete(first, limit=4) == complete(second, limit=4)
    first.close(), second.close()
  finally:
    model.close()


@pytest.mark.parametrize("prompt_length", [520, 1032])
def test_prefix_cache_aliases_share_physical_blocks(library, weights, prompt_length):
  """test_qwen35.py:249-272: four sequences that restore the same prefix bind the same physical K/V blocks, so the
  bytes ever bound do not grow while the shared blocks suffice, and a later sequence reuses the prefix again."""
  model = engine_of(library, weights, context=4096)
  try:
    source, aliases = model.sequence(), [model.sequence() for _ in range(4)]
    prompt = tokens_of(7, prompt_length)
    expected = one(source, prompt)
    mapped = model.mapped_bytes
    assert parallel([lambda s=s: one(s, prompt) for s in aliases]) == [expected] * 4
    assert all(prompt_length <= s.length < prompt_length + 100 for s in aliases)
    # the blocks up to the last 512 boundary are shared; each alias owns only the one block after it
    assert model.mapped_bytes <= mapped + 4 * BLOCK_BYTES
    source.close()
    for sequence in aliases:
      sequence.close()
    reused = model.sequence()
    rows = model.step_counters()["rows"]
    assert one(reused, prompt) == expected and reused.length >= prompt_length
    assert model.step_counters()["rows"] - rows <= prompt_length % 512 + 8
    reused.close()
  finally:
    model.close()


def test_evicted_prefix_is_recomputed(library, weights):
  """test_qwen35.py:295-309: with a pool of one context, a second long prompt evicts the first one's blocks and with
  them its checkpoint; the first prompt is then computed again and gives the same token."""
  model = engine_of(library, weights, context=1024)
  try:
    prompt = tokens_of(8, 520)
    sequence = model.sequence()
    expected = one(sequence, prompt)
    sequence.close()
    for other in (tokens_of(9, 520), tokens_of(10, 520)):
      sequence = model.sequence()
      one(sequence, other)
      sequence.close()
    sequence = model.sequence()
    rows = model.step_counters()["rows"]
    assert one(sequence, prompt) == expected and sequence.length >= 520
    assert model.step_counters()["rows"] - rows >= 520
    sequence.close()
  finally:
    model.close()


def test_all_slots_ninth_sequence_and_bound_bytes(library, weights):
  """test_qwen35.py:275-292: 8 slots in parallel == serial, one block each (8 x K+V tiles), a 9th sequence refused."""
  model = engine_of(library, weights, context=1024)
  try:
    prompts = [[row * 32 + token + 1 for token in range(16)] for row in range(8)]
    references = []
    for prompt in prompts:
      sequence = model.sequence()
      references.append(one(sequence, prompt))
      sequence.close()
    sequences = [model.sequence() for _ in range(8)]
    assert parallel([lambda row=row: one(sequences[row], prompts[row]) for row in range(8)]) == references
    assert model.mapped_bytes == 8 * BLOCK_BYTES
    with pytest.raises(RuntimeError, match="maximum live sequence count"):
      model.sequence()
    for sequence in sequences:
      sequence.close()
  finally:
    model.close()


def test_allocator_failure_is_atomic(library, weights):
  """test_qwen35.py:233-246."""
  model = engine_of(library, weights, context=16)
  try:
    owner, blocked = model.sequence(), model.sequence()
    one(owner, [1, 2, 3])
    length = owner.length
    with pytest.raises(RuntimeError, match="no evictable capacity"):
      one(blocked, [4, 5, 6])
    assert owner.length == length and blocked.length == 0
    owner.close()
    assert one(blocked, []) is not None
    blocked.close()
  finally:
    model.close()


def test_error_codes_of_append(library, weights):
  model = engine_of(library, weights, context=64)
  try:
    sequence = model.sequence()
    with pytest.raises(RuntimeError, match="no available model context"):
      sequence.append([])
    with pytest.raises(RuntimeError, match="no available model context"):
      sequence.append([VOCAB])  # outside the vocabulary
    with pytest.raises(RuntimeError, match="no available model context"):
      sequence.append(list(range(65)))  # longer than the context
    assert model.step_counters()["passes"] == 0
    output = complete(sequence, [1, 2, 3, 4])
    assert sequence.length == 64 and len(output) == 61  # generation stops at the context limit
    with pytest.raises(RuntimeError, match="at most 64 stop tokens"):
      model.sequence(stop_token_ids=list(range(65)))
    sequence.close()
  finally:
    model.close()


def test_device_failure_reaches_the_reader_and_the_engine_recovers(library, weights):
  """A failed commit is reported to every sequence of the batch as -5 (the path of a capacity failure,
  engine.cpp:200-201), nothing of the failed pass is kept, and the next request runs normally."""
  model = engine_of(library, weights)
  try:
    healthy = model.sequence()
    expected = complete(healthy, [5, 6, 7], 3)
    healthy.close()
    sequence = model.sequence()
    library.fake_infdev_fail_commits(1)
    with pytest.raises(RuntimeError, match="no evictable capacity"):
      one(sequence, [5, 6, 7])
    assert sequence.length == 0
    assert complete(sequence, [], 3) == expected  # the prompt is still queued: a retry needs no new tokens
    sequence.close()
  finally:
    library.fake_infdev_fail_commits(0)
    model.close()


def test_speculative_contracts(library, weights):
  """test_qwen35.py:118-176 with the stand-in's drafter (right except at every fourth position): speculative ==
  plain greedy; a stop token inside an accepted draft is emitted and ends the sequence there; a sequence one token
  short of a 512 boundary does not speculate; a rejected draft rolls the state back."""
  model = engine_of(library, weights, drafter=True, INFENG_DRAFT_WIDTH=WIDTH)
  try:
    assert model.drafter == "mtp" and model.draft_width == WIDTH
    prompt = tokens_of(11, 45)
    plain, speculative = model.sequence(), model.sequence(speculative=True)
    want = complete(plain, prompt, 24)
    assert complete(speculative, prompt, 24) == want
    counters = speculative.speculative_counters()
    assert 0 < counters["accepted_tokens"] < counters["drafted_tokens"]
    plain.close(), speculative.close()

    # the stop token is the second token of a speculative step whose first proposal was accepted
    stopper = model.sequence(stop_token_ids=[want[2]], speculative=True)
    assert one(stopper, prompt) == want[0]
    assert complete(stopper) == [want[1]]
    assert stopper.length == len(prompt) + 2
    accepted = stopper.speculative_counters()["accepted_tokens"]
    assert accepted in (0, 1)  # 1 when the drafter had proposed want[2] itself
    stopper.close()

    # stop and resume after every step: each speculative step starts from the state its predecessor's acceptance left
    rollback_reference, rollback = model.sequence(), model.sequence(speculative=True)
    straight = complete(rollback_reference, [30, 31, 32], 40)
    cursor, stepwise = rollback.append([30, 31, 32]), []
    for _ in range(6):
      stepwise.append(rollback.read(cursor))
      cursor += 1
      rollback.cancel()
      while (token := rollback.read(cursor)) is not None:
        stepwise.append(token)
        cursor += 1
      assert rollback.append([]) == cursor
    rollback.cancel()
    assert 6 <= len(stepwise) <= 40 and stepwise == straight[:len(stepwise)]
    rollback_reference.close(), rollback.close()
  finally:
    model.close()


def test_no_speculation_across_a_checkpoint_boundary(library, weights):
  """test_qwen35.py:130-147: with one token of room to the next 512 boundary a sequence decodes a plain row. The
  context limit of 512 ends the sequence there, so the counters are exact."""
  model = engine_of(library, weights, context=512, drafter=True, INFENG_DRAFT_WIDTH=WIDTH, INFENG_KV_BLOCKS=16)
  try:
    prompt = tokens_of(12, 511)
    plain, edge = model.sequence(), model.sequence(speculative=True)
    assert complete(edge, prompt) == complete(plain, prompt)
    assert edge.length == 512 and edge.speculative_counters()["drafted_tokens"] == 0
    # with room for a whole draft the same engine does speculate
    short = model.sequence(speculative=True)
    complete(short, tokens_of(13, 20), 6)
    assert short.speculative_counters()["drafted_tokens"] >= WIDTH
    for sequence in (plain, edge, short):
      sequence.close()
  finally:
    model.close()


def test_slot_reuse_during_generation(library, weights):
  """test_qwen35.py:312-335: sequences come and go on four threads while others generate."""
  model = engine_of(library, weights, context=1024, drafter=True, INFENG_DRAFT_WIDTH=WIDTH)
  try:
    prompts = [[row * 32 + token + 1 for token in range(16)] for row in range(4)]
    expected = []
    for prompt in prompts:
      sequence = model.sequence(speculative=True)
      expected.append(complete(sequence, prompt, 4))
      sequence.close()

    def cycle(row):
      for _ in range(4):
        sequence = model.sequence(speculative=True)
        try:
          assert complete(sequence, prompts[row], 4) == expected[row]
        finally:
          sequence.close()

    parallel([lambda row=row: cycle(row) for row in range(4)])
  finally:
    model.close()


def test_engine_outlives_close_while_sequences_live(library, weights):
  """test_qwen35.py:179-188."""
  model = engine_of(library, weights, context=256)
  sequence = model.sequence()
  model.close()
  assert len(complete(sequence, [7, 8, 9], 2)) == 2
  sequence.close()


def test_requests_arriving_together_compute_a_shared_prefix_once(library, weights):
  """Eight requests with the same 1024-token prefix and different suffixes start at the same moment. One of them
  computes each 512-token block of the prefix while the others sit those passes out and then restore the published
  checkpoint, so the engine prefills the prefix once plus the suffixes, and every request still gets the tokens it
  gets alone."""
  model = engine_of(library, weights, context=2048, INFENG_KV_BLOCKS=128, INFENG_CHECKPOINTS=32)
  try:
    prefix = tokens_of(40, 1024)
    prompts = [prefix + tokens_of(41 + i, 30 + 7 * i) for i in range(8)]
    alone = []
    for prompt in prompts[:3]:
      fresh = engine_of(library, weights, context=2048)
      sequence = fresh.sequence()
      alone.append(complete(sequence, prompt, 3))
      sequence.close()
      fresh.close()
    sequences = [model.sequence() for _ in range(8)]
    before = model.step_counters()["prefill_rows"]
    together = parallel([lambda s=s, p=p: complete(s, p, 3) for s, p in zip(sequences, prompts)])
    computed = model.step_counters()["prefill_rows"] - before
    assert together[:3] == alone
    suffixes = sum(len(p) - 1024 for p in prompts)
    assert 1024 + suffixes <= computed <= 1024 + suffixes + 64, (computed, suffixes)
    for sequence in sequences:
      sequence.close()
  finally:
    model.close()
