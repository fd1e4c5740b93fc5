"""Latency / throughput report of one engine in the terms of the reference's benchmarks/benchmark_qwen35.py:
TTFT (append to first token of all sessions), TPOT (decode time per token), TTL, aggregate / prefill / decode
tokens per second, mapped K/V bytes, MBU (weight bytes / TPOT against the memory bandwidth) and MFU
(2 * parameters * prompt tokens / TTFT against the tensor peak), drafted / accepted counts. Same sessions, same
timing points and same formulas (benchmark_qwen35.py:24-54, 93-111); the machine constants are a B200's instead of an
M2 Pro's, read from MEASURED_PEAKS.json at the repository root when it is there.

  python -m mtlqwen_b200.benchmark [--weights FILE] [--draft-weights FILE] [--batch 8] [--prefill 128] [--decode 256]

Without --weights it runs on the random-init Qwen3.5-9B-shaped GGUF that the tests and bench.py use (written on
first use, about 5.7 GB under /tmp).
"""
import argparse
import json
import random
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from time import perf_counter

from .inference import InferenceEngine

ROOT = Path(__file__).resolve().parents[1]
BANDWIDTH_BPS, FLOPS = 7.7e12, 2.25e15  # nominal HBM3e and dense bf16 / fp16 of a B200


def machine_constants():
  path = ROOT / "MEASURED_PEAKS.json"
  if path.exists():
    peaks = json.loads(path.read_text())
    return peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12, "measured on this machine"
  return BANDWIDTH_BPS, FLOPS, "nominal"


def run(model, tokens, decode, batch, speculative=False):
  """One timed round (benchmark_qwen35.py:24-54): `batch` sessions take the same prompt at once; TTFT ends when every
  one of them has its first token, the decode time when every one has `decode` more."""
  sessions = [model.sequence(speculative=speculative) for _ in range(batch)]

  def first(session):
    cursor = session.append(tokens)
    assert session.read(cursor) is not None
    return cursor + 1

  def finish(item):
    session, cursor = item
    for _ in range(decode):
      if session.read(cursor) is None: break
      cursor += 1
    session.cancel()
    return cursor

  def stop(item):
    session, cursor = item
    while session.read(cursor) is not None:
      cursor += 1

  with ThreadPoolExecutor(max_workers=batch) as pool:
    start = perf_counter()
    cursors = list(pool.map(first, sessions))
    ttft = perf_counter() - start
    start = perf_counter()
    cursors = list(pool.map(finish, zip(sessions, cursors)))
    elapsed = perf_counter() - start
    list(pool.map(stop, zip(sessions, cursors)))
  mapped = model.mapped_bytes
  spec = [session.speculative_counters() for session in sessions]
  for session in sessions:
    session.close()
  return ttft, elapsed, mapped, sum(item["drafted_tokens"] for item in spec), sum(item["accepted_tokens"] for item in spec)


def report(model, tokens, decode, batch, speculative, warmup, iters):
  """Mean over `iters` rounds after `warmup` untimed ones; returns the figures as a dict."""
  bandwidth, flops, source = machine_constants()
  for _ in range(warmup):
    run(model, tokens, decode, batch, speculative)
  ttft, decode_times, mapped, drafted, accepted = [], [], 0, 0, 0
  for _ in range(iters):
    first, rest, mapped, proposed, kept = run(model, tokens, decode, batch, speculative)
    ttft.append(first)
    decode_times.append(rest)
    drafted += proposed
    accepted += kept
  ttft_s, decode_s = sum(ttft) / len(ttft), sum(decode_times) / len(decode_times)
  tpot_s, ttl_s, prefill = decode_s / decode, ttft_s + decode_s, len(tokens)
  return {
    "batch": batch, "prefill": prefill, "decode": decode, "speculative": speculative, "TTFT_ms": ttft_s * 1e3, "TPOT_ms": tpot_s * 1e3, "TTL_s": ttl_s,
    "aggregate_tok_s": batch * (prefill + decode) / ttl_s, "prefill_aggregate_tok_s": batch * prefill / ttft_s, "decode_aggregate_tok_s": batch / tpot_s,
    "session_decode_tok_s": 1 / tpot_s, "mapped_kv_MiB": mapped / 2**20,
    "MBU_pct": None if speculative else model.weight_bytes / tpot_s / bandwidth * 100,
    "MFU_pct": 2 * model.parameter_count * batch * prefill / ttft_s / flops * 100, "drafted": drafted, "accepted": accepted,
    "acceptance_pct": accepted / drafted * 100 if drafted else 0.0, "machine_constants": source,
  }


def main():
  p = argparse.ArgumentParser()
  p.add_argument("--weights", type=Path)
  p.add_argument("--draft-weights", type=Path)
  p.add_argument("--max-context", type=int, default=4096)
  p.add_argument("--prefill", type=int, default=128)
  p.add_argument("--prompt-ids", help="comma-separated token IDs; overrides --prefill random input")
  p.add_argument("--decode", type=int, default=256)
  p.add_argument("--batch", type=int, default=8)
  p.add_argument("--warmup", type=int, default=1)
  p.add_argument("--iters", type=int, default=3)
  p.add_argument("--speculative", action="store_true")
  a = p.parse_args()
  if a.weights is None:
    from .testing import synth
    a.weights = synth.ensure_full_model()
    if a.speculative and a.draft_weights is None:
      a.draft_weights = a.weights  # the synthetic file carries an MTP block
  model = InferenceEngine(a.weights, draft_weights=a.draft_weights, max_context=a.max_context)
  if not 1 <= a.batch <= model.max_batch_sequences:
    p.error(f"--batch must be between 1 and {model.max_batch_sequences}")
  if a.speculative and model.drafter == "none":
    p.error("--speculative requires --draft-weights")
  rng = random.Random(1)
  tokens = [int(t) for t in a.prompt_ids.split(",")] if a.prompt_ids else [rng.randrange(model.vocab_size) for _ in range(a.prefill)]
  figures = report(model, tokens, a.decode, a.batch, a.speculative, a.warmup, a.iters)
  model.close()
  print(f"# Qwen3.5 CUDA benchmark\nweights={a.weights} drafter={model.drafter} draft_width={model.draft_width}")
  print(" ".join(f"{key}={value:.2f}" if isinstance(value, float) else f"{key}={value}" for key, value in figures.items()))
  print(json.dumps(figures))


if __name__ == "__main__":
  main()
