"""Benchmark of the ragged continuous-batching forward step.

Metric (BASELINE.json): aggregate decode tokens/s at 8 live sequences per GPU, plus the Q4_K GEMV fraction of
HBM peak. Headline workload (config 4): the full Qwen3.5-9B-shaped decoder (32 layers = 8 x (3 GDN + 1 gated
attention), hidden 4096, SwiGLU 12288, vocabulary 248320; all projections Q4_K, embedding / lm_head Q6_K) with
random-init weights in a GGUF file written on the fly, 8 sequences with seeded token-id prompts of ragged length
uniform in [128, 4096], greedy sampling, prefill chunks mixed with decodes in one packed pass. A "step" is one pass
in which every one of the 8 live sequences decodes one token.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--case NAME]

N > 1 runs N independent engine replicas (one process per GPU under torchrun, no data-path collective); `value`
is the whole-job rate. The same line carries `cfg5` (64 request streams with a shared 2048-token prefix routed over
the replicas, MTP drafting of width 4, temperature / top-p / top-k sampling, 512 tokens each, with and without
speculation) and `configs` (the single-kernel configurations 1 to 3, lm_head and the prefill GEMM, on rank 0's GPU).
`--impl reference` times the CPU oracle (the scalar restatement of the reference's Metal kernels; Metal itself
cannot run on Linux) on the host cores for the same decode step. `--case` runs one small case alone (the commands
of the profile summaries).
"""
import argparse
import json
import os
import queue
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LAYERS, VOCAB, SEQUENCES, SEED = 32, 248320, 8, 1234
WEIGHT_BYTES_PER_STEP = 24 * 123_896_576 + 8 * 117_999_616 + 834_355_200  # Q4_K/Q6_K bytes read by one decode pass
STATE_BYTES_PER_STEP = 8 * 24 * (8192 * 4 * 4 + 32 * 128 * 128 * 4) * 2  # GDN conv + recurrent state, read and written
# DRAM bytes (read + write) of one launch of the Q4_K decode GEMV at the config-1 shape with 8 rows, from an ncu capture
# of that launch (dram__bytes_read.sum + dram__bytes_write.sum): the weights once, the result stays in L2.
GEMV_DRAM_BYTES_PER_LAUNCH = 28_399_488
DTYPE = ("f32 activations in HBM; Q4_K GEMV (<= 8 rows): u8 x int16-per-256-block integer MMA; prefill GEMM: fp16 operands, fp32 accumulate; "
         "K/V fp16")


def prompts(vocab=VOCAB, longest=4096):
  rng = np.random.default_rng(SEED + 4)
  lengths = rng.integers(min(128, longest), longest + 1, SEQUENCES)
  return [[int(t) for t in rng.integers(0, vocab, int(n))] for n in lengths]


class ClockSampler:
  """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
  FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

  def __init__(self, gpu):
    self.gpu, self.process, self.lines = gpu, None, []

  def start(self):
    try:
      self.process = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                                      stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
      threading.Thread(target=lambda: self.lines.extend(self.process.stdout), daemon=True).start()
    except OSError:
      self.process = None

  def stop(self, busy_from, busy_to, started):
    if not self.process:
      return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
    time.sleep(0.25)
    self.process.terminate()
    # nvidia-smi emits one line per 200 ms from `started`; keep those that fall inside the timed region
    rows = [[field.strip() for field in line.split(",")] for line in self.lines if line.count(",") >= 7]
    inside = [row for i, row in enumerate(rows) if busy_from - 0.25 <= started + 0.2 * i <= busy_to + 0.25] or rows
    clocks = [float(row[1]) for row in inside if row[1].replace(".", "").isdigit()]
    reasons = set()
    for row in inside:
      for name, value in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), row[4:8]):
        if value == "Active":
          reasons.add(name)
    return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": float(rows[0][2]) if rows else None,
            "reasons": sorted(reasons), "samples": len(inside)}


def measured_peak():
  path = ROOT / "MEASURED_PEAKS.json"
  if path.exists():
    return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
  return 6650.0, "fallback"


# ---- CPU baseline: the oracle decoding the same 8 sequences ---------------------------------------------------------
def host_threads():
  """The oracle parallelises with OpenMP. torchrun exports OMP_NUM_THREADS=1 to its workers, which would turn the
  baseline into a single-thread run: the count is set explicitly, before the oracle's library is loaded."""
  cores = os.cpu_count() or 1
  os.environ["OMP_NUM_THREADS"] = str(cores)
  return cores


def cpu_decode(path, contexts, steps, warmup, seconds_budget=None):
  """Times the CPU oracle on the decode step the GPU arm is timed on: 8 sequences, one token each per step, in one
  batched pass (a weight row is dequantised once for all 8, as the engine reads it once). The sequences' contexts are
  set to `contexts` without computing the prompts on the CPU (that alone would take the better part of an hour): K/V
  caches and recurrent states are filled with seeded values of the distributions the benchmark configurations give
  them, which leaves the work of a decode step - weights, states and K/V of the same sizes - unchanged.
  Returns tokens/s, steps timed, seconds, threads."""
  cores = host_threads()
  import oracle
  from mtlqwen_b200.testing import synth
  tensors = synth.read_gguf(path)
  room = max(contexts) + warmup + (steps or 64) + 8
  rng = np.random.default_rng(SEED + 9)
  models = []
  for context in contexts:
    model = oracle.Model(tensors, LAYERS, VOCAB, room)
    model._keys[:, :context] = rng.standard_normal((model._keys.shape[0], context, 1024), dtype=np.float32).astype(np.float16)
    model._values[:, :context] = rng.standard_normal((model._values.shape[0], context, 1024), dtype=np.float32).astype(np.float16)
    model._S[:] = 0.01 * rng.standard_normal(model._S.shape, dtype=np.float32)
    model._conv[:] = rng.standard_normal(model._conv.shape, dtype=np.float32)
    model._state.length = context
    models.append(model)
  tokens = [17 + i for i in range(len(models))]
  for _ in range(warmup):
    tokens = [int(np.argmax(row)) for row in oracle.decode_batch(models, tokens)[1]]
  started, done = time.perf_counter(), 0
  while (steps is not None and done < steps) or (steps is None and (done < 2 or time.perf_counter() - started < seconds_budget)):
    tokens = [int(np.argmax(row)) for row in oracle.decode_batch(models, tokens)[1]]
    done += 1
  elapsed = time.perf_counter() - started
  return len(models) * done / elapsed, done, elapsed, cores


def cpu_configs():
  """BASELINE configs 1 to 3 on the CPU oracle, single-threaded and on all host cores (median of 5 runs each), on the
  seeded inputs of the GPU cases: the Q4_K linear 12288 x 4096 with 8 rows, one GDN layer decode step of 8 sequences,
  and decode attention over 8 contexts uniform in [1, 32768]."""
  cores = host_threads()
  import oracle
  from mtlqwen_b200.testing import synth
  rng = np.random.default_rng(SEED + 11)
  w, x = synth.weight(oracle.Q4_K, 12288, 4096, 1235), synth.activations(8, 4096, 1236)
  gdn = dict(x=synth.activations(8, 4096, 8), mixed=synth.activations(8, 8192, 9), z=synth.activations(8, 4096, 10),
             wb=(rng.standard_normal((32, 4096)) / 64).astype(np.float32), wa=(rng.standard_normal((32, 4096)) / 64).astype(np.float32),
             A=(-rng.uniform(1, 16, 32)).astype(np.float32), dt=(0.1 * rng.standard_normal(32)).astype(np.float32),
             conv=(0.5 * rng.standard_normal((8192, 4))).astype(np.float32), norm=np.ones(128, np.float32),
             taps=rng.standard_normal((8, 8192, 4)).astype(np.float32), S=(0.01 * rng.standard_normal((8, 32, 128, 128))).astype(np.float32))
  contexts = [int(c) for c in np.random.default_rng(7).integers(1, 32769, 8)]
  blocks = [-(-c // 16) for c in contexts]
  table = np.zeros((8, max(blocks)), np.int32)
  order, at = rng.permutation(sum(blocks)).astype(np.int32), 0
  for i, count in enumerate(blocks):
    table[i, :count] = order[at:at + count]
    at += count
  keys = rng.standard_normal((sum(blocks), 4, 16, 256), dtype=np.float32).astype(np.float16).view(np.uint16)
  values = rng.standard_normal((sum(blocks), 4, 16, 256), dtype=np.float32).astype(np.float16).view(np.uint16)
  q, qg = rng.standard_normal((8, 16, 256)).astype(np.float32), rng.standard_normal((8, 16, 512)).astype(np.float32)

  def gdn_step():
    for i in range(8):
      beta, g = oracle.gdn_ba(gdn["x"][i:i + 1], gdn["wb"], gdn["wa"], gdn["A"], gdn["dt"])
      qo, ko, vo, _ = oracle.gdn_conv(gdn["mixed"][i:i + 1], gdn["conv"], gdn["taps"][i])
      o, _, _ = oracle.delta_rule(qo, ko, vo, g, beta, gdn["S"][i])
      oracle.gated_rms_norm(o, gdn["z"][i:i + 1], gdn["norm"])

  cases = {"cfg1_m8": lambda: oracle.linear(w, oracle.Q4_K, 12288, 4096, x), "cfg2_gdn_decode": gdn_step,
           "cfg3_attention": lambda: oracle.attention(q, qg, keys, values, table, contexts, 16)}
  out = {}
  for name, call in cases.items():
    entry = {}
    for label, threads in (("one_thread_ms", 1), ("all_cores_ms", cores)):
      oracle.set_threads(threads)
      samples = []
      for _ in range(5):
        started = time.perf_counter()
        call()
        samples.append(time.perf_counter() - started)
      entry[label] = 1e3 * statistics.median(samples)
    entry["cores"] = cores
    out[name] = entry
  oracle.set_threads(cores)
  return out


def reference_contexts(warmup):
  return [len(p) + warmup for p in prompts()]


def run_reference(args, rank, world):
  if rank != 0:
    return
  from mtlqwen_b200.testing import synth
  path = synth.ensure_full_model()
  contexts = reference_contexts(args.warmup)
  warmup = min(args.warmup, 2)
  rate, done, elapsed, cores = cpu_decode(path, contexts, steps=args.steps, warmup=warmup)
  sample = (f"{done} batched decode steps of the same 8 sequences of the 32-layer model at contexts {min(contexts)}..{max(contexts)} "
            f"(mean {sum(contexts) // len(contexts)}); K/V caches and recurrent states filled with seeded synthetic values instead of computing the "
            "prompts on the CPU")
  print(json.dumps({
    "impl": "reference", "metric": "decode_tokens_per_second", "value": rate, "unit": "tok/s", "n_gpus": args.gpus, "steps": done,
    "warmup": warmup, "ms_per_step": 1e3 * elapsed / done, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
    "dtype": "f32", "data": "synthetic", "config": workload_config(),
    "cpu_baseline": {"value": rate, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
    "e2e": {"value": rate, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0,
    "note": "CPU oracle port of the reference's Metal kernels (Metal is unavailable on this box); all host cores via OpenMP; one host, one "
            "replica whatever --gpus says"
  }))


def workload_config():
  return {"workload": "config 4: Qwen3.5-9B-shaped 32-layer decoder, Q4_K projections + Q6_K embedding/lm_head, random init, "
                      "8 live sequences, ragged prompts U[128,4096], greedy decode", "live_sequences_per_gpu": SEQUENCES,
          "parallelism": "replicas", "l2_policy": "inputs larger than L2: 4.75 GB of weights streamed per step"}


# ---- config 4: the headline ---------------------------------------------------------------------------------------
def run_config4(args, local, path, dist, longest=4096):
  from mtlqwen_b200.inference import InferenceEngine
  os.environ.update(INFENG_KV_BLOCKS="384", INFENG_SEED=str(SEED), INFENG_DEVICE=str(local))
  engine = InferenceEngine(path, max_context=8192)
  texts = prompts(longest=longest)
  sequences = [engine.sequence() for _ in range(SEQUENCES)]
  warmup, steps = args.warmup, args.steps
  stamps = [[] for _ in range(SEQUENCES)]
  counters = [[] for _ in range(SEQUENCES)]
  finished = threading.Event()

  def reader(i):
    cursor = sequences[i].append(texts[i])
    while not finished.is_set():
      token = sequences[i].read(cursor)
      if token is None:
        break
      cursor += 1
      stamps[i].append(time.perf_counter())
      counters[i].append(engine.step_counters())
    sequences[i].cancel()

  if dist:
    dist.barrier()
  sampler = ClockSampler(local)
  sampler_started = time.perf_counter()
  sampler.start()
  threads = [threading.Thread(target=reader, args=(i, )) for i in range(SEQUENCES)]
  for thread in threads:
    thread.start()
  # The timed region opens when the last sequence has decoded `warmup` tokens (so all 8 are live and only decode
  # passes run) and closes `steps` passes later, on the clock of that last sequence.
  while any(len(s) < warmup + 1 for s in stamps):
    time.sleep(0.002)
  last = max(range(SEQUENCES), key=lambda i: stamps[i][warmup])
  first_index = len(stamps[last]) - 1  # the pass that just completed
  while len(stamps[last]) < first_index + steps + 1:
    time.sleep(0.002)
  finished.set()
  for thread in threads:
    thread.join()
  t0, t1 = stamps[last][first_index], stamps[last][first_index + steps]
  c0, c1 = counters[last][first_index], counters[last][first_index + steps]
  result = {
    # every pass of the window is a decode pass of all live sequences: its rows are the tokens handed to the readers
    "tokens": c1["rows"] - c0["rows"], "wall": t1 - t0, "clocks": sampler.stop(t0, t1, sampler_started),
    "device_seconds": (c1["device_ns"] - c0["device_ns"]) / 1e9, "passes": c1["passes"] - c0["passes"], "rows": c1["rows"] - c0["rows"],
    "launches": c1["launches"] - c0["launches"], "contexts": [sequence.length for sequence in sequences], "c0": c0, "c1": c1}
  for sequence in sequences:
    sequence.close()
  engine.close()
  return result


# ---- config 5: request streams over replicas ----------------------------------------------------------------------
STREAMS, PREFIX_TOKENS, GENERATED, DRAFT_WIDTH = 64, 2048, 512, 4


def config5_streams():
  rng = np.random.default_rng(SEED + 5)
  prefix = [int(t) for t in rng.integers(0, VOCAB, PREFIX_TOKENS)]
  return [prefix + [int(t) for t in rng.integers(0, VOCAB, int(rng.integers(64, 1025)))] for _ in range(STREAMS)]


def run_config5(local, rank, world, path, dist, speculative, generated=GENERATED, streams=None):
  """This rank's share of the streams, 8 live at a time, the rest queued behind slot release. Returns the tokens
  generated, wall seconds from the first append to the last token, and the engine's counters."""
  from mtlqwen_b200 import replicas
  from mtlqwen_b200.inference import InferenceEngine
  streams = streams or config5_streams()
  mine = replicas.route(streams, world)[rank]
  # 64 cache entries of 53 MB each and 1024 K/V blocks: the shared prefix stays restorable while 8 streams publish their own
  os.environ.update(INFENG_KV_BLOCKS="1024", INFENG_CHECKPOINTS="64", INFENG_SEED=str(SEED), INFENG_DEVICE=str(local),
                    INFENG_DRAFT_WIDTH=str(DRAFT_WIDTH))
  try:
    engine = InferenceEngine(path, draft_weights=path, max_context=4096)
  finally:
    os.environ.pop("INFENG_CHECKPOINTS"), os.environ.pop("INFENG_DRAFT_WIDTH")
  pending = queue.Queue()
  for index in mine:
    pending.put(index)
  produced, drafted, accepted, lock = [0], [0], [0], threading.Lock()

  def worker():
    while True:
      try:
        index = pending.get_nowait()
      except queue.Empty:
        return
      sequence = engine.sequence(temperature=0.7, top_p=0.9, top_k=40, speculative=speculative, seed=SEED + index)
      cursor, count = sequence.append(streams[index]), 0
      while count < generated and sequence.read(cursor) is not None:
        cursor += 1
        count += 1
      sequence.cancel()
      while sequence.read(cursor) is not None:
        cursor += 1
      counters = sequence.speculative_counters()
      sequence.close()
      with lock:
        produced[0] += count
        drafted[0] += counters["drafted_tokens"]
        accepted[0] += counters["accepted_tokens"]

  if dist:
    dist.barrier()
  before, started = engine.step_counters(), time.perf_counter()
  threads = [threading.Thread(target=worker) for _ in range(SEQUENCES)]
  for thread in threads:
    thread.start()
  for thread in threads:
    thread.join()
  wall, after = time.perf_counter() - started, engine.step_counters()
  engine.close()
  return {"tokens": produced[0], "wall": wall, "device_seconds": (after["device_ns"] - before["device_ns"]) / 1e9, "passes": after["passes"] - before["passes"],
          "rows": after["rows"] - before["rows"], "prefill_rows": after["prefill_rows"] - before["prefill_rows"],
          "prompt_tokens": sum(len(streams[i]) for i in mine), "drafted": drafted[0], "accepted": accepted[0], "streams": len(mine)}


def config5_block(local, rank, world, path, dist, generated=GENERATED):
  from mtlqwen_b200 import replicas
  block = {"workload": f"config 5: {STREAMS} streams = shared {PREFIX_TOKENS}-token prefix + suffix U[64,1024], routed over the replicas, 8 live per "
                       f"replica, MTP draft width {DRAFT_WIDTH} (random-init head), temperature 0.7 / top-p 0.9 / top-k 40, seeded Philox, "
                       f"{generated} tokens per stream"}
  for name, speculative in (("speculative", True), ("plain", False)):
    r = run_config5(local, rank, world, path, dist, speculative, generated)
    tokens, wall = replicas.combine(dist, r["tokens"], r["wall"])
    _, device = replicas.combine(dist, 0, r["device_seconds"])
    prefill, _ = replicas.combine(dist, r["prefill_rows"], 0.0)
    prompt, _ = replicas.combine(dist, r["prompt_tokens"], 0.0)
    drafted, _ = replicas.combine(dist, r["drafted"], 0.0)
    accepted, _ = replicas.combine(dist, r["accepted"], 0.0)
    block[name] = {"tok_per_s": tokens / wall, "tokens": int(tokens), "wall_s": wall, "device_s_slowest_replica": device,
                   "prefill_rows": int(prefill), "prompt_tokens_requested": int(prompt),
                   "acceptance_rate": accepted / drafted if drafted else None, "drafted": int(drafted), "accepted": int(accepted),
                   "passes_rank0": int(r["passes"]), "streams_rank0": r["streams"]}
  return block


# ---- single-kernel configurations ---------------------------------------------------------------------------------
def kernel_configs(local, contexts):
  """Configs 1 to 3, lm_head, the prefill GEMM and one attention layer at the decode step's contexts on one GPU:
  microseconds per launch and the algorithmic rate."""
  from mtlqwen_b200 import device as D
  from mtlqwen_b200.testing import cases
  dev = D.Device(local)
  peak, _ = measured_peak()
  try:
    out = {"cfg1_m8": cases.linear_case(dev)}
    out["cfg1_m8_fp32_activations"] = cases.linear_case(dev, supplied_image=False, replays=10)
    out["cfg1_m1"] = cases.linear_case(dev, m=1, replays=10)
    out["cfg1_m1_fp32_activations"] = cases.linear_case(dev, m=1, supplied_image=False, replays=10)
    out["lm_head_q6k_m8"] = cases.linear_case(dev, qtype=D.Q6_K, n=VOCAB, copies=1, replays=10)
    out["cfg2_gdn_decode"] = cases.gdn_case(dev)
    out["cfg2_gdn_prefill"] = cases.gdn_prefill_case(dev)
    out["cfg3_attention"] = cases.attention_case(dev)
    out["attention_layer_at_step_contexts"] = cases.attention_case(dev, contexts=contexts, block_tokens=128, layers=8, replays=20)
    prefill = cases.linear_case(dev, m=128, copies=8, replays=5)
    prefill["TFLOPs"] = 2.0 * 128 * 12288 * 4096 / prefill["us"] / 1e6
    out["prefill_gemm_m128"] = prefill
    for entry in out.values():
      if "GBs" in entry:
        entry["frac_of_measured_hbm"] = entry["GBs"] / peak
    return out
  finally:
    dev.close()


def run_ours(args, rank, world):
  local = int(os.environ.get("LOCAL_RANK", 0))
  dist = None
  if world > 1:
    import torch.distributed as dist
    dist.init_process_group("gloo")  # bookkeeping only: replicas exchange no data
  from mtlqwen_b200 import replicas
  from mtlqwen_b200.testing import synth
  if local == 0:
    synth.ensure_full_model()
  if dist:
    dist.barrier()
  path = synth.full_model_path()
  r = run_config4(args, local, path, dist)
  kernels = kernel_configs(local, r["contexts"]) if rank == 0 else None
  cfg5 = None if args.no_cfg5 else config5_block(local, rank, world, path, dist)
  peak, peak_kind = measured_peak()

  # whole job = all replicas; time = max over ranks
  total_rows, worst_device = replicas.combine(dist, r["rows"], r["device_seconds"])
  total_tokens, worst_wall = replicas.combine(dist, r["tokens"], r["wall"])
  total_launches, _ = replicas.combine(dist, r["launches"], 0.0)
  if dist:
    dist.barrier()
  if rank != 0:
    return
  c0, c1, passes, contexts = r["c0"], r["c1"], r["passes"], r["contexts"]
  headline = kernels["cfg1_m8"]
  kv_bytes = sum(contexts) * 32768  # K+V, 8 attention layers, 4 kv heads x 256 x fp16
  step_bytes = WEIGHT_BYTES_PER_STEP + STATE_BYTES_PER_STEP + kv_bytes
  step_seconds = r["device_seconds"] / max(passes, 1)
  line = {
    "metric": "decode_tokens_per_second", "value": total_rows / worst_device, "unit": "tok/s", "n_gpus": world, "steps": int(passes),
    "warmup": args.warmup, "ms_per_step": 1e3 * step_seconds, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": DTYPE,
    "data": "synthetic", "config": workload_config(), "clocks": r["clocks"], "gpu_launches": int(total_launches),
    "e2e": {"value": total_tokens / worst_wall, "unit": "tok/s", "h2d_bytes_per_step": SEQUENCES * (64 + 4) + 128,
            "d2h_bytes_per_step": SEQUENCES * 4 + 4 + SEQUENCES * 12,
            # rank 0: wall ms per step seen by the readers, and the part of it the scheduler spends inside a pass
            # (record, graph launch, wait for the stream); the rest is batch building and token hand-over
            "wall_ms_per_step": 1e3 * r["wall"] / max(1, passes), "in_pass_ms_per_step": (c1["micros"] - c0["micros"]) / 1e3 / max(1, passes),
            "scheduler_ms_per_step": {key: (c1[key + "_micros"] - c0[key + "_micros"]) / 1e3 / max(1, passes) for key in ("build", "lock", "publish")},
            "note": "through infeng_sequence_append/read with host token buffers; token ids, query records, sampled tokens and acceptance "
                    "verdicts cross PCIe every step"},
    "roofline": {"bound": "hbm", "kernel": "q4k_decode_kernel 12288x4096 M=8 (BASELINE config 1), quantised activations supplied as in a decode pass",
                 "achieved": headline["GBs"], "peak": peak, "unit": "GB/s", "frac": headline["GBs"] / peak, "of": peak_kind,
                 "traffic": GEMV_DRAM_BYTES_PER_LAUNCH, "frac_of_nominal_8TBs": headline["GBs"] / 8000.0, "us_per_launch": headline["us"],
                 "launches_timed": headline["launches_timed"], "algorithmic_bytes": headline["bytes"]},
    "step_hbm": {"bytes_per_step": step_bytes, "achieved_GBs": step_bytes / step_seconds / 1e9, "frac_of_measured": step_bytes / step_seconds / 1e9 / peak,
                 "frac_of_nominal_8TBs": step_bytes / step_seconds / 8e12, "mean_context": sum(contexts) / len(contexts)},
    "configs": kernels,
  }
  if cfg5:
    line["cfg5"] = cfg5
  # Everything before the timed window is prompt processing (128-row passes of prefill chunks, with the decode rows of the
  # sequences that finished their prompt earlier mixed in): reported beside the headline, not part of it.
  if c0["device_ns"]:
    line["prefill"] = {"rows_per_s": c0["rows"] / (c0["device_ns"] / 1e9), "rows": int(c0["rows"]), "passes": int(c0["passes"]),
                       "note": "rank 0, all passes before the timed decode window"}
  if world == 1:
    rate, done, elapsed, cores = cpu_decode(path, reference_contexts(args.warmup), None, 1, seconds_budget=12.0)
    for name, entry in cpu_configs().items():  # the oracle on the single-kernel configurations, beside the GPU figures
      kernels[name]["cpu_oracle"] = entry
    line["cpu_baseline"] = {"value": rate, "unit": "tok/s", "cores": cores, "kind": "port",
                            "sample": f"{done} batched decode steps of the same 8 sequences at the same contexts on the host cores ({elapsed:.1f} s); "
                                      "K/V and recurrent states filled with seeded synthetic values"}
  print(json.dumps(line))


def run_case(args):
  """One small case alone: what the ncu captures of the profile summaries run."""
  from mtlqwen_b200 import device as D
  from mtlqwen_b200.testing import cases, synth
  local = int(os.environ.get("LOCAL_RANK", 0))
  if args.case in ("step", "cfg5"):
    path = synth.ensure_full_model()
    if args.case == "step":  # decode steps of config 4; --context bounds the prompt lengths (short ones: few launches before the timed passes)
      r = run_config4(args, local, path, None, longest=max(args.context, 1))
      print(json.dumps({"case": "step", "ms_per_step": 1e3 * r["device_seconds"] / max(r["passes"], 1), "passes": int(r["passes"]),
                        "launches": int(r["launches"]), "contexts": r["contexts"]}))
    else:
      print(json.dumps({"case": "cfg5", **config5_block(local, 0, 1, path, None, generated=args.steps)}))
    return
  dev = D.Device(local)
  try:
    small = dict(copies=8, replays=2)
    table = {
      "cfg1": lambda: cases.linear_case(dev, **small), "cfg1_m1": lambda: cases.linear_case(dev, m=1, **small),
      "lm_head": lambda: cases.linear_case(dev, qtype=D.Q6_K, n=65536, copies=2, replays=2),
      "prefill": lambda: cases.linear_case(dev, m=128, **small), "cfg2": lambda: cases.gdn_case(dev, replays=2),
      "cfg2_prefill": lambda: cases.gdn_prefill_case(dev, replays=1), "cfg3": lambda: cases.attention_case(dev, replays=2),
      # one attention layer at contexts like those of the config-4 decode step
      "attention_step": lambda: cases.attention_case(dev, contexts=[2728, 4044, 899, 546, 1176, 3424, 3129, 2627], block_tokens=128, layers=8, replays=2),
    }
    print(json.dumps({"case": args.case, **table[args.case]()}))
  finally:
    dev.close()


def main():
  parser = argparse.ArgumentParser()
  parser.add_argument("--gpus", type=int, default=1)
  parser.add_argument("--steps", type=int, default=128)
  parser.add_argument("--warmup", type=int, default=16)
  parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
  parser.add_argument("--case", default=None, choices=("cfg1", "cfg1_m1", "lm_head", "prefill", "cfg2", "cfg2_prefill", "cfg3", "attention_step", "step", "cfg5"),
                      help="run one small case alone and print its line (the commands of the profile summaries)")
  parser.add_argument("--context", type=int, default=160, help="--case step only: upper bound of the ragged prompt lengths (4096 = the headline workload; 1 = no prefill passes, for launch lists)")
  parser.add_argument("--no-cfg5", action="store_true", help="leave the config-5 block out of the line")
  args = parser.parse_args()
  args.warmup = max(args.warmup, 3)
  if args.case:
    return run_case(args)
  rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
  if args.impl == "reference":
    run_reference(args, rank, world)
  else:
    run_ours(args, rank, world)


if __name__ == "__main__":
  main()
