"""Benchmark of the ragged continuous-batching forward step.

Metric (BASELINE.json): aggregate decode tokens/s at 8 live sequences per GPU, plus the Q4_K GEMV fraction of
HBM peak. Workload: the full Qwen3.5-9B-shaped decoder (32 layers = 8 x (3 GDN + 1 gated attention), hidden
4096, SwiGLU 12288, vocabulary 248320; all projections Q4_K, embedding / lm_head Q6_K) with random-init
weights in a GGUF file written on the fly, 8 sequences with seeded token-id prompts of ragged length uniform
in [128, 4096], greedy sampling, prefill chunks mixed with decodes in one packed pass. A "step" is one pass in
which every one of the 8 live sequences decodes one token.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N > 1 runs N independent engine replicas (one process per GPU under torchrun, no data-path collective);
`value` is the whole-job rate. `--impl reference` times the CPU oracle (the scalar restatement of the
reference's Metal kernels; Metal itself cannot run on Linux) on the host cores for the same model.
"""
import argparse
import json
import os
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


def model_path():
  override = os.environ.get("MTLQWEN_BENCH_GGUF")
  return Path(override) if override else Path(f"/tmp/mtlqwen_b200_bench_{LAYERS}x{VOCAB}_seed{SEED}.gguf")


def ensure_model(path, layers=LAYERS, vocab=VOCAB):
  from mtlqwen_b200.testing import synth
  if not path.exists():
    temporary = path.with_suffix(f".{os.getpid()}.tmp")
    synth.write_gguf(temporary, layers=layers, vocab=vocab, mtp=False, seed=SEED)
    os.replace(temporary, path)
  return path


def prompts(vocab=VOCAB, longest=4096):
  rng = np.random.default_rng(SEED + 4)
  lengths = rng.integers(128, longest + 1, SEQUENCES)
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


# dram__bytes_read.sum + dram__bytes_write.sum of one q4k_decode_kernel launch at the config-1 shape, from the ncu capture
# summarised in profiles/q4k_decode_12288x4096_m8.md (the same shape and launch as the roofline leg below).
GEMV_DRAM_BYTES_PER_LAUNCH = 28_399_488


def gemv_roofline(device_index, copies=24, replays=20, xsplit=None, qtype=None, n=12288, k=4096, m=8):
  """The dominant kernel alone: Q4_K GEMV 12288 x 4096 with 8 activation rows (BASELINE config 1), launched over a
  ring of 24 distinct weight copies (680 MB, larger than L2) and timed with CUDA events on the launching stream."""
  from mtlqwen_b200 import device as D
  from mtlqwen_b200.testing import synth
  dev = D.Device(device_index)
  qtype = qtype or D.Q4_K
  if xsplit:  # asks for the fp16-MMA kernel with this activation split
    dev.set_xsplit(xsplit)
    dev.set_integer_decode(False)
  base = synth.weight(qtype, n, k, 1235)
  ring = [dev.array(base) for _ in range(copies)]
  x, y = dev.array(synth.activations(m, k, 1236)), dev.empty((m, n))
  # Q4_K: the integer kernel reads the quantised image of the activations, which a decode pass gets from the kernel
  # before the GEMV; it is prepared once here so that the timed launches are the GEMV kernel alone.
  image = None
  if qtype == D.Q4_K and not xsplit and m <= 8:
    image = dev.empty(dev.image_bytes(m, k), np.uint8)
    dev.quantize(x, m, k, image)

  def launch(w):
    if image is not None:
      dev.image_supply(image)
    dev.linear(qtype, w, n, k, x, m, y)

  for w in ring:  # warm-up, also builds the kernel's attributes before capture
    launch(w)
  dev.commit()
  dev.check(dev.lib.infdev_graph_begin(dev.ctx))
  for w in ring:
    launch(w)
  graph = dev.lib.infdev_graph_end(dev.ctx)
  for _ in range(10):
    dev.check(dev.lib.infdev_graph_launch(dev.ctx, graph))
  dev.commit()
  start, stop = dev.event(), dev.event()
  dev.record(start)
  for _ in range(replays):
    dev.check(dev.lib.infdev_graph_launch(dev.ctx, graph))
  dev.record(stop)
  dev.commit()
  seconds = dev.elapsed_ms(start, stop) / 1e3 / (copies * replays)
  algorithmic = base.nbytes + (dev.image_bytes(m, k) if image is not None else m * k * 4) + m * n * 4
  dev.lib.infdev_graph_destroy(dev.ctx, graph)
  dev.close()
  return algorithmic, seconds, copies * replays


def measured_peak():
  path = ROOT / "MEASURED_PEAKS.json"
  if path.exists():
    return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
  return 6650.0, "fallback"


def cpu_decode(path, seconds_budget, steps=None, warmup=0):
  """Times the CPU oracle decoding one sequence of the same model, one token per step, with every host core
  (OpenMP over output rows). Returns tokens/s, steps timed, seconds."""
  import oracle
  from mtlqwen_b200.testing import synth
  model = oracle.Model(synth.read_gguf(path), LAYERS, VOCAB, 4096)
  token = 17
  for _ in range(warmup):
    token = int(np.argmax(model.step(token)[1]))
  started, done = time.perf_counter(), 0
  while (steps is not None and done < steps) or (steps is None and (done < 4 or time.perf_counter() - started < seconds_budget)):
    token = int(np.argmax(model.step(token)[1]))
    done += 1
  elapsed = time.perf_counter() - started
  return done / elapsed, done, elapsed


def run_reference(args, rank, world):
  if rank != 0:
    return
  path = ensure_model(model_path())
  rate, done, elapsed = cpu_decode(path, 0, steps=args.steps, warmup=args.warmup)
  cores = os.cpu_count()
  sample = f"{done} single-sequence decode steps of the 32-layer model (1 of the 8 live sequences per step), context < {done + args.warmup + 1}"
  print(json.dumps({
    "impl": "reference", "metric": "decode_tokens_per_second", "value": rate, "unit": "tok/s", "n_gpus": args.gpus, "steps": done,
    "warmup": args.warmup, "ms_per_step": 1e3 * elapsed / done, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
    "data": "synthetic", "config": workload_config(), "cpu_baseline": {"value": rate, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
    "e2e": {"value": rate, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0,
    "note": "CPU oracle port of the reference's Metal kernels (Metal is unavailable on this box); all host cores via OpenMP"
  }))


def workload_config():
  return {"workload": "config 4: Qwen3.5-9B-shaped 32-layer decoder, Q4_K projections + Q6_K embedding/lm_head, random init, "
                      "8 live sequences, ragged prompts U[128,4096], greedy decode", "live_sequences_per_gpu": SEQUENCES,
          "parallelism": "replicas", "l2_policy": "inputs larger than L2: 4.75 GB of weights streamed per step"}


def run_ours(args, rank, world):
  local = int(os.environ.get("LOCAL_RANK", 0))
  dist = None
  if world > 1:
    import torch.distributed as dist
    dist.init_process_group("gloo")  # bookkeeping only: replicas exchange no data
  path = model_path()
  if local == 0:
    ensure_model(path)
  if dist:
    dist.barrier()
  from mtlqwen_b200.inference import InferenceEngine
  os.environ.setdefault("INFENG_KV_BLOCKS", "384")
  os.environ.setdefault("INFENG_SEED", str(SEED))
  os.environ["INFENG_DEVICE"] = str(local)
  engine = InferenceEngine(path, max_context=8192)
  texts = prompts(longest=args.prompt_max)
  sequences = [engine.sequence() for _ in range(SEQUENCES)]
  warmup, steps = args.warmup, args.steps
  need = warmup + steps + 1
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
  if args.ncu_range:  # lets `ncu --profile-from-start off` see only the timed decode passes
    from mtlqwen_b200 import device as D
    profiler = D.library().infdev_profiler_range
    profiler(None, 1)
  while len(stamps[last]) < first_index + steps + 1:
    time.sleep(0.002)
  if args.ncu_range:
    profiler(None, 0)
  finished.set()
  for thread in threads:
    thread.join()
  t0, t1 = stamps[last][first_index], stamps[last][first_index + steps]
  c0, c1 = counters[last][first_index], counters[last][first_index + steps]
  tokens = sum(sum(1 for t in s if t0 < t <= t1 + 1e-4) for s in stamps)
  clocks = sampler.stop(t0, t1, sampler_started)
  wall = t1 - t0
  device_seconds = (c1["device_ns"] - c0["device_ns"]) / 1e9
  passes, rows, launches = c1["passes"] - c0["passes"], c1["rows"] - c0["rows"], c1["launches"] - c0["launches"]
  contexts = [sequence.length for sequence in sequences]
  for sequence in sequences:
    sequence.close()
  engine.close()

  algorithmic, kernel_seconds, kernel_launches = gemv_roofline(local)
  peak, peak_kind = measured_peak()

  # whole job = all replicas; time = max over ranks
  from mtlqwen_b200 import replicas
  total_rows, worst_device = replicas.combine(dist, rows, device_seconds)
  total_tokens, worst_wall = replicas.combine(dist, tokens, wall)
  total_launches, _ = replicas.combine(dist, launches, 0.0)
  totals, worst = [total_rows, total_tokens, total_launches], [worst_device, worst_wall]
  if dist:
    dist.barrier()
  if rank != 0:
    return
  kv_bytes = sum(contexts) * 32768  # K+V, 8 attention layers, 4 kv heads x 256 x fp16
  step_bytes = WEIGHT_BYTES_PER_STEP + STATE_BYTES_PER_STEP + kv_bytes
  step_seconds = device_seconds / max(passes, 1)
  line = {
    "metric": "decode_tokens_per_second", "value": totals[0] / worst[0], "unit": "tok/s", "n_gpus": world, "steps": int(passes), "warmup": warmup,
    "ms_per_step": 1e3 * step_seconds, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
    "config": workload_config(), "clocks": clocks, "gpu_launches": int(totals[2]),
    "e2e": {"value": totals[1] / worst[1], "unit": "tok/s", "h2d_bytes_per_step": SEQUENCES * (64 + 4) + 128,
            "d2h_bytes_per_step": SEQUENCES * 4 + 4,
            # rank 0: wall ms per step seen by the readers, and the part of it the scheduler spends inside a pass
            # (record, graph launch, wait for the stream); the rest is batch building and token hand-over
            "wall_ms_per_step": 1e3 * wall / max(1, passes), "in_pass_ms_per_step": (c1["micros"] - c0["micros"]) / 1e3 / max(1, passes),
            "scheduler_ms_per_step": {key: (c1[key + "_micros"] - c0[key + "_micros"]) / 1e3 / max(1, passes) for key in ("build", "lock", "publish")},
            "note": "through infeng_sequence_append/read with host token buffers; token ids, query records and sampled tokens cross PCIe every step"},
    "roofline": {"bound": "hbm", "kernel": "q4k_decode_kernel 12288x4096 M=8 (BASELINE config 1)", "achieved": algorithmic / kernel_seconds / 1e9,
                 "peak": peak, "unit": "GB/s", "frac": algorithmic / kernel_seconds / 1e9 / peak, "of": peak_kind, "traffic": GEMV_DRAM_BYTES_PER_LAUNCH,
                 "frac_of_nominal_8TBs": algorithmic / kernel_seconds / 8e12, "us_per_launch": kernel_seconds * 1e6, "launches_timed": kernel_launches},
    "step_hbm": {"bytes_per_step": step_bytes, "achieved_GBs": step_bytes / step_seconds / 1e9, "frac_of_measured": step_bytes / step_seconds / 1e9 / peak,
                 "frac_of_nominal_8TBs": step_bytes / step_seconds / 8e12, "mean_context": sum(contexts) / len(contexts)},
  }
  # Everything before the timed window is prompt processing (128-row passes of prefill chunks, with the decode rows of the
  # sequences that finished their prompt earlier mixed in): reported beside the headline, not part of it.
  if c0["device_ns"]:
    line["prefill"] = {"rows_per_s": c0["rows"] / (c0["device_ns"] / 1e9), "rows": int(c0["rows"]), "passes": int(c0["passes"]),
                       "note": "rank 0, all passes before the timed decode window"}
  if world == 1:
    rate, done, elapsed = cpu_decode(path, 12.0)
    line["cpu_baseline"] = {"value": rate, "unit": "tok/s", "cores": os.cpu_count(), "kind": "port",
                            "sample": f"{done} single-sequence decode steps of the same 32-layer model on the host cores ({elapsed:.1f} s)"}
  print(json.dumps(line))


def main():
  parser = argparse.ArgumentParser()
  parser.add_argument("--gpus", type=int, default=1)
  parser.add_argument("--steps", type=int, default=128)
  parser.add_argument("--warmup", type=int, default=16)
  parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
  parser.add_argument("--kernel-only", default=None, choices=("q4k", "q6k", "prefill"),
                      help="run only the isolated GEMV kernel on a small ring (the case profiled with ncu) and print its rate")
  parser.add_argument("--xsplit", type=int, default=None, choices=(1, 2))
  parser.add_argument("--prompt-max", type=int, default=4096, help="upper bound of the ragged prompt lengths (profiling runs use a small one)")
  parser.add_argument("--ncu-range", action="store_true", help="bracket the timed passes with cudaProfilerStart/Stop")
  args = parser.parse_args()
  if args.kernel_only:
    q6, prefill = args.kernel_only == "q6k", args.kernel_only == "prefill"
    n, m = 65536 if q6 else 12288, 128 if prefill else 8  # 128 rows take the tcgen05 prefill GEMM (two launches: prepare + GEMM)
    algorithmic, seconds, launches = gemv_roofline(int(os.environ.get("LOCAL_RANK", 0)), copies=2 if q6 else 8, replays=2, xsplit=args.xsplit,
                                                   qtype=14 if q6 else 12, n=n, m=m)
    line = {"kernel": args.kernel_only, "n": n, "k": 4096, "m": m, "us_per_launch": seconds * 1e6, "GBs": algorithmic / seconds / 1e9, "launches": launches}
    if prefill:
      line["TFLOPs"] = 2.0 * m * n * 4096 / seconds / 1e12
    print(json.dumps(line))
    return
  args.warmup = max(args.warmup, 3)
  rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
  if args.impl == "reference":
    run_reference(args, rank, world)
  else:
    run_ours(args, rank, world)


if __name__ == "__main__":
  main()
