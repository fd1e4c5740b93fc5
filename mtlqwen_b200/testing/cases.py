"""Timed single-kernel cases of the benchmark configurations (BASELINE configs 1 to 3, the lm_head GEMV and the
prefill GEMM), on synthetic inputs of the configured shapes. Every case keeps its inputs resident in device memory,
defeats the L2 (operands larger than it, or a ring of operand copies larger than it), times with CUDA events on the
launching stream after warm-up, and returns microseconds per launch with the algorithmic bytes it moves.
Used by bench.py; the parity of the same kernels is the business of tests/."""
import numpy as np

from .. import device as D
from . import synth

L2_BYTES = 126 << 20


def timed(dev, launch, items, replays, warm=2, graph=True):
  """Microseconds per item. `launch(item)` queues one case on item; the sequence over all items is captured into a
  CUDA graph when `graph` (short kernels: no launch gaps), replayed `replays` times between two events."""
  for item in items:  # also sets kernel attributes before any capture
    launch(item)
  dev.commit()
  handle = None
  if graph:
    dev.check(dev.lib.infdev_graph_begin(dev.ctx))
    for item in items:
      launch(item)
    handle = dev.lib.infdev_graph_end(dev.ctx)
    assert handle, dev.error()

  def once():
    if handle:
      dev.check(dev.lib.infdev_graph_launch(dev.ctx, handle))
    else:
      for item in items:
        launch(item)

  for _ in range(warm):
    once()
  dev.commit()
  start, stop = dev.event(), dev.event()
  dev.record(start)
  for _ in range(replays):
    once()
  dev.record(stop)
  dev.commit()
  micros = dev.elapsed_ms(start, stop) * 1e3 / (len(items) * replays)
  if handle:
    dev.lib.infdev_graph_destroy(dev.ctx, handle)
  return micros


def linear_case(dev, qtype=D.Q4_K, n=12288, k=4096, m=8, copies=24, replays=20, supplied_image=True):
  """y = x W^T over a ring of `copies` distinct weight matrices. supplied_image: the integer Q4_K kernel gets the
  quantised activations ready-made, as in a decode pass where the producing kernel writes them; otherwise every call
  quantises its fp32 activations first (one more small launch, counted in the time)."""
  base = synth.weight(qtype, n, k, 1235)
  ring = [dev.array(base) for _ in range(copies)]
  x, y = dev.array(synth.activations(m, k, 1236)), dev.empty((m, n))
  image = None
  if supplied_image and qtype == D.Q4_K and m <= 8:
    image = dev.empty(dev.image_bytes(m, k), np.uint8)
    dev.quantize(x, m, k, image)

  def launch(w):
    if image is not None:
      dev.image_supply(image)
    dev.linear(qtype, w, n, k, x, m, y)

  micros = timed(dev, launch, ring, replays)
  activations = dev.image_bytes(m, k) if image is not None else m * k * 4
  algorithmic = base.nbytes + activations + m * n * 4
  for w in ring:
    w.free()
  return {"us": micros, "bytes": int(algorithmic), "GBs": algorithmic / micros / 1e3, "n": n, "k": k, "m": m,
          "activations": "quantised image supplied" if image is not None else "fp32", "launches_timed": copies * replays}


def gdn_case(dev, sequences=8, layers=8, replays=20, seed=7):
  """BASELINE config 2, decode: one gated-delta-rule layer step for `sequences` sequences (causal conv + SiLU, beta / g,
  the recurrence on the fp32 128 x 128 state of 32 heads, gated norm) in one launch, cycling over `layers` sets of
  state records so that the 2 x 2.16 MB per sequence come from HBM every time, as across the 24 GDN layers of the model."""
  rng = np.random.default_rng(seed)
  record = D.GDN_LAYER_STATE_BYTES
  weights = dict(w_beta=(rng.standard_normal((32, 4096)) / 64), w_alpha=(rng.standard_normal((32, 4096)) / 64), ssm_a=-rng.uniform(1, 16, 32),
                 ssm_dt=0.1 * rng.standard_normal(32), conv=0.5 * rng.standard_normal((8192, 4)), norm=1 + 0.01 * rng.standard_normal(128))
  w = {name: dev.array(value.astype(np.float32)) for name, value in weights.items()}
  x, mixed = dev.array(synth.activations(sequences, 4096, seed + 1)), dev.array(synth.activations(sequences, 8192, seed + 2))
  z, out = dev.array(synth.activations(sequences, 4096, seed + 3)), dev.empty((sequences, 32, 128))
  items = []
  for _ in range(layers):
    states = np.concatenate([rng.standard_normal((sequences, 8192 * 4)), 0.01 * rng.standard_normal((sequences, 32 * 128 * 128))], axis=1)
    previous, following = dev.array(states.astype(np.float32)), dev.empty((sequences, record // 4))
    queries = []
    for i in range(sequences):
      q = D.Query()
      q.previous, q.next = previous.ptr + i * record, following.ptr + i * record
      q.start, q.count, q.position, q.slot, q.state = i, 1, 77, i, D.UNBOUND
      queries.append(q)
    items.append((dev.queries(queries), previous, following))

  def launch(item):
    dev.gdn_decode(x, mixed, w["w_beta"], w["w_alpha"], w["ssm_a"], w["ssm_dt"], w["conv"], z, w["norm"], item[0], sequences, 0, D.CONV_STATE_BYTES,
                   record, out)

  micros = timed(dev, launch, items, replays)
  algorithmic = sequences * (2 * record + (4096 + 8192 + 4096 + 4096) * 4)
  return {"us": micros, "bytes": int(algorithmic), "GBs": algorithmic / micros / 1e3, "sequences": sequences, "launches_timed": layers * replays}


def gdn_prefill_case(dev, sequences=8, seed=9, replays=3):
  """BASELINE config 2, prefill: ragged chunks with lengths uniform in [1, 512], one launch of the preparation kernel
  and the chunked delta rule over all of them (a sequential dependency chain per head, so rows per second is the
  figure of merit)."""
  rng = np.random.default_rng(seed)
  lengths = [int(v) for v in rng.integers(1, 513, sequences)]
  rows, record = sum(lengths), D.GDN_LAYER_STATE_BYTES
  weights = dict(w_beta=(rng.standard_normal((32, 4096)) / 64), w_alpha=(rng.standard_normal((32, 4096)) / 64), ssm_a=-rng.uniform(1, 16, 32),
                 ssm_dt=0.1 * rng.standard_normal(32), conv=0.5 * rng.standard_normal((8192, 4)), norm=1 + 0.01 * rng.standard_normal(128))
  w = {name: dev.array(value.astype(np.float32)) for name, value in weights.items()}
  x, mixed, z = (dev.array(synth.activations(rows, width, seed + i)) for i, width in enumerate((4096, 8192, 4096)))
  states = np.concatenate([rng.standard_normal((sequences, 8192 * 4)), 0.01 * rng.standard_normal((sequences, 32 * 128 * 128))], axis=1)
  previous, following = dev.array(states.astype(np.float32)), dev.empty((sequences, record // 4))
  queries, start = [], 0
  for i, count in enumerate(lengths):
    q = D.Query()
    q.previous, q.next = previous.ptr + i * record, following.ptr + i * record
    q.start, q.count, q.position, q.slot, q.state = start, count, 77, i, D.UNBOUND
    queries.append(q)
    start += count
  dq = dev.queries(queries)
  q_out, k_out, v_out = dev.empty((rows, 16, 128)), dev.empty((rows, 16, 128)), dev.empty((rows, 32, 128))
  beta, g, out = dev.empty((rows, 32)), dev.empty((rows, 32)), dev.empty((rows, 32, 128))

  def launch(_):
    dev.gdn_prepare(x, mixed, w["w_beta"], w["w_alpha"], w["ssm_a"], w["ssm_dt"], w["conv"], dq, sequences, rows, 0, record, q_out, k_out, v_out, beta, g)
    dev.delta_rule(q_out, k_out, v_out, g, beta, z, w["norm"], dq, sequences, D.CONV_STATE_BYTES, record, out, prefill=True)

  micros = timed(dev, launch, [None], replays, warm=1, graph=False)
  return {"us": micros, "rows": rows, "rows_per_s": rows / micros * 1e6, "longest_chunk": max(lengths), "lengths": lengths}


def attention_case(dev, sequences=8, longest=32768, block_tokens=16, replays=10, seed=7, contexts=None, layers=1):
  """BASELINE config 3: decode attention of `sequences` rows over paged fp16 K/V with contexts uniform in [1, longest],
  16-token blocks bound through a random permutation of the pool; scan + reduce, 4096 bytes of K and V per attended
  token. The pool (about half a gigabyte) is larger than the L2. With `contexts` given (the decode step's: a few
  thousand tokens, where one layer's K/V would fit the L2) the launches cycle over `layers` pools, as the attention
  layers of the model do."""
  rng = np.random.default_rng(seed)
  contexts = [int(c) for c in contexts] if contexts is not None else [int(c) for c in rng.integers(1, longest + 1, sequences)]
  sequences = len(contexts)
  blocks = [-(-c // block_tokens) for c in contexts]
  stride, physical = max(blocks), int(sum(blocks))
  permutation = rng.permutation(physical).astype(np.int32)
  table, at = np.zeros((sequences, stride), np.int32), 0
  for i, count in enumerate(blocks):
    table[i, :count] = permutation[at:at + count]
    at += count
  pool = (physical, 4, block_tokens, 256)
  pools = []
  for _ in range(layers):
    pools.append((dev.array(rng.standard_normal(pool, dtype=np.float32).astype(np.float16).view(np.uint16)),
                  dev.array(rng.standard_normal(pool, dtype=np.float32).astype(np.float16).view(np.uint16))))
  queries = []
  for i, context in enumerate(contexts):
    q = D.Query()
    q.start, q.count, q.position, q.slot, q.state = i, 1, context - 1, i, D.UNBOUND
    queries.append(q)
  dq, dtable = dev.queries(queries), dev.array(table)
  qg = dev.array(rng.standard_normal((sequences, 16, 512)).astype(np.float32))
  q, out = dev.array(rng.standard_normal((sequences, 16, 256)).astype(np.float32)), dev.empty((sequences, 16, 256))
  partials = dev.empty(dev.attention_scratch_bytes(sequences, 32) // 4)

  def launch(item):
    dev.attention(q, qg, item[0], item[1], dq, sequences, sequences, dtable, stride, block_tokens, 32, partials, out)

  micros = timed(dev, launch, pools, replays, graph=layers > 1)
  algorithmic = sum(contexts) * 4096
  return {"us": micros, "bytes": int(algorithmic), "GBs": algorithmic / micros / 1e3, "contexts": contexts, "launches_timed": replays * layers}
