"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations:
raw-field GGUF Q4_K / Q6_K weight blocks, activations, and a random-init GGUF writer.

K-quant `quantize` is not needed: blocks are drawn field by field (quants uniform, 6-bit scales and mins
uniform, fp16 super-block scales chosen so the dequantised weights are about N(0, 0.02)).
"""
import numpy as np

Q4_K, Q6_K, F32 = 12, 14, 0


def q4k_blocks(count, rng, target_std=0.02, subnormal=False):
  """`count` Q4_K super-blocks (144 B): fp16 d, fp16 dmin, 12 B of 6-bit scales/mins, 128 B of nibbles.
  With q ~ U{0..15}, sc, m ~ U{0..63}: E[sc q] = 236.25, E[m] = 31.5 so dmin = 7.5 d centres the weights,
  and std(w) = 258.3 d."""
  blocks = np.frombuffer(rng.bytes(count * 144), dtype=np.uint8).reshape(count, 144).copy()
  d = (target_std / 258.3) * rng.uniform(0.8, 1.2, count)
  if subnormal:
    d = d * 0.05
  d16 = d.astype(np.float16)
  m16 = (d16.astype(np.float32) * 7.5).astype(np.float16)
  blocks[:, 0:2] = d16.view(np.uint8).reshape(count, 2)
  blocks[:, 2:4] = m16.view(np.uint8).reshape(count, 2)
  return blocks


def q6k_blocks(count, rng, target_std=0.02):
  """`count` Q6_K super-blocks (210 B): ql[128], qh[64], int8 scales[16], fp16 d. q-32 ~ U{-32..31},
  sc ~ U{-128..127}: std(w) = 18.47 * 73.9 * d."""
  blocks = np.frombuffer(rng.bytes(count * 210), dtype=np.uint8).reshape(count, 210).copy()
  d16 = ((target_std / (18.47 * 73.9)) * rng.uniform(0.8, 1.2, count)).astype(np.float16)
  blocks[:, 208:210] = d16.view(np.uint8).reshape(count, 2)
  return blocks


def weight(qtype, n, k, seed):
  rng = np.random.default_rng(seed)
  count = n * (k // 256)
  return q4k_blocks(count, rng) if qtype == Q4_K else q6k_blocks(count, rng)


def activations(m, k, seed):
  return np.random.default_rng(seed).standard_normal((m, k)).astype(np.float32)


# ---- random-init GGUF files with the reference's tensor names and shapes (model/qwen35/forward.cpp:74-127) ----
GGUF_MAGIC, GGUF_ALIGNMENT = 0x46554747, 32
HIDDEN, INTERMEDIATE = 4096, 12288


def model_tensors(layers=32, vocab=248320, mtp=False, seed=1234):
  """Yields (name, ggml type, shape as (n, k) or (dim,), generator of the raw bytes). Projections Q4_K, embedding
  and lm_head Q6_K, norms F32 at 1 +- 0.01, GDN parameters as in the gated-delta-rule benchmark configuration."""
  counter = [seed]

  def rng():
    counter[0] += 1
    return np.random.default_rng(counter[0])

  def q4(n, k):
    return (Q4_K, (n, k), lambda: q4k_blocks(n * k // 256, rng()))

  def q6(n, k):
    return (Q6_K, (n, k), lambda: q6k_blocks(n * k // 256, rng()))

  def norm(dim):
    return (F32, (dim, ), lambda: (1 + 0.01 * rng().standard_normal(dim)).astype(np.float32))

  def f32(shape, make):
    return (F32, shape, lambda: make(rng()).astype(np.float32))

  yield ("token_embd.weight", *q6(vocab, HIDDEN))
  yield ("output_norm.weight", *norm(HIDDEN))
  yield ("output.weight", *q6(vocab, HIDDEN))

  def ffn(prefix):
    yield (prefix + "post_attention_norm.weight", *norm(HIDDEN))
    yield (prefix + "ffn_gate.weight", *q4(INTERMEDIATE, HIDDEN))
    yield (prefix + "ffn_up.weight", *q4(INTERMEDIATE, HIDDEN))
    yield (prefix + "ffn_down.weight", *q4(HIDDEN, INTERMEDIATE))

  def attention(prefix):
    yield (prefix + "attn_norm.weight", *norm(HIDDEN))
    yield (prefix + "attn_q.weight", *q4(8192, HIDDEN))
    yield (prefix + "attn_k.weight", *q4(1024, HIDDEN))
    yield (prefix + "attn_v.weight", *q4(1024, HIDDEN))
    yield (prefix + "attn_q_norm.weight", *norm(256))
    yield (prefix + "attn_k_norm.weight", *norm(256))
    yield (prefix + "attn_output.weight", *q4(HIDDEN, HIDDEN))
    yield from ffn(prefix)

  for layer in range(layers):
    prefix = f"blk.{layer}."
    if (layer + 1) % 4 == 0:
      yield from attention(prefix)
      continue
    yield (prefix + "attn_norm.weight", *norm(HIDDEN))
    yield (prefix + "attn_qkv.weight", *q4(8192, HIDDEN))
    yield (prefix + "attn_gate.weight", *q4(HIDDEN, HIDDEN))
    yield (prefix + "ssm_beta.weight", *f32((32, HIDDEN), lambda r: r.standard_normal((32, HIDDEN)) / 64))
    yield (prefix + "ssm_alpha.weight", *f32((32, HIDDEN), lambda r: r.standard_normal((32, HIDDEN)) / 64))
    yield (prefix + "ssm_a", *f32((32, ), lambda r: -r.uniform(1, 16, 32)))
    yield (prefix + "ssm_dt.bias", *f32((32, ), lambda r: 0.1 * r.standard_normal(32)))
    yield (prefix + "ssm_conv1d.weight", *f32((8192, 4), lambda r: 0.5 * r.standard_normal((8192, 4))))
    yield (prefix + "ssm_norm.weight", *norm(128))
    yield (prefix + "ssm_out.weight", *q4(HIDDEN, HIDDEN))
    yield from ffn(prefix)
  if mtp:
    prefix = f"blk.{layers}."
    yield (prefix + "nextn.enorm.weight", *norm(HIDDEN))
    yield (prefix + "nextn.hnorm.weight", *norm(HIDDEN))
    yield (prefix + "nextn.eh_proj.weight", *q4(HIDDEN, 2 * HIDDEN))
    yield (prefix + "nextn.shared_head_norm.weight", *norm(HIDDEN))
    yield from attention(prefix)


def _gguf_string(text):
  raw = text.encode()
  return np.uint64(len(raw)).tobytes() + raw


def write_gguf(path, layers=32, vocab=248320, mtp=False, seed=1234):
  """Writes a GGUF v3 file. ne[0] is the contiguous dimension: a weight [n, k] is stored with shape (k, n),
  which the engine reads back as n = shape[1], k = shape[0] (forward.cpp:18-22)."""
  tensors = list(model_tensors(layers, vocab, mtp, seed))
  sizes = []
  for _, qtype, shape, _ in tensors:
    elements = int(np.prod(shape))
    sizes.append(elements * 4 if qtype == F32 else elements // 256 * (144 if qtype == Q4_K else 210))
  header = bytearray()
  header += np.uint32(GGUF_MAGIC).tobytes() + np.uint32(3).tobytes() + np.uint64(len(tensors)).tobytes() + np.uint64(3).tobytes()
  header += _gguf_string("general.architecture") + np.uint32(8).tobytes() + _gguf_string("qwen35")
  header += _gguf_string("general.alignment") + np.uint32(4).tobytes() + np.uint32(GGUF_ALIGNMENT).tobytes()
  header += _gguf_string("qwen35.block_count") + np.uint32(4).tobytes() + np.uint32(layers).tobytes()
  offset, offsets = 0, []
  for (name, qtype, shape, _), size in zip(tensors, sizes):
    dims = tuple(reversed(shape))
    header += _gguf_string(name) + np.uint32(len(dims)).tobytes() + b"".join(np.uint64(d).tobytes() for d in dims)
    header += np.uint32(qtype).tobytes() + np.uint64(offset).tobytes()
    offsets.append(offset)
    offset += -(-size // GGUF_ALIGNMENT) * GGUF_ALIGNMENT
  data_offset = -(-len(header) // GGUF_ALIGNMENT) * GGUF_ALIGNMENT
  with open(path, "wb") as out:
    out.write(header)
    out.write(b"\0" * (data_offset - len(header)))
    for (_, _, _, make), size, at in zip(tensors, sizes, offsets):
      out.seek(data_offset + at)
      raw = np.ascontiguousarray(make()).tobytes()
      assert len(raw) == size
      out.write(raw)
    out.truncate(data_offset + offset)
  return path


def read_gguf(path):
  """Independent reader for tests: name -> (numpy view of the raw tensor bytes or float32 values, ggml type)."""
  raw = np.memmap(path, dtype=np.uint8, mode="r")
  at = [0]

  def take(dtype, count=1):
    width = np.dtype(dtype).itemsize * count
    value = np.frombuffer(raw[at[0]:at[0] + width].tobytes(), dtype=dtype)
    at[0] += width
    return value if count > 1 else value[0]

  def text():
    length = int(take(np.uint64))
    value = raw[at[0]:at[0] + length].tobytes().decode()
    at[0] += length
    return value

  assert take(np.uint32) == GGUF_MAGIC and take(np.uint32) == 3
  tensor_count, pair_count = int(take(np.uint64)), int(take(np.uint64))
  alignment = GGUF_ALIGNMENT
  for _ in range(pair_count):
    key, kind = text(), int(take(np.uint32))
    if kind == 8:
      text()
    elif kind == 4:
      value = int(take(np.uint32))
      alignment = value if key == "general.alignment" else alignment
    else:
      raise ValueError("read_gguf handles only the metadata types write_gguf emits")
  infos = []
  for _ in range(tensor_count):
    name, rank = text(), int(take(np.uint32))
    dims = [int(take(np.uint64)) for _ in range(rank)]
    infos.append((name, dims, int(take(np.uint32)), int(take(np.uint64))))
  data_offset = -(-at[0] // alignment) * alignment
  tensors = {}
  for name, dims, qtype, offset in infos:
    elements = int(np.prod(dims))
    size = elements * 4 if qtype == F32 else elements // 256 * (144 if qtype == Q4_K else 210)
    view = raw[data_offset + offset:data_offset + offset + size]
    tensors[name] = (np.frombuffer(view, dtype=np.float32) if qtype == F32 else np.frombuffer(view, dtype=np.uint8), qtype)
  return tensors


# ---- the full-size model of the benchmark configurations, written once per machine ----
FULL_LAYERS, FULL_VOCAB, FULL_SEED = 32, 248320, 1234


def full_model_path():
  """Where the random-init Qwen3.5-9B-shaped GGUF (with the MTP block) lives; MTLQWEN_BENCH_GGUF overrides."""
  import os
  from pathlib import Path
  override = os.environ.get("MTLQWEN_BENCH_GGUF")
  return Path(override) if override else Path(f"/tmp/mtlqwen_b200_{FULL_LAYERS}x{FULL_VOCAB}_seed{FULL_SEED}_mtp.gguf")


def ensure_full_model():
  """Writes the file if it is not there yet (about 5.7 GB, some twenty seconds) and returns its path. Passed as
  `weights` alone it loads as the plain target model; passed as `draft_weights` the MTP drafter is active."""
  import os
  path = full_model_path()
  if not path.exists():
    temporary = path.with_suffix(f".{os.getpid()}.tmp")
    write_gguf(temporary, layers=FULL_LAYERS, vocab=FULL_VOCAB, mtp=True, seed=FULL_SEED)
    os.replace(temporary, path)
  return path
