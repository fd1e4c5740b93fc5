"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations:
raw-field GGUF Q4_K / Q6_K weight blocks, activations, and a random-init GGUF writer.

K-quant `quantize` is not needed: blocks are drawn field by field (quants uniform, 6-bit scales and mins
uniform, fp16 super-block scales chosen so the dequantised weights are about N(0, 0.02)).
"""
import numpy as np

Q4_K, Q6_K, F32 = 12, 14, 0
F16, Q8_0, Q5_K, IQ4_XS = 1, 8, 13, 23
BLOCK_BYTES = {Q4_K: 144, Q6_K: 210, Q5_K: 176, IQ4_XS: 136, Q8_0: 34}
BLOCK_VALUES = {Q4_K: 256, Q6_K: 256, Q5_K: 256, IQ4_XS: 256, Q8_0: 32}


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


def q5k_blocks(count, rng, target_std=0.02):
  """`count` Q5_K super-blocks (176 B): as Q4_K plus 32 bytes of fifth bits, q ~ U{0..31}. E[sc q] = 488.25 and
  E[m] = 31.5 so dmin = 15.5 d centres the weights; std(w) = 527 d."""
  blocks = np.frombuffer(rng.bytes(count * 176), dtype=np.uint8).reshape(count, 176).copy()
  d16 = ((target_std / 527.0) * rng.uniform(0.8, 1.2, count)).astype(np.float16)
  m16 = (d16.astype(np.float32) * 15.5).astype(np.float16)
  blocks[:, 0:2] = d16.view(np.uint8).reshape(count, 2)
  blocks[:, 2:4] = m16.view(np.uint8).reshape(count, 2)
  return blocks


def q8_0_blocks(count, rng, target_std=0.02):
  """`count` Q8_0 blocks (34 B per 32 values): fp16 d, 32 int8 ~ U{-128..127} (std 73.9)."""
  blocks = np.frombuffer(rng.bytes(count * 34), dtype=np.uint8).reshape(count, 34).copy()
  blocks[:, 0:2] = ((target_std / 73.9) * rng.uniform(0.8, 1.2, count)).astype(np.float16).view(np.uint8).reshape(count, 2)
  return blocks


def iq4xs_blocks(count, rng, target_std=0.02):
  """`count` IQ4_XS super-blocks (136 B): fp16 d, 6-bit sub-block scales ls ~ U{0..63} (factor ls - 32), 4-bit indices
  into the non-linear grid (std about 72): std(w) is about 1330 d."""
  blocks = np.frombuffer(rng.bytes(count * 136), dtype=np.uint8).reshape(count, 136).copy()
  blocks[:, 0:2] = ((target_std / 1330.0) * rng.uniform(0.8, 1.2, count)).astype(np.float16).view(np.uint8).reshape(count, 2)
  return blocks


GENERATORS = {Q4_K: q4k_blocks, Q6_K: q6k_blocks, Q5_K: q5k_blocks, Q8_0: q8_0_blocks, IQ4_XS: iq4xs_blocks}


def weight(qtype, n, k, seed):
  rng = np.random.default_rng(seed)
  return GENERATORS[qtype](n * (k // BLOCK_VALUES[qtype]), rng)


def activations(m, k, seed):
  return np.random.default_rng(seed).standard_normal((m, k)).astype(np.float32)


# ---- random-init GGUF files with the reference's tensor names and shapes (model/qwen35/forward.cpp:74-127) ----
GGUF_MAGIC, GGUF_ALIGNMENT = 0x46554747, 32
HIDDEN, INTERMEDIATE = 4096, 12288


def model_tensors(layers=32, vocab=248320, mtp=False, seed=1234, mixed=False):
  """Yields (name, ggml type, shape as (n, k) or (dim,), generator of the raw bytes). Projections Q4_K, embedding
  and lm_head Q6_K, norms F32 at 1 +- 0.01, GDN parameters as in the gated-delta-rule benchmark configuration.
  mixed: the type mix of the real Qwen3.5 GGUF files instead - projections cycle through Q4_K, Q5_K, IQ4_XS, Q6_K and
  Q8_0 (a gate / up pair shares its type), the embedding table is Q4_K, ssm_beta / ssm_alpha are F16 and the MTP
  projection eh_proj is Q8_0."""
  counter = [seed]
  cycle = [0]

  def rng():
    counter[0] += 1
    return np.random.default_rng(counter[0])

  def quantised(qtype, n, k):
    return (qtype, (n, k), lambda: GENERATORS[qtype](n * k // BLOCK_VALUES[qtype], rng()))

  def q4(n, k, advance=True):
    if not mixed:
      return quantised(Q4_K, n, k)
    if advance:
      cycle[0] += 1
    return quantised((Q4_K, Q5_K, IQ4_XS, Q6_K, Q8_0)[cycle[0] % 5], n, k)

  def q6(n, k):
    return quantised(Q6_K, n, k)

  def norm(dim):
    return (F32, (dim, ), lambda: (1 + 0.01 * rng().standard_normal(dim)).astype(np.float32))

  def f32(shape, make):
    return (F32, shape, lambda: make(rng()).astype(np.float32))

  yield ("token_embd.weight", *(quantised(Q4_K, vocab, HIDDEN) if mixed else q6(vocab, HIDDEN)))
  yield ("output_norm.weight", *norm(HIDDEN))
  yield ("output.weight", *q6(vocab, HIDDEN))

  def ffn(prefix):
    yield (prefix + "post_attention_norm.weight", *norm(HIDDEN))
    yield (prefix + "ffn_gate.weight", *q4(INTERMEDIATE, HIDDEN))
    yield (prefix + "ffn_up.weight", *q4(INTERMEDIATE, HIDDEN, advance=False))
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
    if mixed:
      yield (prefix + "ssm_beta.weight", F16, (32, HIDDEN), lambda: (rng().standard_normal((32, HIDDEN)) / 64).astype(np.float16))
      yield (prefix + "ssm_alpha.weight", F16, (32, HIDDEN), lambda: (rng().standard_normal((32, HIDDEN)) / 64).astype(np.float16))
    else:
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
    yield (prefix + "nextn.eh_proj.weight", *(quantised(Q8_0, HIDDEN, 2 * HIDDEN) if mixed else q4(HIDDEN, 2 * HIDDEN)))
    yield (prefix + "nextn.shared_head_norm.weight", *norm(HIDDEN))
    yield from attention(prefix)


def _gguf_string(text):
  raw = text.encode()
  return np.uint64(len(raw)).tobytes() + raw


def tensor_bytes(qtype, elements):
  return elements * 4 if qtype == F32 else elements * 2 if qtype == F16 else elements // BLOCK_VALUES[qtype] * BLOCK_BYTES[qtype]


def write_gguf(path, layers=32, vocab=248320, mtp=False, seed=1234, mixed=False):
  """Writes a GGUF v3 file. ne[0] is the contiguous dimension: a weight [n, k] is stored with shape (k, n),
  which the engine reads back as n = shape[1], k = shape[0] (forward.cpp:18-22)."""
  tensors = list(model_tensors(layers, vocab, mtp, seed, mixed))
  sizes = [tensor_bytes(qtype, int(np.prod(shape))) for _, qtype, shape, _ in tensors]
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
    size = tensor_bytes(qtype, int(np.prod(dims)))
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
