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
