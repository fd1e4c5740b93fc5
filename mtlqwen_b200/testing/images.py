"""Host-side reader of activation images (the operand format of the integer Q4_K decode kernel, see
csrc/act_image.cuh): used by the tests and handy when debugging a pass.

Per 8-row slice and 256-value block, 4384 bytes:
  [8 sub-blocks][8 rows][4 quarters][8 high bytes | 8 low bytes]   x_int = 256 * int8(high) + uint8(low)
  [8 rows][4][fp16 hi(S_2t), hi(S_2t+1), lo(S_2t), lo(S_2t+1)]     S_j = sum of x_int over sub-block j, stored / 32
  [8 rows] fp32                                                    xs: x ~= xs * x_int
"""
import numpy as np

BLOCK_BYTES, LEVELS = 4384, 32767


def decode(image, rows, k):
  """image: uint8 array of at least ceil(rows/8) * (k/256) * 4384 bytes. Returns (x_int [rows,k] int32,
  xs [rows,k/256] float32, sums [rows,k/256,8] float64 = the stored sub-block sums times 32)."""
  blocks, slices = k // 256, (rows + 7) // 8
  raw = np.asarray(image, dtype=np.uint8).reshape(-1)[:slices * blocks * BLOCK_BYTES].reshape(slices, blocks, BLOCK_BYTES)
  quants = raw[:, :, :4096].reshape(slices, blocks, 8, 8, 4, 16)  # [slice, block, sub-block, row, quarter, 16]
  high = quants[..., :8].view(np.int8).astype(np.int32)
  low = quants[..., 8:].astype(np.int32)
  value = 256 * high + low                                         # [slice, block, j, row, t, 8]
  x_int = value.transpose(0, 3, 1, 2, 4, 5).reshape(slices * 8, k)[:rows]
  sums16 = raw[:, :, 4096:4352].copy().view(np.float16).astype(np.float64).reshape(slices, blocks, 8, 4, 4)  # [.., row, t, (hi0, hi1, lo0, lo1)]
  pair = sums16[..., 0:2] + sums16[..., 2:4]                       # [.., row, t, 2] -> sub-blocks 2t, 2t+1
  sums = (32.0 * pair.reshape(slices, blocks, 8, 8)).transpose(0, 2, 1, 3).reshape(slices * 8, blocks, 8)[:rows]
  xs = raw[:, :, 4352:4384].copy().view(np.float32).reshape(slices, blocks, 8).transpose(0, 2, 1).reshape(slices * 8, blocks)[:rows]
  return x_int, xs, sums


def quantize(x):
  """numpy statement of the quantisation: per (row, 256-value block) xs = max|x| / 32767, x_int = rint(x * (32767 / max|x|))."""
  x = np.asarray(x, dtype=np.float32)
  rows, k = x.shape
  blocks = x.reshape(rows, k // 256, 256)
  amax = np.abs(blocks).max(axis=-1)
  xs = (amax / np.float32(LEVELS)).astype(np.float32)
  with np.errstate(divide="ignore"):
    inv = np.where(amax > 0, np.float32(LEVELS) / amax, np.float32(0)).astype(np.float32)
  x_int = np.clip(np.rint(blocks * inv[..., None]), -LEVELS, LEVELS).astype(np.int32)
  return x_int.reshape(rows, k), xs, x_int.reshape(rows, k // 256, 8, 32).sum(axis=-1).astype(np.float64)
