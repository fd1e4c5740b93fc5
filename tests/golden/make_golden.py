"""Regenerates tests/golden/kquant_dequant.npz from gguf-py (`gguf.quants.dequantize`, gguf 0.19.0), the
third-party implementation of the GGUF K-quant block formats that the reference's kernels re-implement
(backend/metal/kernel/quant_linear.metal:12-85). Run from the repository root:

    python tests/golden/make_golden.py

The fixture pins the oracle's (and through it the CUDA kernels') Q4_K / Q6_K / Q5_K / Q8_0 / IQ4_XS dequantisers bit for bit.
"""
import sys
from pathlib import Path

import numpy as np
from gguf import GGMLQuantizationType
from gguf.quants import dequantize

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from mtlqwen_b200.testing import synth


def main():
  rng = np.random.default_rng(20251125)
  q4 = synth.q4k_blocks(96, rng)
  q4[90:96] = synth.q4k_blocks(6, rng, subnormal=True)  # fp16-subnormal super-block scales
  q4[0, 0:4] = 0  # d = dmin = 0
  q4[1, 4:16] = 0xff  # all scales / mins at 63
  q4[2, 16:144] = 0xff  # all quants at 15
  q4[3, 16:144] = 0x00
  q4[4, 0:2] = np.array([0.5], np.float16).view(np.uint8)  # large d
  q6 = synth.q6k_blocks(96, rng)
  q6[0, 208:210] = 0
  q6[1, 192:208] = 0x80  # all scales -128
  q6[2, 192:208] = 0x7f
  q6[3, 0:192] = 0xff
  q6[4, 0:192] = 0x00
  q6[5, 208:210] = np.array([0.25], np.float16).view(np.uint8)
  # Q5_K (176 B): as Q4_K plus 32 bytes of fifth bits; Q8_0 (34 B per 32 values); IQ4_XS (136 B): 6-bit sub-block scales
  # around 32 and indices into a 16-entry non-linear grid. Raw random fields with fp16 scales of sensible size, plus corners.
  def scaled(count, size, at, low, high):
    blocks = np.frombuffer(rng.bytes(count * size), dtype=np.uint8).reshape(count, size).copy()
    for offset in at:
      blocks[:, offset:offset + 2] = rng.uniform(low, high, count).astype(np.float16).view(np.uint8).reshape(count, 2)
    return blocks
  q5 = scaled(64, 176, (0, 2), 2e-5, 2e-4)
  q5[0, 0:4] = 0
  q5[1, 16:48] = 0xff  # every fifth bit set
  q5[2, 16:48] = 0x00
  q5[3, 4:16] = 0xff
  q8 = scaled(64, 34, (0, ), 1e-4, 1e-3)
  q8[0, 2:] = 0x80  # all -128
  q8[1, 2:] = 0x7f
  q8[2, 0:2] = 0
  iq4 = scaled(64, 136, (0, ), 1e-5, 1e-4)
  iq4[0, 2:8] = 0xff  # all sub-block scales at 63
  iq4[1, 2:8] = 0x00  # all at 0 (factor -32)
  iq4[2, 8:] = 0xff
  out = Path(__file__).resolve().parent / "kquant_dequant.npz"
  np.savez_compressed(out, q4k_blocks=q4, q4k_values=dequantize(q4, GGMLQuantizationType.Q4_K).astype(np.float32), q6k_blocks=q6,
                      q6k_values=dequantize(q6, GGMLQuantizationType.Q6_K).astype(np.float32), q5k_blocks=q5,
                      q5k_values=dequantize(q5, GGMLQuantizationType.Q5_K).astype(np.float32), q8_0_blocks=q8,
                      q8_0_values=dequantize(q8, GGMLQuantizationType.Q8_0).astype(np.float32), iq4xs_blocks=iq4,
                      iq4xs_values=dequantize(iq4, GGMLQuantizationType.IQ4_XS).astype(np.float32))
  print("wrote", out, out.stat().st_size, "bytes")


if __name__ == "__main__":
  main()
