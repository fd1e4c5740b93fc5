"""Regenerates tests/golden/kquant_dequant.npz from gguf-py (`gguf.quants.dequantize`, gguf 0.19.0), the
third-party implementation of the GGUF K-quant block formats that the reference's kernels re-implement
(backend/metal/kernel/quant_linear.metal:12-85). Run from the repository root:

    python tests/golden/make_golden.py

The fixture pins the oracle's (and through it the CUDA kernels') Q4_K / Q6_K dequantisers bit for bit.
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
  out = Path(__file__).resolve().parent / "kquant_dequant.npz"
  np.savez_compressed(out, q4k_blocks=q4, q4k_values=dequantize(q4, GGMLQuantizationType.Q4_K).astype(np.float32), q6k_blocks=q6,
                      q6k_values=dequantize(q6, GGMLQuantizationType.Q6_K).astype(np.float32))
  print("wrote", out, out.stat().st_size, "bytes")


if __name__ == "__main__":
  main()
