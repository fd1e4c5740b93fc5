// Activation image: the operand format the integer decode GEMV (q4k_decode.cu) reads.
//
// Up to 8 activation rows x K values are quantised per (row, 256-value block) to 16-bit integers
// x_int = rint(x / xs), xs = max|x| / 32767, and stored split as hi = x_int >> 8 (signed byte) and
// lo = x_int & 255 (unsigned byte), so that sum q * x_int = 256 * sum q * hi + sum q * lo runs as two
// m16n8k32 integer MMAs whose results are kept apart until the end of a super-block.
//
// Per 256-value block (kImageBlockBytes, contiguous, in this order):
//   [8 sub-blocks][8 rows][4 quarters][16 B]   quarter t of sub-block j: 8 hi bytes then 8 lo bytes of the
//                                               values 32j + 8t + 0..7 (exactly the B fragment of lane
//                                               (row, t): registers b0, b1 of the hi MMA, then of the lo MMA)
//   [8 rows][4][8 B]                            sub-block sums S_j / 32 as fp16 hi | lo pairs: entry (row, t) holds
//                                               {hi(S_2t), hi(S_2t+1)}, {lo(S_2t), lo(S_2t+1)}, the B fragment
//                                               of the min-term MMA; S_j = sum of x_int over sub-block j
//   [8 rows] fp32                               xs
// Rows beyond the live ones are zero.
#pragma once
#include "common.cuh"

namespace infdev {

constexpr int kImageQuantBytes = 8 * 8 * 4 * 16;   // 4096
constexpr int kImageSumOffset = kImageQuantBytes;  // 256 B of sums
constexpr int kImageScaleOffset = kImageSumOffset + 256;
constexpr int kImageBlockBytes = kImageScaleOffset + 32;  // 4384, a multiple of 16
constexpr int kImageRows = 8;
constexpr float kImageLevels = 32767.0f;

// One warp quantises one (row, block): lane L holds the 8 consecutive values 8L .. 8L+7 of the block
// (sub-block L/4, quarter L%4). `block` points at the image of this 256-value block.
__device__ __forceinline__ void image_store_block(uint8_t* block, int row, int lane, const float (&v)[8]) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i)
    amax = fmaxf(amax, fabsf(v[i]));
  amax = warp_max(amax);
  const float xs = amax / kImageLevels, inv = amax > 0.f ? kImageLevels / amax : 0.f;
  uint32_t hi[2] = {0, 0}, lo[2] = {0, 0};
  int sum = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    int q = __float2int_rn(v[i] * inv);
    q = max(-32767, min(32767, q));
    sum += q;
    hi[i >> 2] |= (uint32_t(q >> 8) & 0xffu) << (8 * (i & 3));
    lo[i >> 2] |= (uint32_t(q) & 0xffu) << (8 * (i & 3));
  }
  *reinterpret_cast<uint4*>(block + (lane >> 2) * 512 + row * 64 + (lane & 3) * 16) = make_uint4(hi[0], hi[1], lo[0], lo[1]);
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  sum += __shfl_xor_sync(0xffffffffu, sum, 2);  // lanes 4j .. 4j+3 now hold S_j
  const int t = lane & 3;
  const float s0 = float(__shfl_sync(0xffffffffu, sum, 8 * t)) * 0.03125f, s1 = float(__shfl_sync(0xffffffffu, sum, 8 * t + 4)) * 0.03125f;
  if (lane < 4) {
    const uint32_t top = pack_half2(s0, s1);
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&top));
    *reinterpret_cast<uint2*>(block + kImageSumOffset + (row * 4 + lane) * 8) = make_uint2(top, pack_half2(s0 - f.x, s1 - f.y));
  }
  if (lane == 0)
    *reinterpret_cast<float*>(block + kImageScaleOffset + row * 4) = xs;
}

// An all-zero row of a block (rows past the live ones).
__device__ __forceinline__ void image_zero_block(uint8_t* block, int row, int lane) {
  *reinterpret_cast<uint4*>(block + (lane >> 2) * 512 + row * 64 + (lane & 3) * 16) = make_uint4(0, 0, 0, 0);
  if (lane < 4)
    *reinterpret_cast<uint2*>(block + kImageSumOffset + (row * 4 + lane) * 8) = make_uint2(0, 0);
  if (lane == 0)
    *reinterpret_cast<float*>(block + kImageScaleOffset + row * 4) = 0.f;
}

}  // namespace infdev
