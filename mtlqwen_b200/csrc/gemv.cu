// Dequant-fused fp16 tensor-core GEMV for decode (M <= 8 activation rows) over GGUF Q4_K / Q6_K weights. It serves
// every Q6_K matrix (lm_head) and, when the integer kernel of q4k_decode.cu is switched off, the Q4_K ones.
//
// Replaces linear_decode_q4_k[_add] (quant_linear.metal:245-327), linear_decode_q6_k[_add] (:436-512) and
// mlp_gate_up_q4_k_decode (fused_kernels.metal:11-78). The reference re-reads the weights once per
// activation row (grid.y = rows); here up to 8 rows share one pass over the weights.
//
// Design (one persistent CTA per SM, 8 consumer warps + 1 producer warp):
//  * The weight matrix is a contiguous byte stream (row n = K/256 super-blocks). The producer warp moves
//    16-row x 8-super-block slabs into a shared-memory ring with one tiled TMA copy each (a tensor map over
//    the packed rows as 8-byte elements) that completes on an mbarrier; nothing else touches HBM for the weights.
//  * At 8 rows the fp32 FMA pipe cannot keep up with HBM (8 FMAs per 4-bit weight), so the products run
//    on the tensor cores as m16n8k16: A = 16 weight rows x 16 k, B = 16 k x 8 activation rows.
//    The summation index of an MMA is a dummy, so k is permuted freely to suit the packed layout; the
//    activations are staged once per CTA in shared memory already in B-fragment order under the same
//    permutation.
//  * Q4_K: A holds the exact integers sc*q (<= 945, exact in fp16); the super-block scale d is applied to
//    the fp32 accumulator after each super-block, and the -dmin*m term is one more MMA against the
//    per-sub-block activation sums. Q6_K: A holds q-32 exactly and the per-16 scale d*sc is applied to
//    the accumulator after each MMA (one MMA = one scale group).
//  * Activations are split x = hi + lo into two fp16 fragments (XSPLIT = 2) so the result keeps fp32
//    accuracy; XSPLIT = 1 drops lo (relative error ~3e-4, still inside the 1e-3 contract).
//  * Every mbarrier wait is bounded; on a timeout the kernel raises an abort flag, records a status code
//    and all roles leave their loops.
#include "common.cuh"
#include "kernels.h"

namespace infdev {
namespace {

constexpr int kConsumerWarps = 8;   // one warp per super-block of a stage
constexpr int kThreads = (kConsumerWarps + 1) * kWarp;
constexpr int kChunkBlocks = 16;   // super-blocks of K staged per pass (4096 values)
constexpr int kStageBlocks = kGemvStageBlocks;  // super-blocks per ring stage (one per consumer warp)
constexpr int kMaxStages = 8;
constexpr int kTileRows = kGemvTileRows;

struct Q4K {
  static constexpr int kBlockBytes = 144;
  static constexpr int kRowStride = kStageBlocks * kBlockBytes;  // rows of a TMA box are dense in shared memory
  static constexpr bool kMinTerm = true;
  static constexpr int kStageBytes = kTileRows * kRowStride;
};

struct Q6K {
  static constexpr int kBlockBytes = 210;
  static constexpr int kRowStride = kStageBlocks * kBlockBytes;  // 1680 == 16 mod 128
  static constexpr bool kMinTerm = false;
  static constexpr int kStageBytes = kTileRows * kRowStride;
};

struct Smem {
  uint64_t full[kMaxStages], empty[kMaxStages];
  int abort;
};
constexpr int kControlBytes = 256;
static_assert(sizeof(Smem) <= kControlBytes, "control block overlaps the activation fragments");

template <class Q, int NMAT, int XSPLIT> constexpr size_t fixed_bytes() {
  size_t frag = size_t(kChunkBlocks) * 16 * 32 * 8 * XSPLIT;
  size_t sums = Q::kMinTerm ? size_t(kChunkBlocks) * 32 * 8 : 0;
  size_t partial = size_t(2) * NMAT * kConsumerWarps * 128 * 4;
  return kControlBytes + frag + sums + partial;
}

// As many ring stages as fit beside the fragments in the 227 KB a CTA may use.
template <class Q, int NMAT, int XSPLIT> constexpr int stage_count() {
  int stages = int((size_t(227) * 1024 - fixed_bytes<Q, NMAT, XSPLIT>()) / Q::kStageBytes);
  return stages > kMaxStages ? kMaxStages : stages;
}

template <class Q, int NMAT, int XSPLIT> constexpr size_t smem_bytes() {
  return fixed_bytes<Q, NMAT, XSPLIT>() + size_t(stage_count<Q, NMAT, XSPLIT>()) * Q::kStageBytes;
}

__device__ __forceinline__ uint32_t lds_u32_unaligned(const uint8_t* p) {
  return uint32_t(*reinterpret_cast<const uint16_t*>(p)) | (uint32_t(*reinterpret_cast<const uint16_t*>(p + 2)) << 16);
}

// ---- Q4_K: one 16-row x 256-k unit -------------------------------------------------------------
// Lane (g = lane/4, t = lane%4) owns weight rows g and g+8 and, in each, the 16-byte quant chunks t and
// t+4 of the super-block (chunk c = bytes [16c,16c+16) of qs: low nibbles are elements 64*(c/2) +
// 16*(c%2) + [0,16) , high nibbles the same + 32; GGUF layout as read by dequant_tile,
// quant_linear.metal:39-46). MMA i = (chunk select, word j, nibble h) consumes bytes 0..3 of word j.
__device__ __forceinline__ uint4 lds128(uint32_t address) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(address));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t address) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(address));
  return v;
}

// All operands are 32-bit shared-memory addresses: pA / pB the super-block of rows g and g+8, xhi / xlo the B
// fragments of this super-block already offset by the lane's rotated slot for j = 0 (slots for j = 1..3 follow from
// `rot`, the byte offsets of the other three rotations), xsum the lane's min-term fragment.
template <int XSPLIT>
__device__ __forceinline__ void q4k_unit(uint32_t pA, uint32_t pB, int t, uint32_t xhi, uint32_t xlo, const int (&rot)[4], uint32_t xsum,
                                         float (&total)[4]) {
  const uint4 hA = lds128(pA), hB = lds128(pB);
  // 6-bit scales / mins of the 8 sub-blocks, four per word (scale_min_k4, quant_linear.metal:12-20).
  const uint32_t scA[2] = {hA.y & 0x3f3f3f3fu, (hA.w & 0x0f0f0f0fu) | ((hA.y >> 2) & 0x30303030u)};
  const uint32_t mnA[2] = {hA.z & 0x3f3f3f3fu, ((hA.w >> 4) & 0x0f0f0f0fu) | ((hA.z >> 2) & 0x30303030u)};
  const uint32_t scB[2] = {hB.y & 0x3f3f3f3fu, (hB.w & 0x0f0f0f0fu) | ((hB.y >> 2) & 0x30303030u)};
  const uint32_t mnB[2] = {hB.z & 0x3f3f3f3fu, ((hB.w >> 4) & 0x0f0f0f0fu) | ((hB.z >> 2) & 0x30303030u)};
  const int shift = (t >> 1) * 16;
  constexpr uint32_t k1024 = 0x64006400u, kNeg1024 = 0xE400E400u, kSixteenth = 0x2C002C00u, kNeg64 = 0xD400D400u;
  // Four independent accumulator chains: consecutive MMAs never wait on each other's results.
  float acc[4][4];
#pragma unroll
  for (int c = 0; c < 4; ++c)
    acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0.f;
#pragma unroll
  for (int cs = 0; cs < 2; ++cs) {
    // This lane's quant chunk t + 4*cs of both rows. Its low nibbles belong to sub-block 2*(c/2), the high ones to
    // 2*(c/2)+1; their scales are bytes 2*(t/2), 2*(t/2)+1 of the cs-th scale word.
    const uint4 qA = lds128(pA + 16 + 64 * cs + 16 * t), qB = lds128(pB + 16 + 64 * cs + 16 * t);
    const uint32_t pairA = (scA[cs] >> shift) & 0xffffu, pairB = (scB[cs] >> shift) & 0xffffu;
    const uint32_t sLA = hsub2_u32(__byte_perm(pairA, 0x64u, 0x4040), k1024), sHA = hsub2_u32(__byte_perm(pairA, 0x64u, 0x4141), k1024);
    const uint32_t sLB = hsub2_u32(__byte_perm(pairB, 0x64u, 0x4040), k1024), sHB = hsub2_u32(__byte_perm(pairB, 0x64u, 0x4141), k1024);
    const uint32_t nLA = hmul2_u32(sLA, kNeg1024), nLB = hmul2_u32(sLB, kNeg1024);
    const uint32_t mHA = hmul2_u32(sHA, kSixteenth), mHB = hmul2_u32(sHB, kSixteenth);
    const uint32_t nHA = hmul2_u32(sHA, kNeg64), nHB = hmul2_u32(sHB, kNeg64);
    const uint32_t wordsA[4] = {qA.x, qA.y, qA.z, qA.w}, wordsB[4] = {qB.x, qB.y, qB.z, qB.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t wA = wordsA[j], wB = wordsB[j], vA = wA >> 8, vB = wB >> 8;
      const int i = (cs * 4 + j) * 2;          // MMA index of the low-nibble step; i + 1 is the high-nibble step
      const int at = i * 256 + rot[j];         // byte offset of fragment (i, rotated slot): 32 slots x 8 bytes per MMA
      uint32_t a[4];
      // low nibbles: (1024 + q) * sc - 1024 * sc, exact in fp16
      a[0] = hfma2_u32((wA & 0x000f000fu) | k1024, sLA, nLA);
      a[1] = hfma2_u32((wB & 0x000f000fu) | k1024, sLB, nLB);
      a[2] = hfma2_u32((vA & 0x000f000fu) | k1024, sLA, nLA);
      a[3] = hfma2_u32((vB & 0x000f000fu) | k1024, sLB, nLB);
      uint2 b = lds64(xhi + at);
      mma_16816(acc[j & 1], a, b.x, b.y);
      if (XSPLIT == 2) {
        b = lds64(xlo + at);
        mma_16816(acc[j & 1], a, b.x, b.y);
      }
      // high nibbles in place: (1024 + 16 q) * sc/16 - 64 * sc
      a[0] = hfma2_u32((wA & 0x00f000f0u) | k1024, mHA, nHA);
      a[1] = hfma2_u32((wB & 0x00f000f0u) | k1024, mHB, nHB);
      a[2] = hfma2_u32((vA & 0x00f000f0u) | k1024, mHA, nHA);
      a[3] = hfma2_u32((vB & 0x00f000f0u) | k1024, mHB, nHB);
      b = lds64(xhi + at + 256);
      mma_16816(acc[2 + (j & 1)], a, b.x, b.y);
      if (XSPLIT == 2) {
        b = lds64(xlo + at + 256);
        mma_16816(acc[2 + (j & 1)], a, b.x, b.y);
      }
    }
  }
  // min term: sum_j m_j * (sum of the activations of sub-block j); k 0..7 carry the hi half of the sums,
  // k 8..15 the lo half, against the same mins.
  float accm[4] = {0.f, 0.f, 0.f, 0.f};
  {
    const uint32_t wordA = (t & 2) ? mnA[1] : mnA[0], wordB = (t & 2) ? mnB[1] : mnB[0];
    const uint32_t pA2 = (wordA >> ((t & 1) * 16)) & 0xffffu, pB2 = (wordB >> ((t & 1) * 16)) & 0xffffu;
    uint32_t a[4];
    a[0] = a[2] = hsub2_u32(__byte_perm(pA2, 0x64u, 0x4140), k1024);
    a[1] = a[3] = hsub2_u32(__byte_perm(pB2, 0x64u, 0x4140), k1024);
    const uint2 b = lds64(xsum);
    mma_16816(accm, a, b.x, b.y);
  }
  const float2 dA = __half22float2(*reinterpret_cast<const __half2*>(&hA.x)), dB = __half22float2(*reinterpret_cast<const __half2*>(&hB.x));
  total[0] += dA.x * ((acc[0][0] + acc[1][0]) + (acc[2][0] + acc[3][0])) - dA.y * accm[0];
  total[1] += dA.x * ((acc[0][1] + acc[1][1]) + (acc[2][1] + acc[3][1])) - dA.y * accm[1];
  total[2] += dB.x * ((acc[0][2] + acc[1][2]) + (acc[2][2] + acc[3][2])) - dB.y * accm[2];
  total[3] += dB.x * ((acc[0][3] + acc[1][3]) + (acc[2][3] + acc[3][3])) - dB.y * accm[3];
}

// ---- Q6_K: one 16-row x 256-k unit -------------------------------------------------------------
// Block layout (quant_linear.metal:69-85): ql[128] | qh[64] | int8 sc[16] | fp16 d. Element r = 128*hh + 32*s
// + l has its low nibble in ql[64*hh + 32*(s&1) + l] (high half of the byte when s >= 2), its top two bits
// in qh[32*hh + l] >> 2s, and scale sc[r/16]. MMA gi covers elements [16gi, 16gi+16); lane t supplies
// elements 16gi + 4t + {0,1,2,3}. Blocks are only 2-byte aligned, so words are fetched as two halves.
template <int XSPLIT>
__device__ __forceinline__ void q6k_unit(const uint8_t* pA, const uint8_t* pB, int lane, int hh, const uint2* xhi, const uint2* xlo,
                                         float (&total)[4]) {
  const int t = lane & 3;
  const float dA = load_half_bits(pA + 208), dB = load_half_bits(pB + 208);
  constexpr uint32_t k1056 = 0x64206420u;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const uint32_t hiA = lds_u32_unaligned(pA + 128 + 32 * hh + 16 * u + 4 * t), hiB = lds_u32_unaligned(pB + 128 + 32 * hh + 16 * u + 4 * t);
#pragma unroll
      for (int sl = 0; sl < 2; ++sl) {
        const uint32_t loA = lds_u32_unaligned(pA + 64 * hh + 32 * sl + 16 * u + 4 * t), loB = lds_u32_unaligned(pB + 64 * hh + 32 * sl + 16 * u + 4 * t);
#pragma unroll
        for (int sh = 0; sh < 2; ++sh) {
          const int s = sl + 2 * sh, gi = hh * 8 + s * 2 + u;
          const uint32_t bytesA = ((sh ? loA >> 4 : loA) & 0x0f0f0f0fu) | (((hiA >> (2 * s)) & 0x03030303u) << 4);
          const uint32_t bytesB = ((sh ? loB >> 4 : loB) & 0x0f0f0f0fu) | (((hiB >> (2 * s)) & 0x03030303u) << 4);
          uint32_t a[4];
          a[0] = hsub2_u32(__byte_perm(bytesA, 0x64u, 0x4140), k1056);
          a[1] = hsub2_u32(__byte_perm(bytesB, 0x64u, 0x4140), k1056);
          a[2] = hsub2_u32(__byte_perm(bytesA, 0x64u, 0x4342), k1056);
          a[3] = hsub2_u32(__byte_perm(bytesB, 0x64u, 0x4342), k1056);
          float acc[4] = {0.f, 0.f, 0.f, 0.f};
          uint2 b = xhi[gi * 32 + lane];
          mma_16816(acc, a, b.x, b.y);
          if (XSPLIT == 2) {
            b = xlo[gi * 32 + lane];
            mma_16816(acc, a, b.x, b.y);
          }
          const float sA = dA * float(int(reinterpret_cast<const int8_t*>(pA + 192)[gi])), sB = dB * float(int(reinterpret_cast<const int8_t*>(pB + 192)[gi]));
          total[0] += sA * acc[0];
          total[1] += sA * acc[1];
          total[2] += sB * acc[2];
          total[3] += sB * acc[3];
        }
      }
    }
}

__device__ __forceinline__ int find_segment(const GemvParams& p, int tile) {
  int s = 0;
  while (s + 1 < p.nseg && tile >= p.seg[s + 1].tile0)
    ++s;
  return s;
}

template <class Q, int NMAT, int XSPLIT> __global__ void __launch_bounds__(kThreads, 1) gemv_kernel(const __grid_constant__ GemvParams p) {
  constexpr int kStages = stage_count<Q, NMAT, XSPLIT>();
  extern __shared__ __align__(128) uint8_t smemRaw[];
  Smem& ctl = *reinterpret_cast<Smem*>(smemRaw);
  uint2* fragHi = reinterpret_cast<uint2*>(smemRaw + kControlBytes);
  uint2* fragLo = fragHi + (XSPLIT == 2 ? kChunkBlocks * 16 * 32 : 0);
  uint2* fragSum = fragHi + kChunkBlocks * 16 * 32 * XSPLIT;
  float* partial = reinterpret_cast<float*>(fragSum + (Q::kMinTerm ? kChunkBlocks * 32 : 0));
  uint8_t* ring = reinterpret_cast<uint8_t*>(partial + 2 * NMAT * kConsumerWarps * 128);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int blocksPerRow = p.k / 256;
  const size_t rowBytes = size_t(blocksPerRow) * Q::kBlockBytes;
  const int chunks = (blocksPerRow + kChunkBlocks - 1) / kChunkBlocks;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&ctl.full[s], 1);
      mbar_init(&ctl.empty[s], kConsumerWarps);
    }
    ctl.abort = 0;
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();
  volatile int* abortFlag = &ctl.abort;

  if (warp == kConsumerWarps) {
    // ---- producer: stream weight slabs into the ring (they do not depend on the kernels before this one) ----
    uint32_t it = 0;
    for (int chunk = 0; chunk < chunks && !*abortFlag; ++chunk) {
      const int chunkBlocks = min(kChunkBlocks, blocksPerRow - chunk * kChunkBlocks);
      const int groups = (chunkBlocks + kStageBlocks - 1) / kStageBlocks;
      for (int tile = blockIdx.x; tile < p.tiles && !*abortFlag; tile += gridDim.x) {
        const int segment = find_segment(p, tile);
        const size_t row0 = size_t(tile - p.seg[segment].tile0) * kTileRows;
        for (int mat = 0; mat < NMAT; ++mat) {
          for (int grp = 0; grp < groups; ++grp, ++it) {
            const uint32_t slot = it % kStages, round = it / kStages;
            bool ok = true;
            if (lane == 0 && round > 0)
              ok = mbar_wait_bounded(&ctl.empty[slot], (round - 1) & 1, abortFlag);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
              if (lane == 0) {
                *abortFlag = 1;
                atomicExch(p.status, kStatusBarrierTimeout);
              }
              break;
            }
            // One tiled copy moves the whole 16-row x 8-super-block slab; columns past the end of a row are zero-filled
            // and still counted, so the transaction size is always the full box.
            if (lane == 0) {
              mbar_arrive_expect_tx(&ctl.full[slot], uint32_t(Q::kStageBytes));
              tma_load_2d(ring + size_t(slot) * Q::kStageBytes, &p.map[segment][mat], (chunk * (kChunkBlocks / kStageBlocks) + grp) * Q::kBlockBytes,
                          int(row0), &ctl.full[slot]);
            }
            __syncwarp();
          }
        }
      }
    }
    pdl_wait();  // every thread of every kernel waits, so completion stays transitive along the stream
    return;
  }

  // ---- consumers ----
  pdl_wait();  // the activations come from the kernels before this one
  const int g = lane >> 2, t = lane & 3;
  // Shared-memory byte addresses of this lane's B fragments: slot rotated by j inside each 32-entry line.
  const int rotation[4] = {0, (((lane + 1) & 31) - lane) * 8, (((lane + 2) & 31) - lane) * 8, (((lane + 3) & 31) - lane) * 8};
  const uint32_t fragHiAddress = smem_u32(fragHi) + lane * 8, fragLoAddress = smem_u32(fragLo) + lane * 8, fragSumAddress = smem_u32(fragSum) + lane * 8;
  uint32_t it = 0;
  int tileCounter = 0;
  for (int chunk = 0; chunk < chunks; ++chunk) {
    const int chunkBlocks = min(kChunkBlocks, blocksPerRow - chunk * kChunkBlocks);
    const int groups = (chunkBlocks + kStageBlocks - 1) / kStageBlocks;
    const int k0 = chunk * kChunkBlocks * 256;
    // Stage the activations of this K chunk in B-fragment order (hi / lo fp16 split). A warp takes a
    // 64-value span of all 8 rows at a time: lane (row = lane/4, jj = lane%4) loads four float4 at
    // 16*e + 4*jj, so each row contributes whole 64-byte pieces. Q4_K fragments are stored rotated by jj
    // inside their 32-entry line, which makes both these writes and the MMA-time reads conflict-free.
    for (int span = warp; span < chunkBlocks * 4; span += kConsumerWarps) {
        const int row = lane >> 2, jj = lane & 3, sb = span >> 2, tq = span & 3;
        float4 v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          v[e] = row < p.m ? *reinterpret_cast<const float4*>(p.x + size_t(row) * p.ldx + k0 + 64 * span + 16 * e + 4 * jj)
                           : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          uint2 hi;
          float4 r;
          int slot;
          if (Q::kMinTerm) {  // A pairs bytes (0,2) and (1,3) of a quant word
            const int c = 2 * tq + (e & 1), i = ((c >> 2) * 4 + jj) * 2 + (e >> 1);
            slot = (sb * 16 + i) * 32 + ((row * 4 + (c & 3) + jj) & 31);
            hi.x = pack_half2(v[e].x, v[e].z);
            hi.y = pack_half2(v[e].y, v[e].w);
            const float2 f0 = __half22float2(*reinterpret_cast<__half2*>(&hi.x)), f1 = __half22float2(*reinterpret_cast<__half2*>(&hi.y));
            r = make_float4(v[e].x - f0.x, v[e].z - f0.y, v[e].y - f1.x, v[e].w - f1.y);
          } else {
            slot = (sb * 16 + tq * 4 + e) * 32 + lane;
            hi.x = pack_half2(v[e].x, v[e].y);
            hi.y = pack_half2(v[e].z, v[e].w);
            const float2 f0 = __half22float2(*reinterpret_cast<__half2*>(&hi.x)), f1 = __half22float2(*reinterpret_cast<__half2*>(&hi.y));
            r = make_float4(v[e].x - f0.x, v[e].y - f0.y, v[e].z - f1.x, v[e].w - f1.y);
          }
          fragHi[slot] = hi;
          if (XSPLIT == 2)
            fragLo[slot] = make_uint2(pack_half2(r.x, r.y), pack_half2(r.z, r.w));
        }
        if (Q::kMinTerm) {  // sums of the two 32-value sub-blocks of this span, for the min term
          float s[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s[e] = (v[e].x + v[e].y) + (v[e].z + v[e].w);
            s[e] += __shfl_xor_sync(0xffffffffu, s[e], 1);
            s[e] += __shfl_xor_sync(0xffffffffu, s[e], 2);
          }
          const float s0 = s[0] + s[1], s1 = s[2] + s[3];
          if (jj == 0) {
            const uint32_t hi = pack_half2(s0, s1);
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hi));
            fragSum[sb * 32 + row * 4 + tq] = make_uint2(hi, pack_half2(s0 - f.x, s1 - f.y));
          }
        }
      }
    named_barrier(1, kConsumerWarps * kWarp);

    for (int tile = blockIdx.x; tile < p.tiles; tile += gridDim.x, ++tileCounter) {
      // Where this thread's element of the tile goes and what is added to it (the residual, or the sum over the earlier
      // K chunks), looked up and fetched before the arithmetic: the parameter block is reached through a generic address
      // (the segment is a run-time index), and a chain of such reads after the reduction would delay every tile.
      float* destination = nullptr;
      float addend = 0.f;
      if (tid < 128 && (tid >> 4) < p.m) {
        const GemvSeg& seg = p.nseg == 1 ? p.seg[0] : p.seg[find_segment(p, tile)];
        const size_t at = size_t(tid >> 4) * seg.ldy + size_t(tile - seg.tile0) * kTileRows + (tid & 15);
        destination = seg.y + at;
        if (NMAT == 1 && chunk > 0)
          addend = *destination;
        else if (NMAT == 1 && seg.res)
          addend = seg.res[at];
      }
      float total[NMAT][4];
#pragma unroll
      for (int mat = 0; mat < NMAT; ++mat)
        total[mat][0] = total[mat][1] = total[mat][2] = total[mat][3] = 0.f;
#pragma unroll
      for (int mat = 0; mat < NMAT; ++mat)
        for (int grp = 0; grp < groups; ++grp, ++it) {
          const uint32_t slot = it % kStages, round = it / kStages;
          if (*abortFlag)
            continue;
          if (!mbar_wait_bounded(&ctl.full[slot], round & 1, abortFlag)) {
            *abortFlag = 1;
            atomicExch(p.status, kStatusBarrierTimeout);
            continue;
          }
          const int count = min(kStageBlocks, chunkBlocks - grp * kStageBlocks);
          if (warp < count) {
            const uint8_t* base = ring + size_t(slot) * Q::kStageBytes + warp * Q::kBlockBytes;
            const int sb = grp * kStageBlocks + warp;
            if (Q::kMinTerm) {
              const uint32_t rows = smem_u32(base);
              q4k_unit<XSPLIT>(rows + g * Q::kRowStride, rows + (g + 8) * Q::kRowStride, t, fragHiAddress + sb * 4096, fragLoAddress + sb * 4096, rotation,
                               fragSumAddress + sb * 256, total[mat]);
            } else {
#pragma unroll
              for (int half = 0; half < 2; ++half)
                q6k_unit<XSPLIT>(base + g * Q::kRowStride, base + (g + 8) * Q::kRowStride, lane, half, fragHi + sb * 512, fragLo + sb * 512,
                                 total[mat]);
            }
          }
          __syncwarp();
          if (lane == 0)
            mbar_arrive(&ctl.empty[slot]);
        }
      // Cross-warp reduction of the K split, then the epilogue.
      float* mine = partial + size_t(tileCounter & 1) * NMAT * kConsumerWarps * 128;
#pragma unroll
      for (int mat = 0; mat < NMAT; ++mat) {
        float* dst = mine + (mat * kConsumerWarps + warp) * 128;
        dst[(2 * t) * 16 + g] = total[mat][0];
        dst[(2 * t + 1) * 16 + g] = total[mat][1];
        dst[(2 * t) * 16 + g + 8] = total[mat][2];
        dst[(2 * t + 1) * 16 + g + 8] = total[mat][3];
      }
      named_barrier(1, kConsumerWarps * kWarp);
      if (tid < 128) {
        float sum[NMAT];
#pragma unroll
        for (int mat = 0; mat < NMAT; ++mat) {
          sum[mat] = 0.f;
#pragma unroll
          for (int w = 0; w < kConsumerWarps; ++w)
            sum[mat] += mine[(mat * kConsumerWarps + w) * 128 + tid];
        }
        if (destination)
          *destination = NMAT == 2 ? silu_f(sum[0]) * sum[NMAT - 1] : sum[0] + addend;
      }
    }
  }
}

template <class Q, int NMAT, int XSPLIT> cudaError_t launch(const GemvParams& p, int sms, cudaStream_t stream) {
  static PerDeviceOnce configured;
  constexpr size_t bytes = smem_bytes<Q, NMAT, XSPLIT>();
  if (cudaError_t e = configure_shared_memory(gemv_kernel<Q, NMAT, XSPLIT>, bytes, configured))
    return e;
  const int grid = p.tiles < sms ? p.tiles : sms;
  launch_kernel<1>(gemv_kernel<Q, NMAT, XSPLIT>, grid, kThreads, bytes, stream, p);
  return cudaGetLastError();
}

}  // namespace

// type: ggml type id (12 = Q4_K, 14 = Q6_K); pair: gate/up fusion (two matrices, silu(a)*b epilogue).
cudaError_t gemv_launch(int type, bool pair, int xsplit, const GemvParams& p, int sms, cudaStream_t stream) {
  if (type == 12) {
    if (pair)
      return xsplit == 2 ? launch<Q4K, 2, 2>(p, sms, stream) : launch<Q4K, 2, 1>(p, sms, stream);
    return xsplit == 2 ? launch<Q4K, 1, 2>(p, sms, stream) : launch<Q4K, 1, 1>(p, sms, stream);
  }
  if (type == 14 && !pair)
    return xsplit == 2 ? launch<Q6K, 1, 2>(p, sms, stream) : launch<Q6K, 1, 1>(p, sms, stream);
  return cudaErrorInvalidValue;
}

}  // namespace infdev
