// Integer tensor-core GEMV for decode (M <= 8 activation rows) over GGUF Q4_K weights.
//
// Replaces linear_decode_q4_k[_add] (quant_linear.metal:245-327) and mlp_gate_up_q4_k_decode
// (fused_kernels.metal:11-78) like gemv.cu, with a cheaper inner loop: the 4-bit quants feed the tensor cores
// as unsigned bytes (one AND per four weights) against activations quantised to 16-bit integers per
// (row, 256-value block) and split into a signed high and an unsigned low byte (act_image.cuh). One m16n8k32
// integer MMA covers exactly one 32-weight sub-block of 16 weight rows, so the 6-bit sub-block scale is applied
// to the int32 result with one integer multiply-add per accumulator; the super-block scale d, the activation
// scale and the -dmin * m term (one fp16 MMA against the sub-block sums) are applied once per super-block.
// The only approximation is the 16-bit activation grid: absolute error at most 1.6e-5 of the block maximum.
//
// One persistent CTA per SM: 16 consumer warps, 3 finisher warps and 1 producer warp (five warps per scheduler). The producer streams 16-row x
// 8-super-block weight slabs with one tiled TMA copy each into a shared-memory ring. A consumer warp works on the
// same super-block of every tile (warp w of a half takes super-block w of the half's slab), so it keeps the activation
// fragments of that super-block in registers for a whole K chunk, loaded straight from the image in global memory:
// shared memory is read for the weights only, which is what bounds the rate of this kernel (the activation fragments
// of a unit are 4 KB against 2.3 KB of weights). Every wait on an mbarrier is bounded and ends in an abort flag plus a
// device status code.
#include "act_image.cuh"
#include "kernels.h"

namespace infdev {
namespace {

constexpr int kConsumerWarps = 16;  // two halves of 8; consecutive ring stages alternate between the halves
constexpr int kStageWarps = 8;       // one warp per super-block of a stage
constexpr int kFinisherWarps = 3;  // each sums the consumers' partial results of every third tile and stores it
constexpr int kProducerWarp = kConsumerWarps + kFinisherWarps;  // 16 + 3 + 1 warps: five on each scheduler
constexpr int kThreads = (kProducerWarp + 1) * kWarp;
constexpr int kChunkBlocks = 16;  // super-blocks of K per pass over the tiles: two slabs, one per half
constexpr int kStageBlocks = kGemvStageBlocks;
constexpr int kTileRows = kGemvTileRows;
constexpr int kMaxStages = 12;
constexpr int kBlockBytes = 144;
constexpr int kRowPitch = kStageBlocks * kBlockBytes + kDecodePadBytes;  // 1184
constexpr int kStageBytes = kTileRows * kRowPitch;                       // 18,944
static_assert(kChunkBlocks == 2 * kStageBlocks, "a consumer warp's super-block within a chunk is fixed by its half");

struct Control {
  uint64_t full[kMaxStages], empty[kMaxStages];
  uint64_t partialReady[kFinisherWarps], partialFree[kFinisherWarps];  // per partial-sum buffer: consumers -> its finisher and back
  int abort;
};
constexpr int kControlBytes = 256;
static_assert(sizeof(Control) <= kControlBytes, "control block overlaps the partial sums");

template <int NMAT> constexpr size_t fixed_bytes() { return kControlBytes + size_t(kFinisherWarps) * NMAT * kConsumerWarps * 128 * 4; }
template <int NMAT> constexpr int stage_count() {
  int stages = int((size_t(227) * 1024 - fixed_bytes<NMAT>()) / kStageBytes);
  return stages > kMaxStages ? kMaxStages : stages;
}
template <int NMAT> constexpr size_t smem_bytes() { return fixed_bytes<NMAT>() + size_t(stage_count<NMAT>()) * kStageBytes; }

// Ordinary loads (not volatile asm): the compiler may hoist and interleave them with the MMAs, but not move them
// above the mbarrier wait, which clobbers memory.
__device__ __forceinline__ uint4 lds128(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ uint2 lds64(const uint8_t* p) { return *reinterpret_cast<const uint2*>(p); }

// D(16x8,s32) = A(16x32,u8,row) * B(32x8,s8 or u8,col)
__device__ __forceinline__ void imma_u8s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void imma_u8u8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}

// What one lane keeps of the image of one super-block (act_image.cuh) while its warp walks the tiles: lane
// (g = lane/4, t = lane%4) holds, per sub-block j, the B fragments of activation row g, quarter t: registers b0, b1 of
// the high-byte MMA in x, y and of the low-byte MMA in z, w.
struct Fragments {
  uint4 quant[8];
  uint2 sums;    // min-term fragment: fp16 pairs of S_j / 32, high halves in x, low halves in y
  uint2 scales;  // fp32 bits of the activation scales of rows 2t and 2t+1
};

__device__ __forceinline__ Fragments load_fragments(const uint8_t* block, int lane) {
  Fragments f;
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int j = 0; j < 8; ++j)
    f.quant[j] = *reinterpret_cast<const uint4*>(block + j * 512 + g * 64 + t * 16);
  f.sums = *reinterpret_cast<const uint2*>(block + kImageSumOffset + lane * 8);
  f.scales = *reinterpret_cast<const uint2*>(block + kImageScaleOffset + t * 8);
  return f;
}

// One 16-row x 256-k unit. Lane (g, t) owns weight rows g and g+8 (shared-memory addresses pA, pB) and, in each
// 32-byte quant chunk c, bytes 8t .. 8t+7: their low nibbles are values 8t .. 8t+7 of sub-block 2c, their high
// nibbles the same values of sub-block 2c+1 (GGUF layout as read by dequant_tile, quant_linear.metal:39-46). The four
// bytes of a word fill four consecutive summation slots of the MMA, which is the order the image stores the
// activations in.
__device__ __forceinline__ void q4k_unit(const uint8_t* pA, const uint8_t* pB, int t, const Fragments& f, float (&total)[4]) {
  const uint4 hA = lds128(pA), hB = lds128(pB);
  // 6-bit scales / mins of the 8 sub-blocks, four per word (scale_min_k4, quant_linear.metal:12-20).
  const uint32_t scA[2] = {hA.y & 0x3f3f3f3fu, (hA.w & 0x0f0f0f0fu) | ((hA.y >> 2) & 0x30303030u)};
  const uint32_t mnA[2] = {hA.z & 0x3f3f3f3fu, ((hA.w >> 4) & 0x0f0f0f0fu) | ((hA.z >> 2) & 0x30303030u)};
  const uint32_t scB[2] = {hB.y & 0x3f3f3f3fu, (hB.w & 0x0f0f0f0fu) | ((hB.y >> 2) & 0x30303030u)};
  const uint32_t mnB[2] = {hB.z & 0x3f3f3f3fu, ((hB.w >> 4) & 0x0f0f0f0fu) | ((hB.z >> 2) & 0x30303030u)};
  // 16 x the sum over the 8 sub-blocks of scale * (integer dot product), separately for the low and the high activation
  // byte: |low| <= 16 * 8 * 63 * 15 * 32 * 255 < 2^30 and |high| <= 16 * 8 * 63 * 15 * 32 * 128 both stay inside int32.
  int sumLow[4] = {0, 0, 0, 0}, sumHigh[4] = {0, 0, 0, 0};
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint2 qA = lds64(pA + 16 + 32 * c + 8 * t), qB = lds64(pB + 16 + 32 * c + 8 * t);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int j = 2 * c + h;
      uint32_t a[4];
      // Low nibbles as they are, high nibbles in place as 16 q (still a byte); the sub-block scale of the low ones is
      // taken 16-fold instead, and the common factor leaves with d at the end.
      const uint32_t mask = h == 0 ? 0x0f0f0f0fu : 0xf0f0f0f0u;
      a[0] = qA.x & mask, a[1] = qB.x & mask, a[2] = qA.y & mask, a[3] = qB.y & mask;
      const uint4 b = f.quant[j];
      int high[4], low[4];
      imma_u8s8(high, a, b.x, b.y);
      imma_u8u8(low, a, b.z, b.w);
      const int byteA = int(__byte_perm(scA[j >> 2], 0u, 0x4440 + (j & 3))), byteB = int(__byte_perm(scB[j >> 2], 0u, 0x4440 + (j & 3)));
      const int sA = h == 0 ? byteA * 16 : byteA, sB = h == 0 ? byteB * 16 : byteB;
      sumLow[0] += sA * low[0], sumHigh[0] += sA * high[0];
      sumLow[1] += sA * low[1], sumHigh[1] += sA * high[1];
      sumLow[2] += sB * low[2], sumHigh[2] += sB * high[2];
      sumLow[3] += sB * low[3], sumHigh[3] += sB * high[3];
    }
  }
  // min term: sum_j m_j * S_j / 32; summation slots 0..7 carry the fp16 high halves of the sums, 8..15 the low halves.
  float accm[4] = {0.f, 0.f, 0.f, 0.f};
  {
    constexpr uint32_t k1024 = 0x64006400u;
    const uint32_t wordA = (t & 2) ? mnA[1] : mnA[0], wordB = (t & 2) ? mnB[1] : mnB[0];
    const uint32_t pairA = (wordA >> ((t & 1) * 16)) & 0xffffu, pairB = (wordB >> ((t & 1) * 16)) & 0xffffu;
    uint32_t a[4];
    a[0] = a[2] = hsub2_u32(__byte_perm(pairA, 0x64u, 0x4140), k1024);
    a[1] = a[3] = hsub2_u32(__byte_perm(pairB, 0x64u, 0x4140), k1024);
    mma_16816(accm, a, f.sums.x, f.sums.y);
  }
  const float xs0 = __uint_as_float(f.scales.x), xs1 = __uint_as_float(f.scales.y);
  const float2 dA = __half22float2(*reinterpret_cast<const __half2*>(&hA.x)), dB = __half22float2(*reinterpret_cast<const __half2*>(&hB.x));
  const float mA = 32.f * dA.y, mB = 32.f * dB.y, sixteenthA = 0.0625f * dA.x, sixteenthB = 0.0625f * dB.x;
  total[0] += xs0 * (sixteenthA * fmaf(float(sumHigh[0]), 256.f, float(sumLow[0])) - mA * accm[0]);
  total[1] += xs1 * (sixteenthA * fmaf(float(sumHigh[1]), 256.f, float(sumLow[1])) - mA * accm[1]);
  total[2] += xs0 * (sixteenthB * fmaf(float(sumHigh[2]), 256.f, float(sumLow[2])) - mB * accm[2]);
  total[3] += xs1 * (sixteenthB * fmaf(float(sumHigh[3]), 256.f, float(sumLow[3])) - mB * accm[3]);
}

__device__ __forceinline__ int find_segment(const GemvParams& p, int tile) {
  int s = 0;
  while (s + 1 < p.nseg && tile >= p.seg[s + 1].tile0)
    ++s;
  return s;
}

template <int NMAT> __global__ void __launch_bounds__(kThreads, 1) q4k_decode_kernel(const __grid_constant__ GemvParams p) {
  constexpr int kStages = stage_count<NMAT>();
  extern __shared__ __align__(128) uint8_t smemRaw[];
  Control& ctl = *reinterpret_cast<Control*>(smemRaw);
  float* partial = reinterpret_cast<float*>(smemRaw + kControlBytes);
  uint8_t* ring = reinterpret_cast<uint8_t*>(partial + kFinisherWarps * NMAT * kConsumerWarps * 128);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int blocksPerRow = p.k / 256;
  const int chunks = (blocksPerRow + kChunkBlocks - 1) / kChunkBlocks;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&ctl.full[s], 1);
      mbar_init(&ctl.empty[s], kStageWarps);
    }
    for (int b = 0; b < kFinisherWarps; ++b) {
      mbar_init(&ctl.partialReady[b], kConsumerWarps);
      mbar_init(&ctl.partialFree[b], 1);
    }
    ctl.abort = 0;
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();
  volatile int* abortFlag = &ctl.abort;

  if (warp == kProducerWarp) {
    // ---- producer (one thread): weight slabs into the ring. The weights do not depend on the kernels before this
    // one, so the ring fills while they finish.
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int chunk = 0; chunk < chunks && ok; ++chunk) {
        const int chunkBlocks = min(kChunkBlocks, blocksPerRow - chunk * kChunkBlocks);
        const int groups = (chunkBlocks + kStageBlocks - 1) / kStageBlocks;
        for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x) {
          const int segment = find_segment(p, tile);
          const int row0 = (tile - p.seg[segment].tile0) * kTileRows;
          for (int mat = 0; mat < NMAT && ok; ++mat) {
            for (int grp = 0; grp < groups; ++grp, ++it) {
              const uint32_t slot = it % kStages, round = it / kStages;
              if (round > 0 && !mbar_wait_bounded(&ctl.empty[slot], (round - 1) & 1, abortFlag)) {
                *abortFlag = 1;
                atomicExch(p.status, kStatusBarrierTimeout);
                ok = false;
                break;
              }
              // One tiled copy moves the whole slab; bytes past the end of a row are zero-filled and still counted, so
              // the transaction size is always the full box.
              mbar_arrive_expect_tx(&ctl.full[slot], uint32_t(kStageBytes));
              tma_load_2d(ring + size_t(slot) * kStageBytes, &p.map[segment][mat], (chunk * (kChunkBlocks / kStageBlocks) + grp) * (kStageBlocks * kBlockBytes / 8),
                          row0, &ctl.full[slot]);
            }
          }
        }
      }
    }
    __syncwarp();
    pdl_wait();  // every thread of every kernel waits, so completion stays transitive along the stream
    return;
  }

  // The partial sums of a tile go through one of three buffers, taken in turn within a K chunk, and each buffer has
  // its own finisher warp and two mbarriers: partialReady[b] "every consumer warp has stored its partial sums" and
  // partialFree[b] "the finisher has read them", which a consumer tests before it stores into the buffer again.
  // Nobody waits for a warp of its own role, each barrier is watched phase by phase by the same warps, and a tile of
  // the result has the same finisher in every K chunk, so the sum over the earlier chunks it adds is its own store.
  if (warp >= kConsumerWarps) {
    // ---- finishers: four elements of a tile's 16 x 8 result per lane ----
    pdl_wait();
    const int buffer = warp - kConsumerWarps;
    uint32_t uses = 0;
    for (int chunk = 0; chunk < chunks; ++chunk)
      for (int tile = blockIdx.x + buffer * gridDim.x; tile < p.tiles; tile += kFinisherWarps * gridDim.x, ++uses) {
        // Lane (g = lane/4, t = lane%4) sums what the same lane of every consumer warp holds: weight rows g and g+8 for
        // activation rows 2t and 2t+1. What is added to them (the residual, or the sum over the earlier K chunks) is
        // fetched before the wait.
        const GemvSeg& seg = p.nseg == 1 ? p.seg[0] : p.seg[find_segment(p, tile)];
        const int g = lane >> 2, t = lane & 3;
        float* destination[2] = {nullptr, nullptr};  // activation rows 2t, 2t+1 at weight row g; g + 8 is 8 floats on
        float addend[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < 2; ++r)
          if (2 * t + r < p.m) {
            const size_t at = size_t(2 * t + r) * seg.ldy + size_t(tile - seg.tile0) * kTileRows + g;
            destination[r] = seg.y + at;
            if (NMAT == 1 && chunk > 0)
              addend[r] = destination[r][0], addend[2 + r] = destination[r][8];
            else if (NMAT == 1 && seg.res)
              addend[r] = seg.res[at], addend[2 + r] = seg.res[at + 8];
          }
        const float4* sums = reinterpret_cast<const float4*>(partial + size_t(buffer) * NMAT * kConsumerWarps * 128) + lane;
        if (!mbar_wait_bounded(&ctl.partialReady[buffer], uses & 1, abortFlag)) {
          *abortFlag = 1;
          atomicExch(p.status, kStatusBarrierTimeout);
          return;
        }
        float4 sum[NMAT];
#pragma unroll
        for (int mat = 0; mat < NMAT; ++mat) {
          float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;  // two chains in a fixed order: the result does not depend on timing
#pragma unroll
          for (int w = 0; w < kConsumerWarps; w += 2) {
            const float4 u = sums[(mat * kConsumerWarps + w) * 32], v = sums[(mat * kConsumerWarps + w + 1) * 32];
            a.x += u.x, a.y += u.y, a.z += u.z, a.w += u.w;
            b.x += v.x, b.y += v.y, b.z += v.z, b.w += v.w;
          }
          sum[mat] = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
        }
        __syncwarp();
        if (lane == 0)
          mbar_arrive(&ctl.partialFree[buffer]);
        const float4 first = sum[0], second = sum[NMAT - 1];
        const float lowRows[2] = {NMAT == 2 ? silu_f(first.x) * second.x : first.x + addend[0], NMAT == 2 ? silu_f(first.y) * second.y : first.y + addend[1]};
        const float highRows[2] = {NMAT == 2 ? silu_f(first.z) * second.z : first.z + addend[2], NMAT == 2 ? silu_f(first.w) * second.w : first.w + addend[3]};
#pragma unroll
        for (int r = 0; r < 2; ++r)
          if (destination[r])
            destination[r][0] = lowRows[r], destination[r][8] = highRows[r];
      }
    return;
  }

  // ---- consumers ----
  pdl_wait();  // the image comes from the kernels before this one
  const int g = lane >> 2, t = lane & 3, half = warp / kStageWarps, unit = warp % kStageWarps;
  const int laneRow = g * kRowPitch + unit * kBlockBytes;
  uint32_t it = 0, mine = half, slot = half, phase = 0;
  uint32_t bufferState = 0;  // bit b: parity of the next use of partial-sum buffer b; bit 4 + b: it has been used before
  for (int chunk = 0; chunk < chunks; ++chunk) {
    const int chunkBlocks = min(kChunkBlocks, blocksPerRow - chunk * kChunkBlocks);
    const int groups = (chunkBlocks + kStageBlocks - 1) / kStageBlocks;
    // With two slabs per tile the stages of a tile alternate between the halves (a chunk starts at an even stage,
    // only the last chunk of a row can be a single slab), with one slab every stage is slab 0: either way this warp
    // meets the same super-block in every tile of the chunk.
    const int myBlock = (groups == 2 ? half * kStageBlocks : 0) + unit;
    const bool live = myBlock < chunkBlocks;
    Fragments fragments;
    if (live)
      fragments = load_fragments(p.image + size_t(chunk * kChunkBlocks + myBlock) * kImageBlockBytes, lane);
    int buffer = 0;
    for (int tile = blockIdx.x; tile < p.tiles; tile += gridDim.x, buffer = buffer == kFinisherWarps - 1 ? 0 : buffer + 1) {
      float total[NMAT][4];
#pragma unroll
      for (int mat = 0; mat < NMAT; ++mat)
        total[mat][0] = total[mat][1] = total[mat][2] = total[mat][3] = 0.f;
      // `mine` is the next stage of this half (they are the stages congruent to `half` modulo 2), `slot` and `phase`
      // its place in the ring.
      const int perTile = NMAT * groups;
      for (; mine < it + perTile; mine += 2, slot += 2) {
        if (slot >= kStages) {
          slot -= kStages;
          phase ^= 1;
        }
        const int mat = NMAT == 2 && int(mine - it) >= groups;
        if (!mbar_wait_bounded(&ctl.full[slot], phase, abortFlag)) {  // also leaves when another role raised the abort flag
          *abortFlag = 1;
          atomicExch(p.status, kStatusBarrierTimeout);
          break;
        }
        if (live) {
          const uint8_t* rows = ring + slot * kStageBytes + laneRow;
          if (NMAT == 2 && mat)
            q4k_unit(rows, rows + 8 * kRowPitch, t, fragments, total[NMAT - 1]);
          else
            q4k_unit(rows, rows + 8 * kRowPitch, t, fragments, total[0]);
        }
        __syncwarp();
        if (lane == 0)
          mbar_arrive(&ctl.empty[slot]);
      }
      it += perTile;
      // Hand the partial sums of the K split to the buffer's finisher and go on with the next tile.
      const uint32_t parity = (bufferState >> buffer) & 1u;
      if (((bufferState >> (4 + buffer)) & 1u) && !mbar_wait_bounded(&ctl.partialFree[buffer], parity ^ 1u, abortFlag)) {
        *abortFlag = 1;
        atomicExch(p.status, kStatusBarrierTimeout);
      }
      bufferState = (bufferState ^ (1u << buffer)) | (16u << buffer);
      float* sums = partial + size_t(buffer) * NMAT * kConsumerWarps * 128;
#pragma unroll
      for (int mat = 0; mat < NMAT; ++mat) {
        reinterpret_cast<float4*>(sums + (mat * kConsumerWarps + warp) * 128)[lane] = make_float4(total[mat][0], total[mat][1], total[mat][2], total[mat][3]);
      }
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&ctl.partialReady[buffer]);
    }
  }
}

// One warp per (row, 256-value block).
__global__ void __launch_bounds__(256) activation_image_kernel(const float* x, int ldx, int m, int blocks, uint8_t* image) {
  pdl_launch_dependents();
  pdl_wait();
  const int item = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= blocks * kImageRows)
    return;
  const int block = item >> 3, row = item & 7;
  uint8_t* out = image + size_t(block) * kImageBlockBytes;
  if (row >= m) {
    image_zero_block(out, row, lane);
    return;
  }
  const float4* src = reinterpret_cast<const float4*>(x + size_t(row) * ldx + size_t(block) * 256 + lane * 8);
  const float4 lo = src[0], hi = src[1];
  const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
  image_store_block(out, row, lane, v);
}

template <int NMAT> cudaError_t launch(const GemvParams& p, int sms, cudaStream_t stream) {
  static PerDeviceOnce configured;
  constexpr size_t bytes = smem_bytes<NMAT>();
  if (cudaError_t e = configure_shared_memory(q4k_decode_kernel<NMAT>, bytes, configured))
    return e;
  const int grid = p.tiles < sms ? p.tiles : sms;
  launch_kernel<1>(q4k_decode_kernel<NMAT>, grid, kThreads, bytes, stream, p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t q4k_decode_launch(bool pair, const GemvParams& p, int sms, cudaStream_t stream) {
  return pair ? launch<2>(p, sms, stream) : launch<1>(p, sms, stream);
}

cudaError_t activation_image_launch(const float* x, int ldx, int m, int k, uint8_t* image, cudaStream_t stream) {
  const int blocks = k / 256;
  launch_kernel<2>(activation_image_kernel, (blocks * kImageRows + 7) / 8, 256, 0, stream, x, ldx, m, blocks, image);
  return cudaGetLastError();
}

}  // namespace infdev
