// Q4_K linear on the 5th-generation tensor cores (tcgen05) with TMEM operands.
//
// Replaces, for weight matrices whose row count is a multiple of 128 and whose K is a multiple of 2048, the
// decode GEMVs linear_decode_q4_k[_add] (quant_linear.metal:245-327) and mlp_gate_up_q4_k_decode
// (fused_kernels.metal:11-78). The mma.sync kernel in gemv.cu is bound by its instruction count (fragment
// loads, HMMA issue, per-lane scale selection, cross-warp reduction); here
//   * one thread owns one weight row: it reads the row's 144-byte super-block from a TMA-filled slab,
//     builds the exact integers sc*q as fp16 pairs (one LOP3 + one HFMA2 per two weights, scales held as
//     per-thread scalars) and writes them to tensor memory with tcgen05.st;
//   * tcgen05.mma (kind::f16, M = 128 weight rows, N = 16 activation columns, K = 16) takes A from TMEM and
//     B, the activations, from shared memory through a matrix descriptor. The activations were split
//     hi + lo into fp16 beforehand (umma_prepare_kernel), already laid out as canonical no-swizzle K-major
//     core matrices under the same K permutation that the nibble extraction produces;
//   * every super-block accumulates into its own 16 TMEM columns, so the epilogue applies the fp32
//     super-block scale d exactly: y = sum_sb d_sb * D_sb - dmin_sb * sum_j m_j * xsum_j, the latter added up
//     on the CUDA cores by the row's thread;
//   * accumulators are double-buffered per 8-super-block chunk, so the epilogue of one chunk overlaps the
//     MMAs of the next.
// Warp roles: 0 = TMA producer, 1 = MMA issuer (owns the TMEM allocation), 4..11 = dequant (two groups of
// four, one TMEM lane quadrant each), 12..15 = epilogue. Every mbarrier wait is bounded; on a timeout the
// kernel raises an abort flag, records a status code, and every role leaves its loops.
#include "common.cuh"
#include "kernels.h"

namespace infdev {
namespace {

constexpr int kRows = kUmmaTileRows;  // weight rows per tile = TMEM lanes
constexpr int kChunkSb = 8;           // super-blocks per accumulator buffer (decode mode)
constexpr int kSlabBytes = kRows * 144;  // 18,432
constexpr int kThreads = 512;
// Two modes, selected by the MMA N dimension:
//  NACT = 16  decode: up to 8 activation rows; columns 0..7 carry their fp16 hi halves, columns 8..15 the lo halves, so
//             one MMA per k-step yields both products. A holds the exact integers sc*q; one accumulator per super-block.
//  NACT = 128 prefill: up to 128 activation rows in fp16 (hi only); A holds the dequantised weight d*sc*q - dmin*m
//             rounded to fp16, one accumulator per tile (the GEMM of linear_prefill, quant_linear.metal:151-233).
// Shared-memory rings. Decode: 7 stages of one weight slab + its activations (26,624 bytes). Prefill: the fp16
// activations of a super-block are 64 KB, so slab and activations travel separately and the activations in two halves
// of eight k-steps each: 3 slab stages + 5 half stages keep two and a half super-blocks in flight (with whole
// super-blocks as stages only two fit, and every dequantisation group then waited out a full TMA latency per block).
template <int NACT> struct Mode {
  static constexpr int kActBytesPerSb = 16 * NACT * 16 * 2;             // 16 k-steps x [NACT x 16] fp16
  static constexpr int kStageBytes = NACT == 16 ? kSlabBytes + kActBytesPerSb : kSlabBytes;  // 26,624 / 18,432
  static constexpr int kStages = NACT == 16 ? 7 : 3;
  static constexpr int kActStages = 5, kActHalfBytes = kActBytesPerSb / 2;  // prefill only
  static constexpr uint32_t kInstruction = (1u << 4) | (uint32_t(NACT >> 3) << 17) | (uint32_t(kRows >> 4) << 24);
};
constexpr int kTmemCols = 512;
constexpr uint32_t kColA = 0, kColD = 256;  // A: 2 x 128 columns; D: 2 x (8 super-blocks x 16 columns)

struct Control {
  uint64_t full[8], slotFree[8], actFull[8], actFree[8], aReady[2], aFree[2], dReady[2], dFree[2];
  uint32_t tmemBase;
  int abort;
};
constexpr int kControlBytes = 512;
static_assert(sizeof(Control) <= kControlBytes, "control block too large");
constexpr int kScaleBytes = 2 * kChunkSb * kRows * 4;  // d of every (buffer, super-block, row): 8,192
constexpr int kMinBytes = 2 * 2 * kRows * 8 * 4;       // min-term partials [buffer][group][row][8]: 16,384
template <int NACT> constexpr size_t smem_bytes() {  // the scale / min tables belong to decode mode
  return NACT == 16 ? 1024 + kControlBytes + kScaleBytes + kMinBytes + size_t(Mode<NACT>::kStages) * Mode<NACT>::kStageBytes
                    : 1024 + kControlBytes + size_t(Mode<NACT>::kStages) * Mode<NACT>::kStageBytes +
                          size_t(Mode<NACT>::kActStages) * Mode<NACT>::kActHalfBytes;
}

__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[128 x N] (+)= A[128 x 16] (TMEM) * B[16 x N] (shared memory descriptor)
__device__ __forceinline__ void umma_ts(uint32_t d, uint32_t a, uint64_t bDesc, uint32_t iDesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(d),
      "r"(a), "l"(bDesc), "r"(iDesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// 32 lanes x 32 consecutive columns, one 32-bit value per (lane, column)
__device__ __forceinline__ void tmem_store32(uint32_t address, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"
      "%28,%29,%30,%31,%32};" ::"r"(address),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]),
      "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]),
      "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_load8(uint32_t address, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(address)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i)
    v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major, no-swizzle operand: 8-row x 16-byte core matrices, the two K halves
// `leading` bytes apart, successive 8-row groups `stride` bytes apart (descriptor version 1 = Blackwell).
__device__ __forceinline__ uint64_t smem_descriptor(uint32_t address, uint32_t leading, uint32_t stride) {
  return uint64_t((address & 0x3FFFFu) >> 4) | (uint64_t(leading >> 4) << 16) | (uint64_t(stride >> 4) << 32) | (uint64_t(1) << 46);
}

// (Mode<NACT>::kInstruction is the kind::f16 instruction descriptor: fp32 accumulate, fp16 A and B, both K-major, M = 128.)

template <int NMAT, int NACT> __global__ void __launch_bounds__(kThreads, 1) umma_linear_kernel(const __grid_constant__ UmmaParams p) {
  using M = Mode<NACT>;
  constexpr bool kDecode = NACT == 16;
  constexpr int kStages = M::kStages, kStageBytes = M::kStageBytes;
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
  Control& ctl = *reinterpret_cast<Control*>(smem);
  float* dScale = reinterpret_cast<float*>(smem + kControlBytes);                 // [2][8][128], decode mode
  float* minPart = reinterpret_cast<float*>(smem + kControlBytes + kScaleBytes);  // [2][2][128][8], decode mode
  uint8_t* ring = smem + kControlBytes + (kDecode ? kScaleBytes + kMinBytes : 0);
  uint8_t* actRing = ring + size_t(kStages) * kStageBytes;  // prefill mode: halves of a super-block's activations

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // With p.splits > 1 (prefill mode, one matrix) the work items are (tile, K slice) pairs, so that a matrix of few
  // 128-row tiles still fills the GPU; `blocksPerRow` is then the super-blocks of one slice.
  const int blocksPerRow = p.k / 256 / p.splits, items = p.tiles * p.splits;
  // A "unit" owns one accumulator buffer: 8 super-blocks in decode mode, a whole (tile, matrix) in prefill mode.
  const int unitsPerMat = kDecode ? blocksPerRow / kChunkSb : 1, blocksPerUnit = kDecode ? kChunkSb : blocksPerRow;
  volatile int* abortFlag = &ctl.abort;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&ctl.full[s], 1);
      mbar_init(&ctl.slotFree[s], kDecode ? 5 : 4);  // four dequant warps (+ the MMA commit where the stage holds activations)
    }
    for (int s = 0; s < M::kActStages; ++s) {
      mbar_init(&ctl.actFull[s], 1);
      mbar_init(&ctl.actFree[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&ctl.aReady[b], 4);
      mbar_init(&ctl.aFree[b], 1);
      mbar_init(&ctl.dReady[b], 1);
      mbar_init(&ctl.dFree[b], 4);
    }
    ctl.abort = 0;
    mbar_fence_init();
  }
  if (warp == 1)
    tmem_alloc(&ctl.tmemBase, kTmemCols);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = ctl.tmemBase;

  if (warp == 0) {
    // ---------------- producer: one weight slab + its activation fragments per super-block ----------------
    uint32_t it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const int tile = item % p.tiles, firstBlock = (item / p.tiles) * blocksPerRow;
      int segment = 0;
      while (segment + 1 < p.nseg && tile >= p.seg[segment + 1].tile0)
        ++segment;
      const int row0 = (tile - p.seg[segment].tile0) * kRows;
      for (int mat = 0; mat < NMAT && ok; ++mat)
        for (int sb = firstBlock; sb < firstBlock + blocksPerRow && ok; ++sb, ++it) {
          const uint32_t slot = it % kStages, round = it / kStages;
          if (lane == 0) {
            if (round > 0)
              ok = mbar_wait_bounded(&ctl.slotFree[slot], (round - 1) & 1, abortFlag);
            if (ok) {
              uint8_t* stage = ring + size_t(slot) * kStageBytes;
              mbar_arrive_expect_tx(&ctl.full[slot], kStageBytes);
              tma_load_2d(stage, &p.map[segment][mat], sb * 18, row0, &ctl.full[slot]);
              if (kDecode)
                bulk_load(stage + kSlabBytes, p.acts + size_t(sb) * M::kActBytesPerSb, M::kActBytesPerSb, &ctl.full[slot]);
            }
            for (int h = 0; h < 2 && ok && !kDecode; ++h) {  // the two activation halves of this super-block
              const uint32_t half = 2 * it + h, actSlot = half % M::kActStages, actRound = half / M::kActStages;
              if (actRound > 0)
                ok = mbar_wait_bounded(&ctl.actFree[actSlot], (actRound - 1) & 1, abortFlag);
              if (ok) {
                mbar_arrive_expect_tx(&ctl.actFull[actSlot], M::kActHalfBytes);
                bulk_load(actRing + size_t(actSlot) * M::kActHalfBytes, p.acts + size_t(sb) * M::kActBytesPerSb + size_t(h) * M::kActHalfBytes,
                          M::kActHalfBytes, &ctl.actFull[actSlot]);
              }
            }
            if (!ok) {
              *abortFlag = 1;
              atomicExch(p.status, kStatusBarrierTimeout);
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
        }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (lane 0) ----------------
    if (lane == 0) {
      uint32_t it = 0, unit = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x)
        for (int mat = 0; mat < NMAT && ok; ++mat)
          for (int chunk = 0; chunk < unitsPerMat && ok; ++chunk, ++unit) {
            const uint32_t buffer = unit & 1;
            if (unit >= 2)
              ok = mbar_wait_bounded(&ctl.dFree[buffer], ((unit >> 1) - 1) & 1, abortFlag);
            for (int j = 0; j < blocksPerUnit && ok; ++j, ++it) {
              const uint32_t slot = it % kStages, aBuffer = it & 1;
              ok = mbar_wait_bounded(&ctl.aReady[aBuffer], (it >> 1) & 1, abortFlag);
              if (!ok)
                break;
              fence_after_sync();
              // decode: 16 columns per super-block; prefill: one 128-column accumulator per unit
              const uint32_t dColumn = tmem + kColD + buffer * 128 + (kDecode ? j * 16 : 0);
              if (kDecode) {
                const uint32_t actBase = smem_u32(ring + size_t(slot) * kStageBytes + kSlabBytes);
#pragma unroll
                for (int step = 0; step < 16; ++step)
                  umma_ts(dColumn, tmem + kColA + aBuffer * 128 + step * 8, smem_descriptor(actBase + step * (NACT * 32), 128, 256), M::kInstruction,
                            step != 0);
                umma_commit(&ctl.aFree[aBuffer]);
                umma_commit(&ctl.slotFree[slot]);
              } else {
                for (int h = 0; h < 2 && ok; ++h) {  // eight k-steps per activation half
                  const uint32_t half = 2 * it + h, actSlot = half % M::kActStages;
                  ok = mbar_wait_bounded(&ctl.actFull[actSlot], (half / M::kActStages) & 1, abortFlag);
                  if (!ok)
                    break;
                  fence_after_sync();
                  const uint32_t actBase = smem_u32(actRing + size_t(actSlot) * M::kActHalfBytes);
#pragma unroll
                  for (int step = 0; step < 8; ++step)
                    umma_ts(dColumn, tmem + kColA + aBuffer * 128 + (8 * h + step) * 8, smem_descriptor(actBase + step * (NACT * 32), 128, 256),
                              M::kInstruction, (j | h | step) != 0);
                  umma_commit(&ctl.actFree[actSlot]);
                }
                if (!ok)
                  break;
                umma_commit(&ctl.aFree[aBuffer]);
              }
              if (j == blocksPerUnit - 1)
                umma_commit(&ctl.dReady[buffer]);
            }
          }
      if (!ok) {
        *abortFlag = 1;
        atomicExch(p.status, kStatusBarrierTimeout);
      }
    }
  }
  else if (warp >= 4 && warp < 12) {
    // ---------------- dequant: thread = weight row; group g takes the super-blocks with (index & 1) == g ----------------
    const int group = (warp - 4) >> 2, quadrant = warp & 3, row = quadrant * 32 + lane;
    constexpr uint32_t k1024 = 0x64006400u, kNeg1024 = 0xE400E400u, kSixteenth = 0x2C002C00u, kNeg64 = 0xD400D400u;
    uint32_t it = 0, unit = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < items && ok; item += gridDim.x)
      for (int mat = 0; mat < NMAT && ok; ++mat)
        for (int chunk = 0; chunk < unitsPerMat && ok; ++chunk, ++unit) {
          const uint32_t buffer = unit & 1;
          // decode: the epilogue of the unit that last used this accumulator buffer also read its scale / min tables
          if (kDecode && unit >= 2)
            ok = mbar_wait_bounded(&ctl.dFree[buffer], ((unit >> 1) - 1) & 1, abortFlag);
          float minAcc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          for (int j = 0; j < blocksPerUnit && ok; ++j, ++it) {
            if ((it & 1) != uint32_t(group))
              continue;
            const uint32_t slot = it % kStages, round = it / kStages;
            ok = mbar_wait_bounded(&ctl.full[slot], round & 1, abortFlag);
            if (ok && it >= 2)
              ok = mbar_wait_bounded(&ctl.aFree[it & 1], ((it >> 1) - 1) & 1, abortFlag);
            if (!ok)
              break;
            fence_after_sync();
            const uint8_t* block = ring + size_t(slot) * kStageBytes + row * 144;
            const uint4 header = *reinterpret_cast<const uint4*>(block);
            const float2 dm = __half22float2(*reinterpret_cast<const __half2*>(&header.x));
            // 6-bit scales / mins, four per word (scale_min_k4, quant_linear.metal:12-20)
            const uint32_t scales[2] = {header.y & 0x3f3f3f3fu, (header.w & 0x0f0f0f0fu) | ((header.y >> 2) & 0x30303030u)};
            const uint32_t mins[2] = {header.z & 0x3f3f3f3fu, ((header.w >> 4) & 0x0f0f0f0fu) | ((header.z >> 2) & 0x30303030u)};
            if (kDecode) {
              dScale[(buffer * kChunkSb + j) * kRows + row] = dm.x;
              // min term: dmin * sum_sub m_sub * (sum of the 32 activations of the sub-block), for 8 activation rows
              const float* sums = p.actSums + size_t(chunk * kChunkSb + j) * 64;  // [8 sub-blocks][8 rows]
#pragma unroll
              for (int sub = 0; sub < 8; ++sub) {
                const float m = dm.y * float((mins[sub >> 2] >> (8 * (sub & 3))) & 0xffu);
                const float4 lo = __ldg(reinterpret_cast<const float4*>(sums + sub * 8)), hi = __ldg(reinterpret_cast<const float4*>(sums + sub * 8 + 4));
                minAcc[0] = fmaf(m, lo.x, minAcc[0]), minAcc[1] = fmaf(m, lo.y, minAcc[1]), minAcc[2] = fmaf(m, lo.z, minAcc[2]);
                minAcc[3] = fmaf(m, lo.w, minAcc[3]), minAcc[4] = fmaf(m, hi.x, minAcc[4]), minAcc[5] = fmaf(m, hi.y, minAcc[5]);
                minAcc[6] = fmaf(m, hi.z, minAcc[6]), minAcc[7] = fmaf(m, hi.w, minAcc[7]);
              }
              float4* mine = reinterpret_cast<float4*>(minPart + ((buffer * 2 + group) * kRows + row) * 8);
              mine[0] = make_float4(minAcc[0], minAcc[1], minAcc[2], minAcc[3]);  // running total: final after the group's last super-block
              mine[1] = make_float4(minAcc[4], minAcc[5], minAcc[6], minAcc[7]);
            }
            const uint32_t aAddress = tmem + (uint32_t(quadrant * 32) << 16) + kColA + (it & 1) * 128;
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                // 32 quant bytes: low nibbles belong to sub-block 2t, high nibbles to sub-block 2t+1
                const uint32_t pair = (scales[t >> 1] >> (16 * (t & 1))) & 0xffffu;
                const uint4 q0 = *reinterpret_cast<const uint4*>(block + 16 + 32 * t), q1 = *reinterpret_cast<const uint4*>(block + 32 + 32 * t);
                const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                uint32_t v[32];
                if (kDecode) {
                  const uint32_t sL = hsub2_u32(__byte_perm(pair, 0x64u, 0x4040), k1024), sH = hsub2_u32(__byte_perm(pair, 0x64u, 0x4141), k1024);
                  const uint32_t nL = hmul2_u32(sL, kNeg1024), mH = hmul2_u32(sH, kSixteenth), nH = hmul2_u32(sH, kNeg64);
#pragma unroll
                  for (int w = 0; w < 8; ++w) {
                    const uint32_t a = words[w], b = a >> 8;
                    v[2 * w] = hfma2_u32((a & 0x000f000fu) | k1024, sL, nL);           // (1024 + q) * sc - 1024 sc: bytes 0, 2, low nibble
                    v[2 * w + 1] = hfma2_u32((b & 0x000f000fu) | k1024, sL, nL);       // bytes 1, 3, low nibble
                    v[16 + 2 * w] = hfma2_u32((a & 0x00f000f0u) | k1024, mH, nH);      // (1024 + 16 q) * sc/16 - 64 sc: bytes 0, 2, high nibble
                    v[16 + 2 * w + 1] = hfma2_u32((b & 0x00f000f0u) | k1024, mH, nH);  // bytes 1, 3, high nibble
                  }
                } else {
                  // dequantised weight d*sc*q - dmin*m, in fp16: q is made exact first, then one fused multiply-add
                  const uint32_t minPair = (mins[t >> 1] >> (16 * (t & 1))) & 0xffffu;
                  const uint32_t sL = pack_half2(dm.x * float(pair & 0xffu), dm.x * float(pair & 0xffu));
                  const uint32_t sH = pack_half2(dm.x * float(pair >> 8), dm.x * float(pair >> 8));
                  const uint32_t nL = pack_half2(-dm.y * float(minPair & 0xffu), -dm.y * float(minPair & 0xffu));
                  const uint32_t nH = pack_half2(-dm.y * float(minPair >> 8), -dm.y * float(minPair >> 8));
#pragma unroll
                  for (int w = 0; w < 8; ++w) {
                    const uint32_t a = words[w];
                    v[2 * w] = hfma2_u32(hsub2_u32((a & 0x000f000fu) | k1024, k1024), sL, nL);
                    v[2 * w + 1] = hfma2_u32(hsub2_u32(((a >> 8) & 0x000f000fu) | k1024, k1024), sL, nL);
                    v[16 + 2 * w] = hfma2_u32(hsub2_u32(((a >> 4) & 0x000f000fu) | k1024, k1024), sH, nH);
                    v[16 + 2 * w + 1] = hfma2_u32(hsub2_u32(((a >> 12) & 0x000f000fu) | k1024, k1024), sH, nH);
                  }
                }
                tmem_store32(aAddress + 32 * t, v);
              }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            fence_before_sync();
            __syncwarp();
            if (lane == 0) {
              mbar_arrive(&ctl.aReady[it & 1]);
              mbar_arrive(&ctl.slotFree[slot]);
            }
          }
        }
    if (!ok && lane == 0) {
      *abortFlag = 1;
      atomicExch(p.status, kStatusBarrierTimeout);
    }
  }
  else if (warp >= 12) {
    // ---------------- epilogue: thread = weight row ----------------
    const int quadrant = warp & 3, row = quadrant * 32 + lane;
    const uint32_t laneBase = tmem + (uint32_t(quadrant * 32) << 16) + kColD;
    uint32_t unit = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const int tile = item % p.tiles, slice = item / p.tiles;
      int segment = 0;
      while (segment + 1 < p.nseg && tile >= p.seg[segment + 1].tile0)
        ++segment;
      const GemvSeg& seg = p.seg[segment];
      const size_t column = size_t(tile - seg.tile0) * kRows + row;
      if (kDecode) {
        float total[NMAT][8];
#pragma unroll
        for (int mat = 0; mat < NMAT; ++mat) {
#pragma unroll
          for (int m = 0; m < 8; ++m)
            total[mat][m] = 0.f;
          for (int chunk = 0; chunk < unitsPerMat && ok; ++chunk, ++unit) {
            const uint32_t buffer = unit & 1;
            ok = mbar_wait_bounded(&ctl.dReady[buffer], (unit >> 1) & 1, abortFlag);
            if (!ok)
              break;
            fence_after_sync();
#pragma unroll
            for (int j = 0; j < kChunkSb; ++j) {
              float hi[8], lo[8];
              tmem_load8(laneBase + buffer * 128 + j * 16, hi);
              tmem_load8(laneBase + buffer * 128 + j * 16 + 8, lo);
              const float d = dScale[(buffer * kChunkSb + j) * kRows + row];
#pragma unroll
              for (int m = 0; m < 8; ++m)
                total[mat][m] = fmaf(d, hi[m] + lo[m], total[mat][m]);
            }
#pragma unroll
            for (int g = 0; g < 2; ++g) {
              const float4* part = reinterpret_cast<const float4*>(minPart + ((buffer * 2 + g) * kRows + row) * 8);
              const float4 a = part[0], b = part[1];
              total[mat][0] -= a.x, total[mat][1] -= a.y, total[mat][2] -= a.z, total[mat][3] -= a.w;
              total[mat][4] -= b.x, total[mat][5] -= b.y, total[mat][6] -= b.z, total[mat][7] -= b.w;
            }
            fence_before_sync();
            __syncwarp();
            if (lane == 0)
              mbar_arrive(&ctl.dFree[buffer]);
          }
        }
        if (!ok)
          break;
#pragma unroll
        for (int m = 0; m < 8; ++m)
          if (m < p.m) {
            const size_t at = size_t(m) * seg.ldy + column;
            float value = NMAT == 2 ? silu_f(total[0][m]) * total[NMAT - 1][m] : total[0][m];
            if (NMAT == 1 && seg.res)
              value += seg.res[at];
            seg.y[at] = value;
          }
      } else {
        for (int mat = 0; mat < NMAT && ok; ++mat, ++unit) {
          const uint32_t buffer = unit & 1;
          ok = mbar_wait_bounded(&ctl.dReady[buffer], (unit >> 1) & 1, abortFlag);
          if (!ok)
            break;
          fence_after_sync();
          for (int c = 0; c < NACT / 8; ++c) {
            float v[8];
            tmem_load8(laneBase + buffer * 128 + c * 8, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int m = c * 8 + i;
              if (m < p.m) {
                const size_t at = size_t(m) * seg.ldy + column;
                float value = v[i];
                if (NMAT == 1 && p.splits > 1) {  // a K slice: the partial sums are added up, with the residual, by umma_reduce_kernel
                  p.partial[(size_t(slice) * p.m + m) * seg.ldy + column] = value;
                  continue;
                }
                if (NMAT == 2)  // the gate half parks in y until the up half arrives (post == 2 epilogue, quant_linear.metal:224-232)
                  value = mat == 0 ? value : silu_f(seg.y[at]) * value;
                else if (seg.res)
                  value += seg.res[at];
                seg.y[at] = value;
              }
            }
          }
          fence_before_sync();
          __syncwarp();
          if (lane == 0)
            mbar_arrive(&ctl.dFree[buffer]);
        }
      }
    }
    if (!ok && lane == 0) {
      *abortFlag = 1;
      atomicExch(p.status, kStatusBarrierTimeout);
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1)
    tmem_dealloc(tmem, kTmemCols);
}

// Lays the activations out as the B operand, per 256-wide super-block: [16 k-steps][NACT/8 row groups][2 K halves][8 rows]
// [8 values] fp16. K inside a step follows the order in which the dequantiser emits weights: step s covers quant bytes of
// 64-group t = s / 4, nibble side (s / 2) % 2, words 4 * (s % 2) .. +3; TMEM column c of a step holds the nibbles of bytes
// (c % 2, c % 2 + 2) of word c / 2. Decode mode (NACT = 16): rows 0..7 are the fp16 hi halves of up to 8 activation rows,
// rows 8..15 their lo halves (x - hi), and the per-sub-block sums [super-block][8 sub-blocks][8 rows] for the min term
// are written too. Prefill mode (NACT = 128): rows are up to 128 activation rows rounded to fp16.
// grid = k / 256 super-blocks, 256 threads.
template <int NACT> __global__ void __launch_bounds__(256) umma_prepare_kernel(const float* x, int ldx, int m, __half* acts, float* sums) {
  const int sb = blockIdx.x, tid = threadIdx.x;
  const int step = tid >> 4, kk = tid & 15;  // this thread's (k-step, position inside the step)
  const int t = step >> 2, side = (step >> 1) & 1, half = step & 1, c = kk >> 1, upper = kk & 1;
  const int word = 4 * half + (c >> 1), byte = (c & 1) + 2 * upper;
  const int element = 64 * t + 32 * side + 4 * word + byte;
  __half* out = acts + size_t(sb) * (Mode<NACT>::kActBytesPerSb / 2) + size_t(step) * (NACT * 16);
  const int inner = (kk >> 3) * 64 + (kk & 7);  // K half, then position inside the 16-byte core-matrix row
  if (NACT == 16) {
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const float v = n < m ? x[size_t(n) * ldx + size_t(sb) * 256 + element] : 0.f;
      const __half hi = __float2half_rn(v), lo = __float2half_rn(v - __half2float(hi));
      out[inner + n * 8] = hi;         // row group 0
      out[128 + inner + n * 8] = lo;   // row group 1
    }
    if (tid < 64) {
      const int sub = tid >> 3, n = tid & 7;
      float s = 0.f;
      if (n < m)
        for (int e = 0; e < 32; ++e)
          s += x[size_t(n) * ldx + size_t(sb) * 256 + sub * 32 + e];
      sums[size_t(sb) * 64 + tid] = s;
    }
  } else {
    for (int n = 0; n < NACT; ++n) {
      const float v = n < m ? x[size_t(n) * ldx + size_t(sb) * 256 + element] : 0.f;
      out[(n >> 3) * 128 + inner + (n & 7) * 8] = __float2half_rn(v);
    }
  }
}

// Prefill-mode form of the same layout, vectorised: eight consecutive k of a super-block are one 16-byte core-matrix
// row of a k-step (in the order 0,2,1,3,4,6,5,7), so a thread turns two float4 loads into one 16-byte store.
// grid (k / 256, 4), 256 threads: 128 rows x 32 groups of eight per super-block, four items per thread; a warp reads one
// activation row's 256 values at a time.
__global__ void __launch_bounds__(256) umma_prepare_rows_kernel(const float* x, int ldx, int m, __half* acts) {
  constexpr int kRowsB = 128;
  const int sb = blockIdx.x;
  __half* out = acts + size_t(sb) * (Mode<kRowsB>::kActBytesPerSb / 2);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int item = (blockIdx.y * 4 + j) * 256 + threadIdx.x, n = item >> 5, group = item & 31;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
    if (n < m) {
      const float4* src = reinterpret_cast<const float4*>(x + size_t(n) * ldx + size_t(sb) * 256 + group * 8);
      a = src[0], b = src[1];
    }
    const __half2 h0 = __floats2half2_rn(a.x, a.z), h1 = __floats2half2_rn(a.y, a.w), h2 = __floats2half2_rn(b.x, b.z), h3 = __floats2half2_rn(b.y, b.w);
    uint4 packed;
    packed.x = *reinterpret_cast<const uint32_t*>(&h0), packed.y = *reinterpret_cast<const uint32_t*>(&h1);
    packed.z = *reinterpret_cast<const uint32_t*>(&h2), packed.w = *reinterpret_cast<const uint32_t*>(&h3);
    *reinterpret_cast<uint4*>(out + size_t(group >> 1) * (kRowsB * 16) + (n >> 3) * 128 + (group & 1) * 64 + (n & 7) * 8) = packed;
  }
}

// y = partial[0] + partial[1] + ... (+ residual), four values per thread.
__global__ void __launch_bounds__(256) umma_reduce_kernel(const float* partial, int splits, size_t count, const float* residual, float* y) {
  const size_t at = (size_t(blockIdx.x) * 256 + threadIdx.x) * 4;
  if (at >= count)
    return;
  float4 sum = *reinterpret_cast<const float4*>(partial + at);
  for (int s = 1; s < splits; ++s) {
    const float4 v = *reinterpret_cast<const float4*>(partial + s * count + at);
    sum.x += v.x, sum.y += v.y, sum.z += v.z, sum.w += v.w;
  }
  if (residual) {
    const float4 v = *reinterpret_cast<const float4*>(residual + at);
    sum.x += v.x, sum.y += v.y, sum.z += v.z, sum.w += v.w;
  }
  *reinterpret_cast<float4*>(y + at) = sum;
}

template <int NMAT, int NACT> cudaError_t launch_mode(const UmmaParams& p, const float* x, int ldx, int sms, cudaStream_t stream) {
  static PerDeviceOnce configured;
  constexpr size_t bytes = smem_bytes<NACT>();
  if (const cudaError_t e = configure_shared_memory(umma_linear_kernel<NMAT, NACT>, bytes, configured))
    return e;
  {
    if (NACT == 128 && ldx % 4 == 0)
      umma_prepare_rows_kernel<<<dim3(p.k / 256, 4), 256, 0, stream>>>(x, ldx, p.m, reinterpret_cast<__half*>(const_cast<uint8_t*>(p.acts)));
    else
      umma_prepare_kernel<NACT><<<p.k / 256, 256, 0, stream>>>(x, ldx, p.m, reinterpret_cast<__half*>(const_cast<uint8_t*>(p.acts)),
                                                                const_cast<float*>(p.actSums));
  }
  const int items = p.tiles * p.splits, grid = items < sms ? items : sms;
  umma_linear_kernel<NMAT, NACT><<<grid, kThreads, bytes, stream>>>(p);
  if (p.splits > 1) {
    const size_t count = size_t(p.m) * p.seg[0].ldy;
    umma_reduce_kernel<<<unsigned((count / 4 + 255) / 256), 256, 0, stream>>>(p.partial, p.splits, count, p.seg[0].res, p.seg[0].y);
  }
  return cudaGetLastError();
}

}  // namespace

// p.m <= 8 runs the exact decode mode, p.m <= 128 the fp16-weight prefill mode.
cudaError_t umma_launch(bool pair, const UmmaParams& p, const float* x, int ldx, int sms, cudaStream_t stream) {
  if (p.m <= 8)
    return pair ? launch_mode<2, 16>(p, x, ldx, sms, stream) : launch_mode<1, 16>(p, x, ldx, sms, stream);
  return pair ? launch_mode<2, 128>(p, x, ldx, sms, stream) : launch_mode<1, 128>(p, x, ldx, sms, stream);
}

}  // namespace infdev
