// Q4_K prefill GEMM on the 5th-generation tensor cores (tcgen05) with the weight operand in tensor memory.
//
// Replaces linear_prefill / linear_prefill_small (quant_linear.metal:151-233, epilogues 0 / 1 / 2) for weight matrices
// whose row count is a multiple of 128 and whose K is a multiple of 2048, for 9 to 128 activation rows per launch:
//   * one thread owns one weight row of a 128-row tile: it reads the row's 144-byte super-block from a TMA-filled slab,
//     dequantises it to fp16 (d*sc*q - dmin*m, q made exact first, then one fused multiply-add per two weights) and
//     writes it to tensor memory with tcgen05.st;
//   * tcgen05.mma (kind::f16, M = 128 weight rows, N = 128 activation rows, K = 16) takes A from TMEM and B, the
//     activations, from shared memory through a matrix descriptor. The activations were rounded to fp16 beforehand
//     (umma_prepare_rows_kernel), already laid out as canonical no-swizzle K-major core matrices under the same K
//     permutation that the nibble extraction produces;
//   * one 128-column fp32 accumulator per (tile, matrix), double-buffered, so the epilogue of one overlaps the MMAs of
//     the next.
// Warp roles: 0 = TMA producer, 1 = MMA issuer (owns the TMEM allocation), 4..11 = dequant (two groups of four, one
// TMEM lane quadrant each), 12..15 = epilogue. Every mbarrier wait is bounded; on a timeout the kernel raises an abort
// flag, records a status code, and every role leaves its loops.
// The fp16 activations of a super-block are 64 KB, so weight slabs and activations travel through separate rings, the
// activations in two halves of eight k-steps each: 3 slab stages + 5 half stages keep two and a half super-blocks in
// flight. The producer warp first asks the L2 for the whole tile (and the next one of this CTA) with bulk prefetches,
// which need no shared memory, so that three 18 KB slab copies in flight are enough.
// The kernel is launched programmatically dependent on the kernel that lays out the activations: set-up, the
// prefetches and the first weight slab run while that one is still at work, and only the activation copies and the
// epilogue wait for it.
// Measured at 12288 x 4096 x 128 rows: 1.18 us per super-block (the 16 MMAs of a super-block keep the tensor pipe busy
// for about two thirds of that), 31 us per call of which 4 us are the layout kernel; 96 tiles occupy 96 of 148 SMs.
#include "common.cuh"
#include "kernels.h"

namespace infdev {
namespace {

constexpr int kRows = kUmmaTileRows;      // weight rows per tile = TMEM lanes
constexpr int kActs = 128;                // most activation rows per launch; the MMA N is the live rows rounded up to 16
constexpr int kSlabBytes = kRows * 144;   // 18,432
constexpr int kThreads = 512;
constexpr int kStages = 3, kActStages = 5;
constexpr int kActHalfBytes = 8 * kActs * 16 * 2;  // ring stage: 8 k-steps x [128 x 16] fp16; a launch of N rows uses N x 256 of it
// kind::f16 instruction descriptor: fp32 accumulate, fp16 A and B, both K-major, M = 128
__device__ __forceinline__ uint32_t instruction_descriptor(int n) { return (1u << 4) | (uint32_t(n >> 3) << 17) | (uint32_t(kRows >> 4) << 24); }
constexpr int kTmemCols = 512;
constexpr uint32_t kColA = 0, kColD = 256;  // A: 2 x 128 columns; D: 2 x 128 columns

struct Control {
  uint64_t full[8], slotFree[8], actFull[8], actFree[8], aReady[2], aFree[2], dReady[2], dFree[2];
  uint32_t tmemBase;
  int abort;
};
constexpr int kControlBytes = 512;
static_assert(sizeof(Control) <= kControlBytes, "control block too large");
constexpr size_t kSharedBytes = 1024 + kControlBytes + size_t(kStages) * kSlabBytes + size_t(kActStages) * kActHalfBytes;

__device__ __forceinline__ void prefetch_l2(const void* address, uint32_t bytes) {  // 16-byte aligned, bytes a multiple of 16
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(address), "r"(bytes) : "memory");
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

// The epilogue of one (item, matrix) accumulator for the 32 TMEM lanes (= weight rows = output columns) of the calling
// warp: groups of eight activation rows `first`, `first + stride`, ... of the 16. Everything the store loop needs is
// copied out of the parameter block first: the segment is a run-time index, so the block is reached through a generic
// address, and the compiler must assume that the stores change it and would read pointer and pitch again after every
// one of them (measured: 110 ns per store instead of 10).
template <int NMAT> __device__ __forceinline__ void store_accumulator(const UmmaParams& p, int item, int mat, uint32_t accumulator, int row, int first,
                                                                      int stride) {
  const int tile = item % p.tiles, slice = item / p.tiles;
  int segment = 0;
  while (segment + 1 < p.nseg && tile >= p.seg[segment + 1].tile0)
    ++segment;
  float* const y = p.seg[segment].y;
  const float* const residual = p.seg[segment].res;
  const size_t pitch = size_t(p.seg[segment].ldy), column = size_t(tile - p.seg[segment].tile0) * kRows + row;
  const int liveRows = p.m;
  float* const partial = NMAT == 1 && p.splits > 1 ? p.partial + size_t(slice) * p.m * pitch : nullptr;
  for (int c = first; c < kActs / 8 && c * 8 < liveRows; c += stride) {
    float v[8];
    tmem_load8(accumulator + c * 8, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int m = c * 8 + i;
      if (m < liveRows) {
        const size_t at = size_t(m) * pitch + column;
        float value = v[i];
        if (partial) {  // a K slice: the partial sums are added up, with the residual, by umma_reduce_kernel
          partial[at] = value;
          continue;
        }
        if (NMAT == 2)  // the gate half parks in y until the up half arrives (post == 2 epilogue, quant_linear.metal:224-232)
          value = mat == 0 ? value : silu_f(y[at]) * value;
        else if (residual)
          value += residual[at];
        y[at] = value;
      }
    }
  }
}

template <int NMAT> __global__ void __launch_bounds__(kThreads, 1) umma_linear_kernel(const __grid_constant__ UmmaParams p) {
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
  Control& ctl = *reinterpret_cast<Control*>(smem);
  uint8_t* ring = smem + kControlBytes;
  uint8_t* actRing = ring + size_t(kStages) * kSlabBytes;  // halves of a super-block's activations

  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // With p.splits > 1 (one matrix) the work items are (tile, K slice) pairs, so that a matrix of few 128-row tiles still
  // fills the GPU; `blocksPerRow` is then the super-blocks of one slice. One accumulator buffer per (item, matrix).
  const int blocksPerRow = p.k / 256 / p.splits, items = p.tiles * p.splits;
  const uint32_t units = int(blockIdx.x) < items ? uint32_t((items - 1 - int(blockIdx.x)) / int(gridDim.x) + 1) * NMAT : 0u;  // accumulators of this CTA
  volatile int* abortFlag = &ctl.abort;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&ctl.full[s], 1);
      mbar_init(&ctl.slotFree[s], 4);  // four dequant warps
    }
    for (int s = 0; s < kActStages; ++s) {
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
    // ---------------- producer: one weight slab and two activation halves per super-block ----------------
    // L2 prefetch of an item's weights: 128 rows x (blocksPerRow x 144) bytes per matrix, four rows per lane.
    auto prefetch = [&](int item) {
      const int tile = item % p.tiles, firstBlock = (item / p.tiles) * blocksPerRow;
      int segment = 0;
      while (segment + 1 < p.nseg && tile >= p.seg[segment + 1].tile0)
        ++segment;
      const size_t rowBytes = size_t(p.k / 256) * 144, row0 = size_t(tile - p.seg[segment].tile0) * kRows;
      for (int mat = 0; mat < NMAT; ++mat) {
        const uint8_t* base = (mat ? p.seg[segment].w2 : p.seg[segment].w) + row0 * rowBytes + size_t(firstBlock) * 144;
        for (int r = lane; r < kRows; r += 32)
          prefetch_l2(base + r * rowBytes, uint32_t(blocksPerRow) * 144);
      }
    };
    if (int(blockIdx.x) < items)
      prefetch(blockIdx.x);
    const uint32_t halfBytes = uint32_t(p.actRows) * 256;  // 8 k-steps x [actRows x 16] fp16
    uint32_t it = 0;
    bool ok = true, waited = false;
    for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
      if (item + int(gridDim.x) < items)
        prefetch(item + gridDim.x);
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
              mbar_arrive_expect_tx(&ctl.full[slot], kSlabBytes);
              tma_load_2d(ring + size_t(slot) * kSlabBytes, &p.map[segment][mat], sb * 18, row0, &ctl.full[slot]);
            }
            if (!waited) {  // the activations are the preceding kernel's output
              pdl_wait();
              waited = true;
            }
            for (int h = 0; h < 2 && ok; ++h) {  // the two activation halves of this super-block
              const uint32_t half = 2 * it + h, actSlot = half % kActStages, actRound = half / kActStages;
              if (actRound > 0)
                ok = mbar_wait_bounded(&ctl.actFree[actSlot], (actRound - 1) & 1, abortFlag);
              if (ok) {
                mbar_arrive_expect_tx(&ctl.actFull[actSlot], halfBytes);
                bulk_load(actRing + size_t(actSlot) * kActHalfBytes, p.acts + (size_t(sb) * 2 + h) * halfBytes, halfBytes, &ctl.actFull[actSlot]);
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
      const uint32_t instruction = instruction_descriptor(p.actRows), stepBytes = uint32_t(p.actRows) * 32;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x)
        for (int mat = 0; mat < NMAT && ok; ++mat, ++unit) {
          const uint32_t buffer = unit & 1;
          if (unit >= 2)
            ok = mbar_wait_bounded(&ctl.dFree[buffer], ((unit >> 1) - 1) & 1, abortFlag);
          const uint32_t dColumn = tmem + kColD + buffer * 128;
          for (int j = 0; j < blocksPerRow && ok; ++j, ++it) {
            const uint32_t aBuffer = it & 1;
            ok = mbar_wait_bounded(&ctl.aReady[aBuffer], (it >> 1) & 1, abortFlag);
            for (int h = 0; h < 2 && ok; ++h) {  // eight k-steps per activation half
              const uint32_t half = 2 * it + h, actSlot = half % kActStages;
              ok = mbar_wait_bounded(&ctl.actFull[actSlot], (half / kActStages) & 1, abortFlag);
              if (!ok)
                break;
              fence_after_sync();
              const uint32_t actBase = smem_u32(actRing + size_t(actSlot) * kActHalfBytes);
#pragma unroll
              for (int step = 0; step < 8; ++step)
                umma_ts(dColumn, tmem + kColA + aBuffer * 128 + (8 * h + step) * 8, smem_descriptor(actBase + step * stepBytes, 128, 256), instruction,
                        (j | h | step) != 0);
              umma_commit(&ctl.actFree[actSlot]);
            }
            if (!ok)
              break;
            umma_commit(&ctl.aFree[aBuffer]);
            if (j == blocksPerRow - 1)
              umma_commit(&ctl.dReady[buffer]);
          }
        }
      if (!ok) {
        *abortFlag = 1;
        atomicExch(p.status, kStatusBarrierTimeout);
      }
    }
  } else if (warp >= 4 && warp < 12) {
    // ---------------- dequant: thread = weight row; group g takes the super-blocks with (index & 1) == g ----------------
    const int group = (warp - 4) >> 2, quadrant = warp & 3, row = quadrant * 32 + lane;
    constexpr uint32_t k1024 = 0x64006400u;
    uint32_t it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < items && ok; item += gridDim.x)
      for (int mat = 0; mat < NMAT && ok; ++mat)
        for (int j = 0; j < blocksPerRow && ok; ++j, ++it) {
          if ((it & 1) != uint32_t(group))
            continue;
          const uint32_t slot = it % kStages, round = it / kStages;
          ok = mbar_wait_bounded(&ctl.full[slot], round & 1, abortFlag);
          if (ok && it >= 2)
            ok = mbar_wait_bounded(&ctl.aFree[it & 1], ((it >> 1) - 1) & 1, abortFlag);
          if (!ok)
            break;
          fence_after_sync();
          const uint8_t* block = ring + size_t(slot) * kSlabBytes + row * 144;
          const uint4 header = *reinterpret_cast<const uint4*>(block);
          const float2 dm = __half22float2(*reinterpret_cast<const __half2*>(&header.x));
          // 6-bit scales / mins, four per word (scale_min_k4, quant_linear.metal:12-20)
          const uint32_t scales[2] = {header.y & 0x3f3f3f3fu, (header.w & 0x0f0f0f0fu) | ((header.y >> 2) & 0x30303030u)};
          const uint32_t mins[2] = {header.z & 0x3f3f3f3fu, ((header.w >> 4) & 0x0f0f0f0fu) | ((header.z >> 2) & 0x30303030u)};
          const uint32_t aAddress = tmem + (uint32_t(quadrant * 32) << 16) + kColA + (it & 1) * 128;
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            // 32 quant bytes: low nibbles belong to sub-block 2t, high nibbles to sub-block 2t+1
            const uint32_t pair = (scales[t >> 1] >> (16 * (t & 1))) & 0xffffu, minPair = (mins[t >> 1] >> (16 * (t & 1))) & 0xffffu;
            const uint4 q0 = *reinterpret_cast<const uint4*>(block + 16 + 32 * t), q1 = *reinterpret_cast<const uint4*>(block + 32 + 32 * t);
            const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
            // dequantised weight d*sc*q - dmin*m, in fp16: q is made exact first, then one fused multiply-add
            const uint32_t sL = pack_half2(dm.x * float(pair & 0xffu), dm.x * float(pair & 0xffu));
            const uint32_t sH = pack_half2(dm.x * float(pair >> 8), dm.x * float(pair >> 8));
            const uint32_t nL = pack_half2(-dm.y * float(minPair & 0xffu), -dm.y * float(minPair & 0xffu));
            const uint32_t nH = pack_half2(-dm.y * float(minPair >> 8), -dm.y * float(minPair >> 8));
            uint32_t v[32];
#pragma unroll
            for (int w = 0; w < 8; ++w) {
              const uint32_t a = words[w];
              v[2 * w] = hfma2_u32(hsub2_u32((a & 0x000f000fu) | k1024, k1024), sL, nL);
              v[2 * w + 1] = hfma2_u32(hsub2_u32(((a >> 8) & 0x000f000fu) | k1024, k1024), sL, nL);
              v[16 + 2 * w] = hfma2_u32(hsub2_u32(((a >> 4) & 0x000f000fu) | k1024, k1024), sH, nH);
              v[16 + 2 * w + 1] = hfma2_u32(hsub2_u32(((a >> 12) & 0x000f000fu) | k1024, k1024), sH, nH);
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
    if (ok && units > 0) {
      // their share of the CTA's last accumulator (see the epilogue warps): groups of eight activation rows 1 + group,
      // 4 + group, ...; the accumulator has no later user, so nobody waits for these reads
      const uint32_t unit = units - 1, buffer = unit & 1;
      pdl_wait();
      ok = mbar_wait_bounded(&ctl.dReady[buffer], (unit >> 1) & 1, abortFlag);
      if (ok && NMAT == 2)  // the up half reads the gate half that the epilogue warps parked in y: wait until they are through with it
        ok = mbar_wait_bounded(&ctl.dFree[(unit - 1) & 1], ((unit - 1) >> 1) & 1, abortFlag);
      if (ok) {
        fence_after_sync();
        const int lastItem = int(blockIdx.x) + int((units - 1) / NMAT) * int(gridDim.x);
        store_accumulator<NMAT>(p, lastItem, NMAT - 1, tmem + (uint32_t(quadrant * 32) << 16) + kColD + buffer * 128, row, 1 + group, 3);
      }
    }
    if (!ok && lane == 0) {
      *abortFlag = 1;
      atomicExch(p.status, kStatusBarrierTimeout);
    }
  } else if (warp >= 12) {
    // ---------------- epilogue: thread = weight row ----------------
    pdl_wait();  // residuals, the parked gate half and the partial-sum buffer belong to earlier kernels
    const int quadrant = warp & 3, row = quadrant * 32 + lane;
    const uint32_t laneBase = tmem + (uint32_t(quadrant * 32) << 16) + kColD;
    uint32_t unit = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < items && ok; item += gridDim.x)
      for (int mat = 0; mat < NMAT && ok; ++mat, ++unit) {
        const uint32_t buffer = unit & 1;
        ok = mbar_wait_bounded(&ctl.dReady[buffer], (unit >> 1) & 1, abortFlag);
        if (!ok)
          break;
        fence_after_sync();
        // the CTA's last accumulator: the dequant warps, idle by then, take two thirds of it
        const bool last = unit + 1 == units;
        store_accumulator<NMAT>(p, item, mat, laneBase + buffer * 128, row, 0, last ? 3 : 1);
        fence_before_sync();
        __syncwarp();
        if (lane == 0)
          mbar_arrive(&ctl.dFree[buffer]);
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

// Lays the activations out as the B operand, per 256-wide super-block: [16 k-steps][16 row groups][2 K halves][8 rows]
// [8 values] fp16, rows rounded to fp16, rows from m up zero. K inside a step follows the order in which the
// dequantiser emits weights: step s covers the quant bytes of 64-group t = s / 4, nibble side (s / 2) % 2, words
// 4 * (s % 2) .. +3; TMEM column c of a step holds the nibbles of bytes (c % 2, c % 2 + 2) of word c / 2. Eight
// consecutive k of a super-block are thus one 16-byte core-matrix row of a k-step (in the order 0,2,1,3,4,6,5,7), and a
// thread turns two float4 loads into one 16-byte store.
// grid (k / 256, actRows / 8), 256 threads: actRows x 32 groups of eight per super-block, one per thread; a warp reads
// one activation row's 256 values.
__global__ void __launch_bounds__(256) umma_prepare_rows_kernel(const float* x, int ldx, int m, int actRows, __half* acts) {
  pdl_launch_dependents();
  pdl_wait();
  const int sb = blockIdx.x;
  __half* out = acts + size_t(sb) * (actRows * 256);
  {
    const int item = blockIdx.y * 256 + threadIdx.x, n = item >> 5, group = item & 31;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
    if (n < m) {
      const float4* src = reinterpret_cast<const float4*>(x + size_t(n) * ldx + size_t(sb) * 256 + group * 8);
      a = src[0], b = src[1];
    }
    const __half2 h0 = __floats2half2_rn(a.x, a.z), h1 = __floats2half2_rn(a.y, a.w), h2 = __floats2half2_rn(b.x, b.z), h3 = __floats2half2_rn(b.y, b.w);
    uint4 packed;
    packed.x = *reinterpret_cast<const uint32_t*>(&h0), packed.y = *reinterpret_cast<const uint32_t*>(&h1);
    packed.z = *reinterpret_cast<const uint32_t*>(&h2), packed.w = *reinterpret_cast<const uint32_t*>(&h3);
    *reinterpret_cast<uint4*>(out + size_t(group >> 1) * (actRows * 16) + (n >> 3) * 128 + (group & 1) * 64 + (n & 7) * 8) = packed;
  }
}

// y = partial[0] + partial[1] + ... (+ residual), four values per thread.
__global__ void __launch_bounds__(256) umma_reduce_kernel(const float* partial, int splits, size_t count, const float* residual, float* y) {
  pdl_launch_dependents();
  pdl_wait();
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

template <int NMAT> cudaError_t launch_tiles(const UmmaParams& params, const float* x, int ldx, int sms, cudaStream_t stream) {
  static PerDeviceOnce configured;
  if (const cudaError_t e = configure_shared_memory(umma_linear_kernel<NMAT>, kSharedBytes, configured))
    return e;
  // The MMA is as wide as the launch has rows, in steps of 16: a speculative pass of 40 rows moves 24 KB of activations
  // per super-block instead of 64 KB and spends a third of the tensor time.
  UmmaParams p = params;
  p.actRows = (p.m + 15) / 16 * 16;
  launch_kernel(umma_prepare_rows_kernel, dim3(p.k / 256, p.actRows / 8), 256, 0, stream, x, ldx, p.m, p.actRows,
                reinterpret_cast<__half*>(const_cast<uint8_t*>(p.acts)));
  const int items = p.tiles * p.splits, grid = items < sms ? items : sms;
  launch_kernel<1>(umma_linear_kernel<NMAT>, grid, kThreads, kSharedBytes, stream, p);
  if (p.splits > 1) {
    const size_t count = size_t(p.m) * p.seg[0].ldy;
    launch_kernel(umma_reduce_kernel, unsigned((count / 4 + 255) / 256), 256, 0, stream, p.partial, p.splits, count, p.seg[0].res, p.seg[0].y);
  }
  return cudaGetLastError();
}

}  // namespace

// 9 to 128 activation rows (p.m), rows of x `ldx` floats apart (a multiple of 4).
cudaError_t umma_launch(bool pair, const UmmaParams& p, const float* x, int ldx, int sms, cudaStream_t stream) {
  return pair ? launch_tiles<2>(p, x, ldx, sms, stream) : launch_tiles<1>(p, x, ldx, sms, stream);
}

}  // namespace infdev
