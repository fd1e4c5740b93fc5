// Gated GQA attention over the paged fp16 K/V pool.
//
// attention_prepare_kernel <- attention_prepare (attention.metal:14-50) + the cache append that the
//                             reference does inside attention_scan (:126-133)
// attention_scan_kernel    <- attention_scan   (attention.metal:103-183)
// attention_reduce_kernel  <- attention_reduce (attention.metal:185-216)
//
// K/V pool of one layer: [physical block][4 kv heads][blockTokens][256] fp16, so the 16 tokens of a tile of
// one kv head are 8 KB contiguous. A per-slot block table maps logical to physical blocks (the reference
// reaches the same effect through Metal sparse-buffer page mappings, device.cpp:147-198).
//
// Split-K: the reference uses max(1, 8/rows) splits (forward.cpp:92), which leaves a 148-SM part idle on a
// long single-row context and makes the reduction order depend on the batch. Here the number of splits of a
// row depends only on how many tokens that row attends to, so a sequence gets the same arithmetic whether
// it runs alone or batched. One CTA serves the four query heads that share a kv head, so K and V are read
// once per group.
#include <mutex>
#include "act_image.cuh"
#include "ops.h"

namespace infdev {
namespace {

constexpr int kQHeads = 16, kKvHeads = 4, kDim = 256, kGroup = kQHeads / kKvHeads, kTile = 16;
constexpr int kPartialStride = kDim + 4;  // 260 floats keeps every record 16-byte aligned for the float4 stores

// Row -> query. In a decode pass every query is one row, so query `row` is the answer; probing it first saves a chain
// of dependent loads at the head of every CTA (queryCount bounds the probe).
__device__ __forceinline__ const infdev_query& query_of_row(const infdev_query* queries, int queryCount, uint32_t row) {
  const infdev_query& guess = queries[min(row, uint32_t(queryCount - 1))];
  if (row >= guess.start && row < guess.start + guess.count)
    return guess;
  while (row >= queries->start + queries->count)
    ++queries;
  return *queries;
}

// Splits of a row that attends to `attended` tokens: 64-token pieces, at most maxSplits, each a multiple of
// the 16-token tile. The piece length trades the fixed cost of a CTA (query load, first tile fetch, partial store)
// against the number of CTAs in flight; it depends only on the row's own context, never on the batch.
__device__ __forceinline__ void split_range(uint32_t attended, uint32_t maxSplits, uint32_t split, uint32_t& begin, uint32_t& end, uint32_t& count) {
  count = min(maxSplits, (attended + 63u) / 64u);
  const uint32_t per = (((attended + count - 1) / count) + kTile - 1) / kTile * kTile;
  begin = min(attended, split * per);
  end = min(attended, begin + per);
}

// grid (rows * 20), 256 threads: heads 0..15 are queries, 16..19 keys (which also store the value head).
__global__ void __launch_bounds__(256) attention_prepare_kernel(const float* qg, const float* rawK, const float* rawV, const float* qNorm,
                                                                const float* kNorm, const float* rope, const infdev_query* queries, int queryCount,
                                                                const int32_t* table, int tableStride, int blockTokens, float* q, __half* cacheK,
                                                                __half* cacheV) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x / 20, head = blockIdx.x % 20, lane = threadIdx.x;
  const bool query = head < kQHeads;
  if (query && !qg)  // K/V store only (mtp_store_kv, attention.metal:53-100)
    return;
  const int local = query ? head : head - kQHeads;
  const float* source = query ? qg + (size_t(row) * kQHeads + local) * kDim * 2 : rawK + (size_t(row) * kKvHeads + local) * kDim;
  const float* weight = query ? qNorm : kNorm;
  const float value = source[lane];
  __shared__ float partial[8], scale;
  const float sum = warp_sum(value * value);
  if ((lane & 31) == 0)
    partial[lane >> 5] = sum;
  __syncthreads();
  if (lane == 0) {
    float total = 0.f;
    for (int i = 0; i < 8; ++i)
      total += partial[i];
    scale = rsqrtf(total / float(kDim) + 1.0e-6f);
  }
  __syncthreads();
  const infdev_query& info = query_of_row(queries, queryCount, row);
  const uint32_t position = info.position + row - info.start;
  float result = value * scale * weight[lane];
  if (lane < 64) {
    const int other = lane < 32 ? lane + 32 : lane - 32, pair = lane & 31;
    const float paired = source[other] * scale * weight[other];
    const float2 cs = *reinterpret_cast<const float2*>(rope + (size_t(position) * 32 + pair) * 2);
    result = result * cs.x + (lane < 32 ? -paired : paired) * cs.y;
  }
  if (query) {
    q[(size_t(row) * kQHeads + local) * kDim + lane] = result;
  } else {
    const size_t block = table[size_t(info.slot) * tableStride + position / blockTokens];
    const size_t at = ((block * kKvHeads + local) * blockTokens + position % blockTokens) * kDim + lane;
    cacheK[at] = __float2half_rn(result);
    cacheV[at] = __float2half_rn(rawV[(size_t(row) * kKvHeads + local) * kDim + lane]);
  }
}

// 16-byte asynchronous copy global -> shared; `bytes` = 0 writes zeros instead (a token past the end of the piece).
__device__ __forceinline__ void copy_async16(void* dst, const void* src, uint32_t bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}

// grid (maxSplits, 4 kv heads, rows), 128 threads. The 16-token K and V tiles of the piece are copied into a
// double buffer in shared memory with cp.async one tile ahead of the arithmetic, so the walk over the piece is not a
// chain of load latencies. Both contractions run on the tensor cores as m16n8k16 with fp16 operands split hi + lo where
// they are not fp16 already: warp 0 scores the tile's 16 tokens for the four query heads of the group, then warp w
// accumulates the weighted values of dims 64w .. 64w+63 for all four heads.
__global__ void __launch_bounds__(128, 6) attention_scan_kernel(const float* q, const __half* cacheK, const __half* cacheV,
                                                                const infdev_query* queries, int queryCount, const int32_t* table, int tableStride,
                                                                int blockTokens, uint32_t maxSplits, float* partials) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t split = blockIdx.x, kvHead = blockIdx.y, row = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const infdev_query& info = query_of_row(queries, queryCount, row);
  const uint32_t attended = info.position + (row - info.start) + 1;
  uint32_t begin, end, count;
  split_range(attended, maxSplits, split, begin, end, count);
  if (split >= count)
    return;
  __shared__ float scores[kGroup][kTile];
  // [buffer][K, V][token][dim]; rows padded by 16 bytes so that the eight token rows one ldmatrix phase reads hit different banks
  __shared__ __align__(16) __half tiles[2][2][kTile][kDim + 8];
  const int32_t* slotTable = table + size_t(info.slot) * tableStride;
  auto fetch = [&](uint32_t tile, int buffer) {
    const size_t block = slotTable[tile / blockTokens];
    const size_t base = ((block * kKvHeads + kvHead) * blockTokens + tile % blockTokens) * kDim;
    // 16 tokens x 512 bytes per tensor = 512 chunks of 16 bytes, four per thread
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int chunk = c * 128 + threadIdx.x, token = chunk >> 5, offset = (chunk & 31) * 8;
      const uint32_t bytes = tile + token < end ? 16u : 0u;
      copy_async16(&tiles[buffer][0][token][offset], cacheK + base + token * kDim + offset, bytes);
      copy_async16(&tiles[buffer][1][token][offset], cacheV + base + token * kDim + offset, bytes);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  fetch(begin, 0);
  // Scores on the tensor cores too (warp 0): A = the K tile (16 tokens x 256 dims, 16 dims per MMA), B = q of the four
  // heads as 8 columns, columns 0..3 the fp16 high halves, columns 4..7 the low halves (q - hi). Lane (g, t) keeps column
  // g of B for all 16 dim steps: 32 registers.
  const int g = lane >> 2, t = lane & 3, myHead = g & 3;
  uint32_t qFragment[16][2];
  if (warp == 0) {
    const float* src = q + (size_t(row) * kQHeads + kvHead * kGroup + myHead) * kDim;
#pragma unroll
    for (int step = 0; step < 16; ++step) {
      const float2 a = *reinterpret_cast<const float2*>(src + 16 * step + 2 * t), b = *reinterpret_cast<const float2*>(src + 16 * step + 2 * t + 8);
      __half2 h0 = __floats2half2_rn(a.x, a.y), h1 = __floats2half2_rn(b.x, b.y);
      if (g >= 4) {
        const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
        h0 = __floats2half2_rn(a.x - f0.x, a.y - f0.y), h1 = __floats2half2_rn(b.x - f1.x, b.y - f1.y);
      }
      qFragment[step][0] = *reinterpret_cast<const uint32_t*>(&h0), qFragment[step][1] = *reinterpret_cast<const uint32_t*>(&h1);
    }
  }
  // Value accumulation on the tensor cores (m16n8k16, fp16 operands, fp32 accumulate): warp w owns value dims 64w .. 64w+63
  // in four 16-dim chunks; A = V^T of the tile (dims x tokens, read transposed by ldmatrix), B = the tile's softmax weights
  // (tokens x 8 columns: columns 0..3 the fp16 high halves for the four heads, columns 4..7 the low halves, so the result is
  // accurate to fp32 rounding of the weights). Lane (g, t) builds column g of B, i.e. head g % 4, and tracks that head's
  // running maximum and, over its four tokens of every tile, its share of the norm.
  float runningMax = -1.0e30f, runningNorm = 0.f, acc[4][4];
#pragma unroll
  for (int c = 0; c < 4; ++c)
    acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0.f;
  int buffer = 0;
  for (uint32_t tile = begin; tile < end; tile += kTile, buffer ^= 1) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // this tile is complete for every thread, and every thread is done with the previous tile and its scores
    if (tile + kTile < end)
      fetch(tile + kTile, buffer ^ 1);  // lands while this tile is worked on
    if (warp == 0) {
      // scores of the tile's 16 tokens for the four heads: two accumulator chains over the 16 dim steps
      float score[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const int matrix = lane >> 3, tokenRow = (lane & 7) + 8 * (matrix & 1), dimOffset = 8 * (matrix >> 1);
#pragma unroll
      for (int step = 0; step < 16; ++step) {
        uint32_t a[4];
        const uint32_t address = smem_u32(&tiles[buffer][0][tokenRow][16 * step + dimOffset]);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(address));
        mma_16816(score[step & 1], a, qFragment[step][0], qFragment[step][1]);
      }
      // columns 4..7 (lanes t = 2, 3) carry the low-half products of heads 0..3
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        score[0][i] += score[1][i];
        score[0][i] += __shfl_xor_sync(0xffffffffu, score[0][i], 2);
      }
      if (t < 2) {
        scores[2 * t][g] = tile + g < end ? score[0][0] * (1.0f / 16.0f) : -INFINITY;
        scores[2 * t + 1][g] = tile + g < end ? score[0][1] * (1.0f / 16.0f) : -INFINITY;
        scores[2 * t][g + 8] = tile + g + 8 < end ? score[0][2] * (1.0f / 16.0f) : -INFINITY;
        scores[2 * t + 1][g + 8] = tile + g + 8 < end ? score[0][3] * (1.0f / 16.0f) : -INFINITY;
      }
    }
    __syncthreads();
    // online softmax. A token past the end has score -inf: weight 0 against a zero-filled value row.
    float tileMax = -INFINITY;
#pragma unroll
    for (int i = 0; i < kTile; i += 4) {
      const float4 four = *reinterpret_cast<const float4*>(&scores[myHead][i]);
      tileMax = fmaxf(fmaxf(tileMax, fmaxf(four.x, four.y)), fmaxf(four.z, four.w));
    }
    const float nextMax = fmaxf(runningMax, tileMax), rescale = expf(runningMax - nextMax);
    runningMax = nextMax;
    // weights of this lane's four tokens (the summation slots 2t, 2t+1, 2t+8, 2t+9 of the B fragment)
    const float w0 = expf(scores[myHead][2 * t] - nextMax), w1 = expf(scores[myHead][2 * t + 1] - nextMax);
    const float w2 = expf(scores[myHead][2 * t + 8] - nextMax), w3 = expf(scores[myHead][2 * t + 9] - nextMax);
    runningNorm = runningNorm * rescale + ((w0 + w1) + (w2 + w3));
    __half2 b0 = __floats2half2_rn(w0, w1), b1 = __floats2half2_rn(w2, w3);
    if (g >= 4) {  // the low halves
      const float2 f0 = __half22float2(b0), f1 = __half22float2(b1);
      b0 = __floats2half2_rn(w0 - f0.x, w1 - f0.y), b1 = __floats2half2_rn(w2 - f1.x, w3 - f1.y);
    }
    // this lane's accumulators are columns 2t and 2t+1: heads (2t) % 4 and (2t+1) % 4
    const float r0 = __shfl_sync(0xffffffffu, rescale, ((2 * t) & 3) * 4), r1 = __shfl_sync(0xffffffffu, rescale, ((2 * t + 1) & 3) * 4);
    const int matrix = lane >> 3, tokenRow = (lane & 7) + 8 * (matrix >> 1), dimOffset = 8 * (matrix & 1);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t a[4];
      const uint32_t address = smem_u32(&tiles[buffer][1][tokenRow][64 * warp + 16 * c + dimOffset]);
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(address));
      acc[c][0] *= r0, acc[c][1] *= r1, acc[c][2] *= r0, acc[c][3] *= r1;
      mma_16816(acc[c], a, *reinterpret_cast<const uint32_t*>(&b0), *reinterpret_cast<const uint32_t*>(&b1));
    }
  }
  // columns 4..7 (lanes t = 2, 3) hold the low-half products of heads 0..3: add them to columns 0..3 (lanes t = 0, 1)
#pragma unroll
  for (int c = 0; c < 4; ++c)
#pragma unroll
    for (int i = 0; i < 4; ++i)
      acc[c][i] += __shfl_xor_sync(0xffffffffu, acc[c][i], 2);
  runningNorm += __shfl_xor_sync(0xffffffffu, runningNorm, 1);
  runningNorm += __shfl_xor_sync(0xffffffffu, runningNorm, 2);
  float* base = partials + ((size_t(row) * kQHeads + kvHead * kGroup) * maxSplits + split) * kPartialStride;
  const size_t headStride = size_t(maxSplits) * kPartialStride;
  if (t < 2) {
    float *first = base + (2 * t) * headStride, *second = base + (2 * t + 1) * headStride;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int dim = 64 * warp + 16 * c + g;
      first[dim] = acc[c][0], second[dim] = acc[c][1];
      first[dim + 8] = acc[c][2], second[dim + 8] = acc[c][3];
    }
  }
  if (warp == 0 && g < 4 && t == 0) {
    base[g * headStride + kDim] = runningMax;
    base[g * headStride + kDim + 1] = runningNorm;
  }
}

// grid (rows * 16), 256 threads: merge the splits, normalise, multiply by sigmoid(gate).
// `image`, when not null, also receives the activation image of the output rows: a head is one 256-value block.
__global__ void __launch_bounds__(256) attention_reduce_kernel(const float* partials, const float* qg, const infdev_query* queries, int queryCount,
                                                               uint32_t maxSplits, float* out, uint8_t* image) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t headRow = blockIdx.x, row = headRow / kQHeads, dim = threadIdx.x;
  const infdev_query& info = query_of_row(queries, queryCount, row);
  const uint32_t attended = info.position + (row - info.start) + 1;
  uint32_t begin, end, count;
  split_range(attended, maxSplits, 0, begin, end, count);
  const float* src = partials + size_t(headRow) * maxSplits * kPartialStride;
  // Lane s of every warp fetches the running maximum and norm of split s (at most 32 splits) in one trip to the L2; the
  // weights of the splits then travel by shuffle, and the loop below has only independent loads, taken in split order
  // so the sums are those of a sequential merge.
  const uint32_t lane = dim & 31;
  float splitMaximum = -1.0e30f, splitNorm = 0.f;
  if (lane < count) {
    const float2 pair = *reinterpret_cast<const float2*>(src + lane * kPartialStride + kDim);
    splitMaximum = pair.x, splitNorm = pair.y;
  }
  const float maximum = warp_max(splitMaximum);
  const float splitWeight = lane < count ? expf(splitMaximum - maximum) : 0.f;
  float norm = 0.f, numerator = 0.f;
#pragma unroll 8
  for (uint32_t s = 0; s < count; ++s) {
    const float w = __shfl_sync(0xffffffffu, splitWeight, int(s));
    norm += __shfl_sync(0xffffffffu, splitNorm, int(s)) * w;
    numerator += src[s * kPartialStride + dim] * w;
  }
  const float gate = qg[size_t(headRow) * kDim * 2 + kDim + dim];
  const float value = (numerator / norm) / (1.0f + expf(-gate));
  out[size_t(headRow) * kDim + dim] = value;
  if (image) {
    __shared__ __align__(16) float staged[kDim];
    staged[dim] = value;
    __syncthreads();
    if (dim < 32) {
      const float4 a = *reinterpret_cast<const float4*>(&staged[dim * 8]), b = *reinterpret_cast<const float4*>(&staged[dim * 8 + 4]);
      const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
      image_store_block(image + (size_t(row >> 3) * kQHeads + headRow % kQHeads) * kImageBlockBytes, row & 7, dim, v);
    }
  }
}

}  // namespace

cudaError_t attention_prepare_launch(const float* qg, const float* rawK, const float* rawV, const float* qNorm, const float* kNorm, const float* rope,
                                     const infdev_query* queries, int queryCount, const int32_t* table, int tableStride, int blockTokens, int64_t rows, float* q,
                                     void* cacheK, void* cacheV, cudaStream_t stream) {
  if (rows <= 0)
    return cudaSuccess;
  launch_kernel<2>(attention_prepare_kernel, unsigned(rows * 20), 256, 0, stream, qg, rawK, rawV, qNorm, kNorm, rope, queries, queryCount, table, tableStride, blockTokens, q,
                                                                     static_cast<__half*>(cacheK), static_cast<__half*>(cacheV));
  return cudaGetLastError();
}

cudaError_t attention_launch(const float* q, const float* qg, const void* cacheK, const void* cacheV, const infdev_query* queries,
                             int queryCount, const int32_t* table, int tableStride, int blockTokens, int64_t rows, uint32_t maxSplits, float* partials, float* out,
                             uint8_t* image, cudaStream_t stream) {
  if (rows <= 0)
    return cudaSuccess;
  launch_kernel(attention_scan_kernel, dim3(maxSplits, kKvHeads, unsigned(rows)), 128, 0, stream, q, static_cast<const __half*>(cacheK),
                                                                                       static_cast<const __half*>(cacheV), queries, queryCount, table,
                                                                                       tableStride, blockTokens, maxSplits, partials);
  launch_kernel(attention_reduce_kernel, unsigned(rows * kQHeads), 256, 0, stream, partials, qg, queries, queryCount, maxSplits, out, image);
  return cudaGetLastError();
}

// ---- attention without any allocation -------------------------------------------------------------
// Some users of this library cannot give the attention call a scratch buffer: a serving process that sized its
// K/V pool to whatever device memory was free at start-up has nothing left for a later cudaMalloc, and a
// latency-critical decode loop cannot afford an allocation call that synchronises the whole device. For them the
// split-K partials of up to kStaticRows packed rows live in this file-scope array (about 2 MiB), which every GPU
// that loads the library keeps until the process exits.
constexpr int kStaticRows = 8, kStaticSplits = 16;
static __device__ __align__(256) float staticPartials[size_t(kStaticRows) * kQHeads * kStaticSplits * kPartialStride];

cudaError_t attention_static_launch(const float* q, const float* qg, const void* cacheK, const void* cacheV, const infdev_query* queries,
                                    int queryCount, const int32_t* table, int tableStride, int blockTokens, int64_t rows, int device, float* out,
                                    cudaStream_t stream) {
  // In host code `staticPartials` is only a handle; the kernels need the device address, looked up once per
  // device (with that device current, which the caller guarantees) and remembered.
  static std::mutex guard;
  static float* address[64] = {nullptr};
  if (device < 0 || device >= 64 || rows > kStaticRows)
    return cudaErrorInvalidValue;
  if (rows <= 0)
    return cudaSuccess;
  float* partials;
  {
    std::lock_guard<std::mutex> lock(guard);
    if (!address[device]) {
      void* found = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&found, staticPartials);
      if (e != cudaSuccess)
        return e;
      address[device] = static_cast<float*>(found);
    }
    partials = address[device];
  }
  // Nothing has to start at zero: the reduction reads exactly the (row, head, split) records that the scan of the
  // same call wrote; whatever an earlier call left in the array is never read.
  launch_kernel(attention_scan_kernel, dim3(kStaticSplits, kKvHeads, unsigned(rows)), 128, 0, stream, q, static_cast<const __half*>(cacheK),
                                                                                          static_cast<const __half*>(cacheV), queries, queryCount, table,
                                                                                          tableStride, blockTokens, kStaticSplits, partials);
  launch_kernel(attention_reduce_kernel, unsigned(rows * kQHeads), 256, 0, stream, partials, qg, queries, queryCount, kStaticSplits, out, nullptr);
  return cudaGetLastError();
}

int attention_static_max_rows() { return kStaticRows; }

}  // namespace infdev
