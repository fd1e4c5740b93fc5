// Small memory-bound kernels of the forward step: block dequantisation, embedding gather, RMS norms and
// the per-row token selection.
#include "act_image.cuh"
#include "ops.h"

namespace infdev {
namespace {

// scale_min_k4, quant_linear.metal:12-20
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t* q, int& d, int& m) {
  if (j < 4) {
    d = q[j] & 63;
    m = q[j + 4] & 63;
  } else {
    d = (q[j + 4] & 15) | ((q[j - 4] >> 6) << 4);
    m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

// Element r of a Q4_K super-block, with the multiplication order of dequant_tile (quant_linear.metal:38-45)
// and no fused multiply-add so the result is bit-identical to a plain fp32 evaluation.
__device__ __forceinline__ float dequant_q4k_element(const uint8_t* b, int r) {
  const float d = __half2float(*reinterpret_cast<const __half*>(b)), dm = __half2float(*reinterpret_cast<const __half*>(b + 2));
  int sc, mn;
  scale_min_k4(r >> 5, b + 4, sc, mn);
  const uint8_t q = b[16 + (r >> 6) * 32 + (r & 31)];
  const int v = (r & 32) ? (q >> 4) : (q & 15);
  return __fsub_rn(__fmul_rn(__fmul_rn(d, float(sc)), float(v)), __fmul_rn(dm, float(mn)));
}

// Element r of a Q6_K super-block (quant_linear.metal:75-82).
__device__ __forceinline__ float dequant_q6k_element(const uint8_t* b, int r) {
  const float d = __half2float(*reinterpret_cast<const __half*>(b + 208));
  const int h = r >> 7, rr = r & 127, l = r & 31, s = rr >> 5;
  const uint8_t q = b[h * 64 + ((rr & 32) ? 32 : 0) + l];
  const int lo = (rr & 64) ? (q >> 4) : (q & 15), hi = (b[128 + h * 32 + l] >> (2 * s)) & 3;
  const int sc = int(reinterpret_cast<const int8_t*>(b)[192 + h * 8 + (rr >> 4)]);
  return __fmul_rn(__fmul_rn(d, float(sc)), float(((hi << 4) | lo) - 32));
}

template <int TYPE> __global__ void dequant_kernel(const uint8_t* blocks, int64_t count, float* out) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int bytes = TYPE == 12 ? 144 : 210;
  const int64_t block = blockIdx.x;
  if (block >= count)
    return;
  const uint8_t* b = blocks + block * bytes;
  const int r = threadIdx.x;
  out[block * 256 + r] = TYPE == 12 ? dequant_q4k_element(b, r) : dequant_q6k_element(b, r);
}

template <int TYPE> __global__ void embedding_kernel(const uint8_t* table, int blocksPerRow, const int32_t* tokens, float* out) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int bytes = TYPE == 12 ? 144 : 210;
  const int64_t row = blockIdx.y, token = tokens[row];
  const int block = blockIdx.x, r = threadIdx.x;
  const uint8_t* b = table + (token * blocksPerRow + block) * bytes;
  out[(row * blocksPerRow + block) * 256 + r] = TYPE == 12 ? dequant_q4k_element(b, r) : dequant_q6k_element(b, r);
}

__device__ __forceinline__ const infdev_query& query_of_row(const infdev_query* queries, uint32_t row) {  // batch.hpp:19-23
  while (row >= queries->start + queries->count)
    ++queries;
  return *queries;
}

__device__ __forceinline__ const infdev_query& query_of_logit(const infdev_query* queries, uint32_t row) {  // batch.hpp:25-29
  while (!queries->samples || row >= queries->logit + queries->samples)
    ++queries;
  return *queries;
}

__global__ void gather_tokens_kernel(const infdev_query* queries, int queryCount, const int32_t* requestData, uint32_t capacity,
                                     const int32_t* proposals, uint32_t mode, int32_t* rowTokens) {
  pdl_launch_dependents();
  pdl_wait();
  const int q = blockIdx.x;
  if (q >= queryCount)
    return;
  const infdev_query info = queries[q];
  for (uint32_t p = threadIdx.x; p < info.count; p += blockDim.x) {
    const uint32_t row = info.start + p;
    int32_t token;
    if (mode == 2)
      token = proposals[row];
    else if (info.state != 0xffffffffu && p)
      token = proposals[p * 8 + info.state / info.count];
    else
      token = requestData[size_t(info.slot) * capacity + info.position + p];
    rowTokens[row] = token;
  }
}

// `image`, when not null, also receives the activation image of the normalised rows (act_image.cuh; needs dim to
// be a multiple of 256): 8-row slices of dim/256 blocks each.
template <bool GATHER>
__global__ void __launch_bounds__(256) rms_norm_kernel(const float* x, const float* w, const infdev_query* queries, int dim, float* y, uint8_t* image) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const float* src = x + size_t(row) * dim;
  if (GATHER) {
    const infdev_query& info = query_of_logit(queries, row);
    src = x + size_t(info.start + info.count - info.samples + (row - info.logit)) * dim;
  }
  __shared__ float sums[9];
  float sum = 0.f;
  for (int d = threadIdx.x * 4; d < dim; d += 1024) {
    const float4 v = *reinterpret_cast<const float4*>(src + d);
    sum += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  sum = warp_sum(sum);
  if ((threadIdx.x & 31) == 0)
    sums[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < 8 ? sums[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0)
      sums[8] = rsqrtf(v / float(dim) + 1.0e-6f);
  }
  __syncthreads();
  const float scale = sums[8];
  if (image) {
    // one warp per 256-value block, eight consecutive values per lane: the layout image_store_block wants
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, blocks = dim / 256;
    uint8_t* slice = image + size_t(row >> 3) * blocks * kImageBlockBytes;
    for (int block = warp; block < blocks; block += 8) {
      const int d = block * 256 + lane * 8;
      const float4 a = *reinterpret_cast<const float4*>(src + d), b = *reinterpret_cast<const float4*>(src + d + 4);
      const float4 ga = *reinterpret_cast<const float4*>(w + d), gb = *reinterpret_cast<const float4*>(w + d + 4);
      const float v[8] = {a.x * scale * ga.x, a.y * scale * ga.y, a.z * scale * ga.z, a.w * scale * ga.w,
                          b.x * scale * gb.x, b.y * scale * gb.y, b.z * scale * gb.z, b.w * scale * gb.w};
      if (y) {
        *reinterpret_cast<float4*>(y + size_t(row) * dim + d) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(y + size_t(row) * dim + d + 4) = make_float4(v[4], v[5], v[6], v[7]);
      }
      image_store_block(slice + size_t(block) * kImageBlockBytes, row & 7, lane, v);
    }
    return;
  }
  for (int d = threadIdx.x * 4; d < dim; d += 1024) {
    const float4 v = *reinterpret_cast<const float4*>(src + d), g = *reinterpret_cast<const float4*>(w + d);
    *reinterpret_cast<float4*>(y + size_t(row) * dim + d) = make_float4(v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w);
  }
}

// The same for dim = 4096 in one pass over the row: 512 threads, each keeps its eight consecutive values in registers
// between the sum of squares and the scaling (a warp holds one 256-value block, which is also the unit of the image).
template <bool GATHER>
__global__ void __launch_bounds__(512) rms_norm_4096_kernel(const float* x, const float* w, const infdev_query* queries, float* y, uint8_t* image) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int kDim = 4096;
  const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, d = threadIdx.x * 8;
  const float* src = x + size_t(row) * kDim;
  if (GATHER) {
    const infdev_query& info = query_of_logit(queries, row);
    src = x + size_t(info.start + info.count - info.samples + (row - info.logit)) * kDim;
  }
  const float4 a = *reinterpret_cast<const float4*>(src + d), b = *reinterpret_cast<const float4*>(src + d + 4);
  const float4 ga = *reinterpret_cast<const float4*>(w + d), gb = *reinterpret_cast<const float4*>(w + d + 4);
  __shared__ float sums[16];
  const float sum = warp_sum((a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w) + (b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w));
  if (lane == 0)
    sums[warp] = sum;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i)
    total += sums[i];
  const float scale = rsqrtf(total / float(kDim) + 1.0e-6f);
  const float v[8] = {a.x * scale * ga.x, a.y * scale * ga.y, a.z * scale * ga.z, a.w * scale * ga.w,
                      b.x * scale * gb.x, b.y * scale * gb.y, b.z * scale * gb.z, b.w * scale * gb.w};
  if (y) {
    *reinterpret_cast<float4*>(y + size_t(row) * kDim + d) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(y + size_t(row) * kDim + d + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
  if (image)
    image_store_block(image + (size_t(row >> 3) * (kDim / 256) + warp) * kImageBlockBytes, row & 7, lane, v);
}

// mtp_fuse (native_ops.metal:43-87): y[row] = [rmsnorm(embedding[row]) * enorm | rmsnorm(h) * hnorm], 8192 wide.
// h by mode: 2 = the slot's MTP seed (the target's hidden state of the last committed position, kept at the end
// of the state record); 1 = seed for a query's first row, else the target hidden of the previous row; 0 = the
// hidden of the same row (previous MTP step). A fresh sequence's first row has no predecessor: h = 0.
// Mode 1 also stores the target hidden of each candidate row (speculative) or of the last row as the next seed.
__global__ void __launch_bounds__(256) mtp_fuse_kernel(const float* embedding, const float* hidden, const infdev_query* queries, const float* enorm,
                                                       const float* hnorm, uint32_t mode, uint64_t seedOffset, uint64_t stateBytes, float* y) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t row = blockIdx.x, tid = threadIdx.x;
  const infdev_query& info = query_of_row(queries, row);
  const uint32_t token = row - info.start;
  const float* seed = reinterpret_cast<const float*>(info.previous + seedOffset);
  const float* h = mode == 2 ? seed : (mode == 1 && !token) ? seed : hidden + size_t(mode == 1 ? row - 1 : row) * 4096;
  // Without a predecessor record there is no seed to read: the first row of a fresh sequence (`initial`,
  // native_ops.metal:57), and every row that would take the seed in a frame the engine never builds that way.
  const bool initial = !info.previous && (token == 0 || mode == 2);
  __shared__ float sums[18];
  float es = 0.f, hs = 0.f;
  for (int d = tid; d < 4096; d += 256) {
    const float ev = embedding[size_t(row) * 4096 + d], hv = initial ? 0.f : h[d];
    es += ev * ev;
    hs += hv * hv;
  }
  es = warp_sum(es);
  hs = warp_sum(hs);
  if ((tid & 31) == 0) {
    sums[tid >> 5] = es;
    sums[8 + (tid >> 5)] = hs;
  }
  __syncthreads();
  if (tid < 32) {
    es = warp_sum(tid < 8 ? sums[tid] : 0.f);
    hs = warp_sum(tid < 8 ? sums[8 + tid] : 0.f);
    if (tid == 0) {
      sums[16] = rsqrtf(es / 4096.f + 1.0e-6f);
      sums[17] = rsqrtf(hs / 4096.f + 1.0e-6f);
    }
  }
  __syncthreads();
  const bool speculative = info.state != 0xffffffffu;
  float* nextSeed = nullptr;
  if (mode == 1 && (speculative || token + 1 == info.count))
    nextSeed = reinterpret_cast<float*>(info.next + (speculative ? uint64_t(token) * stateBytes : 0) + seedOffset);
  for (int d = tid; d < 4096; d += 256) {
    const float hv = initial ? 0.f : h[d];
    y[size_t(row) * 8192 + d] = embedding[size_t(row) * 4096 + d] * sums[16] * enorm[d];
    y[size_t(row) * 8192 + 4096 + d] = hv * sums[17] * hnorm[d];
    if (nextSeed)
      nextSeed[d] = hidden[size_t(row) * 4096 + d];
  }
}

// Health check of the abort path every waiting kernel shares: one thread waits, with an iteration limit, for a barrier
// phase that cannot complete (two arrivals expected, one made). The wait must give up, raise the abort flag and leave
// kStatusBarrierTimeout in the status word; the kernel returns normally and the context stays usable.
__global__ void bounded_wait_probe_kernel(uint32_t limit, int* status) {
  __shared__ uint64_t barrier;
  __shared__ int abortFlag;
  if (threadIdx.x == 0) {
    mbar_init(&barrier, 2);
    abortFlag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    mbar_arrive(&barrier);
    if (!mbar_wait_bounded(&barrier, 0, &abortFlag, limit)) {
      abortFlag = 1;
      atomicExch(status, kStatusBarrierTimeout);
    }
  }
}

}  // namespace

cudaError_t bounded_wait_probe_launch(uint32_t limit, int* status, cudaStream_t stream) {
  bounded_wait_probe_kernel<<<1, 32, 0, stream>>>(limit, status);
  return cudaGetLastError();
}

cudaError_t mtp_fuse_launch(const float* embedding, const float* hidden, const infdev_query* queries, const float* enorm, const float* hnorm,
                            int64_t rows, uint32_t mode, uint64_t seedOffset, uint64_t stateBytes, float* y, cudaStream_t stream) {
  if (rows <= 0)
    return cudaSuccess;
  launch_kernel(mtp_fuse_kernel, unsigned(rows), 256, 0, stream, embedding, hidden, queries, enorm, hnorm, mode, seedOffset, stateBytes, y);
  return cudaGetLastError();
}

cudaError_t dequant_launch(int type, const void* blocks, int64_t count, float* out, cudaStream_t stream) {
  if (count <= 0)
    return cudaSuccess;
  if (type == 12)
    launch_kernel(dequant_kernel<12>, unsigned(count), 256, 0, stream, static_cast<const uint8_t*>(blocks), count, out);
  else
    launch_kernel(dequant_kernel<14>, unsigned(count), 256, 0, stream, static_cast<const uint8_t*>(blocks), count, out);
  return cudaGetLastError();
}

cudaError_t embedding_launch(int type, const void* table, int64_t k, const int32_t* tokens, int64_t rows, float* out, cudaStream_t stream) {
  if (rows <= 0)
    return cudaSuccess;
  const dim3 grid(unsigned(k / 256), unsigned(rows));
  if (type == 12)
    launch_kernel(embedding_kernel<12>, grid, 256, 0, stream, static_cast<const uint8_t*>(table), int(k / 256), tokens, out);
  else
    launch_kernel(embedding_kernel<14>, grid, 256, 0, stream, static_cast<const uint8_t*>(table), int(k / 256), tokens, out);
  return cudaGetLastError();
}

cudaError_t gather_tokens_launch(const infdev_query* queries, int queryCount, const int32_t* requestData, uint32_t capacity,
                                 const int32_t* proposals, uint32_t mode, int32_t* rowTokens, cudaStream_t stream) {
  if (queryCount <= 0)
    return cudaSuccess;
  launch_kernel(gather_tokens_kernel, queryCount, 128, 0, stream, queries, queryCount, requestData, capacity, proposals, mode, rowTokens);
  return cudaGetLastError();
}

cudaError_t rms_norm_launch(const float* x, const float* w, const infdev_query* queries, int64_t rows, int64_t dim, float* y, uint8_t* image,
                            cudaStream_t stream) {
  if (rows <= 0)
    return cudaSuccess;
  if (dim == 4096) {
    if (queries)
      launch_kernel<2>(rms_norm_4096_kernel<true>, unsigned(rows), 512, 0, stream, x, w, queries, y, image);
    else
      launch_kernel<2>(rms_norm_4096_kernel<false>, unsigned(rows), 512, 0, stream, x, w, nullptr, y, image);
    return cudaGetLastError();
  }
  if (queries)
    launch_kernel<2>(rms_norm_kernel<true>, unsigned(rows), 256, 0, stream, x, w, queries, int(dim), y, image);
  else
    launch_kernel<2>(rms_norm_kernel<false>, unsigned(rows), 256, 0, stream, x, w, nullptr, int(dim), y, image);
  return cudaGetLastError();
}

}  // namespace infdev
