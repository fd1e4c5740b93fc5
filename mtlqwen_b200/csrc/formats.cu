// The GGUF block formats of the real Qwen3.5 files beyond Q4_K / Q6_K: Q5_K, Q8_0, IQ4_XS (and plain F16).
//
// Replaces dequant_tile for q5_k / q8_0 / iq4_xs (quant_linear.metal:50-67, 87-115), linear_decode_q5_k and
// linear_decode_q8_0 (:329-434, 514-570), the q5_k / iq4_xs variants of mlp_gate_up (fused_kernels.metal:80-200) and the
// embedding gather for tables of these types. The synthetic benchmark models are all Q4_K / Q6_K, so these kernels
// are written for correctness and moderate speed, not for the roofline: one warp per weight row, the row's blocks
// dequantised in registers (bit-exact with the CPU oracle's values), fp32 multiply-adds against up to 8 activation rows
// at a time, a shuffle reduction, and the residual add or SiLU * up epilogue.
#include "common.cuh"
#include "ops.h"

namespace infdev {
namespace {

constexpr int kF16 = 1, kQ8_0 = 8, kQ5K = 13, kIQ4XS = 23;

__device__ __forceinline__ float half_at(const uint8_t* p) { return __half2float(*reinterpret_cast<const __half*>(p)); }

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

__constant__ float kIq4nl[16] = {-127.0f, -104.0f, -83.0f, -65.0f, -49.0f, -35.0f, -22.0f, -10.0f, 1.0f, 13.0f, 25.0f, 38.0f, 53.0f, 69.0f, 89.0f, 113.0f};

template <int TYPE> struct Format;
template <> struct Format<kQ5K> {
  static constexpr int kBytes = 176, kValues = 256;
  // Element r of a super-block, in the multiplication order of dequant_tile (quant_linear.metal:57-64), no contraction.
  static __device__ __forceinline__ float element(const uint8_t* b, int r) {
    const float d = half_at(b), dm = half_at(b + 2);
    int sc, mn;
    scale_min_k4(r >> 5, b + 4, sc, mn);
    const uint8_t q = b[48 + (r >> 6) * 32 + (r & 31)], hm = b[16 + (r & 31)];
    const int v = ((r & 32) ? (q >> 4) : (q & 15)) + ((hm & (1u << (r >> 5))) ? 16 : 0);
    return __fsub_rn(__fmul_rn(__fmul_rn(d, float(sc)), float(v)), __fmul_rn(dm, float(mn)));
  }
};
template <> struct Format<kQ8_0> {
  static constexpr int kBytes = 34, kValues = 32;
  static __device__ __forceinline__ float element(const uint8_t* b, int r) { return __fmul_rn(half_at(b), float(int8_t(b[2 + r]))); }
};
template <> struct Format<kIQ4XS> {
  static constexpr int kBytes = 136, kValues = 256;
  static __device__ __forceinline__ float element(const uint8_t* b, int r) {
    const int j = r >> 5, l = r & 31;
    const unsigned sh = unsigned(b[2]) | (unsigned(b[3]) << 8);
    const int ls = int((b[4 + (j >> 1)] >> (4 * (j & 1))) & 15) | int(((sh >> (2 * j)) & 3) << 4);
    const uint8_t q = b[8 + j * 16 + (l & 15)];
    return __fmul_rn(__fmul_rn(half_at(b), float(ls - 32)), kIq4nl[(l & 16) ? (q >> 4) : (q & 15)]);
  }
};
template <> struct Format<kF16> {
  static constexpr int kBytes = 512, kValues = 256;  // "block" = 256 consecutive halves
  static __device__ __forceinline__ float element(const uint8_t* b, int r) { return half_at(b + 2 * r); }
};

template <int TYPE> __global__ void __launch_bounds__(256) format_dequant_kernel(const uint8_t* blocks, int64_t count, float* out) {
  using F = Format<TYPE>;
  const int64_t item = int64_t(blockIdx.x) * 256 + threadIdx.x;
  if (item >= count * F::kValues)
    return;
  out[item] = F::element(blocks + (item / F::kValues) * F::kBytes, int(item % F::kValues));
}

template <int TYPE> __global__ void __launch_bounds__(256) format_embedding_kernel(const uint8_t* table, int k, const int32_t* tokens, float* out) {
  using F = Format<TYPE>;
  pdl_launch_dependents();
  pdl_wait();
  const int64_t row = blockIdx.y, token = tokens[row];
  const int column = blockIdx.x * 256 + threadIdx.x;
  if (column >= k)
    return;
  const uint8_t* source = table + token * int64_t(k / F::kValues) * F::kBytes;
  out[row * k + column] = F::element(source + int64_t(column / F::kValues) * F::kBytes, column % F::kValues);
}

// One warp per weight row (or per gate / up row pair), up to 8 activation rows per launch. Lane l takes the 8 consecutive
// values 8 l .. 8 l + 7 of every 256-value span of the row.
template <int TYPE, int NMAT>
__global__ void __launch_bounds__(256) format_gemv_kernel(const uint8_t* w, const uint8_t* w2, int64_t n, int k, const float* x, int m, float* y,
                                                          const float* residual) {
  using F = Format<TYPE>;
  pdl_launch_dependents();
  pdl_wait();
  const int64_t row = int64_t(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n)
    return;
  const int64_t rowBytes = int64_t(k / F::kValues) * F::kBytes;
  float acc[NMAT][8];
#pragma unroll
  for (int mat = 0; mat < NMAT; ++mat)
#pragma unroll
    for (int r = 0; r < 8; ++r)
      acc[mat][r] = 0.f;
  for (int base = 0; base < k; base += 256) {
    const int first = base + lane * 8;
    float values[NMAT][8];
#pragma unroll
    for (int mat = 0; mat < NMAT; ++mat) {
      const uint8_t* source = (mat ? w2 : w) + row * rowBytes;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        values[mat][i] = F::element(source + int64_t((first + i) / F::kValues) * F::kBytes, (first + i) % F::kValues);
    }
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (r < m) {
        const float4 a = *reinterpret_cast<const float4*>(x + int64_t(r) * k + first), b = *reinterpret_cast<const float4*>(x + int64_t(r) * k + first + 4);
#pragma unroll
        for (int mat = 0; mat < NMAT; ++mat) {
          float sum = acc[mat][r];
          sum = fmaf(values[mat][0], a.x, sum), sum = fmaf(values[mat][1], a.y, sum), sum = fmaf(values[mat][2], a.z, sum), sum = fmaf(values[mat][3], a.w, sum);
          sum = fmaf(values[mat][4], b.x, sum), sum = fmaf(values[mat][5], b.y, sum), sum = fmaf(values[mat][6], b.z, sum), sum = fmaf(values[mat][7], b.w, sum);
          acc[mat][r] = sum;
        }
      }
  }
#pragma unroll
  for (int r = 0; r < 8; ++r)
    if (r < m) {
      const float first = warp_sum(acc[0][r]);
      const float second = NMAT == 2 ? warp_sum(acc[NMAT - 1][r]) : 0.f;
      if (lane == 0) {
        const int64_t at = int64_t(r) * n + row;
        y[at] = NMAT == 2 ? silu_f(first) * second : residual ? first + residual[at] : first;
      }
    }
}

template <int TYPE> cudaError_t gemv_for(bool pair, const void* w, const void* w2, int64_t n, int64_t k, const float* x, int64_t m, float* y,
                                         const float* residual, cudaStream_t stream) {
  const auto* a = static_cast<const uint8_t*>(w);
  const auto* b = static_cast<const uint8_t*>(w2);
  for (int64_t row = 0; row < m; row += 8) {  // more than 8 activation rows: slices that re-read the weights from L2
    const int rows = int(m - row < 8 ? m - row : 8);
    const float* res = residual ? residual + row * n : nullptr;
    if (pair)
      launch_kernel(format_gemv_kernel<TYPE, 2>, unsigned((n + 7) / 8), 256, 0, stream, a, b, n, int(k), x + row * k, rows, y + row * n, res);
    else
      launch_kernel(format_gemv_kernel<TYPE, 1>, unsigned((n + 7) / 8), 256, 0, stream, a, b, n, int(k), x + row * k, rows, y + row * n, res);
  }
  return cudaGetLastError();
}

}  // namespace

bool format_supported(int type) { return type == kQ5K || type == kQ8_0 || type == kIQ4XS; }
int format_block_values(int type) { return type == kQ8_0 ? 32 : 256; }

cudaError_t format_dequant_launch(int type, const void* blocks, int64_t count, float* out, cudaStream_t stream) {
  if (count <= 0)
    return cudaSuccess;
  const auto* source = static_cast<const uint8_t*>(blocks);
  const unsigned grid = unsigned((count * format_block_values(type) + 255) / 256);
  switch (type) {
    case kQ5K: format_dequant_kernel<kQ5K><<<grid, 256, 0, stream>>>(source, count, out); break;
    case kQ8_0: format_dequant_kernel<kQ8_0><<<grid, 256, 0, stream>>>(source, count, out); break;
    case kIQ4XS: format_dequant_kernel<kIQ4XS><<<grid, 256, 0, stream>>>(source, count, out); break;
    case kF16: format_dequant_kernel<kF16><<<grid, 256, 0, stream>>>(source, count, out); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t format_embedding_launch(int type, const void* table, int64_t k, const int32_t* tokens, int64_t rows, float* out, cudaStream_t stream) {
  if (rows <= 0)
    return cudaSuccess;
  const dim3 grid(unsigned((k + 255) / 256), unsigned(rows));
  const auto* source = static_cast<const uint8_t*>(table);
  switch (type) {
    case kQ5K: launch_kernel(format_embedding_kernel<kQ5K>, grid, 256, 0, stream, source, int(k), tokens, out); break;
    case kQ8_0: launch_kernel(format_embedding_kernel<kQ8_0>, grid, 256, 0, stream, source, int(k), tokens, out); break;
    case kIQ4XS: launch_kernel(format_embedding_kernel<kIQ4XS>, grid, 256, 0, stream, source, int(k), tokens, out); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

// y[m,n] = x[m,k] . W[n,k]^T (+ residual), or silu(x . W^T) * (x . W2^T) for a pair; launches ceil(m / 8) kernels.
cudaError_t format_linear_launch(int type, bool pair, const void* w, const void* w2, int64_t n, int64_t k, const float* x, int64_t m, float* y,
                                 const float* residual, cudaStream_t stream) {
  switch (type) {
    case kQ5K: return gemv_for<kQ5K>(pair, w, w2, n, k, x, m, y, residual, stream);
    case kQ8_0: return gemv_for<kQ8_0>(pair, w, w2, n, k, x, m, y, residual, stream);
    case kIQ4XS: return gemv_for<kIQ4XS>(pair, w, w2, n, k, x, m, y, residual, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace infdev
