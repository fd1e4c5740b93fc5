// Gated delta-rule (GDN) layer kernels.
//
// gdn_prepare_kernel <- gdn_ba_prepare_4096x32 (native_ops.metal:89-113) and gdn_causal_conv_silu
//                      (fused_kernels.metal:202-232) in one launch
// delta_rule_kernel <- delta_rule_decode (delta_rule.metal:256-363) for every query length, fused with
//                      gated_rms_norm_128 (fused_kernels.metal:234-254).
//
// The recurrence keeps the whole 128x128 fp32 state of one (sequence, value head) in the registers of one
// CTA (256 threads x 64 values): it is read from HBM once, updated for every token of the query, and
// written once (or once per token for speculative queries, whose every row must stay selectable). The
// reference makes two passes over the state in device memory per token (delta_rule.metal:320-333, 351-360).
#include "act_image.cuh"
#include "kernels.h"
#include "ops.h"

namespace infdev {
namespace {

constexpr int kChannels = 8192, kHeadDim = 128, kValueHeads = 32, kKeyHeads = 16;
constexpr uint32_t kUnbound = 0xffffffffu;

// The four products of a gate dot-product step with the roundings spelled out: the preparation kernel and the fused
// decode kernel must agree bit for bit (a token's result may not depend on which kind of pass computed it), and the
// compiler is otherwise free to contract a.x*b.x + a.y*b.y + ... differently in the two.
__device__ __forceinline__ float dot4(const float4& a, const float4& b) {
  return __fmaf_rn(a.w, b.w, __fmaf_rn(a.z, b.z, __fmaf_rn(a.y, b.y, __fmul_rn(a.x, b.x))));
}

__device__ __forceinline__ const infdev_query& query_of_row(const infdev_query* queries, uint32_t row) {
  while (row >= queries->start + queries->count)
    ++queries;
  return *queries;
}

// gdn_prepare_kernel: both preparation steps of a GDN layer in one launch of 256-thread CTAs.
//  * CTAs [0, rows * 32): causal conv + SiLU, one thread per (row, channel). State layout: conv taps fp32 [8192][4]
//    at record + stateOffset.
//  * CTAs [rows * 32, rows * 32 + ceil(rows / 8) * 32): beta / g of eight rows and one value head: warps 0..3 share the
//    4096-long dot products with wBeta, warps 4..7 those with wAlpha; the head's weight rows are fetched once for the
//    eight rows (a CTA per row moved 32 KB of weights for 16 KB of input: 134 MB through the L2 per layer at 128 rows).
__global__ void __launch_bounds__(256) gdn_prepare_kernel(const float* x, const float* wBeta, const float* wAlpha, const float* A, const float* dt,
                                                          const float* mixed, const float* w, const infdev_query* queries, int rows,
                                                          uint64_t stateOffset, uint64_t stateBytes, float* q, float* k, float* v, float* beta,
                                                          float* g) {
  pdl_launch_dependents();
  pdl_wait();
  const int convBlocks = rows * (kChannels / 256);
  if (int(blockIdx.x) >= convBlocks) {
    const int item = blockIdx.x - convBlocks, row0 = (item / kValueHeads) * 8, head = item % kValueHeads;
    const int live = min(8, rows - row0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, which = warp >> 2, quarter = warp & 3;
    const float* weights = (which ? wAlpha : wBeta) + size_t(head) * 4096 + quarter * 1024;
    const float* src = x + size_t(row0) * 4096 + quarter * 1024;
    float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 b = *reinterpret_cast<const float4*>(weights + i * 128 + lane * 4);
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < live)
          sum[r] += dot4(*reinterpret_cast<const float4*>(src + size_t(r) * 4096 + i * 128 + lane * 4), b);
    }
    __shared__ float parts[8][8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const float total = warp_sum(sum[r]);
      if (lane == 0)
        parts[r][warp] = total;
    }
    __syncthreads();
    const int r = threadIdx.x & 127;
    if (r < live) {
      if (threadIdx.x < 128) {
        const float dot = (parts[r][0] + parts[r][1]) + (parts[r][2] + parts[r][3]);
        beta[(row0 + r) * kValueHeads + head] = 1.0f / (1.0f + expf(-dot));
      } else {
        const float dot = (parts[r][4] + parts[r][5]) + (parts[r][6] + parts[r][7]);
        g[(row0 + r) * kValueHeads + head] = A[head] * logf(1.0f + expf(dot + dt[head]));
      }
    }
    return;
  }
  const int64_t tid = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t row = tid / kChannels, c = tid % kChannels;
  const infdev_query& info = query_of_row(queries, uint32_t(row));
  const int64_t p = row - info.start;
  const bool speculative = info.state != kUnbound;
  const float* prev = reinterpret_cast<const float*>(info.previous + stateOffset);
  float context[4], acc = 0.f;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int64_t position = p - 3 + r;
    context[r] = position >= 0 ? mixed[(info.start + position) * kChannels + c] : info.previous ? prev[c * 4 + position + 4] : 0.f;
    acc = fmaf(context[r], w[c * 4 + r], acc);
  }
  const float value = silu_f(acc);
  if (c < 2048)
    q[row * 2048 + c] = value;
  else if (c < 4096)
    k[row * 2048 + c - 2048] = value;
  else
    v[row * 4096 + c - 4096] = value;
  if (speculative || p + 1 == info.count) {
    float* state = reinterpret_cast<float*>(info.next + stateOffset + (speculative ? uint64_t(p) * stateBytes : 0)) + c * 4;
    *reinterpret_cast<float4*>(state) = make_float4(context[0], context[1], context[2], context[3]);
  }
}

// grid (32 value heads, queries), 256 threads. Thread (part = tid/32, lane) owns S[k][4*lane .. 4*lane+3]
// for k = part + 8*i, i < 16.
// `image`, when not null, also receives the activation image of `out`. A 256-value block holds two heads, which two
// CTAs produce: each adds one to the block's entry in `counters` (zero between launches) after its stores, and the
// second to arrive reads both halves back and writes the block's image, then clears the entry.
// FUSED: the preparation of gdn_prepare_kernel happens here as well, for this CTA's channels only: the conv + SiLU of
// its 128 q, k and v channels (the taps of the q / k channels are written by the first of the two value heads that
// share a key head) and its beta / g dot products, with the same arithmetic and summation order; q, k, v, g, beta
// are then not read. One launch less per layer for passes without prefill chunks.
//
// What bounds a decode launch is latency, not bytes: all 256 CTAs are resident at once, so the time is the longest
// dependent chain of one CTA. The kernel therefore asks for everything up front and keeps block-wide barriers to two per
// token:
//  * before griddepcontrol.wait (these depend on nothing the preceding kernel writes): the gate-projection rows of the
//    head, the conv weights and taps go to shared memory with cp.async (no registers held while in flight), then the 64
//    KB state goes to registers; after the wait the token's input row follows. The small operands, which hit the L2,
//    arrive and are consumed while the state is still on its way from HBM.
//  * after the first barrier every thread derives the q / k norms and the two gates itself from the partial sums
//    (redundantly; a second barrier to broadcast them costs more than 256 threads repeating a few instructions);
//  * after the second barrier (partial products with the state) every warp sums the eight partials of its own four
//    columns, so each has delta and the output for them without another barrier; warp 0 alone normalises, gates and
//    stores the 128 outputs and runs the image protocol while the others update and store the state.
struct GdnInputs {
  const float *x, *wBeta, *wAlpha, *A, *dt, *mixed, *convWeight;
  uint64_t convStateOffset;
  bool ahead;  // the query table and the state records may be read before griddepcontrol.wait (see the kernel)
};

struct GdnStage {                      // dynamic shared memory of the fused form
  float4 x[1024];                      // the token's input row (4096 values)
  float4 wBeta[1024], wAlpha[1024];    // this head's rows of the two gate projections
  float4 window[3][kHeadDim];          // conv taps of this CTA's q, k and v channels, rolled forward token by token
  float4 convWeight[3][kHeadDim];
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

template <bool FUSED>
__global__ void __launch_bounds__(256, 2) delta_rule_kernel(const float* q, const float* k, const float* v, const float* g, const float* beta,
                                                         const float* z, const float* normWeight, const infdev_query* queries,
                                                         uint64_t stateOffset, uint64_t stateBytes, float* out, uint8_t* image, int* counters,
                                                         uint32_t chunkedFrom, GdnInputs in) {
  pdl_launch_dependents();
  // The weights never change. The query table and the state records were written by the first kernels of this pass and
  // by the pass before it: when only the GEMV kernels and their followers are launched early, those have completed
  // before the preceding kernel could start, and both may be read ahead of the wait. When every kernel of the pass is
  // launched early nothing bounds how far ahead this one runs, and it waits first.
  if (!in.ahead)
    pdl_wait();
  const infdev_query info = queries[blockIdx.y];
  const int head = blockIdx.x, keyHead = head % kKeyHeads, tid = threadIdx.x, part = tid >> 5, lane = tid & 31;
  const bool speculative = info.state != kUnbound;
  if (chunkedFrom && !speculative && info.count >= chunkedFrom)  // delta_rule_chunked_kernel takes this query
    return;
  extern __shared__ float4 stageRaw[];
  GdnStage& stage = *reinterpret_cast<GdnStage*>(stageRaw);
  __shared__ float qraw[kHeadDim], kraw[kHeadDim], vraw[kHeadDim], red[12], dots[8];
  __shared__ float4 partialPred[8][32], partialQ[8][32];
  const int channels[3] = {keyHead * kHeadDim + (tid & 127), 2048 + keyHead * kHeadDim + (tid & 127), 4096 + head * kHeadDim + (tid & 127)};
  float headA = 0.f, headDt = 0.f;

  if (FUSED) {
    const float4* wb = reinterpret_cast<const float4*>(in.wBeta + size_t(head) * 4096);
    const float4* wa = reinterpret_cast<const float4*>(in.wAlpha + size_t(head) * 4096);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      cp_async16(&stage.wBeta[tid + 256 * i], wb + tid + 256 * i);
      cp_async16(&stage.wAlpha[tid + 256 * i], wa + tid + 256 * i);
    }
    if (tid < kHeadDim) {
      const float4* taps = reinterpret_cast<const float4*>(info.previous + in.convStateOffset);
#pragma unroll
      for (int which = 0; which < 3; ++which) {
        cp_async16(&stage.convWeight[which][tid], reinterpret_cast<const float4*>(in.convWeight) + channels[which]);
        if (info.previous)
          cp_async16(&stage.window[which][tid], taps + channels[which]);
        else
          stage.window[which][tid] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    cp_async_commit();
    headA = in.A[head], headDt = in.dt[head];
  }

  float4 S[16];
  if (info.previous) {
    const float4* src = reinterpret_cast<const float4*>(info.previous + stateOffset) + size_t(head) * kHeadDim * 32;
#pragma unroll
    for (int i = 0; i < 16; ++i)
      S[i] = src[(part + 8 * i) * 32 + lane];
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      S[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (in.ahead)
    pdl_wait();

  for (uint32_t t = 0; t < info.count; ++t) {
    const size_t row = info.start + t;
    const size_t at = (row * kValueHeads + head) * kHeadDim + 4 * lane;  // warp 0: this lane's four outputs
    float qv = 0.f, kv = 0.f, vv = 0.f, decay = 0.f, betaValue = 0.f;
    if (FUSED) {
      float mixedNow[3] = {0.f, 0.f, 0.f};
      if (tid < kHeadDim) {
#pragma unroll
        for (int which = 0; which < 3; ++which)
          mixedNow[which] = in.mixed[row * kChannels + channels[which]];
      }
      const float4* xrow = reinterpret_cast<const float4*>(in.x + row * 4096);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        cp_async16(&stage.x[tid + 256 * i], xrow + tid + 256 * i);
      cp_async_commit();
      cp_async_wait_all();
      __syncthreads();
      // beta / g: warps 0..3 share the dot product with wBeta, warps 4..7 the one with wAlpha (as gdn_prepare_kernel)
      const float4* weights = ((part >> 2) ? stage.wAlpha : stage.wBeta) + (part & 3) * 256;
      const float4* src = stage.x + (part & 3) * 256;
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 a = src[i * 32 + lane], b = weights[i * 32 + lane];
        sum += dot4(a, b);
      }
      sum = warp_sum(sum);
      if (lane == 0)
        dots[part] = sum;
      if (tid < kHeadDim) {
        // causal conv + SiLU of this head's q, k and v channel `tid` (gdn_causal_conv_silu, fused_kernels.metal:202-232):
        // the window holds the three tokens before this one, oldest first in .y (.x is the tap that falls out)
        float values[3];
#pragma unroll
        for (int which = 0; which < 3; ++which) {
          const float4 taps = stage.window[which][tid], w4 = stage.convWeight[which][tid];
          const float4 context = make_float4(taps.y, taps.z, taps.w, mixedNow[which]);
          float acc = fmaf(context.x, w4.x, 0.f);
          acc = fmaf(context.y, w4.y, acc), acc = fmaf(context.z, w4.z, acc), acc = fmaf(context.w, w4.w, acc);
          values[which] = silu_f(acc);
          stage.window[which][tid] = context;
          if ((speculative || t + 1 == info.count) && (which == 2 || head < kKeyHeads)) {
            float* state = reinterpret_cast<float*>(info.next + in.convStateOffset + (speculative ? uint64_t(t) * stateBytes : 0)) + channels[which] * 4;
            *reinterpret_cast<float4*>(state) = context;
          }
        }
        qv = values[0], kv = values[1], vv = values[2];
      }
    } else {
      if (tid < kHeadDim) {
        qv = q[(row * kKeyHeads + keyHead) * kHeadDim + tid];
        kv = k[(row * kKeyHeads + keyHead) * kHeadDim + tid];
        vv = v[(row * kValueHeads + head) * kHeadDim + tid];
      }
      decay = expf(g[row * kValueHeads + head]);
      betaValue = beta[row * kValueHeads + head];
    }
    // L2-normalise q (scaled by 1/sqrt(128)) and k; q.k of the normalised vectors (delta_rule.metal:281-311).
    if (tid < kHeadDim) {
      qraw[tid] = qv, kraw[tid] = kv, vraw[tid] = vv;
      const float a = warp_sum(qv * qv), b = warp_sum(kv * kv), c = warp_sum(qv * kv);
      if (lane == 0) {
        red[part] = a;
        red[4 + part] = b;
        red[8 + part] = c;
      }
    }
    __syncthreads();
    float4 gate = make_float4(0.f, 0.f, 0.f, 0.f), weight = gate;
    if (part == 0 && z)  // needed after the next barrier; asked for here
      gate = *reinterpret_cast<const float4*>(z + at), weight = *reinterpret_cast<const float4*>(normWeight + 4 * lane);
    const float qn = rsqrtf(red[0] + red[1] + red[2] + red[3] + 1.0e-6f) * 0.08838834764831845f;
    const float kn = rsqrtf(red[4] + red[5] + red[6] + red[7] + 1.0e-6f);
    const float qk = (red[8] + red[9] + red[10] + red[11]) * qn * kn;
    if (FUSED) {
      const float dotBeta = (dots[0] + dots[1]) + (dots[2] + dots[3]), dotAlpha = (dots[4] + dots[5]) + (dots[6] + dots[7]);
      decay = expf(headA * logf(1.0f + expf(dotAlpha + headDt)));
      betaValue = 1.0f / (1.0f + expf(-dotBeta));
    }
    float4 pred = make_float4(0.f, 0.f, 0.f, 0.f), qstate = pred;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float kk = kraw[part + 8 * i] * kn, qq = qraw[part + 8 * i] * qn;
      S[i].x *= decay, S[i].y *= decay, S[i].z *= decay, S[i].w *= decay;
      pred.x = fmaf(S[i].x, kk, pred.x), pred.y = fmaf(S[i].y, kk, pred.y), pred.z = fmaf(S[i].z, kk, pred.z), pred.w = fmaf(S[i].w, kk, pred.w);
      qstate.x = fmaf(S[i].x, qq, qstate.x), qstate.y = fmaf(S[i].y, qq, qstate.y), qstate.z = fmaf(S[i].z, qq, qstate.z),
      qstate.w = fmaf(S[i].w, qq, qstate.w);
    }
    partialPred[part][lane] = pred;
    partialQ[part][lane] = qstate;
    __syncthreads();
    // every warp: the sums of the eight partials for its lanes' four columns, delta and the output there
    float4 p4 = make_float4(0.f, 0.f, 0.f, 0.f), s4 = p4;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const float4 a = partialPred[w][lane], b = partialQ[w][lane];
      p4.x += a.x, p4.y += a.y, p4.z += a.z, p4.w += a.w;
      s4.x += b.x, s4.y += b.y, s4.z += b.z, s4.w += b.w;
    }
    const float4 v4 = *reinterpret_cast<const float4*>(&vraw[4 * lane]);
    const float4 d4 = make_float4((v4.x - p4.x) * betaValue, (v4.y - p4.y) * betaValue, (v4.z - p4.z) * betaValue, (v4.w - p4.w) * betaValue);
    if (part == 0) {
      float4 o = make_float4(s4.x + d4.x * qk, s4.y + d4.y * qk, s4.z + d4.z * qk, s4.w + d4.w * qk);
      if (z) {  // gated_rms_norm_128
        const float scale = rsqrtf(warp_sum(o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w) / float(kHeadDim) + 1.0e-6f);
        o = make_float4(o.x * scale * weight.x * silu_f(gate.x), o.y * scale * weight.y * silu_f(gate.y), o.z * scale * weight.z * silu_f(gate.z),
                        o.w * scale * weight.w * silu_f(gate.w));
      }
      *reinterpret_cast<float4*>(out + at) = o;
      if (image && row < kImageCounters / (kValueHeads / 2)) {  // later rows have no counter and get no image
        const int entry = int(row) * (kValueHeads / 2) + (head >> 1);
        __syncwarp();
        int arrivals = 0;
        if (lane == 0) {
          __threadfence();
          arrivals = atomicAdd(&counters[entry], 1);
        }
        if (__shfl_sync(0xffffffffu, arrivals, 0) == 1) {
          __threadfence();
          const float* src = out + (row * kValueHeads + (head & ~1)) * kHeadDim + lane * 8;
          const float4 a = __ldcg(reinterpret_cast<const float4*>(src)), b = __ldcg(reinterpret_cast<const float4*>(src + 4));
          const float values[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
          image_store_block(image + (size_t(row >> 3) * (kValueHeads / 2) + (head >> 1)) * kImageBlockBytes, int(row & 7), lane, values);
          if (lane == 0)
            counters[entry] = 0;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float kk = kraw[part + 8 * i] * kn;
      S[i].x = fmaf(kk, d4.x, S[i].x), S[i].y = fmaf(kk, d4.y, S[i].y), S[i].z = fmaf(kk, d4.z, S[i].z), S[i].w = fmaf(kk, d4.w, S[i].w);
    }
    if (speculative || t + 1 == info.count) {
      float4* dst = reinterpret_cast<float4*>(info.next + stateOffset + (speculative ? uint64_t(t) * stateBytes : 0)) + size_t(head) * kHeadDim * 32;
#pragma unroll
      for (int i = 0; i < 16; ++i)
        dst[(part + 8 * i) * 32 + lane] = S[i];
    }
    if (t + 1 < info.count)
      __syncthreads();  // the shared arrays are rewritten for the next token
  }
}

// ---- chunked form for long prefill queries -----------------------------------------------------------
// Replaces delta_rule_prefill (delta_rule.metal:19-253): 16 tokens per step instead of one. With S0 the state
// before the chunk, d_t the decay of token t, G_t = d_0 ... d_t and R[t][i] = G_t / G_i, the recurrence of
// delta_rule_kernel unrolls to
//   delta_t = beta_t * (v_t - G_t * S0^T k_t - sum_{i<t} R[t][i] (k_i . k_t) delta_i)        (a unit lower-triangular system)
//   o_t     = G_t * S0^T q_t + sum_{i<=t} R[t][i] (k_i . q_t) delta_i
//   S       = G_15 * S0 + sum_i (G_15 / G_i) k_i delta_i^T
// All in fp32 on the CUDA cores, like the sequential kernel (so both agree to rounding): the two S0 products cost what
// 16 sequential steps cost, but a chunk needs 5 block-wide barriers instead of 64, which is what bounds a prefill query
// (one CTA per head, 128 dependent steps per pass).
// grid (32 value heads, queries), 256 threads, same state ownership as delta_rule_kernel; serves the non-speculative
// queries of at least `chunkedFrom` tokens. A last chunk of fewer than 16 tokens is padded with tokens of beta = 0,
// k = q = 0 and decay 1, which change nothing.
constexpr int kChunk = 16;
struct ChunkShared {
  float k[kChunk][kHeadDim + 4], q[kChunk][kHeadDim + 4], v[kChunk][kHeadDim];  // rows of k, q padded: column reads over 16 rows hit 16 banks
  float partialK[kChunk][8][kHeadDim], partialQ[kChunk][8][kHeadDim];  // per-warp partial S0^T k_t, S0^T q_t
  float ks[kChunk][kHeadDim], qs[kChunk][kHeadDim];                    // S0^T k_t, S0^T q_t
  float u[kChunk][kHeadDim], o[kChunk][kHeadDim];                      // (G_15 / G_t) delta_t, o_t
  float kk[kChunk][kChunk], qk[kChunk][kChunk];                        // R[t][i] (k_i . k_t), R[t][i] (k_i . q_t)
  float cumulative[kChunk], beta[kChunk];                              // log G_t, beta_t
};

__global__ void __launch_bounds__(256) delta_rule_chunked_kernel(const float* q, const float* k, const float* v, const float* g, const float* beta,
                                                                 const float* z, const float* normWeight, const infdev_query* queries,
                                                                 uint64_t stateOffset, float* out, uint32_t chunkedFrom) {
  pdl_launch_dependents();
  pdl_wait();
  const infdev_query info = queries[blockIdx.y];
  if (info.state != kUnbound || info.count < chunkedFrom)  // delta_rule_kernel takes this query
    return;
  extern __shared__ __align__(16) uint8_t chunkRaw[];
  ChunkShared& sh = *reinterpret_cast<ChunkShared*>(chunkRaw);
  const int head = blockIdx.x, keyHead = head % kKeyHeads, tid = threadIdx.x, part = tid >> 5, lane = tid & 31;

  float4 S[16];
  if (info.previous) {
    const float4* src = reinterpret_cast<const float4*>(info.previous + stateOffset) + size_t(head) * kHeadDim * 32;
#pragma unroll
    for (int i = 0; i < 16; ++i)
      S[i] = src[(part + 8 * i) * 32 + lane];
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      S[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }

  for (uint32_t first = 0; first < info.count; first += kChunk) {
    const uint32_t live = min(uint32_t(kChunk), info.count - first);
    // (a) normalised q (scaled by 1/sqrt(128)) and k, raw v, gates: warp w prepares tokens 2w and 2w+1
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint32_t t = 2 * part + j;
      float4 qv = make_float4(0.f, 0.f, 0.f, 0.f), kv = qv, vv = qv;
      if (t < live) {
        const size_t row = info.start + first + t;
        qv = *reinterpret_cast<const float4*>(q + (row * kKeyHeads + keyHead) * kHeadDim + 4 * lane);
        kv = *reinterpret_cast<const float4*>(k + (row * kKeyHeads + keyHead) * kHeadDim + 4 * lane);
        vv = *reinterpret_cast<const float4*>(v + (row * kValueHeads + head) * kHeadDim + 4 * lane);
      }
      const float qq = warp_sum(qv.x * qv.x + qv.y * qv.y + qv.z * qv.z + qv.w * qv.w);
      const float kq = warp_sum(kv.x * kv.x + kv.y * kv.y + kv.z * kv.z + kv.w * kv.w);
      const float qn = rsqrtf(qq + 1.0e-6f) * 0.08838834764831845f, kn = rsqrtf(kq + 1.0e-6f);
      *reinterpret_cast<float4*>(&sh.q[t][4 * lane]) = make_float4(qv.x * qn, qv.y * qn, qv.z * qn, qv.w * qn);
      *reinterpret_cast<float4*>(&sh.k[t][4 * lane]) = make_float4(kv.x * kn, kv.y * kn, kv.z * kn, kv.w * kn);
      *reinterpret_cast<float4*>(&sh.v[t][4 * lane]) = vv;
    }
    if (tid == 0) {
      float running = 0.f;
      for (uint32_t t = 0; t < kChunk; ++t) {
        const size_t row = info.start + first + t;
        running += t < live ? g[row * kValueHeads + head] : 0.f;
        sh.cumulative[t] = running;
        sh.beta[t] = t < live ? beta[row * kValueHeads + head] : 0.f;
      }
    }
    __syncthreads();
    // (b) per-warp partial products of the chunk's keys and queries with S0, and the token-by-token dot products
#pragma unroll 2
    for (int t = 0; t < kChunk; ++t) {
      float4 pk = make_float4(0.f, 0.f, 0.f, 0.f), pq = pk;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float kv = sh.k[t][part + 8 * i], qv = sh.q[t][part + 8 * i];
        pk.x = fmaf(S[i].x, kv, pk.x), pk.y = fmaf(S[i].y, kv, pk.y), pk.z = fmaf(S[i].z, kv, pk.z), pk.w = fmaf(S[i].w, kv, pk.w);
        pq.x = fmaf(S[i].x, qv, pq.x), pq.y = fmaf(S[i].y, qv, pq.y), pq.z = fmaf(S[i].z, qv, pq.z), pq.w = fmaf(S[i].w, qv, pq.w);
      }
      *reinterpret_cast<float4*>(&sh.partialK[t][part][4 * lane]) = pk;
      *reinterpret_cast<float4*>(&sh.partialQ[t][part][4 * lane]) = pq;
    }
    {
      const int t = tid >> 4, i = tid & 15;  // one (t, i) pair per thread
      float kk = 0.f, qk = 0.f;
      if (i <= t) {
#pragma unroll 8
        for (int d = 0; d < kHeadDim; d += 4) {
          const float4 a = *reinterpret_cast<const float4*>(&sh.k[i][d]), b = *reinterpret_cast<const float4*>(&sh.k[t][d]),
                       c = *reinterpret_cast<const float4*>(&sh.q[t][d]);
          kk += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
          qk += a.x * c.x + a.y * c.y + a.z * c.z + a.w * c.w;
        }
        const float ratio = expf(sh.cumulative[t] - sh.cumulative[i]);
        kk *= ratio, qk *= ratio;
      }
      sh.kk[t][i] = i < t ? kk : 0.f;
      sh.qk[t][i] = i <= t ? qk : 0.f;
    }
    __syncthreads();
    // (c) sum the eight partials: 2048 values each for ks and qs, eight per thread
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int at = tid + 256 * j, t = at >> 7, d = at & 127;
      float a = 0.f, b = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        a += sh.partialK[t][w][d];
        b += sh.partialQ[t][w][d];
      }
      sh.ks[t][d] = a;
      sh.qs[t][d] = b;
    }
    __syncthreads();
    // (d) one thread per value column: forward substitution for delta, then the outputs
    if (tid < kHeadDim) {
      const float last = sh.cumulative[kChunk - 1];
      float delta[kChunk];
#pragma unroll
      for (int t = 0; t < kChunk; ++t) {
        const float decay = expf(sh.cumulative[t]);
        float r = sh.v[t][tid] - decay * sh.ks[t][tid], o = decay * sh.qs[t][tid];
#pragma unroll
        for (int i = 0; i < t; ++i) {
          r = fmaf(-sh.kk[t][i], delta[i], r);
          o = fmaf(sh.qk[t][i], delta[i], o);
        }
        delta[t] = r * sh.beta[t];
        o = fmaf(sh.qk[t][t], delta[t], o);
        sh.u[t][tid] = delta[t] * expf(last - sh.cumulative[t]);
        sh.o[t][tid] = o;
      }
    }
    __syncthreads();
    // (e) new state, and the outputs of the chunk through the gated norm: warp w writes tokens 2w and 2w+1
    {
      const float decay = expf(sh.cumulative[kChunk - 1]);
#pragma unroll
      for (int i = 0; i < 16; ++i)
        S[i].x *= decay, S[i].y *= decay, S[i].z *= decay, S[i].w *= decay;
#pragma unroll 4
      for (int t = 0; t < kChunk; ++t) {
        const float4 u = *reinterpret_cast<const float4*>(&sh.u[t][4 * lane]);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float kv = sh.k[t][part + 8 * i];
          S[i].x = fmaf(kv, u.x, S[i].x), S[i].y = fmaf(kv, u.y, S[i].y), S[i].z = fmaf(kv, u.z, S[i].z), S[i].w = fmaf(kv, u.w, S[i].w);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint32_t t = 2 * part + j;
      if (t < live) {
        const size_t at = ((info.start + first + t) * kValueHeads + head) * kHeadDim + 4 * lane;
        float4 o = *reinterpret_cast<const float4*>(&sh.o[t][4 * lane]);
        if (z) {  // gated_rms_norm_128
          const float scale = rsqrtf(warp_sum(o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w) / float(kHeadDim) + 1.0e-6f);
          const float4 w = *reinterpret_cast<const float4*>(normWeight + 4 * lane), gate = *reinterpret_cast<const float4*>(z + at);
          o = make_float4(o.x * scale * w.x * silu_f(gate.x), o.y * scale * w.y * silu_f(gate.y), o.z * scale * w.z * silu_f(gate.z),
                          o.w * scale * w.w * silu_f(gate.w));
        }
        *reinterpret_cast<float4*>(out + at) = o;
      }
    }
    __syncthreads();  // the chunk's shared arrays are rewritten by the next chunk
  }
  float4* dst = reinterpret_cast<float4*>(info.next + stateOffset) + size_t(head) * kHeadDim * 32;
#pragma unroll
  for (int i = 0; i < 16; ++i)
    dst[(part + 8 * i) * 32 + lane] = S[i];
}

}  // namespace

cudaError_t gdn_prepare_launch(const float* x, const float* mixed, const float* wBeta, const float* wAlpha, const float* A, const float* dt,
                               const float* convWeight, const infdev_query* queries, int64_t rows, uint64_t stateOffset, uint64_t stateBytes,
                               float* q, float* k, float* v, float* beta, float* g, cudaStream_t stream) {
  if (rows <= 0)
    return cudaSuccess;
  launch_kernel<2>(gdn_prepare_kernel, unsigned(rows * (kChannels / 256) + (rows + 7) / 8 * kValueHeads), 256, 0, stream, x, wBeta, wAlpha, A, dt, mixed, convWeight, queries,
                int(rows), stateOffset, stateBytes, q, k, v, beta, g);
  return cudaGetLastError();
}

cudaError_t delta_rule_launch(const float* q, const float* k, const float* v, const float* g, const float* beta, const float* z,
                              const float* normWeight, const infdev_query* queries, int queryCount, uint64_t stateOffset, uint64_t stateBytes,
                              float* out, uint8_t* image, int* counters, uint32_t chunkedFrom, cudaStream_t stream) {
  if (queryCount <= 0)
    return cudaSuccess;
  if (chunkedFrom) {
    static PerDeviceOnce configured;
    if (cudaError_t e = configure_shared_memory(delta_rule_chunked_kernel, sizeof(ChunkShared), configured))
      return e;
    launch_kernel(delta_rule_chunked_kernel, dim3(kValueHeads, unsigned(queryCount)), 256, sizeof(ChunkShared), stream, q, k, v, g, beta, z, normWeight,
                  queries, stateOffset, out, chunkedFrom);
  }
  launch_kernel(delta_rule_kernel<false>, dim3(kValueHeads, unsigned(queryCount)), 256, 0, stream, q, k, v, g, beta, z, normWeight, queries, stateOffset,
                stateBytes, out, image, counters, chunkedFrom, GdnInputs{});
  return cudaGetLastError();
}

cudaError_t gdn_decode_launch(const float* x, const float* mixed, const float* wBeta, const float* wAlpha, const float* A, const float* dt,
                              const float* convWeight, const float* z, const float* normWeight, const infdev_query* queries, int queryCount,
                              uint64_t convStateOffset, uint64_t stateOffset, uint64_t stateBytes, float* out, uint8_t* image, int* counters,
                              cudaStream_t stream) {
  if (queryCount <= 0)
    return cudaSuccess;
  static PerDeviceOnce configured;
  if (cudaError_t e = configure_shared_memory(delta_rule_kernel<true>, sizeof(GdnStage), configured))
    return e;
  launch_kernel<1>(delta_rule_kernel<true>, dim3(kValueHeads, unsigned(queryCount)), 256, sizeof(GdnStage), stream, nullptr, nullptr, nullptr, nullptr, nullptr, z, normWeight,
                   queries, stateOffset, stateBytes, out, image, counters, 0u, GdnInputs{x, wBeta, wAlpha, A, dt, mixed, convWeight, convStateOffset, pdl_mode() != 1});
  return cudaGetLastError();
}

}  // namespace infdev
