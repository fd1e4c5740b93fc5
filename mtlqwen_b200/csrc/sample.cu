// On-GPU sampling, query packing and draft verification.
//
// sample_kernel <- sample_logits (native_ops.metal:122-224). The reference runs the temperature path on one
// thread (a serial insertion sort over 248,320 logits); here a block finds the top-k set with a radix select
// over the order-preserving integer image of logit/temperature, sorts those <= 64 candidates, and only the
// final <= 64-step softmax / top-p / inverse-CDF walk is serial, in exactly the reference's order.
// RNG: Philox4x32-10 keyed by the slot seed, counter = absolute index of the sampled token in its sequence,
// so a sequence draws the same variates whether it runs alone, batched or speculatively (the reference
// advances an xorshift64 state per sample and commits it on the host, engine.cpp:210-211).
#include "common.cuh"
#include "ops.h"

namespace infdev {
namespace {

constexpr int kThreads = 1024;
constexpr uint32_t kUnbound = 0xffffffffu;

__device__ __forceinline__ const infdev_query& query_of_logit(const infdev_query* queries, uint32_t row) {
  while (!queries->samples || row >= queries->logit + queries->samples)
    ++queries;
  return *queries;
}

__device__ __forceinline__ float philox_uniform(uint64_t key, uint64_t counter) {
  uint32_t c0 = uint32_t(counter), c1 = uint32_t(counter >> 32), c2 = 0, c3 = 0, k0 = uint32_t(key), k1 = uint32_t(key >> 32);
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const uint32_t h0 = __umulhi(0xD2511F53u, c0), l0 = 0xD2511F53u * c0, h1 = __umulhi(0xCD9E8D57u, c2), l1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = h1 ^ c1 ^ k0, n2 = h0 ^ c3 ^ k1;
    c0 = n0, c1 = l1, c2 = n2, c3 = l0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return float(c0 >> 8) * (1.0f / 16777216.0f);
}

// Order-preserving map float -> uint32 (larger float = larger key).
__device__ __forceinline__ uint32_t sortable(float v) {
  const uint32_t bits = __float_as_uint(v);
  return bits ^ ((bits & 0x80000000u) ? 0xffffffffu : 0x80000000u);
}

// grid (count), 1024 threads. mode 0: target sampling; mode 1: MTP drafting (always argmax, and bumps the
// drafter query's position, native_ops.metal:128-129).
__global__ void __launch_bounds__(kThreads) sample_kernel(const float* logits, int vocab, infdev_query* queries, uint32_t mode, int32_t* tokens) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t i = blockIdx.x;
  const int tid = threadIdx.x;
  const infdev_query info = query_of_logit(queries, i);
  const float* row = logits + size_t(i) * vocab;
  __shared__ float redValue[32];
  __shared__ int redIndex[32];
  __shared__ uint32_t histogram[256];
  __shared__ uint32_t selPrefix, selRemaining, candidateCount, tieCount;
  __shared__ float candValue[128];
  __shared__ int candIndex[128];

  if (mode == 1 && tid == 0) {
    infdev_query* q = queries;
    while (!q->samples || i >= q->logit + q->samples)
      ++q;
    ++q->position;
  }
  if (mode || info.temperature <= 0.f) {
    // first-index argmax (native_ops.metal:137-158)
    float best = -INFINITY;
    int index = 0;
    if (vocab % 4 == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {  // four logits per load, visited in ascending order
      const float4* row4 = reinterpret_cast<const float4*>(row);
#pragma unroll 4
      for (int j = tid; j < vocab / 4; j += kThreads) {
        const float4 v = row4[j];
        if (v.x > best)
          best = v.x, index = 4 * j;
        if (v.y > best)
          best = v.y, index = 4 * j + 1;
        if (v.z > best)
          best = v.z, index = 4 * j + 2;
        if (v.w > best)
          best = v.w, index = 4 * j + 3;
      }
    } else {
      for (int j = tid; j < vocab; j += kThreads) {
        const float v = row[j];
        if (v > best) {
          best = v;
          index = j;
        }
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, index, o);
      if (ov > best || (ov == best && oi < index)) {
        best = ov;
        index = oi;
      }
    }
    if ((tid & 31) == 0) {
      redValue[tid >> 5] = best;
      redIndex[tid >> 5] = index;
    }
    __syncthreads();
    if (tid < 32) {
      best = redValue[tid];
      index = redIndex[tid];
#pragma unroll
      for (int o = 16; o; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, index, o);
        if (ov > best || (ov == best && oi < index)) {
          best = ov;
          index = oi;
        }
      }
      if (tid == 0)
        tokens[i] = index;
    }
    return;
  }

  const float temperature = info.temperature;
  const float random = philox_uniform(info.seed, uint64_t(info.position) + info.count - info.samples + (i - info.logit) + 1);
  if (info.topK == 0) {
    // plain temperature sampling over the vocabulary, top-p ignored (native_ops.metal:172-188)
    float maximum = -INFINITY;
    for (int j = tid; j < vocab; j += kThreads)
      maximum = fmaxf(maximum, row[j] / temperature);
    maximum = warp_max(maximum);
    if ((tid & 31) == 0)
      redValue[tid >> 5] = maximum;
    __syncthreads();
    maximum = redValue[0];
    for (int w = 1; w < 32; ++w)
      maximum = fmaxf(maximum, redValue[w]);
    __syncthreads();
    // contiguous chunk per thread so the cumulative order is the vocabulary order
    const int chunk = (vocab + kThreads - 1) / kThreads, first = tid * chunk, last = min(vocab, first + chunk);
    double local = 0.0;
    for (int j = first; j < last; ++j)
      local += double(expf(row[j] / temperature - maximum));
    __shared__ double sums[kThreads];
    sums[tid] = local;
    __syncthreads();
    if (tid == 0) {
      double total = 0.0;
      for (int t = 0; t < kThreads; ++t)
        total += sums[t];
      const double target = double(random) * total;
      double cumulative = 0.0;
      int owner = kThreads - 1;
      for (int t = 0; t < kThreads; ++t) {
        if (cumulative + sums[t] >= target) {
          owner = t;
          break;
        }
        cumulative += sums[t];
      }
      int token = vocab - 1;
      const int a = owner * chunk, b = min(vocab, a + chunk);
      for (int j = a; j < b; ++j) {
        cumulative += double(expf(row[j] / temperature - maximum));
        if (cumulative >= target) {
          token = j;
          break;
        }
      }
      tokens[i] = token;
    }
    return;
  }

  // ---- top-k (<= 64) by radix select on the key of logit / temperature ----
  const uint32_t wanted = min(uint32_t(info.topK), 64u);
  if (tid == 0) {
    selPrefix = 0;
    selRemaining = wanted;
    candidateCount = 0;
    tieCount = 0;
  }
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256)
      histogram[tid] = 0;
    __syncthreads();
    const uint32_t prefix = selPrefix, prefixMask = pass ? (0xffffffffu << (shift + 8)) : 0u;
    for (int j = tid; j < vocab; j += kThreads) {
      const uint32_t key = sortable(row[j] / temperature);
      if ((key & prefixMask) == prefix)
        atomicAdd(&histogram[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t remaining = selRemaining;
      int bin = 255;
      for (; bin > 0; --bin) {
        if (histogram[bin] >= remaining)
          break;
        remaining -= histogram[bin];
      }
      selPrefix = prefix | (uint32_t(bin) << shift);
      selRemaining = remaining;
    }
    __syncthreads();
  }
  // selPrefix is now the key of the wanted-th largest value; selRemaining of the elements equal to it belong
  // to the set (the ones with the smallest indices, as the reference's stable insertion keeps the earliest).
  const uint32_t threshold = selPrefix;
  for (int j = tid; j < vocab; j += kThreads) {
    const float value = row[j] / temperature;
    const uint32_t key = sortable(value);
    if (key > threshold) {
      const uint32_t at = atomicAdd(&candidateCount, 1u);
      if (at < 64) {
        candValue[at] = value;
        candIndex[at] = j;
      }
    } else if (key == threshold) {
      const uint32_t at = atomicAdd(&tieCount, 1u);
      if (at < 64) {
        candValue[64 + at] = value;
        candIndex[64 + at] = j;
      }
    }
  }
  __syncthreads();
  if (tid == 0) {
    // ties at the threshold: take the earliest indices
    uint32_t count = min(candidateCount, 64u), need = selRemaining;
    if (tieCount <= 64) {
      for (uint32_t a = 1; a < tieCount; ++a) {  // order the ties by index
        const int x = candIndex[64 + a];
        int b = int(a) - 1;
        while (b >= 0 && candIndex[64 + b] > x) {
          candIndex[64 + b + 1] = candIndex[64 + b];
          --b;
        }
        candIndex[64 + b + 1] = x;
      }
      for (uint32_t a = 0; a < tieCount && need && count < 64; ++a, --need) {
        candValue[count] = candValue[64];
        candIndex[count] = candIndex[64 + a];
        ++count;
      }
    } else {  // more than 64 equal logits at the cut: serial scan in index order
      for (int j = 0; j < vocab && need && count < 64; ++j) {
        const float value = row[j] / temperature;
        if (sortable(value) == threshold) {
          candValue[count] = value;
          candIndex[count] = j;
          ++count;
          --need;
        }
      }
    }
    // insertion sort: value descending, index ascending
    for (uint32_t a = 1; a < count; ++a) {
      const float v = candValue[a];
      const int x = candIndex[a];
      int b = int(a) - 1;
      while (b >= 0 && (candValue[b] < v || (candValue[b] == v && candIndex[b] > x))) {
        candValue[b + 1] = candValue[b];
        candIndex[b + 1] = candIndex[b];
        --b;
      }
      candValue[b + 1] = v;
      candIndex[b + 1] = x;
    }
    const uint32_t kept = min(count, wanted);
    // softmax over the set, top-p cut, inverse CDF (native_ops.metal:208-223)
    float total = 0.f;
    for (uint32_t j = 0; j < kept; ++j)
      total += expf(candValue[j] - candValue[0]);
    const float limit = info.topP * total;
    float nucleus = 0.f;
    uint32_t keep = 0;
    do {
      nucleus += expf(candValue[keep] - candValue[0]);
      ++keep;
    } while (keep < kept && nucleus < limit);
    const float target = random * nucleus;
    float cumulative = 0.f;
    int token = candIndex[keep - 1];
    for (uint32_t j = 0; j < keep; ++j) {
      cumulative += expf(candValue[j] - candValue[0]);
      if (cumulative >= target) {
        token = candIndex[j];
        break;
      }
    }
    tokens[i] = token;
  }
}

// Finishes the per-query records of one pass on the device: forward()'s packing loop (forward.cpp:171-191).
// in[i] carries slot, count, position, state, sampling parameters, seed and (in `samples`) the slot's
// requested-token count; out gets start, samples, logit offsets and the state addresses.
// meta[0] = rows, meta[1] = logit rows, meta[2] = flags (1 sequential, 2 prefill).
__global__ void pack_queries_kernel(const infdev_query* in, int count, int drafting, uint32_t draftWidth, const uint64_t* statePrevious,
                                    const uint64_t* stateNext, uint64_t candidateBase, uint64_t stateBytes, infdev_query* out, uint32_t* meta) {
  pdl_launch_dependents();
  pdl_wait();
  // One lane per query (at most 32): the records and the state addresses live in host-visible memory, so every read is
  // a trip over PCIe; the lanes make theirs at the same time and the running totals come from a warp scan.
  const uint32_t lane = threadIdx.x;
  if (blockIdx.x || lane >= 32)
    return;
  infdev_query query = {};
  bool keep = false, speculative = false;
  if (int(lane) < count) {
    query = in[lane];
    speculative = query.state != kUnbound;
    keep = !(drafting && !speculative);
  }
  uint32_t flags = 0;
  if (keep) {
    const uint32_t requested = query.samples;
    if (drafting)
      query.count = 1;
    query.samples = drafting ? 1 : speculative ? query.count : (query.position + query.count == requested ? 1u : 0u);
    flags = ((speculative || query.count == 1) ? 1u : 0u) | ((!speculative && query.count > 1) ? 2u : 0u);
    query.previous = query.position ? statePrevious[query.slot] : 0;
    query.next = speculative ? candidateBase + uint64_t(query.state) * stateBytes : stateNext[query.slot];
  }
  // inclusive scans of rows, logit rows and kept queries over the lanes
  uint32_t rows = keep ? query.count : 0u, logits = keep ? query.samples : 0u, packed = keep ? 1u : 0u;
#pragma unroll
  for (int step = 1; step < 32; step <<= 1) {
    const uint32_t r = __shfl_up_sync(0xffffffffu, rows, step), l = __shfl_up_sync(0xffffffffu, logits, step), k = __shfl_up_sync(0xffffffffu, packed, step);
    if (int(lane) >= step)
      rows += r, logits += l, packed += k;
  }
  flags = __reduce_or_sync(0xffffffffu, flags);
  if (keep) {
    query.start = rows - query.count;
    query.logit = logits - query.samples;
    out[packed - 1] = query;
  }
  (void)draftWidth;
  if (lane == 31) {
    meta[0] = rows;
    meta[1] = logits;
    meta[2] = flags;
    meta[3] = packed;
  }
}

// The acceptance loop of Engine::schedule (engine.cpp:205-216) on the device, one thread per query. For query i it
// walks the sampled rows exactly as the host loop does: a sampled token is emitted; a stop token ends the walk after
// this token; a speculative query goes on to the next row only while the sampled token equals the drafter's proposal
// for that row and fewer than draftWidth proposals have been accepted. verdict[3 i .. 3 i + 2] = accepted proposals,
// emitted tokens, stopped (0 / 1). stops: [slot][stopStride] token ids, stopCounts[slot] of them valid.
__global__ void verify_drafts_kernel(const infdev_query* queries, int count, const int32_t* sampled, const int32_t* proposed, uint32_t draftWidth,
                                     const int32_t* stops, uint32_t stopStride, const uint32_t* stopCounts, uint32_t* verdict) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count)
    return;
  const infdev_query& query = queries[i];
  const bool speculative = query.state != kUnbound;
  const uint32_t column = speculative ? query.state / query.count : 0;
  uint32_t accepted = 0, emitted = 0, stopped = 0;
  for (uint32_t s = 0; s < query.samples && !stopped; ++s) {
    const int32_t token = sampled[query.logit + s];
    ++emitted;
    for (uint32_t k = 0; k < stopCounts[query.slot]; ++k)
      stopped |= stops[size_t(query.slot) * stopStride + k] == token ? 1u : 0u;
    if (!speculative || s == draftWidth || token != proposed[(s + 1) * 8 + column])
      break;
    ++accepted;
  }
  verdict[3 * i] = accepted;
  verdict[3 * i + 1] = emitted;
  verdict[3 * i + 2] = stopped;
}

// Copies the accepted candidate state row of each speculative query to the slot's next state buffer
// (engine.cpp:217-218), driven by the verdicts of verify_drafts_kernel. grid (chunks, queries).
__global__ void __launch_bounds__(256) commit_states_kernel(const infdev_query* queries, const uint32_t* verdict, const uint64_t* stateNext,
                                                            uint64_t candidateBase, uint64_t stateBytes) {
  pdl_launch_dependents();
  pdl_wait();
  const infdev_query& query = queries[blockIdx.y];
  if (query.state == kUnbound)
    return;
  const uint4* src = reinterpret_cast<const uint4*>(candidateBase + uint64_t(query.state + verdict[3 * blockIdx.y]) * stateBytes);
  uint4* dst = reinterpret_cast<uint4*>(stateNext[query.slot]);
  const size_t total = stateBytes / 16;
  for (size_t at = size_t(blockIdx.x) * blockDim.x + threadIdx.x; at < total; at += size_t(gridDim.x) * blockDim.x)
    dst[at] = src[at];
}

}  // namespace

cudaError_t sample_launch(const float* logits, int vocab, infdev_query* queries, int64_t count, uint32_t mode, int32_t* tokens,
                          cudaStream_t stream) {
  if (count <= 0)
    return cudaSuccess;
  launch_kernel(sample_kernel, unsigned(count), kThreads, 0, stream, logits, vocab, queries, mode, tokens);
  return cudaGetLastError();
}

cudaError_t pack_queries_launch(const infdev_query* in, int count, int drafting, uint32_t draftWidth, const uint64_t* statePrevious,
                                const uint64_t* stateNext, uint64_t candidateBase, uint64_t stateBytes, infdev_query* out, uint32_t* meta,
                                cudaStream_t stream) {
  launch_kernel(pack_queries_kernel, 1, 32, 0, stream, in, count, drafting, draftWidth, statePrevious, stateNext, candidateBase, stateBytes, out, meta);
  return cudaGetLastError();
}

cudaError_t verify_drafts_launch(const infdev_query* queries, int count, const int32_t* sampled, const int32_t* proposed, uint32_t draftWidth,
                                 const int32_t* stops, uint32_t stopStride, const uint32_t* stopCounts, uint32_t* verdict, cudaStream_t stream) {
  if (count <= 0)
    return cudaSuccess;
  launch_kernel(verify_drafts_kernel, 1, 32, 0, stream, queries, count, sampled, proposed, draftWidth, stops, stopStride, stopCounts, verdict);
  return cudaGetLastError();
}

cudaError_t commit_states_launch(const infdev_query* queries, int count, const uint32_t* verdict, const uint64_t* stateNext,
                                 uint64_t candidateBase, uint64_t stateBytes, cudaStream_t stream) {
  if (count <= 0)
    return cudaSuccess;
  launch_kernel(commit_states_kernel, dim3(64, unsigned(count)), 256, 0, stream, queries, verdict, stateNext, candidateBase, stateBytes);
  return cudaGetLastError();
}

}  // namespace infdev
