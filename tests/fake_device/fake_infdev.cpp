// A host-only stand-in for the infdev_* device layer (include/infdev.h), for tests of the engine's host side:
// scheduler, K/V reservation, prefix-checkpoint cache, acceptance bookkeeping, error paths. It is linked with
// csrc/scheduler.cpp and csrc/forward_pass.cpp into tests/_build/libinfeng_fake.so and never into the product library.
//
// Memory is plain host memory. The arithmetic kernels do nothing; what the host logic can observe is emulated with a
// toy model whose "recurrent state" is a running hash of the tokens fed so far, kept in the first 8 bytes of a state
// record exactly where and when the real kernels update theirs (previous -> next, one snapshot per candidate row of a
// speculative query), and whose "logits" pick the token g(hash). The drafter proposes what the target will sample,
// except at positions with position % 4 == 3, so acceptance is partial. A wrong state record after a prefix restore, a
// wrong candidate row after a rejection or a wrong K/V binding count therefore changes the tokens or the counters.
//
// fake_infdev_fail_commits(n) makes the next n infdev_commit calls report a device failure. A commit takes
// fake_infdev_commit_delay_us (default 10 ms) so that, as on a GPU, a client that reads one token and cancels does so
// well before the next pass has finished.
#include <atomic>
#include <chrono>
#include <thread>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>
#include "../../include/infdev.h"

struct infdev_ctx {
  std::string error;
  std::atomic<uint64_t> launches{0};
  const int32_t* rowTokens = nullptr;  // set by infdev_gather_tokens
  uint64_t rowHash[128] = {};          // state hash after each packed row of the current target pass
  uint64_t carried[8] = {};            // drafter: hash chain of each speculative query across the drafting steps
};

namespace {

std::atomic<int> failingCommits{0}, commitDelayMicros{10000};
constexpr uint32_t kUnbound = 0xffffffffu;

uint64_t mix(uint64_t hash, int32_t token) {
  hash ^= uint64_t(uint32_t(token)) + 0x9e3779b97f4a7c15ull + (hash << 6) + (hash >> 2);
  hash *= 0x100000001b3ull;
  return hash ^ (hash >> 29);
}

int32_t pick(uint64_t hash, int64_t vocab) { return int32_t((hash >> 11) % uint64_t(vocab)); }

const infdev_query& query_of_logit(const infdev_query* queries, uint32_t row) {
  while (!queries->samples || row >= queries->logit + queries->samples)
    ++queries;
  return *queries;
}

// The layer-0 state update of a target pass: hash chain over the rows of every query.
void update_state(infdev_ctx* ctx, const infdev_query* queries, int count, uint64_t stateBytes) {
  for (int i = 0; i < count; ++i) {
    const infdev_query& q = queries[i];
    uint64_t hash = q.previous ? *reinterpret_cast<const uint64_t*>(q.previous) : 0;
    for (uint32_t p = 0; p < q.count; ++p) {
      hash = mix(hash, ctx->rowTokens[q.start + p]);
      ctx->rowHash[q.start + p] = hash;
      if (q.state != kUnbound)
        *reinterpret_cast<uint64_t*>(q.next + uint64_t(p) * stateBytes) = hash;
    }
    if (q.state == kUnbound)
      *reinterpret_cast<uint64_t*>(q.next) = hash;
  }
}

}  // namespace

extern "C" {

void fake_infdev_fail_commits(int count) { failingCommits = count; }
void fake_infdev_commit_delay_us(int micros) { commitDelayMicros = micros; }

infdev_ctx* infdev_create(int, char*) { return new infdev_ctx; }
void infdev_destroy(infdev_ctx* ctx) { delete ctx; }
const char* infdev_error(infdev_ctx* ctx) { return ctx->error.c_str(); }
int infdev_sm_count(infdev_ctx*) { return 1; }
uint64_t infdev_launch_count(infdev_ctx* ctx) { return ctx->launches; }
void* infdev_alloc(infdev_ctx*, size_t bytes, int) { return std::calloc(bytes ? bytes : 16, 1); }
void infdev_free(infdev_ctx*, void* pointer) { std::free(pointer); }
int infdev_upload(infdev_ctx*, void* device, const void* host, size_t bytes) { return std::memcpy(device, host, bytes), 0; }
int infdev_download(infdev_ctx*, void* host, const void* device, size_t bytes) { return std::memcpy(host, device, bytes), 0; }
int infdev_peek(infdev_ctx*, void* host, const void* device, size_t bytes) { return std::memcpy(host, device, bytes), 0; }
int infdev_copy(infdev_ctx*, void* destination, const void* source, size_t bytes) { return std::memmove(destination, source, bytes), 0; }
int infdev_fill(infdev_ctx*, void* device, int byte, size_t bytes) { return std::memset(device, byte, bytes), 0; }
int infdev_commit(infdev_ctx* ctx, uint32_t) {
  std::this_thread::sleep_for(std::chrono::microseconds(commitDelayMicros.load()));
  if (failingCommits > 0) {
    --failingCommits;
    ctx->error = "injected device failure";
    return INFDEV_E_DEVICE;
  }
  return 0;
}
void* infdev_event_create(infdev_ctx*) { return std::malloc(1); }
void infdev_event_destroy(infdev_ctx*, void* event) { std::free(event); }
int infdev_event_record(infdev_ctx*, void*) { return 0; }
float infdev_event_elapsed_ms(infdev_ctx*, void*, void*) { return 0.001f; }
int infdev_graph_begin(infdev_ctx* ctx) { return ctx->error = "the fake device records no graphs", INFDEV_E_ARGUMENT; }
void* infdev_graph_end(infdev_ctx*) { return nullptr; }
int infdev_graph_launch(infdev_ctx*, void*) { return INFDEV_E_ARGUMENT; }
void infdev_graph_destroy(infdev_ctx*, void*) {}
size_t infdev_image_bytes(int64_t rows, int64_t k) { return size_t((rows + 7) / 8) * size_t(k / 256) * 4384; }
int infdev_image_capture(infdev_ctx*, uint8_t*) { return 0; }
int infdev_image_supply(infdev_ctx*, const uint8_t*) { return 0; }
int infdev_set_umma(infdev_ctx*, int) { return 0; }
size_t infdev_attention_scratch_bytes(int64_t rows, uint32_t maxSplits) { return size_t(rows) * 16 * maxSplits * 260 * sizeof(float); }

int infdev_linear(infdev_ctx* ctx, int, const void*, int64_t, int64_t, const float*, int64_t, float*, const float*) { return ++ctx->launches, 0; }
int infdev_linear_group(infdev_ctx* ctx, int, int, const void* const*, const int64_t*, int64_t, const float*, int64_t, float* const*) {
  return ++ctx->launches, 0;
}
int infdev_gate_up(infdev_ctx* ctx, int, const void*, const void*, int64_t, int64_t, const float*, int64_t, float*) { return ++ctx->launches, 0; }
int infdev_embedding(infdev_ctx* ctx, int, const void*, int64_t, const int32_t*, int64_t, float*) { return ++ctx->launches, 0; }
int infdev_dequant(infdev_ctx* ctx, int, const void*, int64_t, float*) { return ++ctx->launches, 0; }
int infdev_rms_norm(infdev_ctx* ctx, const float*, const float*, int64_t, int64_t, float*) { return ++ctx->launches, 0; }
int infdev_rms_norm_gather(infdev_ctx* ctx, const float*, const float*, const infdev_query*, int, int64_t, float*) { return ++ctx->launches, 0; }
int infdev_rope_table(infdev_ctx*, int64_t, float*) { return 0; }
int infdev_attention_prepare(infdev_ctx* ctx, const float*, const float*, const float*, const float*, const float*, const float*, const infdev_query*,
                             int, int64_t, const int32_t*, int32_t, int32_t, float*, void*, void*) {
  return ++ctx->launches, 0;
}
int infdev_attention(infdev_ctx* ctx, const float*, const float*, const void*, const void*, const infdev_query*, int, int64_t, const int32_t*, int32_t,
                     int32_t, uint32_t, float*, float*) {
  return ++ctx->launches, 0;
}
int infdev_mtp_fuse(infdev_ctx* ctx, const float*, const float*, const infdev_query*, int, const float*, const float*, int64_t, uint32_t, uint64_t,
                    uint64_t, float*) {
  return ++ctx->launches, 0;
}

int infdev_gather_tokens(infdev_ctx* ctx, const infdev_query* queries, int queryCount, const int32_t* requestData, uint32_t capacity,
                         const int32_t* proposals, uint32_t mode, int32_t* rowTokens) {
  for (int q = 0; q < queryCount; ++q) {
    const infdev_query& info = queries[q];
    for (uint32_t p = 0; p < info.count; ++p) {
      const uint32_t row = info.start + p;
      if (mode == 2)
        rowTokens[row] = proposals[row];
      else if (info.state != kUnbound && p)
        rowTokens[row] = proposals[p * 8 + info.state / info.count];
      else
        rowTokens[row] = requestData[size_t(info.slot) * capacity + info.position + p];
    }
  }
  ctx->rowTokens = rowTokens;
  return ++ctx->launches, 0;
}

// The first GDN layer of a pass (its conv taps sit at offset 0 of a record) advances the toy state.
int infdev_gdn_prepare(infdev_ctx* ctx, const float*, const float*, const float*, const float*, const float*, const float*, const float*,
                       const infdev_query*, int, int64_t, uint64_t, uint64_t, float*, float*, float*, float*, float*) {
  return ++ctx->launches, 0;
}
int infdev_delta_rule(infdev_ctx* ctx, const float*, const float*, const float*, const float*, const float*, const float*, const float*,
                      const infdev_query* queries, int queryCount, uint64_t stateOffset, uint64_t stateBytes, float*) {
  if (stateOffset == INFDEV_CONV_STATE_BYTES)
    update_state(ctx, queries, queryCount, stateBytes);
  return ++ctx->launches, 0;
}
int infdev_delta_rule_prefill(infdev_ctx* ctx, const float* q, const float* k, const float* v, const float* g, const float* beta, const float* z,
                              const float* normWeight, const infdev_query* queries, int queryCount, uint64_t stateOffset, uint64_t stateBytes,
                              float* out) {
  return infdev_delta_rule(ctx, q, k, v, g, beta, z, normWeight, queries, queryCount, stateOffset, stateBytes, out);
}
int infdev_gdn_decode(infdev_ctx* ctx, const float*, const float*, const float*, const float*, const float*, const float*, const float*, const float*,
                      const float*, const infdev_query* queries, int queryCount, uint64_t convStateOffset, uint64_t, uint64_t stateBytes, float*) {
  if (convStateOffset == 0)
    update_state(ctx, queries, queryCount, stateBytes);
  return ++ctx->launches, 0;
}

int infdev_sample(infdev_ctx* ctx, const float*, int64_t vocab, infdev_query* queries, int, int64_t count, uint32_t mode, int32_t* tokens) {
  for (uint32_t i = 0; i < uint32_t(count); ++i) {
    infdev_query& q = const_cast<infdev_query&>(query_of_logit(queries, i));
    if (mode == 1) {
      // Drafting: one row per speculative query. Its chain was started from the slot's committed state when the
      // drafter frame was packed and is fed the anchor token, then the drafter's own proposals: exactly the hashes
      // the target will see on its candidate rows, so the proposal is what the target will sample there. The token at
      // every position with position % 4 == 3 is proposed wrongly on purpose.
      uint64_t& chain = ctx->carried[q.start];
      chain = mix(chain, ctx->rowTokens[q.start]);
      int32_t proposal = pick(chain, vocab);
      if ((q.position + 1) % 4 == 3)
        proposal = (proposal + 1) % int32_t(vocab);
      tokens[i] = proposal;
      ++q.position;
    } else {
      const uint32_t row = q.start + q.count - q.samples + (i - q.logit);
      tokens[i] = pick(ctx->rowHash[row], vocab);
    }
  }
  return ++ctx->launches, 0;
}

int infdev_pack_queries(infdev_ctx* ctx, const infdev_query* in, int count, int drafting, uint32_t, const uint64_t* statePrevious,
                        const uint64_t* stateNext, uint64_t candidateBase, uint64_t stateBytes, infdev_query* out, uint32_t* meta) {
  uint32_t rows = 0, logits = 0, flags = 0, packed = 0;
  for (int i = 0; i < count; ++i) {
    infdev_query query = in[i];
    const bool speculative = query.state != kUnbound;
    if (drafting && !speculative)
      continue;
    const uint32_t requested = query.samples;
    query.start = rows;
    if (drafting)
      query.count = 1;
    query.samples = drafting ? 1 : speculative ? query.count : (query.position + query.count == requested ? 1u : 0u);
    flags |= (speculative || query.count == 1) ? 1u : 0u;
    flags |= (!speculative && query.count > 1) ? 2u : 0u;
    query.previous = query.position ? statePrevious[query.slot] : 0;
    query.next = speculative ? candidateBase + uint64_t(query.state) * stateBytes : stateNext[query.slot];
    query.logit = logits;
    if (drafting)  // the drafter's hash chain restarts from the slot's committed state
      ctx->carried[packed] = query.previous ? *reinterpret_cast<const uint64_t*>(query.previous) : 0;
    out[packed++] = query;
    logits += query.samples;
    rows += query.count;
  }
  meta[0] = rows, meta[1] = logits, meta[2] = flags, meta[3] = packed;
  return ++ctx->launches, 0;
}

int infdev_verify_drafts(infdev_ctx* ctx, const infdev_query* queries, int count, const int32_t* sampled, const int32_t* proposed,
                         uint32_t draftWidth, const int32_t* stops, uint32_t stopStride, const uint32_t* stopCounts, uint32_t* verdict) {
  for (int i = 0; i < count; ++i) {
    const infdev_query& query = queries[i];
    const bool speculative = query.state != kUnbound;
    uint32_t accepted = 0, emitted = 0, stopped = 0;
    for (uint32_t s = 0; s < query.samples && !stopped; ++s) {
      const int32_t token = sampled[query.logit + s];
      ++emitted;
      for (uint32_t k = 0; k < stopCounts[query.slot]; ++k)
        stopped |= stops[size_t(query.slot) * stopStride + k] == token;
      if (!speculative || s == draftWidth || token != proposed[(s + 1) * 8 + query.state / query.count])
        break;
      ++accepted;
    }
    verdict[3 * i] = accepted, verdict[3 * i + 1] = emitted, verdict[3 * i + 2] = stopped;
  }
  return ++ctx->launches, 0;
}

int infdev_commit_states(infdev_ctx* ctx, const infdev_query* queries, int count, const uint32_t* verdict, const uint64_t* stateNext,
                         uint64_t candidateBase, uint64_t stateBytes) {
  for (int i = 0; i < count; ++i)
    if (queries[i].state != kUnbound)
      std::memcpy(reinterpret_cast<void*>(stateNext[queries[i].slot]),
                  reinterpret_cast<const void*>(candidateBase + uint64_t(queries[i].state + verdict[3 * i]) * stateBytes), stateBytes);
  return ++ctx->launches, 0;
}

}  // extern "C"
