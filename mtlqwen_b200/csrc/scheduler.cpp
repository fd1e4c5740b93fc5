// Engine lifetime, the continuous-batching scheduler thread, K/V block reservation, the prefix-checkpoint
// cache, the commit of sampled tokens, and the infeng_* C ABI. CUDA build of runtime/engine.cpp: the
// behaviour (batch composition, 512-token checkpoint boundaries, LRU block eviction, acceptance rule,
// error codes) follows the reference; the Metal device underneath is replaced by infdev.
#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include "../../include/infeng.h"
#include "runtime.hpp"

namespace infeng::qwen35 {
namespace {

// Chains one 512-token block into a prefix hash (hashCheckpoint, engine.cpp:9-16).
uint64_t hashCheckpoint(uint64_t hash, const int32_t* tokens) {
  hash ^= 0x9e3779b97f4a7c15ull;
  for (uint32_t i = 0; i < checkpointTokens; ++i) {
    hash ^= uint32_t(tokens[i]) + 0x9e3779b9u + (hash << 6) + (hash >> 2);
    hash *= 0x100000001b3ull;
  }
  return hash;
}

uint32_t environment(const char* name, uint32_t fallback) {
  const char* text = std::getenv(name);
  return text && *text ? uint32_t(std::strtoul(text, nullptr, 10)) : fallback;
}

// splitmix64: spreads (base seed, creation index) over the 64-bit Philox key space.
uint64_t mixSeed(uint64_t value) {
  value += 0x9e3779b97f4a7c15ull;
  value = (value ^ (value >> 30)) * 0xbf58476d1ce4e5b9ull;
  value = (value ^ (value >> 27)) * 0x94d049bb133111ebull;
  return value ^ (value >> 31);
}

int deviceIndex() {
  if (const char* text = std::getenv("INFENG_DEVICE"))
    return std::atoi(text);
  if (const char* text = std::getenv("LOCAL_RANK"))
    return std::atoi(text);
  return 0;
}

}  // namespace

// Binds the next logical block of a sequence to a physical block (Engine::bind, engine.cpp:18-22).
void Engine::bind(Sequence& sequence, uint32_t physical) {
  kv->map(sequence.slot * kv->tableStride() + uint32_t(sequence.bindings.size()), physical);
  sequence.bindings.push_back(physical);
  ++blocks[physical].refs;
}

// Makes sure every block the batch will touch is bound, evicting the least recently used unreferenced block
// when a sequence grows; false if no block can be freed (Engine::reserve, engine.cpp:24-46).
bool Engine::reserve(const Batch& batch) {
  for (uint32_t i = 0; i < batch.size; ++i) {
    const infdev_query& query = batch.queries[i];
    Sequence& sequence = *sequences[query.slot];
    const uint32_t first = sequence.kvValid / blockTokens, last = (sequence.kvValid + query.count - 1) / blockTokens;
    for (uint32_t logical = first; logical <= last; ++logical) {
      if (logical == sequence.bindings.size()) {
        uint32_t victim = 0;
        uint64_t oldest = UINT64_MAX;
        bool found = false;
        for (uint32_t b = 0; b < blocks.size(); ++b)
          if (!blocks[b].refs && (!found || blocks[b].touch < oldest)) {
            victim = b;
            oldest = blocks[b].touch;
            found = true;
          }
        if (!found)
          return false;
        kv->ensure(victim + 1);
        // A checkpoint that references the evicted block can no longer be restored.
        for (auto entry = checkpointCache.begin(); entry != checkpointCache.end();)
          if (std::find(entry->bindings.begin(), entry->bindings.end(), victim) != entry->bindings.end()) {
            retire(entry->arena);
            entry = checkpointCache.erase(entry);
          } else
            ++entry;
        bind(sequence, victim);
      }
      blocks[sequence.bindings[logical]].touch = ++clock;
    }
  }
  return true;
}

// Drops a reference to a state record; the last one hands the record to the spare list instead of the driver.
void Engine::retire(Tensor& state) {
  if (state.buffer && state.buffer.use_count() == 1 && state.offset == 0 && state.bytes == stateBytes && spareStates.size() < 3 * maxBatchSequences)
    spareStates.push_back(std::move(state));
  state = Tensor{};
}

// A zeroed state record: a spare one if there is any.
Tensor Engine::freshState() {
  if (spareStates.empty())
    return device.empty(stateBytes);
  Tensor state = std::move(spareStates.back());
  spareStates.pop_back();
  device.check(infdev_fill(device.ctx, state.as<void>(), 0, state.bytes));
  return state;
}

// Finds the deepest published prefix of the request beyond what the sequence already holds and adopts its state arena
// and K/V bindings (Engine::restorePrefix, engine.cpp:48-68). The match is by chained hash only. The reference looks
// once, before a sequence's first pass; here a sequence looks again at every 512-token boundary of its prompt, so it
// also picks up checkpoints that another sequence published while both were being prefilled.
void Engine::restorePrefix(Sequence& sequence) {
  if (sequence.kvValid % checkpointTokens || sequence.bindings.size() != sequence.kvValid / blockTokens)
    return;
  uint64_t hash = sequence.prefixHash;
  auto best = checkpointCache.end();
  const uint32_t fullBlocks = (sequence.requested - 1) / checkpointTokens;
  for (uint32_t index = sequence.kvValid / checkpointTokens; index < fullBlocks; ++index) {
    hash = hashCheckpoint(hash, sequence.request + uint64_t(index) * checkpointTokens);
    for (auto entry = checkpointCache.begin(); entry != checkpointCache.end(); ++entry)
      if (entry->hash == hash) {
        best = entry;
        break;
      }
  }
  if (best == checkpointCache.end() || best->bindings.size() <= sequence.bindings.size())
    return;
  checkpointCache.splice(checkpointCache.end(), checkpointCache, best);
  sequence.prefixHash = best->hash;
  const uint64_t touch = ++clock;
  retire(statePool[sequence.slot].first);
  statePool[sequence.slot].first = best->arena;
  for (size_t logical = sequence.bindings.size(); logical < best->bindings.size(); ++logical) {  // bind() appends one
    bind(sequence, best->bindings[logical]);
    blocks[best->bindings[logical]].touch = touch;
  }
  sequence.kvValid = uint32_t(best->bindings.size()) * blockTokens;
}

// True when another live sequence is right now computing the very 512-token block this sequence would compute next
// (same prefix, same tokens) and is ahead of it, or level with it in a lower slot. The sequence then sits this pass
// out: when the other one reaches the boundary it publishes the checkpoint, and restorePrefix picks it up. A prefix
// shared by several requests that arrive together is thus computed once, with the whole row budget, instead of once
// per request in lockstep. (No counterpart in the reference, which lets them all compute it.)
bool Engine::waitsForSibling(const Sequence& sequence) const {
  const uint32_t boundary = sequence.kvValid;
  if (boundary % checkpointTokens || (sequence.requested - 1) / checkpointTokens <= boundary / checkpointTokens)
    return false;
  for (const Sequence* other : sequences) {
    if (!other || other == &sequence || !other->active || other->kvValid < boundary || other->kvValid >= boundary + checkpointTokens)
      continue;
    if ((other->requested - 1) / checkpointTokens <= boundary / checkpointTokens || other->prefixHash != sequence.prefixHash)
      continue;
    if (other->kvValid == boundary && other->slot > sequence.slot)
      continue;
    if (!std::memcmp(other->request + boundary, sequence.request + boundary, checkpointTokens * sizeof(int32_t)))
      return true;
  }
  return false;
}

// Publishes the sequence's state at every 512-token boundary (Engine::publishPrefix, engine.cpp:70-83).
void Engine::publishPrefix(Sequence& sequence) {
  if (sequence.kvValid % checkpointTokens)
    return;
  sequence.prefixHash = hashCheckpoint(sequence.prefixHash, sequence.request + sequence.kvValid - checkpointTokens);
  for (auto entry = checkpointCache.begin(); entry != checkpointCache.end(); ++entry)
    if (entry->hash == sequence.prefixHash) {
      checkpointCache.splice(checkpointCache.end(), checkpointCache, entry);
      return;
    }
  if (checkpointCache.size() >= maxCheckpoints) {
    retire(checkpointCache.front().arena);
    checkpointCache.pop_front();
  }
  checkpointCache.push_back({sequence.prefixHash, statePool[sequence.slot].first, sequence.bindings});
}

Engine::Engine(const std::filesystem::path& path, uint32_t context, const std::filesystem::path& draftPath)
    : device(deviceIndex()), maxContext(context) {
  blockTokens = environment("INFENG_BLOCK_TOKENS", 128);
  if (!blockTokens || blockTokens % 16 || checkpointTokens % blockTokens)
    throw std::runtime_error("INFENG_BLOCK_TOKENS must be a multiple of 16 that divides 512");
  device.commitTimeoutMs = environment("INFENG_COMMIT_TIMEOUT_MS", 120000);
  useGraphs = environment("INFENG_GRAPHS", 1) != 0;
  maxCheckpoints = std::max(1u, environment("INFENG_CHECKPOINTS", 8));
  batchInvariant = environment("INFENG_BATCH_INVARIANT", 0) != 0;
  if (batchInvariant)
    infdev_set_umma(device.ctx, 0);
  // The reference sizes the physical pool for one sequence of maximum context (engine.cpp:86); INFENG_KV_BLOCKS overrides.
  const uint32_t perSlot = (context + blockTokens - 1) / blockTokens;
  blocks.resize(environment("INFENG_KV_BLOCKS", perSlot));
  loadModel(path, draftPath);
  requestData = device.empty(uint64_t(maxBatchSequences) * (maxContext + 1) * sizeof(int32_t), true);
  draftTokens = device.empty((maxDraftTokens + 1) * maxBatchSequences * sizeof(int32_t), true);
  outputTokens = device.empty(maxLogitRows * sizeof(int32_t), true);
  queryInput = device.empty(maxBatchSequences * sizeof(infdev_query), true);
  stateAddresses = device.empty(2 * maxBatchSequences * sizeof(uint64_t), true);
  queryData = device.empty(2 * maxBatchSequences * sizeof(infdev_query));
  passMeta = device.empty(8 * sizeof(uint32_t));
  stopTokens = device.empty(maxBatchSequences * maxStopTokens * sizeof(int32_t), true);
  stopCounts = device.empty(maxBatchSequences * sizeof(uint32_t), true);
  verdicts = device.empty(3 * maxBatchSequences * sizeof(uint32_t), true);
  for (auto& states : statePool)
    states = {device.empty(stateBytes), device.empty(stateBytes)};
  if (const char* text = std::getenv("INFENG_SEED"))
    baseSeed = std::strtoull(text, nullptr, 10);
  else
    baseSeed = uint64_t(std::chrono::high_resolution_clock::now().time_since_epoch().count());
  kv = std::make_unique<PagedKV>(device, maxBatchSequences, perSlot, uint32_t(blocks.size()), kvLayers + (drafter == Drafter::mtp ? 1 : 0), blockTokens);
  device.check(device.commit());
  passEvents[0] = infdev_event_create(device.ctx);
  passEvents[1] = infdev_event_create(device.ctx);
  worker = std::thread(&Engine::schedule, this);
}

Engine::~Engine() {
  {
    std::lock_guard<std::mutex> lock(mutex);
    closing = true;
  }
  condition.notify_all();
  if (worker.joinable())
    worker.join();
  for (auto& graphs : decodeGraphs)
    for (void* graph : graphs)
      infdev_graph_destroy(device.ctx, graph);
  infdev_event_destroy(device.ctx, passEvents[0]);
  infdev_event_destroy(device.ctx, passEvents[1]);
}

Sequence::Sequence(Engine& owner, const int32_t* stopTokens, uint32_t stopCount, float samplingTemperature, float samplingTopP, int32_t samplingTopK,
                   bool useSpeculation)
    : engine(owner), temperature(samplingTemperature), topP(samplingTopP), topK(samplingTopK), speculative(useSpeculation) {
  std::lock_guard<std::mutex> lock(engine.mutex);
  if (stopCount > maxStopTokens)
    throw std::runtime_error("a sequence takes at most " + std::to_string(maxStopTokens) + " stop tokens");
  stops.assign(stopTokens, stopTokens + stopCount);
  slot = uint32_t(std::find(engine.sequences.begin(), engine.sequences.end(), nullptr) - engine.sequences.begin());
  if (slot == maxBatchSequences)
    throw std::runtime_error("maximum live sequence count reached");
  request = engine.requestData.contents<int32_t>() + uint64_t(slot) * (engine.maxContext + 1);
  // No pass in flight reads this slot's rows of the tables: the previous owner left only after its last pass.
  std::copy_n(stopTokens, stopCount, engine.stopTokens.contents<int32_t>() + uint64_t(slot) * maxStopTokens);
  engine.stopCounts.contents<uint32_t>()[slot] = stopCount;
  engine.seeds[slot] = mixSeed(engine.baseSeed + engine.sequencesCreated++);
  engine.sequences[slot] = this;
  ++engine.owners;
}

Sequence::~Sequence() {
  std::unique_lock<std::mutex> lock(engine.mutex);
  active = false;
  engine.condition.wait(lock, [&] { return !busy; });
  for (uint32_t physical : bindings)
    --engine.blocks[physical].refs;
  engine.sequences[slot] = nullptr;
}

// The scheduler thread (Engine::schedule, engine.cpp:142-230). Each iteration packs every ready sequence into
// one pass of at most 128 rows: decodes take one row (plus the draft rows when speculating), prefills share
// what is left and never cross a 512-token boundary; then reserve K/V, run the drafting and target passes,
// block on the commit, and publish tokens.
void Engine::schedule() {
  std::unique_lock<std::mutex> lock(mutex);
  auto ready = [](Sequence* sequence) { return sequence && sequence->active; };
  while (true) {
    // The readers hear of the tokens of a pass once the next pass has been launched (below): woken while this thread
    // still holds the lock and has a batch to build, they would only queue up behind it, and on a busy host push it
    // off its core for milliseconds. With nothing left to launch they are told here, before this thread sleeps.
    if (!closing && std::none_of(sequences.begin(), sequences.end(), ready))
      condition.notify_all();
    condition.wait(lock, [&] { return closing || std::any_of(sequences.begin(), sequences.end(), ready); });
    if (closing)
      return;
    auto stamp = std::chrono::steady_clock::now();
    auto lap = [&stamp](std::atomic_uint64_t& counter) {
      const auto now = std::chrono::steady_clock::now();
      counter += uint64_t(std::chrono::duration_cast<std::chrono::microseconds>(now - stamp).count());
      stamp = now;
    };
    Batch batch;
    batch.queries = queryInput.contents<infdev_query>();
    std::array<infdev_query*, maxBatchSequences> prefills{};
    uint32_t prefillCount = 0, remaining = maxBatchTokens;
    for (Sequence* sequence : sequences) {
      if (!ready(sequence))
        continue;
      restorePrefix(*sequence);
      if (waitsForSibling(*sequence))
        continue;
      sequence->busy = true;
      // The output state must not be an arena that a checkpoint still shares.
      if (statePool[sequence->slot].second.buffer.use_count() > 1)
        statePool[sequence->slot].second = freshState();
      infdev_query& query = batch.queries[batch.size++];
      query = infdev_query{};
      query.count = 1;
      query.position = sequence->kvValid;
      query.slot = sequence->slot;
      query.state = unbound;
      query.samples = sequence->requested;  // finished into a sample count by the pack step
      query.temperature = sequence->temperature;
      query.topP = sequence->topP;
      query.topK = sequence->topK;
      query.seed = seeds[sequence->slot];
      const uint32_t pending = sequence->requested - sequence->kvValid;
      const uint32_t boundary = std::min(maxContext, (sequence->kvValid / checkpointTokens + 1) * checkpointTokens);
      const uint32_t room = boundary - sequence->kvValid;
      if (pending > 1) {
        query.count = std::min(pending, room);
        prefills[prefillCount++] = &query;
        continue;
      }
      if (sequence->speculative && room > draftWidth) {
        query.count += draftWidth;
        query.state = batch.candidateRows;
        batch.candidateRows += query.count;
      }
      remaining -= query.count;
    }
    for (uint32_t i = 0; i < prefillCount; ++i) {
      infdev_query& query = *prefills[i];
      query.count = std::min(query.count, remaining / (prefillCount - i));
      remaining -= query.count;
    }
    if (!batch.size) {  // every ready sequence waits for a sibling that stopped being ready meanwhile: look again shortly
      condition.wait_for(lock, std::chrono::milliseconds(1));
      continue;
    }
    bool success = reserve(batch);
    lock.unlock();
    lap(buildMicros);
    PassShape shape;
    bool announced = false;
    auto announce = [&] {  // the results of the pass before this one
      if (!announced)
        condition.notify_all();
      announced = true;
    };
    if (success) {
      try {
        // Candidate rows: sized once for the largest speculative pass, because captured graphs hold its address.
        if (batch.candidateRows && !candidateStates)
          candidateStates = device.empty(stateBytes * maxBatchSequences * (draftWidth + 1));
        const auto started = std::chrono::steady_clock::now();
        infdev_event_record(device.ctx, passEvents[0]);
        // Uniform passes have a fixed launch sequence: every query one decode row, or every query a speculative decode.
        const uint32_t kind = batch.candidateRows ? 1 : 0, rowsEach = kind ? draftWidth + 1 : 1;
        bool uniform = useGraphs && batch.candidateRows == kind * batch.size * rowsEach;
        for (uint32_t i = 0; i < batch.size && uniform; ++i)
          uniform = batch.queries[i].count == rowsEach;
        void*& graph = decodeGraphs[batch.size][kind];
        auto launchAll = [&] {
          if (batch.candidateRows)
            forward(*this, batch, true);
          shape = forward(*this, batch);
        };
        if (uniform && graph) {
          shape = forward(*this, batch, false, false);  // host bookkeeping only
          device.check(infdev_graph_launch(device.ctx, graph));
        } else if (uniform && decodeSeen[batch.size][kind]++ >= 1 && infdev_graph_begin(device.ctx) == INFDEV_OK) {
          launchAll();
          graph = infdev_graph_end(device.ctx);
          if (!graph)
            throw std::runtime_error(infdev_error(device.ctx));
          device.check(infdev_graph_launch(device.ctx, graph));
        } else {
          launchAll();  // also the way of a device layer that cannot capture
        }
        infdev_event_record(device.ctx, passEvents[1]);
        announce();
        device.check(device.commit());
        passDeviceNanos += uint64_t(double(infdev_event_elapsed_ms(device.ctx, passEvents[0], passEvents[1])) * 1.0e6);
        passMicros += uint64_t(std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - started).count());
        passRows += shape.rows;
        for (uint32_t i = 0; i < batch.size; ++i)
          if (batch.queries[i].state == unbound && batch.queries[i].count > 1)
            prefillRows += batch.queries[i].count;
        ++passes;
      } catch (const std::exception&) {
        success = false;  // a device failure is reported to every sequence of the batch like a capacity failure
      }
    }
    announce();
    stamp = std::chrono::steady_clock::now();
    lock.lock();
    lap(lockMicros);
    // The device has already walked the sampled rows of every query (infdev_verify_drafts, the loop of engine.cpp:205-216)
    // and copied the accepted candidate states (infdev_commit_states, engine.cpp:217-218); what is left for the host is
    // to hand the emitted tokens over and to advance the bookkeeping.
    const int32_t *sampled = outputTokens.contents<int32_t>(), *proposed = draftTokens.contents<int32_t>();
    const uint32_t* verdict = verdicts.contents<uint32_t>();
    for (uint32_t i = 0; i < batch.size; ++i) {
      const infdev_query& query = success ? batch.finished[i] : batch.queries[i];
      Sequence& sequence = *sequences[query.slot];
      sequence.busy = false;
      sequence.error = !success;
      sequence.active &= success;
      if (!sequence.active)
        continue;
      const bool speculative = query.state != unbound;
      uint32_t accepted = 0, emitted = 0;
      bool stopped = false;
      if (query.samples) {
        accepted = std::min(verdict[3 * i], draftWidth);
        emitted = std::min(verdict[3 * i + 1], query.samples);
        stopped = verdict[3 * i + 2] != 0;
      }
      for (uint32_t s = 0; s < emitted; ++s)
        sequence.request[sequence.requested++] = sampled[query.logit + s];
      if (speculative) {
        sequence.draftAnchor = query.position;
        for (uint32_t s = 0; s < draftWidth; ++s)
          sequence.draftProposals[s] = proposed[(s + 1) * maxBatchSequences + query.state / query.count];
      }
      sequence.kvValid += speculative ? 1 + accepted : query.count;
      sequence.drafted += speculative ? draftWidth : 0;
      sequence.accepted += accepted;
      std::swap(statePool[query.slot].first, statePool[query.slot].second);
      sequence.active = sequence.kvValid < maxContext && !stopped;
      publishPrefix(sequence);
    }
    lap(publishMicros);
  }
}

}  // namespace infeng::qwen35

using namespace infeng::qwen35;

// infeng_engine and infeng_sequence are the opaque names of Engine and Sequence in the C header.
struct infeng_engine : Engine {
  using Engine::Engine;
};
struct infeng_sequence : Sequence {
  using Sequence::Sequence;
};

namespace {
void report(char* error, const std::exception& exception) {
  if (error) {
    std::strncpy(error, exception.what(), 1023);
    error[1023] = 0;
  }
}
}  // namespace

extern "C" {

infeng_engine* infeng_engine_create(const char* weights, const char* draftWeights, const char* kernels, uint32_t context, char* error) {
  (void)kernels;  // the Metal build compiles its kernel sources from this directory; the CUDA kernels are linked in
  try {
    if (!context || context > 65536)
      throw std::runtime_error("context must be between 1 and 65536");
    return new infeng_engine(weights, context, draftWeights ? draftWeights : "");
  } catch (const std::exception& exception) {
    report(error, exception);
    return nullptr;
  }
}

void infeng_engine_release(infeng_engine* engine) {
  if (--engine->owners == 0)
    delete engine;
}

infeng_sequence* infeng_sequence_create(infeng_engine* engine, const int32_t* stops, uint32_t stopCount, float temperature, float topP, int32_t topK,
                                        uint32_t speculative, char* error) {
  try {
    return new infeng_sequence(*engine, stops, stopCount, temperature, topP, topK, speculative != 0 && engine->drafter != Drafter::none);
  } catch (const std::exception& exception) {
    report(error, exception);
    return nullptr;
  }
}

int32_t infeng_sequence_seed(infeng_sequence* sequence, uint64_t seed) {
  Engine& engine = sequence->engine;
  std::lock_guard<std::mutex> lock(engine.mutex);
  if (sequence->active || sequence->busy || sequence->requested)
    return -3;
  engine.seeds[sequence->slot] = mixSeed(seed);
  return 0;
}

void infeng_sequence_release(infeng_sequence* sequence) {
  infeng_engine* engine = static_cast<infeng_engine*>(&sequence->engine);
  delete sequence;
  infeng_engine_release(engine);
}

int32_t infeng_sequence_append(infeng_sequence* sequence, const int32_t* tokens, uint32_t count) {
  Engine& engine = sequence->engine;
  std::lock_guard<std::mutex> lock(engine.mutex);
  if (count == UINT32_MAX) {  // cancel
    sequence->active = false;
    engine.condition.notify_all();
    return 0;
  }
  if (sequence->active || sequence->busy)
    return -3;
  if ((!count && sequence->requested == sequence->kvValid) || uint64_t(sequence->requested) + count > engine.maxContext)
    return -4;
  // The embedding gather indexes the table with these ids; the reference trusts its tokenizer here.
  for (uint32_t i = 0; i < count; ++i)
    if (tokens[i] < 0 || uint32_t(tokens[i]) >= engine.vocab)
      return -4;
  std::copy_n(tokens, count, sequence->request + sequence->requested);
  sequence->requested += count;
  sequence->error = false;
  sequence->active = true;
  engine.condition.notify_all();
  return int32_t(sequence->requested);
}

int32_t infeng_sequence_read(infeng_sequence* sequence, uint32_t cursor) {
  Engine& engine = sequence->engine;
  std::unique_lock<std::mutex> lock(engine.mutex);
  engine.condition.wait(lock, [&] { return cursor < sequence->requested || (!sequence->active && !sequence->busy); });
  if (sequence->error)
    return -5;
  return cursor < sequence->requested ? sequence->request[cursor] : -1;
}

uint64_t infeng_engine_info(infeng_engine* engine, uint32_t field) {
  switch (field) {
    case 0: return engine->parameterCount;
    case 1: return engine->modelBytes;
    case 2: return engine->kv->mappedBytes();
    case 3: return uint64_t(engine->drafter);
    case 4: return engine->draftWidth;
    case 5: return engine->passes.load();
    case 6: return engine->passRows.load();
    case 7: return engine->passMicros.load();
    case 8: return engine->targetLayers;
    case 9: return engine->vocab;
    case 10: return engine->passDeviceNanos.load();
    case 11: return infdev_launch_count(engine->device.ctx);
    case 12: return engine->buildMicros.load();
    case 13: return engine->lockMicros.load();
    case 14: return engine->publishMicros.load();
    case 15: return engine->prefillRows.load();
    default: return 0;
  }
}

uint64_t infeng_sequence_info(infeng_sequence* sequence, uint32_t field) {
  std::lock_guard<std::mutex> lock(sequence->engine.mutex);
  switch (field) {
    case 0: return sequence->drafted;
    case 1: return sequence->accepted;
    case 2: return sequence->kvValid;
    case 3: return sequence->draftAnchor;
    default:
      if (field >= 4 && field < 4 + maxDraftTokens)
        return uint64_t(uint32_t(sequence->draftProposals[field - 4]));
      return 0;
  }
}

int64_t infeng_gguf_describe(const char* path, char* out, uint64_t capacity, char* error) {
  try {
    const std::string text = describeGguf(path);
    if (text.size() + 1 > capacity)
      throw std::runtime_error("the listing needs " + std::to_string(text.size() + 1) + " bytes");
    std::memcpy(out, text.c_str(), text.size() + 1);
    return int64_t(text.size());
  } catch (const std::exception& exception) {
    report(error, exception);
    return -1;
  }
}

int64_t infeng_sequence_state(infeng_sequence* sequence, uint64_t offset, void* out, uint64_t bytes) {
  Engine& engine = sequence->engine;
  std::lock_guard<std::mutex> lock(engine.mutex);
  if (!bytes)
    return int64_t(engine.stateBytes);
  if (sequence->active || sequence->busy)
    return -3;
  if (offset > engine.stateBytes || bytes > engine.stateBytes - offset)
    return -4;
  // No pass touches the records of a sequence that is neither active nor busy, and the copy stays off the stream.
  const infeng::Tensor& state = engine.statePool[sequence->slot].first;
  return infdev_peek(engine.device.ctx, out, state.as<uint8_t>() + offset, bytes) == INFDEV_OK ? int64_t(bytes) : -5;
}

}  // extern "C"
