// Host-side engine types: the CUDA build of model/qwen35/qwen35.hpp. Same roles and field meanings as the
// reference (Engine, Sequence, Weights, Scratch, PhysicalBlock, HybridCheckpoint, Batch; qwen35.hpp:20-116),
// with the layer count and vocabulary read from the GGUF file instead of being compile-time constants so
// that reduced models can be checked against the CPU oracle.
#pragma once
#include <array>
#include <atomic>
#include <condition_variable>
#include <filesystem>
#include <list>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <utility>
#include <vector>
#include "cuda_device.hpp"

namespace infeng::qwen35 {

inline constexpr uint32_t hiddenSize = 4096, intermediateSize = 12288, fullAttentionInterval = 4;
inline constexpr uint32_t maxDraftTokens = 7, maxBatchSequences = 8, maxBatchTokens = 128;
inline constexpr uint32_t maxLogitRows = maxBatchSequences * (maxDraftTokens + 1);
inline constexpr uint32_t checkpointTokens = 512, maxAttentionSplits = 32;
inline constexpr uint32_t maxStopTokens = 64;  // per sequence: the stop lists live in a device-visible table
inline constexpr uint32_t unbound = UINT32_MAX;
inline constexpr uint64_t seedBytes = hiddenSize * sizeof(float);  // MTP seed (last target hidden) at the end of a state record

enum class Drafter : uint8_t { none, mtp, dflash };

struct Weight : Tensor {
  uint32_t n = 0, k = 0, type = 0;
};
using Weights = std::unordered_map<std::string, Weight>;

// Fixed scratch for one pass of up to maxBatchTokens rows (Scratch, qwen35.hpp:41-46); all fp32.
struct Scratch {
  Tensor hidden, norm, temporary, mlpGate;
  Tensor mixed, gate, q, k, v, attnQ, attnPartials;
  Tensor gdnB, gdnG;
  Tensor fused, targetLogits, rowTokens;
  // Activation images (infdev_image_capture / infdev_image_supply) of norm, temporary and mlpGate for passes of at
  // most imageRows rows, where the integer decode GEMV consumes them.
  Tensor normImage, temporaryImage, mlpImage;
};
constexpr uint32_t imageRows = 8;

struct PhysicalBlock {
  uint32_t refs = 0;
  uint64_t touch = 0;
};

// A published 512-token prefix: chained hash, the shared recurrent-state arena and the K/V bindings.
struct HybridCheckpoint {
  uint64_t hash = 0;
  Tensor arena;
  std::vector<uint32_t> bindings;
};

struct Sequence;

struct Batch {
  infdev_query* queries = nullptr;  // raw scheduler records in host-visible memory, read by the device pack kernel
  // The same records finished on the host (start, samples, logit, state addresses): target frame, then drafter frame.
  std::array<infdev_query, 2 * maxBatchSequences> finished{};
  uint32_t size = 0, candidateRows = 0;
};

struct Engine {
  std::atomic_uint32_t owners{1};  // one API handle and one reference per live sequence
  Device device;
  uint32_t maxContext, draftWidth = 0;
  uint32_t targetLayers = 0, kvLayers = 0, gdnLayers = 0, vocab = 0, blockTokens = 128;
  uint32_t maxCheckpoints = 8;  // entries of the prefix-checkpoint cache (qwen35.hpp:24); INFENG_CHECKPOINTS overrides
  // INFENG_BATCH_INVARIANT=1: every row is computed by kernels that treat it on its own (the GEMV kernels for any row
  // count instead of the tensor-core GEMM, the token-by-token delta rule instead of the 16-token chunks), so a
  // sequence's tokens are the same bits whatever shares its passes and however its prompt was cut. Prefill is slower.
  bool batchInvariant = false;
  uint64_t stateBytes = 0;
  std::unique_ptr<PagedKV> kv;
  Weights weights;
  Tensor weightData, rope;
  Drafter drafter = Drafter::none;
  Tensor candidateStates;
  Scratch workspace;
  Tensor requestData, queryInput, queryData, passMeta, stateAddresses;
  Tensor draftTokens, outputTokens;
  // Read by the device-side acceptance step: every slot's stop tokens [slot][maxStopTokens] with their counts, and the
  // verdicts it writes per query of a pass (accepted proposals, emitted tokens, stopped).
  Tensor stopTokens, stopCounts, verdicts;
  // Philox keys. A slot's key is renewed for every sequence that takes the slot, from the base seed and the number of
  // sequences created so far, so a repeated request draws new variates (the reference keeps advancing rng[slot] across
  // sequences, engine.cpp:210-211) while a run with a fixed base seed stays reproducible.
  uint64_t seeds[maxBatchSequences]{}, baseSeed = 0, sequencesCreated = 0;
  std::vector<PhysicalBlock> blocks;
  std::list<HybridCheckpoint> checkpointCache;
  std::array<Sequence*, maxBatchSequences> sequences{};
  std::array<std::pair<Tensor, Tensor>, maxBatchSequences> statePool;
  // State records nobody refers to any more (evicted checkpoints, replaced inputs): kept for the next sequence that
  // needs one, because returning 52 MB to the driver and asking for it again costs milliseconds of scheduler time.
  std::vector<Tensor> spareStates;
  std::mutex mutex;
  std::condition_variable condition;
  std::thread worker;
  bool closing = false;
  uint64_t clock = 0;
  uint64_t parameterCount = 0, modelBytes = 0;
  // step counters for roofline reporting
  std::atomic_uint64_t passes{0}, passRows{0}, passMicros{0}, passDeviceNanos{0};
  std::atomic_uint64_t prefillRows{0};  // rows of prompt chunks among passRows (what a prefix-cache hit saves)
  // host microseconds of the scheduler outside the passes: building a batch, waiting for the engine lock after a
  // pass, handing the sampled tokens over
  std::atomic_uint64_t buildMicros{0}, lockMicros{0}, publishMicros{0};
  void* passEvents[2] = {nullptr, nullptr};  // CUDA events bracketing each pass on the stream
  // Pure-decode passes (every query one row, nothing speculative) have a fixed launch sequence for a given number of
  // live sequences; from its second occurrence such a pass is captured once into a CUDA graph and then replayed.
  // The same holds for passes in which every query is a speculative decode of draftWidth + 1 rows (second index 1).
  void* decodeGraphs[maxBatchSequences + 1][2] = {};
  uint32_t decodeSeen[maxBatchSequences + 1][2] = {};
  bool useGraphs = true;

  Engine(const std::filesystem::path& weights, uint32_t maxContext, const std::filesystem::path& draftWeights);
  ~Engine();
  void loadModel(const std::filesystem::path& weights, const std::filesystem::path& draftWeights);

  bool reserve(const Batch& batch);
  void bind(Sequence& sequence, uint32_t physical);
  void restorePrefix(Sequence& sequence);
  bool waitsForSibling(const Sequence& sequence) const;
  void publishPrefix(Sequence& sequence);
  void retire(Tensor& state);
  Tensor freshState();
  void schedule();
};

struct Sequence {
  Engine& engine;
  int32_t* request;
  uint32_t requested = 0;
  std::vector<uint32_t> bindings;
  std::vector<int32_t> stops;
  bool error = false;
  uint64_t drafted = 0, accepted = 0, prefixHash = 0;
  uint32_t kvValid = 0;
  uint32_t slot;
  float temperature, topP;
  int32_t topK;
  bool speculative, active = false, busy = false;
  // The latest speculative step of this sequence: position of its anchor token and the drafter's proposals.
  uint32_t draftAnchor = 0;
  int32_t draftProposals[maxDraftTokens] = {};
  Sequence(Engine&, const int32_t* stops, uint32_t stopCount, float temperature, float topP, int32_t topK, bool speculative);
  ~Sequence();
};

// Result of finishing the per-query records of a pass on the host (the device does the same in
// infdev_pack_queries; the host needs the counts for launch geometry and the logit offsets to read tokens).
struct PassShape {
  uint32_t rows = 0, logits = 0, queries = 0;
  bool sequential = false, prefill = false;
};

PassShape forward(Engine& engine, Batch& batch, bool drafting = false, bool launch = true);

// Text listing of a GGUF file's header as the loader reads it (one line per tensor); see infeng_gguf_describe.
std::string describeGguf(const std::filesystem::path& path);

}  // namespace infeng::qwen35
