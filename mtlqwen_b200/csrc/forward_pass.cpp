// The ragged continuous-batching forward step on the CUDA device layer: weight index, scratch, and the
// fixed decoder recipe. CUDA counterpart of model/qwen35/forward.cpp; every launch goes through the
// infdev_* C ABI.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include "gguf_reader.hpp"
#include "runtime.hpp"

namespace infeng::qwen35 {

// Read-only mapping of a file.
struct FileMapping {
  void* data = MAP_FAILED;
  uint64_t bytes = 0;
  explicit FileMapping(const std::filesystem::path& path) {
    const int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0)
      throw std::runtime_error("cannot open weights file " + path.string());
    struct stat info{};
    ::fstat(fd, &info);
    bytes = uint64_t(info.st_size);
    data = ::mmap(nullptr, bytes, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (data == MAP_FAILED)
      throw std::runtime_error("cannot map weights file " + path.string());
  }
  FileMapping(const FileMapping&) = delete;
  ~FileMapping() { ::munmap(data, bytes); }
};

std::string describeGguf(const std::filesystem::path& path) {
  FileMapping mapping(path);
  const GgufFile file = gguf_parse(static_cast<const uint8_t*>(mapping.data), mapping.bytes);
  std::string text = "gguf\t" + std::to_string(file.version) + "\t" + std::to_string(file.alignment) + "\t" + std::to_string(file.dataOffset) + "\t" +
                     std::to_string(file.tensors.size()) + "\n";
  for (const GgufTensor& tensor : file.tensors) {
    text += tensor.name + "\t" + std::to_string(tensor.type) + "\t" + std::to_string(file.dataOffset + tensor.offset) + "\t" +
            std::to_string(tensor.bytes) + "\t";
    for (size_t d = 0; d < tensor.shape.size(); ++d)
      text += (d ? "," : "") + std::to_string(tensor.shape[d]);
    text += "\n";
  }
  return text;
}

namespace {

// Reads a GGUF file: header parsed on the host from a private mapping, tensor data copied once into one
// device allocation (the reference hands the mapping itself to the GPU, device.cpp:87-98, which unified
// memory allows and PCIe does not). Returns name -> {device view, n = shape[1], k = shape[0], type}
// (loadWeights, forward.cpp:12-23).
void loadWeights(Engine& engine, const std::filesystem::path& path, Weights& weights, Tensor& storage) {
  FileMapping mapping(path);
  const uint8_t* bytesOfFile = static_cast<const uint8_t*>(mapping.data);
  const GgufFile file = gguf_parse(bytesOfFile, mapping.bytes);
  const uint64_t dataBytes = mapping.bytes - file.dataOffset;
  storage = engine.device.empty(dataBytes);
  // Tensor data goes through two pinned 64 MiB staging buffers: CUDA refuses to copy straight out of a
  // read-only file mapping, and pinned slices let the copy of one slice overlap the page-in of the next.
  const uint64_t sliceBytes = 64ull << 20;
  Tensor staging[2] = {engine.device.empty(sliceBytes, true), engine.device.empty(sliceBytes, true)};
  uint32_t turn = 0;
  for (uint64_t at = 0; at < dataBytes; at += sliceBytes, turn ^= 1) {
    const uint64_t slice = std::min<uint64_t>(sliceBytes, dataBytes - at);
    if (at >= 2 * sliceBytes)
      engine.device.check(engine.device.commit());  // the buffer about to be refilled has been consumed
    std::memcpy(staging[turn].contents<uint8_t>(), bytesOfFile + file.dataOffset + at, slice);
    engine.device.upload(storage.view(at, slice), staging[turn].contents<uint8_t>(), slice);
  }
  engine.device.check(engine.device.commit());
  engine.modelBytes += dataBytes;
  for (const GgufTensor& tensor : file.tensors) {
    if (!tensor.bytes)
      throw std::runtime_error("tensor " + tensor.name + " has unsupported ggml type " + std::to_string(tensor.type));
    Weight weight;
    static_cast<Tensor&>(weight) = storage.view(tensor.offset, tensor.bytes);
    weight.k = uint32_t(tensor.shape[0]);
    weight.n = tensor.shape.size() > 1 ? uint32_t(tensor.shape[1]) : 1;
    weight.type = tensor.type;
    engine.parameterCount += tensor.elements;
    weights.emplace(tensor.name, weight);
  }
}

// One pass over `rows` packed tokens (Ops, forward.cpp:25-131).
struct Ops {
  Engine& engine;
  uint32_t rows = 0, queryCount = 0;
  bool prefill = false;                   // the pass holds a non-speculative query of more than one row
  const infdev_query* queries = nullptr;  // device records of this pass
  Scratch& scratch;
  std::string prefix;
  infdev_ctx* ctx;

  Ops(Engine& owner) : engine(owner), scratch(owner.workspace), ctx(owner.device.ctx) {}

  void check(int code) { engine.device.check(code); }

  Weight& weight(const std::string& name, bool absolute = false) {
    const std::string key = absolute ? name : prefix + name;
    auto found = engine.weights.find(key);
    if (found == engine.weights.end())
      throw std::runtime_error("missing weight " + key);
    return found->second;
  }

  const float* f32(const std::string& name, bool absolute = false) {
    Weight& w = weight(name, absolute);
    if (w.type != INFDEV_F32)
      throw std::runtime_error("weight " + prefix + name + " must be F32");
    return w.as<float>();
  }

  // y = x . W^T (+ residual). Decode and prefill share one entry point; the device layer picks the kernel
  // (Ops::linear, forward.cpp:51-70).
  Tensor linear(const Tensor& x, Weight& w, uint32_t count, Tensor output, const Tensor& residual = {}) {
    check(infdev_linear(ctx, int(w.type), w.as<void>(), w.n, w.k, x.as<float>(), count, output.as<float>(), residual ? residual.as<float>() : nullptr));
    return output;
  }

  // Several projections of the same activations in one launch.
  void linearGroup(const Tensor& x, std::initializer_list<std::pair<Weight*, Tensor>> targets, uint32_t count) {
    const void* w[4];
    int64_t n[4];
    float* y[4];
    int used = 0;
    uint32_t type = 0, k = 0;
    for (auto& [weightPointer, output] : targets) {
      w[used] = weightPointer->as<void>();
      n[used] = weightPointer->n;
      y[used] = output.as<float>();
      if (used && (weightPointer->type != type || weightPointer->k != k)) {  // mixed types: fall back to one launch each
        for (auto& [each, out] : targets)
          linear(x, *each, count, out);
        return;
      }
      type = weightPointer->type;
      k = weightPointer->k;
      ++used;
    }
    check(infdev_linear_group(ctx, int(type), used, w, n, k, x.as<float>(), count, y));
  }

  Tensor logits(const Tensor& x, const float* norm, uint32_t count) {
    if (count == rows)
      check(infdev_rms_norm(ctx, x.as<float>(), norm, rows, hiddenSize, scratch.temporary.as<float>()));
    else
      check(infdev_rms_norm_gather(ctx, x.as<float>(), norm, queries, int(queryCount), count, scratch.temporary.as<float>()));
    return linear(scratch.temporary, weight("output.weight", true), count, scratch.targetLogits);
  }

  // One decoder layer in place on `hidden` (Ops::decoder, forward.cpp:77-120). Layers with (layer+1) % 4 == 0
  // and the MTP layer are gated full attention, the others gated delta networks.
  // Decode-sized passes hand the quantised form of each projection's input from the kernel that produces it to the
  // GEMV that consumes it, which saves the GEMV its own quantisation launch.
  void capture(const Tensor& image) {
    if (rows <= imageRows)
      check(infdev_image_capture(ctx, image.as<uint8_t>()));
  }
  void supply(const Tensor& image) {
    if (rows <= imageRows)
      check(infdev_image_supply(ctx, image.as<uint8_t>()));
  }

  void decoder(uint32_t layer, const Tensor& hidden) {
    prefix = "blk." + std::to_string(layer) + ".";
    const bool fullAttention = layer >= engine.targetLayers || (layer + 1) % fullAttentionInterval == 0;
    const Tensor& x = scratch.norm;
    capture(scratch.normImage);
    check(infdev_rms_norm(ctx, hidden.as<float>(), f32("attn_norm.weight"), rows, hiddenSize, x.as<float>()));
    supply(scratch.normImage);
    if (fullAttention) {
      const uint32_t kvLayer = layer < engine.targetLayers ? layer / fullAttentionInterval : engine.kvLayers + layer - engine.targetLayers;
      linearGroup(x, {{&weight("attn_q.weight"), scratch.mixed}, {&weight("attn_k.weight"), scratch.k}, {&weight("attn_v.weight"), scratch.v}}, rows);
      check(infdev_attention_prepare(ctx, scratch.mixed.as<float>(), scratch.k.as<float>(), scratch.v.as<float>(), f32("attn_q_norm.weight"),
                                     f32("attn_k_norm.weight"), engine.rope.as<float>(), queries, int(queryCount), rows, engine.kv->blockTable(),
                                     int32_t(engine.kv->tableStride()), int32_t(engine.blockTokens), scratch.attnQ.as<float>(),
                                     engine.kv->key(kvLayer).as<void>(), engine.kv->value(kvLayer).as<void>()));
      capture(scratch.temporaryImage);
      check(infdev_attention(ctx, scratch.attnQ.as<float>(), scratch.mixed.as<float>(), engine.kv->key(kvLayer).as<void>(),
                             engine.kv->value(kvLayer).as<void>(), queries, int(queryCount), rows, engine.kv->blockTable(),
                             int32_t(engine.kv->tableStride()), int32_t(engine.blockTokens), maxAttentionSplits, scratch.attnPartials.as<float>(),
                             scratch.temporary.as<float>()));
      supply(scratch.temporaryImage);
      linear(scratch.temporary, weight("attn_output.weight"), rows, hidden, hidden);
    } else {
      linearGroup(x, {{&weight("attn_qkv.weight"), scratch.mixed}, {&weight("attn_gate.weight"), scratch.gate}}, rows);
      const uint64_t offset = uint64_t(layer - layer / fullAttentionInterval) * INFDEV_GDN_LAYER_STATE_BYTES;
      if (!prefill) {
        // every query of the pass is short: preparation and recurrence in one launch
        capture(scratch.temporaryImage);
        check(infdev_gdn_decode(ctx, x.as<float>(), scratch.mixed.as<float>(), f32("ssm_beta.weight"), f32("ssm_alpha.weight"), f32("ssm_a"),
                                f32("ssm_dt.bias"), f32("ssm_conv1d.weight"), scratch.gate.as<float>(), f32("ssm_norm.weight"), queries,
                                int(queryCount), offset, offset + INFDEV_CONV_STATE_BYTES, engine.stateBytes, scratch.temporary.as<float>()));
      } else {
        check(infdev_gdn_prepare(ctx, x.as<float>(), scratch.mixed.as<float>(), f32("ssm_beta.weight"), f32("ssm_alpha.weight"), f32("ssm_a"),
                                 f32("ssm_dt.bias"), f32("ssm_conv1d.weight"), queries, int(queryCount), rows, offset, engine.stateBytes,
                                 scratch.q.as<float>(), scratch.k.as<float>(), scratch.v.as<float>(), scratch.gdnB.as<float>(),
                                 scratch.gdnG.as<float>()));
        capture(scratch.temporaryImage);
        // a pass that carries prefill chunks lets its long queries take the chunked kernel
        check((rows > imageRows && !engine.batchInvariant ? infdev_delta_rule_prefill : infdev_delta_rule)(ctx, scratch.q.as<float>(), scratch.k.as<float>(), scratch.v.as<float>(),
                                                                                 scratch.gdnG.as<float>(), scratch.gdnB.as<float>(),
                                                                                 scratch.gate.as<float>(), f32("ssm_norm.weight"), queries,
                                                                                 int(queryCount), offset + INFDEV_CONV_STATE_BYTES,
                                                                                 engine.stateBytes, scratch.temporary.as<float>()));
      }
      supply(scratch.temporaryImage);
      linear(scratch.temporary, weight("ssm_out.weight"), rows, hidden, hidden);
    }
    capture(scratch.normImage);
    check(infdev_rms_norm(ctx, hidden.as<float>(), f32("post_attention_norm.weight"), rows, hiddenSize, x.as<float>()));
    Weight &gate = weight("ffn_gate.weight"), &up = weight("ffn_up.weight");
    supply(scratch.normImage);
    capture(scratch.mlpImage);
    check(infdev_gate_up(ctx, int(gate.type), gate.as<void>(), up.as<void>(), gate.n, gate.k, x.as<float>(), rows, scratch.mlpGate.as<float>()));
    supply(scratch.mlpImage);
    linear(scratch.mlpGate, weight("ffn_down.weight"), rows, hidden, hidden);
  }

  // MTP input (Ops::mtpInput, forward.cpp:122-130): embed the row tokens, fuse with the previous hidden
  // state, project 8192 -> 4096 into scratch.hidden. tokenMode follows infdev_gather_tokens, fuseMode infdev_mtp_fuse.
  Tensor mtpInput(const int32_t* proposals, const Tensor& hidden, uint32_t tokenMode, uint32_t fuseMode) {
    prefix = "blk." + std::to_string(engine.targetLayers) + ".nextn.";
    check(infdev_gather_tokens(ctx, queries, int(queryCount), engine.requestData.as<int32_t>(), engine.maxContext + 1, proposals, tokenMode,
                               scratch.rowTokens.as<int32_t>()));
    Weight& table = weight("token_embd.weight", true);
    check(infdev_embedding(ctx, int(table.type), table.as<void>(), table.k, scratch.rowTokens.as<int32_t>(), rows, scratch.norm.as<float>()));
    check(infdev_mtp_fuse(ctx, scratch.norm.as<float>(), hidden.as<float>(), queries, int(queryCount), f32("enorm.weight"), f32("hnorm.weight"), rows,
                          fuseMode, engine.stateBytes - seedBytes, engine.stateBytes, scratch.fused.as<float>()));
    return linear(scratch.fused, weight("eh_proj.weight"), rows, scratch.hidden);
  }
};

}  // namespace

void Engine::loadModel(const std::filesystem::path& path, const std::filesystem::path& draftPath) {
  // A drafter file that carries the MTP block holds the whole model (forward.cpp:136-143).
  loadWeights(*this, draftPath.empty() ? path : draftPath, weights, weightData);
  uint32_t blocksWithNorm = 0;
  while (weights.count("blk." + std::to_string(blocksWithNorm) + ".attn_norm.weight"))
    ++blocksWithNorm;
  if (!blocksWithNorm || !weights.count("token_embd.weight") || !weights.count("output.weight"))
    throw std::runtime_error("weights file has no decoder blocks");
  const bool hasMtp = weights.count("blk." + std::to_string(blocksWithNorm - 1) + ".nextn.eh_proj.weight") != 0;
  if (!draftPath.empty() && !hasMtp)
    throw std::runtime_error("draft weights carry no MTP block (blk.N.nextn.*); the DFlash drafter is not supported by this build");
  // The drafter runs only when it was asked for through the draft path (forward.cpp:136-139): a file that carries the
  // MTP block loads as a plain target model when passed as `weights` alone.
  drafter = hasMtp && !draftPath.empty() ? Drafter::mtp : Drafter::none;
  targetLayers = blocksWithNorm - (hasMtp ? 1 : 0);
  if (targetLayers % fullAttentionInterval)
    throw std::runtime_error("decoder block count must be a multiple of 4");
  kvLayers = targetLayers / fullAttentionInterval;
  gdnLayers = targetLayers - kvLayers;
  vocab = weights.at("token_embd.weight").n;
  // Every tensor the passes will touch, with the shape the fixed scratch buffers assume and a type the kernels serve:
  // a file that does not fit is refused here rather than at its first pass.
  auto require = [&](const std::string& name, uint32_t n, uint32_t k, bool quantised) {
    auto found = weights.find(name);
    if (found == weights.end())
      throw std::runtime_error("missing weight " + name);
    const Weight& w = found->second;
    if (w.n != n || w.k != k)
      throw std::runtime_error("weight " + name + " has shape " + std::to_string(w.n) + " x " + std::to_string(w.k) + ", expected " + std::to_string(n) +
                               " x " + std::to_string(k));
    const bool supported = quantised ? (w.type == INFDEV_Q4_K || w.type == INFDEV_Q6_K || w.type == INFDEV_Q5_K || w.type == INFDEV_Q8_0 ||
                                        w.type == INFDEV_IQ4_XS)
                                     : w.type == INFDEV_F32;
    if (!supported)
      throw std::runtime_error("weight " + name + " has ggml type " + std::to_string(w.type) + "; this build runs " +
                               (quantised ? "Q4_K, Q5_K, Q6_K, Q8_0 and IQ4_XS projections" : "F32 norms and GDN parameters"));
  };
  // ssm_beta / ssm_alpha come as F16 in the real files (gdn_ba_prepare_4096x32 takes either, native_ops.metal:89-113); the
  // kernels here read fp32, so such a tensor is widened once at load time.
  auto widen = [&](const std::string& name) {
    auto found = weights.find(name);
    if (found == weights.end() || found->second.type != INFDEV_F16)
      return;
    Weight& w = found->second;
    const uint64_t elements = uint64_t(w.n) * w.k;
    if (elements % 256)
      throw std::runtime_error("weight " + name + ": an F16 tensor must hold a multiple of 256 values");
    Tensor wide = device.empty(elements * sizeof(float));
    device.check(infdev_dequant(device.ctx, INFDEV_F16, w.as<void>(), int64_t(elements / 256), wide.as<float>()));
    static_cast<Tensor&>(w) = wide;
    w.type = INFDEV_F32;
  };
  require("token_embd.weight", vocab, hiddenSize, true);
  require("output.weight", vocab, hiddenSize, true);
  require("output_norm.weight", 1, hiddenSize, false);
  for (uint32_t layer = 0; layer < blocksWithNorm; ++layer) {
    const std::string p = "blk." + std::to_string(layer) + ".";
    require(p + "attn_norm.weight", 1, hiddenSize, false);
    require(p + "post_attention_norm.weight", 1, hiddenSize, false);
    require(p + "ffn_gate.weight", intermediateSize, hiddenSize, true);
    require(p + "ffn_up.weight", intermediateSize, hiddenSize, true);
    require(p + "ffn_down.weight", hiddenSize, intermediateSize, true);
    if (weights.at(p + "ffn_gate.weight").type != weights.at(p + "ffn_up.weight").type)
      throw std::runtime_error("blk." + std::to_string(layer) + ": ffn_gate and ffn_up must share a quantisation type (one fused kernel serves the pair)");
    if (layer >= targetLayers || (layer + 1) % fullAttentionInterval == 0) {
      require(p + "attn_q.weight", 8192, hiddenSize, true);
      require(p + "attn_k.weight", 1024, hiddenSize, true);
      require(p + "attn_v.weight", 1024, hiddenSize, true);
      require(p + "attn_output.weight", hiddenSize, hiddenSize, true);
      require(p + "attn_q_norm.weight", 1, 256, false);
      require(p + "attn_k_norm.weight", 1, 256, false);
    } else {
      require(p + "attn_qkv.weight", 8192, hiddenSize, true);
      require(p + "attn_gate.weight", hiddenSize, hiddenSize, true);
      require(p + "ssm_out.weight", hiddenSize, hiddenSize, true);
      widen(p + "ssm_beta.weight");
      widen(p + "ssm_alpha.weight");
      require(p + "ssm_beta.weight", 32, hiddenSize, false);
      require(p + "ssm_alpha.weight", 32, hiddenSize, false);
      require(p + "ssm_a", 1, 32, false);
      require(p + "ssm_dt.bias", 1, 32, false);
      require(p + "ssm_conv1d.weight", 8192, 4, false);
      require(p + "ssm_norm.weight", 1, 128, false);
    }
  }
  device.check(device.commit());  // the widened copies are complete before their sources could be released
  if (hasMtp) {
    const std::string p = "blk." + std::to_string(targetLayers) + ".nextn.";
    require(p + "enorm.weight", 1, hiddenSize, false);
    require(p + "hnorm.weight", 1, hiddenSize, false);
    require(p + "shared_head_norm.weight", 1, hiddenSize, false);
    require(p + "eh_proj.weight", hiddenSize, 2 * hiddenSize, true);
  }
  stateBytes = uint64_t(gdnLayers) * INFDEV_GDN_LAYER_STATE_BYTES + seedBytes;
  if (drafter == Drafter::mtp) {
    const char* width = std::getenv("INFENG_DRAFT_WIDTH");
    draftWidth = width ? std::clamp(std::atoi(width), 1, int(maxDraftTokens)) : 2;
  }
  Scratch& s = workspace;
  const uint64_t row = uint64_t(maxBatchTokens) * sizeof(float);
  for (Tensor* tensor : {&s.hidden, &s.norm, &s.temporary, &s.gate, &s.v, &s.attnQ})
    *tensor = device.empty(row * hiddenSize);
  s.mixed = device.empty(row * 8192);
  s.fused = device.empty(row * 8192);
  s.q = device.empty(row * 2048);
  s.k = device.empty(row * 2048);
  s.mlpGate = device.empty(row * intermediateSize);
  s.gdnB = device.empty(row * 32);
  s.gdnG = device.empty(row * 32);
  s.attnPartials = device.empty(infdev_attention_scratch_bytes(maxBatchTokens, maxAttentionSplits));
  s.targetLogits = device.empty(uint64_t(maxLogitRows) * vocab * sizeof(float));
  s.rowTokens = device.empty(maxBatchTokens * sizeof(int32_t));
  s.normImage = device.empty(infdev_image_bytes(imageRows, hiddenSize));
  s.temporaryImage = device.empty(infdev_image_bytes(imageRows, hiddenSize));
  s.mlpImage = device.empty(infdev_image_bytes(imageRows, intermediateSize));
  rope = device.empty(uint64_t(maxContext) * 32 * 2 * sizeof(float));
  device.check(infdev_rope_table(device.ctx, maxContext, rope.as<float>()));
}

PassShape forward(Engine& engine, Batch& batch, bool drafting, bool launch) {
  Ops ops(engine);
  PassShape shape;
  // Finish the records on the host exactly as infdev_pack_queries does on the device (forward.cpp:171-191): the
  // host needs the row counts for launch geometry and the logit offsets to read the sampled tokens back.
  infdev_query* frame = batch.finished.data() + (drafting ? maxBatchSequences : 0);
  auto* addresses = engine.stateAddresses.contents<uint64_t>();
  for (uint32_t i = 0; i < batch.size; ++i) {
    infdev_query query = batch.queries[i];
    const bool speculative = query.state != unbound;
    const auto& [state, nextState] = engine.statePool[query.slot];
    addresses[query.slot] = state.address();
    addresses[maxBatchSequences + query.slot] = nextState.address();
    if (drafting && !speculative)
      continue;
    const uint32_t requested = query.samples;  // the scheduler passes the slot's requested-token count here
    query.start = shape.rows;
    query.count = drafting ? 1 : query.count;
    query.samples = drafting ? 1 : speculative ? query.count : (query.position + query.count == requested ? 1 : 0);
    shape.sequential |= speculative || query.count == 1;
    shape.prefill |= !speculative && query.count > 1;
    query.previous = query.position ? state.address() : 0;
    query.next = speculative ? engine.candidateStates.address() + uint64_t(query.state) * engine.stateBytes : nextState.address();
    query.logit = shape.logits;
    frame[shape.queries++] = query;
    shape.logits += query.samples;
    shape.rows += query.count;
  }
  if (!shape.rows || !launch)  // launch == false: a captured graph of this pass shape will be replayed instead
    return shape;
  infdev_ctx* ctx = engine.device.ctx;
  infdev_query* deviceQueries = engine.queryData.as<infdev_query>() + (drafting ? maxBatchSequences : 0);
  // The device builds the same packed records from the raw scheduler inputs; every kernel of the pass reads them there.
  ops.check(infdev_pack_queries(ctx, batch.queries, int(batch.size), drafting, engine.draftWidth, addresses, addresses + maxBatchSequences,
                                engine.candidateStates ? engine.candidateStates.address() : 0, engine.stateBytes, deviceQueries,
                                engine.passMeta.as<uint32_t>() + (drafting ? 4 : 0)));
  ops.rows = shape.rows;
  ops.prefill = shape.prefill && !drafting;
  ops.queryCount = shape.queries;
  ops.queries = deviceQueries;
  Scratch& scratch = engine.workspace;
  const Tensor& hidden = scratch.hidden;
  const uint32_t width = engine.draftWidth;
  for (uint32_t step = 0; step < (drafting ? width : 1); ++step) {
    if (drafting) {
      // step 0 embeds the anchor token and fuses it with the slot's stored seed; later steps embed the previous
      // proposal and fuse it with the previous MTP hidden state.
      ops.mtpInput(engine.draftTokens.as<int32_t>() + step * maxBatchSequences, scratch.hidden, step ? 2 : 0, step ? 0 : 2);
    } else {
      ops.check(infdev_gather_tokens(ctx, deviceQueries, int(shape.queries), engine.requestData.as<int32_t>(), engine.maxContext + 1,
                                     engine.draftTokens.as<int32_t>(), 0, scratch.rowTokens.as<int32_t>()));
      Weight& table = ops.weight("token_embd.weight", true);
      ops.check(infdev_embedding(ctx, int(table.type), table.as<void>(), table.k, scratch.rowTokens.as<int32_t>(), shape.rows, hidden.as<float>()));
    }
    for (uint32_t i = 0; i < (drafting ? 1 : engine.targetLayers); ++i)
      ops.decoder((drafting ? engine.targetLayers : 0) + i, hidden);
    if (shape.logits) {
      const float* norm = drafting ? ops.f32("blk." + std::to_string(engine.targetLayers) + ".nextn.shared_head_norm.weight", true)
                                   : ops.f32("output_norm.weight", true);
      Tensor logits = ops.logits(hidden, norm, shape.logits);
      int32_t* output = drafting ? engine.draftTokens.as<int32_t>() + (step + 1) * maxBatchSequences : engine.outputTokens.as<int32_t>();
      ops.check(infdev_sample(ctx, logits.as<float>(), engine.vocab, deviceQueries, int(shape.queries), shape.logits, drafting ? 1 : 0, output));
    }
  }
  if (!drafting && engine.drafter == Drafter::mtp) {
    // Keep the MTP layer's K/V and seed in step with the target for every row of this pass (forward.cpp:218-232).
    Tensor context = ops.mtpInput(engine.draftTokens.as<int32_t>(), hidden, 0, 1);
    ops.prefix = "blk." + std::to_string(engine.targetLayers) + ".";
    ops.check(infdev_rms_norm(ctx, context.as<float>(), ops.f32("attn_norm.weight"), shape.rows, hiddenSize, scratch.norm.as<float>()));
    ops.linearGroup(scratch.norm, {{&ops.weight("attn_k.weight"), scratch.k}, {&ops.weight("attn_v.weight"), scratch.v}}, shape.rows);
    ops.check(infdev_attention_prepare(ctx, nullptr, scratch.k.as<float>(), scratch.v.as<float>(), ops.f32("attn_k_norm.weight"),
                                       ops.f32("attn_k_norm.weight"), engine.rope.as<float>(), deviceQueries, int(shape.queries), shape.rows,
                                       engine.kv->blockTable(), int32_t(engine.kv->tableStride()), int32_t(engine.blockTokens), nullptr,
                                       engine.kv->key(engine.kvLayers).as<void>(), engine.kv->value(engine.kvLayers).as<void>()));
  }
  if (!drafting && shape.logits) {
    // Acceptance of the proposals and the copy of the accepted candidate states (the MTP seeds of the candidate rows
    // included, hence after the tail above), without a round trip to the host (engine.cpp:205-218).
    ops.check(infdev_verify_drafts(ctx, deviceQueries, int(shape.queries), engine.outputTokens.as<int32_t>(), engine.draftTokens.as<int32_t>(),
                                   engine.draftWidth, engine.stopTokens.as<int32_t>(), maxStopTokens, engine.stopCounts.as<uint32_t>(),
                                   engine.verdicts.as<uint32_t>()));
    if (batch.candidateRows)
      ops.check(infdev_commit_states(ctx, deviceQueries, int(shape.queries), engine.verdicts.as<uint32_t>(), addresses + maxBatchSequences,
                                     engine.candidateStates.address(), engine.stateBytes));
  }
  return shape;
}

}  // namespace infeng::qwen35
