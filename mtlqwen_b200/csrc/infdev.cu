// C-ABI device layer: context, memory, stream, and the typed kernel entry points declared in
// include/infdev.h. This file holds no math; it validates arguments and launches.
#include <atomic>
#include <sys/prctl.h>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>
#include "kernels.h"
#include "ops.h"

struct infdev_ctx {
  int device = 0, sms = 0, xsplit = 2;
  int umma = 1;  // tcgen05 GEMM for Q4_K launches of more than 8 activation rows: 0 off, 1 on
  int integerDecode = 1;     // Q4_K decode GEMV: 1 integer-MMA kernel over an activation image, 0 fp16-MMA kernel
  uint8_t* image = nullptr;  // activation image for the integer decode kernel (K up to 16384)
  int* imageCounters = nullptr;        // arrival counters of the kernels that write images block by block (zero between launches)
  uint8_t* captureImage = nullptr;     // one-shot: where the next producer call writes the image of its result
  const uint8_t* supplyImage = nullptr;  // one-shot: image the next linear call reads instead of quantising x
  float* ummaPartial = nullptr;  // K-slice partial results of the tcgen05 prefill GEMM: [4][128][8192] floats, allocated on first use
  void* ummaActs = nullptr;  // fp16 activations laid out for the tcgen05 prefill GEMM (K up to 16384)
  std::atomic<uint64_t> launches{0};  // kernels launched through this context
  cudaStream_t stream = nullptr;
  cudaEvent_t done = nullptr;
  int* status = nullptr;      // device status word written by kernels that abort a bounded wait
  int* statusHost = nullptr;  // pinned mirror
  std::mutex mutex;
  std::unordered_map<void*, int> allocations;  // pointer -> hostVisible
  std::unordered_map<std::string, CUtensorMap> tensorMaps;  // weight matrix -> tiled-TMA descriptor
  std::unordered_map<void*, uint64_t> graphLaunches;         // captured graph -> kernels it launches per replay
  uint64_t captureStart = 0;
  std::string error;
};

namespace infdev {
int pdl_mode() {
  static const int mode = [] {
    const char* env = std::getenv("INFENG_PDL");
    return env ? std::atoi(env) : 2;
  }();
  return mode;
}
}  // namespace infdev

namespace {

int fail(infdev_ctx* ctx, int code, const std::string& text) {
  if (ctx)
    ctx->error = text;
  return code;
}

int check(infdev_ctx* ctx, cudaError_t e, const char* what) {
  if (e == cudaSuccess)
    return INFDEV_OK;
  return fail(ctx, INFDEV_E_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

struct Bind {  // makes the context's device current for the calling thread
  explicit Bind(infdev_ctx* ctx) { cudaSetDevice(ctx->device); }
};

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// The one-shot image requests are consumed by the first call that could honour them, whether or not it does.
uint8_t* take_capture(infdev_ctx* ctx) {
  uint8_t* image = ctx->captureImage;
  ctx->captureImage = nullptr;
  return image;
}
const uint8_t* take_supply(infdev_ctx* ctx) {
  const uint8_t* image = ctx->supplyImage;
  ctx->supplyImage = nullptr;
  return image;
}

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encoder() {
  static EncodeTiled function = [] {
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &status) != cudaSuccess || status != cudaDriverEntryPointSuccess)
      entry = nullptr;
    return reinterpret_cast<EncodeTiled>(entry);
  }();
  return function;
}

// Descriptor of a packed weight matrix [n][k/256 super-blocks] viewed as 8-byte elements: inner dimension = bytes of a
// row / 8, outer = n rows; box = boxBlocks super-blocks x boxRows rows. Cached per matrix: encoding costs about a microsecond.
int weight_map(infdev_ctx* ctx, const void* w, int64_t n, int64_t k, int blockBytes, int boxBlocks, int boxRows, CUtensorMap* out, int padBytes = 0) {
  const std::string key = std::to_string(reinterpret_cast<uintptr_t>(w)) + ":" + std::to_string(n) + ":" + std::to_string(k) + ":" + std::to_string(blockBytes) + ":" +
                          std::to_string(boxBlocks) + ":" + std::to_string(boxRows) + ":" + std::to_string(padBytes);
  std::lock_guard<std::mutex> lock(ctx->mutex);
  auto found = ctx->tensorMaps.find(key);
  if (found != ctx->tensorMaps.end()) {
    *out = found->second;
    return INFDEV_OK;
  }
  EncodeTiled encode = encoder();
  if (!encode)
    return fail(ctx, INFDEV_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const uint64_t rowBytes = uint64_t(k / 256) * blockBytes;
  const cuuint64_t dims[2] = {rowBytes / 8, cuuint64_t(n)}, strides[1] = {rowBytes};
  // padBytes widens the box past its super-blocks (the extra bytes are whatever follows in the row, or zero fill).
  const cuuint32_t box[2] = {cuuint32_t((boxBlocks * blockBytes + padBytes) / 8), cuuint32_t(boxRows)}, elementStrides[2] = {1, 1};
  CUtensorMap map;
  const CUresult result = encode(&map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(w), dims, strides, box, elementStrides,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (result != CUDA_SUCCESS)
    return fail(ctx, INFDEV_E_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(int(result)));
  ctx->tensorMaps.emplace(key, map);
  *out = map;
  return INFDEV_OK;
}

// fp32 rows -> activation image, one launch per 8-row slice.
int quantize_rows(infdev_ctx* ctx, const float* x, int64_t rows, int64_t k, uint8_t* image) {
  for (int64_t row = 0; row < rows; row += 8) {
    if (int r = check(ctx, infdev::activation_image_launch(x + row * k, int(k), int(rows - row < 8 ? rows - row : 8), int(k),
                                                           image + size_t(row / 8) * size_t(k / 256) * infdev::kActivationImageBlockBytes, ctx->stream),
                      "activation image"))
      return r;
    ++ctx->launches;
  }
  return INFDEV_OK;
}

}  // namespace

extern "C" {

infdev_ctx* infdev_create(int device, char* error) {
  auto report = [&](const std::string& text) {
    if (error) {
      std::strncpy(error, text.c_str(), 1023);
      error[1023] = 0;
    }
    return static_cast<infdev_ctx*>(nullptr);
  };
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    return report(std::string("no CUDA device available: ") + cudaGetErrorString(e));
  if (device < 0 || device >= count)
    return report("device index out of range");
  cudaDeviceProp prop;
  if ((e = cudaSetDevice(device)) != cudaSuccess || (e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess)
    return report(std::string("cudaSetDevice: ") + cudaGetErrorString(e));
  if (prop.major != 10)
    return report("this library contains sm_100a code only; device is sm_" + std::to_string(prop.major * 10 + prop.minor));
  auto* ctx = new infdev_ctx;
  ctx->device = device;
  ctx->sms = prop.multiProcessorCount;
  if (const char* env = std::getenv("INFENG_XSPLIT"))
    ctx->xsplit = std::atoi(env) == 1 ? 1 : 2;
  if (const char* env = std::getenv("INFENG_UMMA"))
    ctx->umma = std::atoi(env) != 0;
  if (const char* env = std::getenv("INFENG_INTEGER_DECODE"))
    ctx->integerDecode = std::atoi(env) != 0;
  if ((e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking)) != cudaSuccess ||
      (e = cudaEventCreateWithFlags(&ctx->done, cudaEventDisableTiming)) != cudaSuccess ||
      (e = cudaMalloc(reinterpret_cast<void**>(&ctx->status), sizeof(int))) != cudaSuccess ||
      (e = cudaMemset(ctx->status, 0, sizeof(int))) != cudaSuccess ||
      (e = cudaMalloc(reinterpret_cast<void**>(&ctx->image), size_t(64) * infdev::kActivationImageBlockBytes)) != cudaSuccess ||
      (e = cudaMalloc(reinterpret_cast<void**>(&ctx->imageCounters), infdev::kImageCounters * sizeof(int))) != cudaSuccess ||
      (e = cudaMemset(ctx->imageCounters, 0, infdev::kImageCounters * sizeof(int))) != cudaSuccess ||
      (e = cudaMalloc(&ctx->ummaActs, size_t(64) * infdev::kUmmaMaxActBytesPerBlock)) != cudaSuccess ||
      (e = cudaHostAlloc(reinterpret_cast<void**>(&ctx->statusHost), sizeof(int), cudaHostAllocDefault)) != cudaSuccess) {
    std::string text = std::string("context setup: ") + cudaGetErrorString(e);
    delete ctx;
    return report(text);
  }
  *ctx->statusHost = 0;
  return ctx;
}

void infdev_destroy(infdev_ctx* ctx) {
  if (!ctx)
    return;
  Bind bind(ctx);
  cudaStreamSynchronize(ctx->stream);
  for (auto& entry : ctx->allocations)
    entry.second ? cudaFreeHost(entry.first) : cudaFree(entry.first);
  cudaFree(ctx->status);
  cudaFree(ctx->image);
  cudaFree(ctx->imageCounters);
  cudaFree(ctx->ummaPartial);
  cudaFree(ctx->ummaActs);
  cudaFreeHost(ctx->statusHost);
  cudaEventDestroy(ctx->done);
  cudaStreamDestroy(ctx->stream);
  delete ctx;
}

const char* infdev_error(infdev_ctx* ctx) { return ctx ? ctx->error.c_str() : "null context"; }

int infdev_sm_count(infdev_ctx* ctx) { return ctx->sms; }

uint64_t infdev_launch_count(infdev_ctx* ctx) { return ctx->launches.load(); }

void* infdev_alloc(infdev_ctx* ctx, size_t bytes, int hostVisible) {
  Bind bind(ctx);
  void* pointer = nullptr;
  if (bytes == 0)
    bytes = 16;
  cudaError_t e;
  if (hostVisible) {
    e = cudaHostAlloc(&pointer, bytes, cudaHostAllocMapped | cudaHostAllocPortable);
    if (e == cudaSuccess)
      std::memset(pointer, 0, bytes);
  } else {
    e = cudaMalloc(&pointer, bytes);
    if (e == cudaSuccess)
      e = cudaMemsetAsync(pointer, 0, bytes, ctx->stream);
  }
  if (check(ctx, e, "infdev_alloc") != INFDEV_OK)
    return nullptr;
  std::lock_guard<std::mutex> lock(ctx->mutex);
  ctx->allocations[pointer] = hostVisible;
  return pointer;
}

void infdev_free(infdev_ctx* ctx, void* pointer) {
  if (!pointer)
    return;
  Bind bind(ctx);
  int hostVisible;
  {
    std::lock_guard<std::mutex> lock(ctx->mutex);
    auto found = ctx->allocations.find(pointer);
    if (found == ctx->allocations.end())
      return;
    hostVisible = found->second;
    ctx->allocations.erase(found);
    ctx->tensorMaps.clear();  // descriptors may point into the freed range
  }
  // Work already queued on the stream may still use the buffer.
  cudaStreamSynchronize(ctx->stream);
  hostVisible ? cudaFreeHost(pointer) : cudaFree(pointer);
}

int infdev_upload(infdev_ctx* ctx, void* device, const void* host, size_t bytes) {
  Bind bind(ctx);
  return check(ctx, cudaMemcpyAsync(device, host, bytes, cudaMemcpyHostToDevice, ctx->stream), "infdev_upload");
}

int infdev_download(infdev_ctx* ctx, void* host, const void* device, size_t bytes) {
  Bind bind(ctx);
  int r = check(ctx, cudaMemcpyAsync(host, device, bytes, cudaMemcpyDeviceToHost, ctx->stream), "infdev_download");
  return r ? r : check(ctx, cudaStreamSynchronize(ctx->stream), "infdev_download");
}

int infdev_peek(infdev_ctx* ctx, void* host, const void* device, size_t bytes) {
  Bind bind(ctx);
  return check(ctx, cudaMemcpy(host, device, bytes, cudaMemcpyDeviceToHost), "infdev_peek");
}

int infdev_copy(infdev_ctx* ctx, void* destination, const void* source, size_t bytes) {
  Bind bind(ctx);
  return check(ctx, cudaMemcpyAsync(destination, source, bytes, cudaMemcpyDefault, ctx->stream), "infdev_copy");
}

int infdev_fill(infdev_ctx* ctx, void* device, int byte, size_t bytes) {
  Bind bind(ctx);
  return check(ctx, cudaMemsetAsync(device, byte, bytes, ctx->stream), "infdev_fill");
}

int infdev_commit(infdev_ctx* ctx, uint32_t timeoutMs) {
  Bind bind(ctx);
  cudaError_t e = cudaMemcpyAsync(ctx->statusHost, ctx->status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream);
  if (e == cudaSuccess)
    e = cudaEventRecord(ctx->done, ctx->stream);
  if (e != cudaSuccess)
    return check(ctx, e, "infdev_commit");
  if (timeoutMs == 0)
    e = cudaEventSynchronize(ctx->done);
  else {
    // Sleeping between polls keeps the core free for the client threads; with the default timer slack of 50 us a
    // 10 us sleep would overshoot the end of a 2 ms pass by several per cent, so the polling thread asks for 1 us.
    static thread_local const bool slackSet = [] { return prctl(PR_SET_TIMERSLACK, 1000UL, 0UL, 0UL, 0UL) == 0; }();
    (void)slackSet;
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeoutMs);
    while ((e = cudaEventQuery(ctx->done)) == cudaErrorNotReady) {
      if (std::chrono::steady_clock::now() > deadline)
        return fail(ctx, INFDEV_E_TIMEOUT, "commit deadline passed with work still queued on the stream");
      std::this_thread::sleep_for(std::chrono::microseconds(10));
    }
  }
  if (e != cudaSuccess)
    return check(ctx, e, "infdev_commit");
  if (*ctx->statusHost != 0) {
    const int status = *ctx->statusHost;
    *ctx->statusHost = 0;
    cudaMemsetAsync(ctx->status, 0, sizeof(int), ctx->stream);
    return fail(ctx, INFDEV_E_DEVICE, "a kernel abandoned a bounded wait (device status " + std::to_string(status) + ")");
  }
  return INFDEV_OK;
}

int infdev_check_abort_path(infdev_ctx* ctx, uint32_t spins) {
  Bind bind(ctx);
  if (!spins || spins > (1u << 16))
    return fail(ctx, INFDEV_E_ARGUMENT, "check_abort_path: 1 to 65536 polls");
  ctx->launches += 1;
  return check(ctx, infdev::bounded_wait_probe_launch(spins, ctx->status, ctx->stream), "check_abort_path");
}

void* infdev_event_create(infdev_ctx* ctx) {
  Bind bind(ctx);
  cudaEvent_t event = nullptr;
  return cudaEventCreate(&event) == cudaSuccess ? event : nullptr;
}

void infdev_event_destroy(infdev_ctx* ctx, void* event) {
  Bind bind(ctx);
  if (event)
    cudaEventDestroy(static_cast<cudaEvent_t>(event));
}

int infdev_event_record(infdev_ctx* ctx, void* event) {
  Bind bind(ctx);
  return check(ctx, cudaEventRecord(static_cast<cudaEvent_t>(event), ctx->stream), "infdev_event_record");
}

float infdev_event_elapsed_ms(infdev_ctx* ctx, void* start, void* stop) {
  Bind bind(ctx);
  float ms = -1.f;
  if (cudaEventSynchronize(static_cast<cudaEvent_t>(stop)) != cudaSuccess)
    return -1.f;
  cudaEventElapsedTime(&ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop));
  return ms;
}

int infdev_set_umma(infdev_ctx* ctx, int enabled) {
  ctx->umma = enabled != 0;
  return INFDEV_OK;
}

size_t infdev_image_bytes(int64_t rows, int64_t k) {
  return size_t((rows + 7) / 8) * size_t(k / 256) * infdev::kActivationImageBlockBytes;
}

int infdev_quantize(infdev_ctx* ctx, const float* x, int64_t rows, int64_t k, uint8_t* image) {
  Bind bind(ctx);
  if (rows < 0 || k <= 0 || k % 256 || !aligned16(x) || !aligned16(image))
    return fail(ctx, INFDEV_E_ARGUMENT, "quantize: k must be a positive multiple of 256 and buffers 16-byte aligned");
  return quantize_rows(ctx, x, rows, k, image);
}

int infdev_image_capture(infdev_ctx* ctx, uint8_t* image) {
  if (!aligned16(image))
    return fail(ctx, INFDEV_E_ARGUMENT, "image_capture: the image must be 16-byte aligned");
  ctx->captureImage = image;
  return INFDEV_OK;
}

int infdev_image_supply(infdev_ctx* ctx, const uint8_t* image) {
  if (!aligned16(image))
    return fail(ctx, INFDEV_E_ARGUMENT, "image_supply: the image must be 16-byte aligned");
  ctx->supplyImage = image;
  return INFDEV_OK;
}

int infdev_set_integer_decode(infdev_ctx* ctx, int enabled) {
  ctx->integerDecode = enabled != 0;
  return INFDEV_OK;
}

int infdev_set_xsplit(infdev_ctx* ctx, int xsplit) {
  if (xsplit != 1 && xsplit != 2)
    return fail(ctx, INFDEV_E_ARGUMENT, "xsplit must be 1 or 2");
  ctx->xsplit = xsplit;
  return INFDEV_OK;
}

int infdev_graph_begin(infdev_ctx* ctx) {
  Bind bind(ctx);
  ctx->captureStart = ctx->launches.load();
  return check(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal), "infdev_graph_begin");
}

void* infdev_graph_end(infdev_ctx* ctx) {
  Bind bind(ctx);
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  if (check(ctx, cudaStreamEndCapture(ctx->stream, &graph), "infdev_graph_end") != INFDEV_OK)
    return nullptr;
  const int r = check(ctx, cudaGraphInstantiate(&exec, graph, 0), "cudaGraphInstantiate");
  cudaGraphDestroy(graph);
  if (r != INFDEV_OK)
    return nullptr;
  ctx->graphLaunches[exec] = ctx->launches.load() - ctx->captureStart;  // counted while capturing, not executed yet
  ctx->launches = ctx->captureStart;
  return exec;
}

int infdev_graph_launch(infdev_ctx* ctx, void* graph) {
  Bind bind(ctx);
  ctx->launches += ctx->graphLaunches[graph];
  return check(ctx, cudaGraphLaunch(static_cast<cudaGraphExec_t>(graph), ctx->stream), "infdev_graph_launch");
}

void infdev_graph_destroy(infdev_ctx* ctx, void* graph) {
  Bind bind(ctx);
  if (graph)
    cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(graph));
}

// ---- quantised linear algebra ----------------------------------------------------------------

int infdev_dequant(infdev_ctx* ctx, int type, const void* blocks, int64_t count, float* out) {
  Bind bind(ctx);
  ctx->launches += 1;
  if (infdev::format_supported(type) || type == INFDEV_F16)
    return check(ctx, infdev::format_dequant_launch(type, blocks, count, out, ctx->stream), "dequant");
  if (type != INFDEV_Q4_K && type != INFDEV_Q6_K)
    return fail(ctx, INFDEV_E_ARGUMENT, "dequant: unsupported block type " + std::to_string(type));
  return check(ctx, infdev::dequant_launch(type, blocks, count, out, ctx->stream), "dequant");
}

// `supplied`: image of x to read instead of quantising it (integer kernel only).
static int linear_run(infdev_ctx* ctx, int type, bool pair, int count, const void* const* w, const void* const* w2, const int64_t* n, int64_t k,
                      const float* x, int64_t m, float* const* y, const float* const* residual, const uint8_t* supplied) {
  if (type != INFDEV_Q4_K && type != INFDEV_Q6_K)
    return fail(ctx, INFDEV_E_ARGUMENT, "linear: weight type must be Q4_K or Q6_K");
  if (pair && type != INFDEV_Q4_K)
    return fail(ctx, INFDEV_E_ARGUMENT, "gate_up: only Q4_K pairs are supported");
  if (count < 1 || count > 4 || m < 0 || k <= 0 || k % 256)
    return fail(ctx, INFDEV_E_ARGUMENT, "linear: need 1..4 matrices and k a positive multiple of 256");
  if (type == INFDEV_Q6_K && k % 2048)
    return fail(ctx, INFDEV_E_ARGUMENT, "linear: Q6_K rows must be 16-byte aligned (k a multiple of 2048)");
  if (pair && k > 4096)
    return fail(ctx, INFDEV_E_ARGUMENT, "gate_up: k must not exceed 4096");
  if (!aligned16(x) || (k % 4))
    return fail(ctx, INFDEV_E_ARGUMENT, "linear: activations must be 16-byte aligned");
  bool umma = ctx->umma && m > 8 && type == INFDEV_Q4_K && k % 2048 == 0 && k <= 16384;
  for (int i = 0; i < count; ++i)
    umma = umma && n[i] > 0 && n[i] % infdev::kUmmaTileRows == 0 && aligned16(w[i]) && (!pair || aligned16(w2[i]));
  if (umma) {
    // tcgen05 path: rows per tile 128, accumulators in tensor memory
    infdev::UmmaParams u{};
    u.nseg = count;
    int tiles = 0;
    for (int i = 0; i < count; ++i) {
      u.seg[i] = {static_cast<const uint8_t*>(w[i]), pair ? static_cast<const uint8_t*>(w2[i]) : nullptr, y[i], residual ? residual[i] : nullptr,
                  int(n[i]), int(n[i]), tiles};
      if (int r = weight_map(ctx, w[i], n[i], k, 144, 1, infdev::kUmmaTileRows, &u.map[i][0]))
        return r;
      if (pair)
        if (int r = weight_map(ctx, w2[i], n[i], k, 144, 1, infdev::kUmmaTileRows, &u.map[i][1]))
          return r;
      tiles += int(n[i] / infdev::kUmmaTileRows);
    }
    u.tiles = tiles;
    u.k = int(k);
    // A matrix of few 128-row tiles (n = 4096: 32 of them) would leave most SMs idle during prefill: cut K into slices.
    u.splits = 1;
    if (!pair && count == 1 && m > 8 && n[0] <= 8192 && n[0] % 4 == 0)
      for (int s = 4; s > 1; --s)
        if ((k / 256) % s == 0 && tiles * s <= ctx->sms) {
          u.splits = s;
          break;
        }
    if (u.splits > 1 && !ctx->ummaPartial)
      if (int r = check(ctx, cudaMalloc(reinterpret_cast<void**>(&ctx->ummaPartial), size_t(4) * 128 * 8192 * sizeof(float)), "prefill partial buffer"))
        return r;
    u.partial = ctx->ummaPartial;
    u.acts = static_cast<const uint8_t*>(ctx->ummaActs);
    u.status = ctx->status;
    const int64_t slice = 128;  // activation rows per launch
    for (int64_t row = 0; row < m; row += slice) {
      u.m = int(m - row < slice ? m - row : slice);
      for (int i = 0; i < count; ++i) {
        u.seg[i].y = y[i] + row * n[i];
        u.seg[i].res = residual && residual[i] ? residual[i] + row * n[i] : nullptr;
      }
      if (int r = check(ctx, infdev::umma_launch(pair, u, x + row * k, int(k), ctx->sms, ctx->stream), "umma launch"))
        return r;
      ctx->launches += u.splits > 1 ? 3 : 2;
    }
    return INFDEV_OK;
  }
  infdev::GemvParams p{};
  p.nseg = count;
  int tiles = 0;
  const bool integer = type == INFDEV_Q4_K && ctx->integerDecode && k <= 16384;
  const int pad = integer ? infdev::kDecodePadBytes : 0;
  for (int i = 0; i < count; ++i) {
    if (n[i] <= 0 || n[i] % 16 || !aligned16(w[i]) || (pair && !aligned16(w2[i])))
      return fail(ctx, INFDEV_E_ARGUMENT, "linear: n must be a positive multiple of 16 and weights 16-byte aligned");
    p.seg[i] = {static_cast<const uint8_t*>(w[i]), pair ? static_cast<const uint8_t*>(w2[i]) : nullptr, y[i], residual ? residual[i] : nullptr,
                int(n[i]), int(n[i]), tiles};
    const int blockBytes = type == INFDEV_Q4_K ? 144 : 210;
    if (int r = weight_map(ctx, w[i], n[i], k, blockBytes, infdev::kGemvStageBlocks, infdev::kGemvTileRows, &p.map[i][0], pad))
      return r;
    if (pair)
      if (int r = weight_map(ctx, w2[i], n[i], k, blockBytes, infdev::kGemvStageBlocks, infdev::kGemvTileRows, &p.map[i][1], pad))
        return r;
    tiles += int(n[i] / 16);
  }
  p.tiles = tiles;
  p.ldx = int(k);
  p.k = int(k);
  p.status = ctx->status;
  // More than 8 activation rows: 8-row slices re-use the weights out of L2.
  for (int64_t row = 0; row < m; row += 8) {
    p.x = x + row * k;
    p.m = int(m - row < 8 ? m - row : 8);
    for (int i = 0; i < count; ++i) {
      p.seg[i].y = y[i] + row * n[i];
      p.seg[i].res = residual && residual[i] ? residual[i] + row * n[i] : nullptr;
    }
    if (integer) {
      if (supplied) {  // 8-row slices of k/256 blocks
        p.image = supplied + size_t(row / 8) * size_t(k / 256) * infdev::kActivationImageBlockBytes;
      } else {
        p.image = ctx->image;
        if (int r = check(ctx, infdev::activation_image_launch(p.x, p.ldx, p.m, p.k, ctx->image, ctx->stream), "activation image"))
          return r;
        ++ctx->launches;
      }
      if (int r = check(ctx, infdev::q4k_decode_launch(pair, p, ctx->sms, ctx->stream), "q4k decode launch"))
        return r;
      ++ctx->launches;
      continue;
    }
    if (int r = check(ctx, infdev::gemv_launch(type, pair, ctx->xsplit, p, ctx->sms, ctx->stream), "gemv launch"))
      return r;
    ++ctx->launches;
  }
  return INFDEV_OK;
}

static int linear_common(infdev_ctx* ctx, int type, bool pair, int count, const void* const* w, const void* const* w2, const int64_t* n, int64_t k,
                         const float* x, int64_t m, float* const* y, const float* const* residual) {
  Bind bind(ctx);
  const uint8_t* supplied = take_supply(ctx);
  uint8_t* captured = take_capture(ctx);
  if (captured && (count != 1 || n[0] % 256))
    return fail(ctx, INFDEV_E_ARGUMENT, "linear: an image of the result needs a single matrix with n a multiple of 256");
  if (infdev::format_supported(type)) {  // Q5_K, Q8_0, IQ4_XS: one plain launch per matrix and 8-row slice
    if (m < 0 || k <= 0 || k % 256 || !aligned16(x))
      return fail(ctx, INFDEV_E_ARGUMENT, "linear: k must be a positive multiple of 256 and the activations 16-byte aligned");
    for (int i = 0; i < count; ++i) {
      if (int r = check(ctx, infdev::format_linear_launch(type, pair, w[i], pair ? w2[i] : nullptr, n[i], k, x, m, y[i], residual ? residual[i] : nullptr, ctx->stream),
                        "linear"))
        return r;
      ctx->launches += uint64_t((m + 7) / 8);
    }
    return captured ? quantize_rows(ctx, y[0], m, n[0], captured) : INFDEV_OK;
  }
  if (int r = linear_run(ctx, type, pair, count, w, w2, n, k, x, m, y, residual, supplied))
    return r;
  // A GEMV tile is 16 outputs wide, a 256-value image block spans 16 tiles on different SMs: the image of the result
  // takes a launch of its own.
  return captured ? quantize_rows(ctx, y[0], m, n[0], captured) : INFDEV_OK;
}

int infdev_linear(infdev_ctx* ctx, int type, const void* w, int64_t n, int64_t k, const float* x, int64_t m, float* y, const float* residual) {
  return linear_common(ctx, type, false, 1, &w, nullptr, &n, k, x, m, &y, &residual);
}

int infdev_linear_group(infdev_ctx* ctx, int type, int count, const void* const* w, const int64_t* n, int64_t k, const float* x, int64_t m,
                        float* const* y) {
  return linear_common(ctx, type, false, count, w, nullptr, n, k, x, m, y, nullptr);
}

int infdev_gate_up(infdev_ctx* ctx, int type, const void* wg, const void* wu, int64_t n, int64_t k, const float* x, int64_t m, float* y) {
  return linear_common(ctx, type, true, 1, &wg, &wu, &n, k, x, m, &y, nullptr);
}

// ---- elementwise / normalisation ---------------------------------------------------------------

int infdev_gather_tokens(infdev_ctx* ctx, const infdev_query* queries, int queryCount, const int32_t* requestData, uint32_t capacity,
                         const int32_t* proposals, uint32_t mode, int32_t* rowTokens) {
  Bind bind(ctx);
  ctx->launches += 1;
  return check(ctx, infdev::gather_tokens_launch(queries, queryCount, requestData, capacity, proposals, mode, rowTokens, ctx->stream),
               "gather_tokens");
}

int infdev_embedding(infdev_ctx* ctx, int type, const void* table, int64_t k, const int32_t* rowTokens, int64_t rows, float* out) {
  Bind bind(ctx);
  if (k % 256)
    return fail(ctx, INFDEV_E_ARGUMENT, "embedding: k must be a multiple of 256");
  ctx->launches += 1;
  if (infdev::format_supported(type))
    return check(ctx, infdev::format_embedding_launch(type, table, k, rowTokens, rows, out, ctx->stream), "embedding");
  if (type != INFDEV_Q4_K && type != INFDEV_Q6_K)
    return fail(ctx, INFDEV_E_ARGUMENT, "embedding: unsupported table type " + std::to_string(type));
  return check(ctx, infdev::embedding_launch(type, table, k, rowTokens, rows, out, ctx->stream), "embedding");
}

int infdev_rms_norm(infdev_ctx* ctx, const float* x, const float* w, int64_t rows, int64_t dim, float* y) {
  Bind bind(ctx);
  if (dim % 4 || !aligned16(x) || !aligned16(w) || !aligned16(y))
    return fail(ctx, INFDEV_E_ARGUMENT, "rms_norm: dim must be a multiple of 4 and buffers 16-byte aligned");
  ctx->launches += 1;
  uint8_t* image = take_capture(ctx);
  if (image && dim % 256)
    return fail(ctx, INFDEV_E_ARGUMENT, "rms_norm: an image needs dim to be a multiple of 256");
  return check(ctx, infdev::rms_norm_launch(x, w, nullptr, rows, dim, y, image, ctx->stream), "rms_norm");
}

int infdev_rms_norm_gather(infdev_ctx* ctx, const float* x, const float* w, const infdev_query* queries, int queryCount, int64_t count, float* y) {
  Bind bind(ctx);
  (void)queryCount;
  ctx->launches += 1;
  return check(ctx, infdev::rms_norm_launch(x, w, queries, count, 4096, y, take_capture(ctx), ctx->stream), "rms_norm_gather");
}

// ---- gated delta rule --------------------------------------------------------------------------

int infdev_gdn_prepare(infdev_ctx* ctx, const float* x, const float* mixed, const float* wBeta, const float* wAlpha, const float* ssmA,
                       const float* ssmDt, const float* convWeight, const infdev_query* queries, int queryCount, int64_t rows,
                       uint64_t stateOffset, uint64_t stateBytes, float* q, float* k, float* v, float* beta, float* g) {
  Bind bind(ctx);
  (void)queryCount;
  if (stateOffset % 16 || stateBytes % 16)
    return fail(ctx, INFDEV_E_ARGUMENT, "gdn_prepare: state offsets must be multiples of 16 bytes");
  ctx->launches += 1;
  return check(ctx,
               infdev::gdn_prepare_launch(x, mixed, wBeta, wAlpha, ssmA, ssmDt, convWeight, queries, rows, stateOffset, stateBytes, q, k, v, beta, g,
                                          ctx->stream),
               "gdn_prepare");
}

int infdev_gdn_decode(infdev_ctx* ctx, const float* x, const float* mixed, const float* wBeta, const float* wAlpha, const float* ssmA,
                      const float* ssmDt, const float* convWeight, const float* z, const float* normWeight, const infdev_query* queries,
                      int queryCount, uint64_t convStateOffset, uint64_t stateOffset, uint64_t stateBytes, float* out) {
  Bind bind(ctx);
  if (convStateOffset % 16 || stateOffset % 16 || stateBytes % 16)
    return fail(ctx, INFDEV_E_ARGUMENT, "gdn_decode: state offsets must be multiples of 16 bytes");
  ctx->launches += 1;
  return check(ctx,
               infdev::gdn_decode_launch(x, mixed, wBeta, wAlpha, ssmA, ssmDt, convWeight, z, normWeight, queries, queryCount, convStateOffset, stateOffset,
                                         stateBytes, out, take_capture(ctx), ctx->imageCounters, ctx->stream),
               "gdn_decode");
}

static int delta_rule_common(infdev_ctx* ctx, const float* q, const float* k, const float* v, const float* g, const float* beta, const float* z,
                             const float* normWeight, const infdev_query* queries, int queryCount, uint64_t stateOffset, uint64_t stateBytes,
                             float* out, uint32_t chunkedFrom) {
  Bind bind(ctx);
  if (stateOffset % 16 || stateBytes % 16)
    return fail(ctx, INFDEV_E_ARGUMENT, "delta_rule: state offsets must be multiples of 16 bytes");
  if (chunkedFrom && ctx->captureImage) {
    take_capture(ctx);
    return fail(ctx, INFDEV_E_ARGUMENT, "delta_rule_prefill: writes no image of its result; use infdev_delta_rule for decode-sized passes");
  }
  ctx->launches += chunkedFrom ? 2 : 1;
  return check(ctx,
               infdev::delta_rule_launch(q, k, v, g, beta, z, normWeight, queries, queryCount, stateOffset, stateBytes, out, take_capture(ctx), ctx->imageCounters,
                                         chunkedFrom, ctx->stream),
               "delta_rule");
}

int infdev_delta_rule(infdev_ctx* ctx, const float* q, const float* k, const float* v, const float* g, const float* beta, const float* z,
                      const float* normWeight, const infdev_query* queries, int queryCount, uint64_t stateOffset, uint64_t stateBytes, float* out) {
  return delta_rule_common(ctx, q, k, v, g, beta, z, normWeight, queries, queryCount, stateOffset, stateBytes, out, 0);
}

int infdev_delta_rule_prefill(infdev_ctx* ctx, const float* q, const float* k, const float* v, const float* g, const float* beta, const float* z,
                              const float* normWeight, const infdev_query* queries, int queryCount, uint64_t stateOffset, uint64_t stateBytes,
                              float* out) {
  return delta_rule_common(ctx, q, k, v, g, beta, z, normWeight, queries, queryCount, stateOffset, stateBytes, out, 16);
}

// ---- attention ---------------------------------------------------------------------------------

int infdev_rope_table(infdev_ctx* ctx, int64_t positions, float* table) {
  Bind bind(ctx);
  std::vector<float> host(size_t(positions) * 64);
  for (int64_t p = 0; p < positions; ++p)
    for (int d = 0; d < 32; ++d) {
      const double angle = double(p) / std::pow(1.0e7, double(d) / 32.0);
      host[(p * 32 + d) * 2] = float(std::cos(angle));
      host[(p * 32 + d) * 2 + 1] = float(std::sin(angle));
    }
  int r = check(ctx, cudaMemcpyAsync(table, host.data(), host.size() * 4, cudaMemcpyHostToDevice, ctx->stream), "rope_table");
  return r ? r : check(ctx, cudaStreamSynchronize(ctx->stream), "rope_table");
}

int infdev_attention_prepare(infdev_ctx* ctx, const float* qg, const float* k, const float* v, const float* qNorm, const float* kNorm,
                             const float* rope, const infdev_query* queries, int queryCount, int64_t rows, const int32_t* table,
                             int32_t tableStride, int32_t blockTokens, float* q, void* cacheK, void* cacheV) {
  Bind bind(ctx);
  if (rows > 0 && queryCount < 1)
    return fail(ctx, INFDEV_E_ARGUMENT, "attention: rows without queries");
  if (blockTokens <= 0 || blockTokens % 16)
    return fail(ctx, INFDEV_E_ARGUMENT, "attention: blockTokens must be a positive multiple of 16");
  ctx->launches += 1;
  return check(ctx,
               infdev::attention_prepare_launch(qg, k, v, qNorm, kNorm, rope, queries, queryCount, table, tableStride, blockTokens, rows, q, cacheK, cacheV,
                                                ctx->stream),
               "attention_prepare");
}

size_t infdev_attention_scratch_bytes(int64_t rows, uint32_t maxSplits) { return size_t(rows) * 16 * maxSplits * 260 * sizeof(float); }

int infdev_attention(infdev_ctx* ctx, const float* q, const float* qg, const void* cacheK, const void* cacheV, const infdev_query* queries,
                     int queryCount, int64_t rows, const int32_t* table, int32_t tableStride, int32_t blockTokens, uint32_t maxSplits,
                     float* partials, float* out) {
  Bind bind(ctx);
  if (rows > 0 && queryCount < 1)
    return fail(ctx, INFDEV_E_ARGUMENT, "attention: rows without queries");
  if (blockTokens <= 0 || blockTokens % 16 || maxSplits < 1 || maxSplits > 64)
    return fail(ctx, INFDEV_E_ARGUMENT, "attention: blockTokens must be a multiple of 16 and maxSplits in 1..64");
  ctx->launches += 2;
  return check(ctx,
               infdev::attention_launch(q, qg, cacheK, cacheV, queries, queryCount, table, tableStride, blockTokens, rows, maxSplits, partials, out,
                                        take_capture(ctx), ctx->stream),
               "attention");
}

int infdev_mtp_fuse(infdev_ctx* ctx, const float* embedding, const float* hidden, const infdev_query* queries, int queryCount, const float* enorm,
                    const float* hnorm, int64_t rows, uint32_t mode, uint64_t seedOffset, uint64_t stateBytes, float* y) {
  Bind bind(ctx);
  (void)queryCount;
  ctx->launches += 1;
  return check(ctx, infdev::mtp_fuse_launch(embedding, hidden, queries, enorm, hnorm, rows, mode, seedOffset, stateBytes, y, ctx->stream),
               "mtp_fuse");
}

int infdev_attention_static(infdev_ctx* ctx, const float* q, const float* qg, const void* cacheK, const void* cacheV, const infdev_query* queries,
                            int queryCount, int64_t rows, const int32_t* table, int32_t tableStride, int32_t blockTokens, float* out) {
  Bind bind(ctx);  // the symbol lookup of the first call on a device needs that device current
  if (take_capture(ctx))  // the one-shot request is consumed by the first call that could honour it; this variant writes no image
    return fail(ctx, INFDEV_E_ARGUMENT, "attention_static: writes no image of its result; use infdev_attention after infdev_image_capture");
  if (rows > 0 && queryCount < 1)
    return fail(ctx, INFDEV_E_ARGUMENT, "attention: rows without queries");
  if (blockTokens <= 0 || blockTokens % 16)
    return fail(ctx, INFDEV_E_ARGUMENT, "attention_static: blockTokens must be a positive multiple of 16");
  if (rows > infdev::attention_static_max_rows())
    return fail(ctx, INFDEV_E_ARGUMENT, "attention_static: at most " + std::to_string(infdev::attention_static_max_rows()) +
                                            " packed rows fit the built-in scratch; use infdev_attention with a caller-provided buffer");
  ctx->launches += 2;
  return check(ctx, infdev::attention_static_launch(q, qg, cacheK, cacheV, queries, queryCount, table, tableStride, blockTokens, rows, ctx->device, out, ctx->stream),
               "attention_static");
}

// ---- sampling, packing, verification -----------------------------------------------------------

int infdev_sample(infdev_ctx* ctx, const float* logits, int64_t vocab, infdev_query* queries, int queryCount, int64_t count, uint32_t mode,
                  int32_t* tokens) {
  Bind bind(ctx);
  (void)queryCount;
  ctx->launches += 1;
  return check(ctx, infdev::sample_launch(logits, int(vocab), queries, count, mode, tokens, ctx->stream), "sample");
}

int infdev_pack_queries(infdev_ctx* ctx, const infdev_query* in, int count, int drafting, uint32_t draftWidth, const uint64_t* statePrevious,
                        const uint64_t* stateNext, uint64_t candidateBase, uint64_t stateBytes, infdev_query* out, uint32_t* meta) {
  Bind bind(ctx);
  if (count < 0 || count > 32)
    return fail(ctx, INFDEV_E_ARGUMENT, "pack_queries: at most 32 queries per pass");
  ctx->launches += 1;
  return check(ctx,
               infdev::pack_queries_launch(in, count, drafting, draftWidth, statePrevious, stateNext, candidateBase, stateBytes, out, meta, ctx->stream),
               "pack_queries");
}

int infdev_verify_drafts(infdev_ctx* ctx, const infdev_query* queries, int count, const int32_t* sampled, const int32_t* proposed,
                         uint32_t draftWidth, const int32_t* stops, uint32_t stopStride, const uint32_t* stopCounts, uint32_t* verdict) {
  Bind bind(ctx);
  if (count > 32)
    return fail(ctx, INFDEV_E_ARGUMENT, "verify_drafts: at most 32 queries");
  ctx->launches += 1;
  return check(ctx, infdev::verify_drafts_launch(queries, count, sampled, proposed, draftWidth, stops, stopStride, stopCounts, verdict, ctx->stream),
               "verify_drafts");
}

int infdev_commit_states(infdev_ctx* ctx, const infdev_query* queries, int count, const uint32_t* verdict, const uint64_t* stateNext,
                         uint64_t candidateBase, uint64_t stateBytes) {
  Bind bind(ctx);
  if (stateBytes % 16 || candidateBase % 16)
    return fail(ctx, INFDEV_E_ARGUMENT, "commit_states: state records must be 16-byte aligned");
  ctx->launches += 1;
  return check(ctx, infdev::commit_states_launch(queries, count, verdict, stateNext, candidateBase, stateBytes, ctx->stream), "commit_states");
}

}  // extern "C"
