// C++ face of the infdev C ABI for the host engine: reference-counted tensors, the device with its
// blocking commit, and the paged K/V pool. It takes the place of backend/metal/device.hpp in the
// reference: same roles (Tensor, Device, SparseKV), CUDA underneath.
#pragma once
#include <cstdint>
#include <filesystem>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>
#include "../../include/infdev.h"

namespace infeng {

struct Allocation {
  infdev_ctx* ctx;
  void* pointer;
  uint64_t bytes;
  bool hostVisible;
  Allocation(infdev_ctx* owner, void* memory, uint64_t size, bool shared) : ctx(owner), pointer(memory), bytes(size), hostVisible(shared) {}
  Allocation(const Allocation&) = delete;
  Allocation& operator=(const Allocation&) = delete;
  ~Allocation() { infdev_free(ctx, pointer); }
};

// A byte range of an allocation. The reference count of `buffer` is load-bearing: the scheduler decides
// copy-on-write of a slot's state by use_count() (engine.cpp:157) and prefix checkpoints share arenas.
struct Tensor {
  std::shared_ptr<Allocation> buffer;
  uint64_t offset = 0, bytes = 0;

  Tensor view(uint64_t start, uint64_t count, uint64_t stride = 1) const { return {buffer, offset + start * stride, count * stride}; }
  uint64_t address() const { return reinterpret_cast<uint64_t>(buffer->pointer) + offset; }
  template <class T> T* as() const { return reinterpret_cast<T*>(static_cast<uint8_t*>(buffer->pointer) + offset); }
  // Host pointer; only meaningful for host-visible allocations.
  template <class T> T* contents() const { return as<T>(); }
  explicit operator bool() const { return bool(buffer); }
};

class Device {
 public:
  infdev_ctx* ctx = nullptr;
  uint32_t commitTimeoutMs = 120000;

  explicit Device(int index) {
    char error[1024] = {0};
    ctx = infdev_create(index, error);
    if (!ctx)
      throw std::runtime_error(std::string("CUDA device unavailable: ") + error);
  }
  Device(const Device&) = delete;
  ~Device() { infdev_destroy(ctx); }

  Tensor empty(uint64_t bytes, bool shared = false) {
    void* pointer = infdev_alloc(ctx, bytes, shared);
    if (!pointer)
      throw std::runtime_error(std::string("device allocation failed: ") + infdev_error(ctx));
    return {std::make_shared<Allocation>(ctx, pointer, bytes, shared), 0, bytes};
  }

  void check(int code) const {
    if (code != INFDEV_OK)
      throw std::runtime_error(std::string(infdev_error(ctx)));
  }

  void upload(const Tensor& destination, const void* host, uint64_t bytes) { check(infdev_upload(ctx, destination.as<void>(), host, bytes)); }
  void copy(const Tensor& source, const Tensor& destination) { check(infdev_copy(ctx, destination.as<void>(), source.as<void>(), destination.bytes)); }
  // Blocks until the stream drains (Device::commit, device.cpp:138-145) but gives up after commitTimeoutMs.
  int commit() { return infdev_commit(ctx, commitTimeoutMs); }
};

// Physical block pool + per-slot block tables: the CUDA form of SparseKV (device.hpp:80-112). The
// reference maps 256 KiB tiles of a sparse Metal buffer; here a table [slot][logical block] -> physical
// block lives in device memory and the attention kernels walk it.
class PagedKV {
  Device& device;
  uint32_t slots, blocksPerSlot, maxPhysical, layers, blockTokens;
  uint32_t physicalBlocks = 0;  // high-water mark of blocks ever bound, for mappedBytes()
  uint64_t layerBytes;
  Tensor keys, values, table;
  std::vector<int32_t> mirror;

 public:
  static constexpr uint64_t tileBytes = 256ull << 10;

  PagedKV(Device& owner, uint32_t slotCount, uint32_t logicalBlocksPerSlot, uint32_t physical, uint32_t layerCount, uint32_t tokensPerBlock)
      : device(owner), slots(slotCount), blocksPerSlot(logicalBlocksPerSlot), maxPhysical(physical), layers(layerCount), blockTokens(tokensPerBlock),
        layerBytes(uint64_t(physical) * 4 * tokensPerBlock * 256 * 2), mirror(size_t(slotCount) * logicalBlocksPerSlot, 0) {
    keys = device.empty(layerBytes * layers);
    values = device.empty(layerBytes * layers);
    table = device.empty(mirror.size() * sizeof(int32_t));
  }

  void ensure(uint32_t blocks) { physicalBlocks = blocks > physicalBlocks ? blocks : physicalBlocks; }

  void map(uint32_t virtualBlock, uint32_t physicalBlock) {
    mirror[virtualBlock] = int32_t(physicalBlock);
    device.upload(table.view(virtualBlock, 1, sizeof(int32_t)), &mirror[virtualBlock], sizeof(int32_t));
  }

  Tensor key(uint32_t layer) const { return keys.view(layer, 1, layerBytes); }
  Tensor value(uint32_t layer) const { return values.view(layer, 1, layerBytes); }
  const int32_t* blockTable() const { return table.as<int32_t>(); }
  uint32_t tableStride() const { return blocksPerSlot; }
  // Bytes of K/V that have ever been bound, in the reference's unit: 2 x layers tiles of 256 KiB per
  // 128-token block (device.hpp:109-111).
  uint64_t mappedBytes() const { return uint64_t(physicalBlocks) * 2 * layers * (uint64_t(blockTokens) * 4 * 256 * 2); }
};

}  // namespace infeng
