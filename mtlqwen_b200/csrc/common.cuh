// Shared device helpers for the sm_100a kernels: bounded mbarrier waits, bulk (TMA) copies, the
// m16n8k16 tensor-core instruction, and small numeric utilities.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <atomic>
#include <cstdint>

namespace infdev {

constexpr int kWarp = 32;

// Error codes written to the per-context device status word by kernels that give up on a wait.
enum DeviceStatus : int { kStatusOk = 0, kStatusBarrierTimeout = 1, kStatusBadArgument = 2 };

// ---- programmatic dependent launch ----
// Every kernel of a pass is launched with programmatic stream serialisation (launch_kernel below): its CTAs may become
// resident while the kernel before it in the stream is still running. A kernel lets its successor start early with
// pdl_launch_dependents() and must call pdl_wait() before it reads anything an earlier kernel wrote or writes
// anything an earlier kernel may still read; the wait returns once the preceding kernel has completed and its
// memory is visible. Because each kernel waits, completion is transitive along the stream. Both are no-ops in a
// kernel launched without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Set once per process from INFENG_PDL: 0 no kernel is launched early, 1 every kernel, 2 only the weight-streaming
// GEMV kernels (which use the time to fill their shared-memory ring), 3 those and the small kernels that follow a
// GEMV in a decoder layer (EARLY = 2).
int pdl_mode();

template <int EARLY = 0, class... Params, class... Args>
cudaError_t launch_kernel(void (*kernel)(Params...), dim3 grid, dim3 block, size_t sharedBytes, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = sharedBytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = (pdl_mode() == 1 || (pdl_mode() == 2 && EARLY == 1) || (pdl_mode() == 3 && EARLY >= 1)) ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// A kernel's opt-in to more than 48 KB of dynamic shared memory is a property of the (kernel, device) pair, and one
// process may hold contexts on several GPUs: the attribute is set once per device, for the device that is current.
constexpr int kMaxDevices = 64;
struct PerDeviceOnce {
  std::atomic<unsigned char> done[kMaxDevices] = {};
};

template <class Kernel> cudaError_t configure_shared_memory(Kernel kernel, size_t bytes, PerDeviceOnce& once) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess)
    return e;
  if (device < 0 || device >= kMaxDevices)
    return cudaErrorInvalidDevice;
  if (once.done[device].load(std::memory_order_acquire))
    return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes));
  // Ask for the largest shared-memory carve-out: kernels sized for two CTAs per SM get both only with all of it.
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, int(cudaSharedmemCarveoutMaxShared));
  if (e == cudaSuccess)
    once.done[device].store(1, std::memory_order_release);
  return e;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Non-blocking test of a phase: unlike try_wait it never suspends the thread, so it answers at once when the phase
// has already completed, which is the common case for a consumer that the producer keeps ahead of.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Waits for a phase with an iteration limit. Returns false when the limit ran out; the caller then
// raises the abort flag so every role of the kernel leaves its loops instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abortFlag, uint32_t limit = 1u << 20) {
  if (mbar_test_wait(bar, parity))  // the common case: the phase has already completed
    return true;
  for (uint32_t spin = 0; spin < limit; ++spin) {
    if (mbar_try_wait(bar, parity))
      return true;
    if ((spin & 1023u) == 1023u && *abortFlag)
      return false;
  }
  return false;
}

// Untiled bulk copy global -> shared, completion reported on an mbarrier. Both addresses must be
// 16-byte aligned and `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)), "l"(src),
               "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Tiled 2-D TMA load global -> shared through a tensor map; x counts elements of the innermost dimension and
// x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* dst, const void* tensorMap, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)),
               "l"(tensorMap), "r"(x), "r"(y), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Counts this thread as arrived at a named barrier without waiting: the signalling half of a producer / consumer pair
// whose other half calls named_barrier with the same id and total thread count.
__device__ __forceinline__ void named_barrier_arrive(int id, int threads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1)
    v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1)
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }

// Reads the two bytes at a 2-byte aligned address (210-byte Q6_K blocks are only 2-byte aligned).
__device__ __forceinline__ float load_half_bits(const uint8_t* p) {
  return __half2float(*reinterpret_cast<const __half*>(p));
}

}  // namespace infdev
