// Internal launch interface between the C-ABI layer (infdev.cu) and the kernel files.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace infdev {

// One weight matrix of a grouped GEMV: all segments of a launch share the activations.
struct GemvSeg {
  const uint8_t* w;   // [n][k/256] super-blocks
  const uint8_t* w2;  // second matrix of a gate/up pair, else null
  float* y;           // [m][ldy]
  const float* res;   // residual added to the result (may alias y), else null
  int n, ldy, tile0;  // tile0: index of this segment's first 16-row tile in the launch
};

struct GemvParams {
  // Tiled-TMA descriptors of the weight matrices, [segment][matrix of a gate/up pair]: a 2-D view of the packed
  // rows as 8-byte elements, box = 8 super-blocks x 16 rows.
  alignas(64) CUtensorMap map[4][2];
  GemvSeg seg[4];
  int nseg, tiles;
  const float* x;  // [m][ldx] fp32, rows 16-byte aligned
  const uint8_t* image;  // quantised activations (act_image.cuh) of all k/256 blocks, for the integer Q4_K kernel
  int ldx, m, k;
  int* status;
};

// Box geometry shared by the host encoder and the kernel.
constexpr int kGemvStageBlocks = 8, kGemvTileRows = 16;
// The integer Q4_K kernel reads 32 bytes past the 8 super-blocks of a box row, which makes the row pitch in shared
// memory 1184 = 32 (mod 128) bytes: the 32-byte pieces of consecutive rows that a warp reads in one load then fall
// into different banks.
constexpr int kDecodePadBytes = 32;
constexpr int kImageCounters = 4096;  // arrival counters a context owns for block-wise image writers
constexpr int kActivationImageBlockBytes = 4384;  // act_image.cuh: image bytes per 256 activations x 8 rows

// ---- tcgen05 path (umma.cu) ----
constexpr int kUmmaTileRows = 128, kUmmaMaxActBytesPerBlock = 16 * 128 * 16 * 2;  // 64 KB of fp16 activations per super-block

struct UmmaParams {
  alignas(64) CUtensorMap map[4][2];  // box = one super-block (18 x 8 bytes) x 128 rows
  GemvSeg seg[4];
  int nseg, tiles;  // tiles of 128 rows
  // One matrix: K is cut into `splits` slices that different CTAs take; their partial results go to
  // `partial` [splits][m][n] and are summed (with the residual) by a second small kernel, in a fixed order.
  int splits;
  float* partial;
  int m, k;
  int actRows;           // MMA N: m rounded up to a multiple of 16 (set by umma_launch)
  const uint8_t* acts;   // prepared activations: k/256 blocks of actRows x 512 bytes
  int* status;
};

cudaError_t umma_launch(bool pair, const UmmaParams& p, const float* x, int ldx, int sms, cudaStream_t stream);

cudaError_t gemv_launch(int type, bool pair, int xsplit, const GemvParams& p, int sms, cudaStream_t stream);

// Integer-MMA Q4_K decode GEMV over an activation image (q4k_decode.cu).
cudaError_t q4k_decode_launch(bool pair, const GemvParams& p, int sms, cudaStream_t stream);
// fp32 activations [m][ldx] -> image of k/256 blocks; rows m..7 are zero-filled.
cudaError_t activation_image_launch(const float* x, int ldx, int m, int k, uint8_t* image, cudaStream_t stream);

}  // namespace infdev
