// Internal launch interface of the non-GEMV kernels.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include "../../include/infdev.h"

namespace infdev {

cudaError_t dequant_launch(int type, const void* blocks, int64_t count, float* out, cudaStream_t stream);
cudaError_t embedding_launch(int type, const void* table, int64_t k, const int32_t* tokens, int64_t rows, float* out, cudaStream_t stream);
cudaError_t gather_tokens_launch(const infdev_query* queries, int queryCount, const int32_t* requestData, uint32_t capacity,
                                 const int32_t* proposals, uint32_t mode, int32_t* rowTokens, cudaStream_t stream);
cudaError_t rms_norm_launch(const float* x, const float* w, const infdev_query* queries, int64_t rows, int64_t dim, float* y, cudaStream_t stream);

}  // namespace infdev
