// Internal launch interface of the non-GEMV kernels.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include "../../include/infdev.h"

namespace infdev {

// Q5_K, Q8_0, IQ4_XS (and F16 for dequantisation): formats.cu
bool format_supported(int type);
int format_block_values(int type);
cudaError_t format_dequant_launch(int type, const void* blocks, int64_t count, float* out, cudaStream_t stream);
cudaError_t format_embedding_launch(int type, const void* table, int64_t k, const int32_t* tokens, int64_t rows, float* out, cudaStream_t stream);
cudaError_t format_linear_launch(int type, bool pair, const void* w, const void* w2, int64_t n, int64_t k, const float* x, int64_t m, float* y,
                                 const float* residual, cudaStream_t stream);
cudaError_t bounded_wait_probe_launch(uint32_t limit, int* status, cudaStream_t stream);
cudaError_t dequant_launch(int type, const void* blocks, int64_t count, float* out, cudaStream_t stream);
cudaError_t embedding_launch(int type, const void* table, int64_t k, const int32_t* tokens, int64_t rows, float* out, cudaStream_t stream);
cudaError_t gather_tokens_launch(const infdev_query* queries, int queryCount, const int32_t* requestData, uint32_t capacity,
                                 const int32_t* proposals, uint32_t mode, int32_t* rowTokens, cudaStream_t stream);
cudaError_t rms_norm_launch(const float* x, const float* w, const infdev_query* queries, int64_t rows, int64_t dim, float* y, uint8_t* image,
                            cudaStream_t stream);

cudaError_t mtp_fuse_launch(const float* embedding, const float* hidden, const infdev_query* queries, const float* enorm, const float* hnorm,
                            int64_t rows, uint32_t mode, uint64_t seedOffset, uint64_t stateBytes, float* y, cudaStream_t stream);
cudaError_t gdn_prepare_launch(const float* x, const float* mixed, const float* wBeta, const float* wAlpha, const float* A, const float* dt,
                               const float* convWeight, const infdev_query* queries, int64_t rows, uint64_t stateOffset, uint64_t stateBytes,
                               float* q, float* k, float* v, float* beta, float* g, cudaStream_t stream);
cudaError_t delta_rule_launch(const float* q, const float* k, const float* v, const float* g, const float* beta, const float* z,
                              const float* normWeight, const infdev_query* queries, int queryCount, uint64_t stateOffset, uint64_t stateBytes,
                              float* out, uint8_t* image, int* counters, uint32_t chunkedFrom, cudaStream_t stream);
cudaError_t gdn_decode_launch(const float* x, const float* mixed, const float* wBeta, const float* wAlpha, const float* A, const float* dt,
                              const float* convWeight, const float* z, const float* normWeight, const infdev_query* queries, int queryCount,
                              uint64_t convStateOffset, uint64_t stateOffset, uint64_t stateBytes, float* out, uint8_t* image, int* counters,
                              cudaStream_t stream);
cudaError_t attention_prepare_launch(const float* qg, const float* rawK, const float* rawV, const float* qNorm, const float* kNorm, const float* rope,
                                     const infdev_query* queries, int queryCount, const int32_t* table, int tableStride, int blockTokens, int64_t rows, float* q,
                                     void* cacheK, void* cacheV, cudaStream_t stream);
cudaError_t attention_launch(const float* q, const float* qg, const void* cacheK, const void* cacheV, const infdev_query* queries,
                             int queryCount, const int32_t* table, int tableStride, int blockTokens, int64_t rows, uint32_t maxSplits, float* partials, float* out,
                             uint8_t* image, cudaStream_t stream);
cudaError_t attention_static_launch(const float* q, const float* qg, const void* cacheK, const void* cacheV, const infdev_query* queries,
                                    int queryCount, const int32_t* table, int tableStride, int blockTokens, int64_t rows, int device, float* out,
                                    cudaStream_t stream);
int attention_static_max_rows();
cudaError_t sample_launch(const float* logits, int vocab, infdev_query* queries, int64_t count, uint32_t mode, int32_t* tokens,
                          cudaStream_t stream);
cudaError_t pack_queries_launch(const infdev_query* in, int count, int drafting, uint32_t draftWidth, const uint64_t* statePrevious,
                                const uint64_t* stateNext, uint64_t candidateBase, uint64_t stateBytes, infdev_query* out, uint32_t* meta,
                                cudaStream_t stream);
cudaError_t verify_drafts_launch(const infdev_query* queries, int count, const int32_t* sampled, const int32_t* proposed, uint32_t draftWidth,
                                 const int32_t* stops, uint32_t stopStride, const uint32_t* stopCounts, uint32_t* verdict, cudaStream_t stream);
cudaError_t commit_states_launch(const infdev_query* queries, int count, const uint32_t* verdict, const uint64_t* stateNext,
                                 uint64_t candidateBase, uint64_t stateBytes, cudaStream_t stream);

}  // namespace infdev
