/* infdev: the thin C-ABI device layer under the MTLQwen Engine.
 *
 * It stands where the reference's Metal backend stands (backend/metal/device.hpp:17-140): buffers, a
 * serial command stream with a blocking commit, the paged K/V pool, and one typed launch function per
 * kernel of backend/metal/kernel/*.metal. The reference dispatches kernels by string name with
 * positional tensors (device.hpp:122-139); here each kernel is a plain C function. All pointers named
 * "device" are CUDA device addresses; no C++ or torch types cross this boundary.
 *
 * Return convention: 0 on success, a negative INFDEV_E_* code otherwise; the text of the last failure
 * of a context is available from infdev_error(). Launches are asynchronous on the context's stream and
 * execute in call order, like the reference's barrier-after-every-dispatch encoder (device.hpp:132).
 */
#ifndef INFDEV_H
#define INFDEV_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct infdev_ctx infdev_ctx;

enum {
  INFDEV_OK = 0,
  INFDEV_E_CUDA = -1,     /* a CUDA call failed */
  INFDEV_E_ARGUMENT = -2, /* shape / alignment / type not supported */
  INFDEV_E_TIMEOUT = -3,  /* commit deadline passed while the stream was still busy */
  INFDEV_E_DEVICE = -4    /* a kernel gave up on a bounded wait and set the device status word */
};

/* ggml tensor type ids used by the GGUF files (forward.cpp:55 indexes kernels by `type - 11`). */
enum { INFDEV_F32 = 0, INFDEV_F16 = 1, INFDEV_Q8_0 = 8, INFDEV_Q4_K = 12, INFDEV_Q5_K = 13, INFDEV_Q6_K = 14, INFDEV_IQ4_XS = 23 };

/* Per-query ragged metadata, the CUDA form of GpuQuery (backend/metal/kernel/batch.hpp:11-16).
 * previous/next are device addresses of the slot's state record (0 = fresh sequence); state is the first
 * candidate-state row of a speculative query or 0xffffffff. `seed` is an addition: the Philox key of the slot. */
typedef struct infdev_query {
  uint64_t previous, next;
  uint32_t start, count, position, slot, state, logit, samples;
  float temperature, topP;
  int32_t topK;
  uint64_t seed;
} infdev_query;

/* Sizes of one per-slot state record (batch.hpp:3-8 with fp32 instead of fp16 conv taps and MTP seed). */
enum {
  INFDEV_CONV_STATE_BYTES = 8192 * 4 * 4,
  INFDEV_RECURRENT_STATE_BYTES = 32 * 128 * 128 * 4,
  INFDEV_GDN_LAYER_STATE_BYTES = INFDEV_CONV_STATE_BYTES + INFDEV_RECURRENT_STATE_BYTES
};

/* ---- context, memory, stream (Device::Device/empty/mapped/copy/command/commit, device.hpp:66-140) ---- */
infdev_ctx* infdev_create(int device, char* error /* >= 1024 bytes, may be null */);
void infdev_destroy(infdev_ctx* ctx);
const char* infdev_error(infdev_ctx* ctx);
int infdev_sm_count(infdev_ctx* ctx);
/* Number of kernels this context has launched so far (for launch accounting in benchmarks). */
uint64_t infdev_launch_count(infdev_ctx* ctx);
/* hostVisible != 0: pinned host memory mapped into the device (Metal "shared" storage, device.cpp:82-85);
 * the returned pointer is valid on both sides. Otherwise device memory, zero-filled. */
void* infdev_alloc(infdev_ctx* ctx, size_t bytes, int hostVisible);
void infdev_free(infdev_ctx* ctx, void* pointer);
int infdev_upload(infdev_ctx* ctx, void* device, const void* host, size_t bytes);
int infdev_download(infdev_ctx* ctx, void* host, const void* device, size_t bytes);
/* Reads device memory without touching the context's stream: a synchronous copy that is not ordered with queued work, so
 * it may be called from any thread while another thread launches (or captures) on the stream. The caller guarantees
 * that nothing queued writes the range. */
int infdev_peek(infdev_ctx* ctx, void* host, const void* device, size_t bytes);
int infdev_copy(infdev_ctx* ctx, void* destination, const void* source, size_t bytes);
int infdev_fill(infdev_ctx* ctx, void* device, int byte, size_t bytes);
/* Device::commit (device.cpp:138-145) with a deadline instead of an unbounded wait: blocks until the
 * stream drains or timeoutMs passes (0 = no deadline), then reports the device status word. */
int infdev_commit(infdev_ctx* ctx, uint32_t timeoutMs);
/* Health check of the failure path behind INFDEV_E_DEVICE (no reference counterpart: Device::wait waits for ever,
 * device.cpp:66-70). Every kernel here that waits on a barrier does so with an iteration limit and, when the limit runs
 * out, records a status code and returns instead of spinning. This launches a one-warp kernel whose wait cannot be
 * satisfied and gives up after `spins` polls (1 .. 65536, milliseconds at most): the next infdev_commit must return
 * INFDEV_E_DEVICE, and the one after it INFDEV_OK, with the context fully usable. Nothing faults or hangs. */
int infdev_check_abort_path(infdev_ctx* ctx, uint32_t spins);
/* Timing on the context's stream. */
void* infdev_event_create(infdev_ctx* ctx);
void infdev_event_destroy(infdev_ctx* ctx, void* event);
int infdev_event_record(infdev_ctx* ctx, void* event);
float infdev_event_elapsed_ms(infdev_ctx* ctx, void* start, void* stop);
/* Which quantised-linear kernel serves Q4_K matrices with n % 128 == 0 and k % 2048 == 0 when a launch has more than 8
 * activation rows (prefill chunks, speculative rows): 1 (default) = the tcgen05 / TMEM GEMM, 0 = the GEMV kernels in
 * slices of 8 rows, which compute every activation row on its own. Environment: INFENG_UMMA. */
int infdev_set_umma(infdev_ctx* ctx, int enabled);
/* Activation split of the fp16 tensor-core GEMV: 2 = hi+lo fp16 (fp32-accurate, default), 1 = hi only. */
int infdev_set_xsplit(infdev_ctx* ctx, int xsplit);
/* Q4_K GEMV for up to 8 rows per launch: 1 (default) = integer-MMA kernel over activations quantised to 16 bits per
 * 256-value block (error at most 1.6e-5 of the block maximum), 0 = the fp16-MMA kernel. Q6_K always takes the
 * fp16-MMA kernel. Environment: INFENG_INTEGER_DECODE. */
int infdev_set_integer_decode(infdev_ctx* ctx, int enabled);

/* ---- activation images (no reference counterpart) ----
 * The integer Q4_K decode kernel reads its activations as an "image": per (row, 256-value block) 16-bit integers
 * split into a high and a low byte plane in tensor-core fragment order, the block's scale and its sub-block sums;
 * rows come in 8-row slices of k/256 blocks (4384 bytes per block and slice). A linear call builds the image from
 * its fp32 activations with one extra small launch; a pass avoids that launch by letting the kernel that produces
 * the activations write their image as well, and handing it to the linear call that follows. */
size_t infdev_image_bytes(int64_t rows, int64_t k);
/* image = quantised x[rows,k] (k a multiple of 256). */
int infdev_quantize(infdev_ctx* ctx, const float* x, int64_t rows, int64_t k, uint8_t* image);
/* One-shot: the next infdev_rms_norm, infdev_rms_norm_gather, infdev_delta_rule (gated, rows below 256),
 * infdev_attention, infdev_linear or infdev_gate_up call on this context also writes the image of its result rows
 * to `image` (infdev_image_bytes(rows, width of the result) bytes); the fp32 result is written as usual. The norm,
 * delta-rule and attention kernels write it themselves; a linear call adds a quantisation launch on its result. */
int infdev_image_capture(infdev_ctx* ctx, uint8_t* image);
/* One-shot: the next infdev_linear, infdev_linear_group or infdev_gate_up call takes the image of its activations
 * from `image` (it must be the image of exactly the x passed) instead of quantising x. Only the integer Q4_K kernel
 * reads images; other kernels ignore the request and read x. */
int infdev_image_supply(infdev_ctx* ctx, const uint8_t* image);
/* CUDA-graph capture of a pass on the context's stream (no reference counterpart: Metal re-encodes every
 * pass). begin/end bracket the launches; launch replays; the handle is freed with graph_destroy. */
int infdev_graph_begin(infdev_ctx* ctx);
void* infdev_graph_end(infdev_ctx* ctx);
int infdev_graph_launch(infdev_ctx* ctx, void* graph);
void infdev_graph_destroy(infdev_ctx* ctx, void* graph);

/* ---- quantised linear algebra ---- */
/* Block dequantisation to fp32, bit-exact with dequant_tile (quant_linear.metal:32-48 Q4_K, :50-67 Q5_K, :69-85 Q6_K,
 * :87-97 Q8_0, :99-115 IQ4_XS); `count` blocks of 256 values (32 for Q8_0). INFDEV_F16 converts count * 256 halves. */
int infdev_dequant(infdev_ctx* ctx, int type, const void* blocks, int64_t count, float* out);
/* y[m,n] = x[m,k] . W[n,k]^T (+ residual[m,n]); replaces Ops::linear (forward.cpp:51-70) over
 * linear_decode_q4_k[_add] (quant_linear.metal:245-327), linear_decode_q6_k[_add] (:436-512) and, for
 * m > 8, linear_prefill (:151-233). x, y, residual fp32 row-major; residual may alias y or be null.
 * Q5_K, Q8_0 and IQ4_XS matrices (linear_decode_q5_k, linear_decode_q8_0, :329-434, 514-570; the types the real
 * Qwen3.5 files mix in) are served by a plain dequantise-and-multiply kernel: correct, not tuned. */
int infdev_linear(infdev_ctx* ctx, int type, const void* w, int64_t n, int64_t k, const float* x, int64_t m, float* y, const float* residual);
/* Up to four weight matrices sharing x in one launch (the q/k/v and qkv/z projections of Ops::decoder,
 * forward.cpp:86-88, 98). */
int infdev_linear_group(infdev_ctx* ctx, int type, int count, const void* const* w, const int64_t* n, int64_t k, const float* x, int64_t m,
                        float* const* y);
/* y[m,n] = silu(x.Wg^T) * (x.Wu^T): mlp_gate_up_q4_k_decode (fused_kernels.metal:11-78) and the post == 2
 * epilogue of linear_prefill (quant_linear.metal:224-232). */
int infdev_gate_up(infdev_ctx* ctx, int type, const void* wg, const void* wu, int64_t n, int64_t k, const float* x, int64_t m, float* y);

/* ---- elementwise / normalisation ---- */
/* Per-row token ids: embedding_q4_k's source selection (quant_linear.metal:581-584). mode 0 target pass
 * (request ids, or draft proposals for speculative rows > 0), mode 2 previous MTP proposal. */
int infdev_gather_tokens(infdev_ctx* ctx, const infdev_query* queries, int queryCount, const int32_t* requestData, uint32_t capacity,
                         const int32_t* proposals, uint32_t mode, int32_t* rowTokens);
/* out[row] = dequant(table[tokens[row]]): embedding_q4_k (quant_linear.metal:572-591), plus a Q6_K table. */
int infdev_embedding(infdev_ctx* ctx, int type, const void* table, int64_t k, const int32_t* rowTokens, int64_t rows, float* out);
/* rms_norm (native_ops.metal:6-34): y = x * rsqrt(mean(x^2) + 1e-6) * w over `dim` = 4096. */
int infdev_rms_norm(infdev_ctx* ctx, const float* x, const float* w, int64_t rows, int64_t dim, float* y);
/* rms_norm_gather (native_ops.metal:12-15): row i of y normalises the i-th sampled row of the pass. */
int infdev_rms_norm_gather(infdev_ctx* ctx, const float* x, const float* w, const infdev_query* queries, int queryCount, int64_t count, float* y);


/* ---- gated delta rule (GDN) ---- */
/* gdn_ba_prepare_4096x32 (native_ops.metal:89-113) and gdn_causal_conv_silu (fused_kernels.metal:202-232) in
 * one call. x: normalised hidden [rows,4096]; mixed: qkv projection [rows,8192]; wBeta/wAlpha f32 [32,4096];
 * ssmA, ssmDt [32]; convWeight f32 [8192,4]. stateOffset: byte offset of this layer's conv taps inside a
 * state record; stateBytes: size of one record (stride between candidate rows). Outputs q,k [rows,16,128]
 * (the reference stores each twice for 32 heads; consumers use head % 16), v [rows,32,128], beta, g [rows,32]. */
int infdev_gdn_prepare(infdev_ctx* ctx, const float* x, const float* mixed, const float* wBeta, const float* wAlpha, const float* ssmA,
                       const float* ssmDt, const float* convWeight, const infdev_query* queries, int queryCount, int64_t rows,
                       uint64_t stateOffset, uint64_t stateBytes, float* q, float* k, float* v, float* beta, float* g);
/* delta_rule_decode / delta_rule_prefill (delta_rule.metal:73-363) for every query length, followed by
 * gated_rms_norm_128 (fused_kernels.metal:234-254) when z is non-null (z [rows,4096], normWeight [128]).
 * stateOffset here addresses the layer's recurrent state S fp32 [32][128][128] inside a record. */
int infdev_delta_rule(infdev_ctx* ctx, const float* q, const float* k, const float* v, const float* g, const float* beta, const float* z,
                      const float* normWeight, const infdev_query* queries, int queryCount, uint64_t stateOffset, uint64_t stateBytes, float* out);
/* infdev_gdn_prepare followed by infdev_delta_rule (gated) in one launch, for passes whose queries are all short (decode
 * rows, speculative rows): every (sequence, head) CTA prepares its own 384 channels and its beta / g. Same arithmetic,
 * same results; the intermediate q, k, v, beta, g are not written. */
int infdev_gdn_decode(infdev_ctx* ctx, const float* x, const float* mixed, const float* wBeta, const float* wAlpha, const float* ssmA,
                      const float* ssmDt, const float* convWeight, const float* z, const float* normWeight, const infdev_query* queries,
                      int queryCount, uint64_t convStateOffset, uint64_t stateOffset, uint64_t stateBytes, float* out);
/* The same for a pass that holds prefill chunks: non-speculative queries of at least 16 tokens take the chunked form
 * (16 tokens per step, the role of delta_rule_prefill, delta_rule.metal:19-253), every other query the sequential one.
 * Results agree with infdev_delta_rule to fp32 rounding. Two launches; no image of the result (a pending
 * infdev_image_capture makes the call fail). */
int infdev_delta_rule_prefill(infdev_ctx* ctx, const float* q, const float* k, const float* v, const float* g, const float* beta, const float* z,
                              const float* normWeight, const infdev_query* queries, int queryCount, uint64_t stateOffset, uint64_t stateBytes,
                              float* out);

/* ---- attention ---- */
/* init_rope (native_ops.metal:115-120): cos/sin table fp32 [positions,32,2] for theta = 1e7, evaluated on
 * the host in double precision and uploaded. */
int infdev_rope_table(infdev_ctx* ctx, int64_t positions, float* table);
/* attention_prepare (attention.metal:14-50) plus the K/V cache append of attention_scan (:126-133).
 * qg [rows,16,512] (q | gate per head), k,v [rows,4,256]; q out [rows,16,256]. The cache of one layer is
 * [physical block][4][blockTokens][256] fp16; table[slot*tableStride + logical block] = physical block
 * (the role of SparseKV::map, device.cpp:178-198). blockTokens must be a multiple of 16. */
int infdev_attention_prepare(infdev_ctx* ctx, const float* qg, const float* k, const float* v, const float* qNorm, const float* kNorm,
                             const float* rope, const infdev_query* queries, int queryCount, int64_t rows, const int32_t* table,
                             int32_t tableStride, int32_t blockTokens, float* q, void* cacheK, void* cacheV);
/* With qg == NULL only the K/V store runs: mtp_store_kv (attention.metal:53-100, drafter_store_kv<256>). */
/* attention_scan + attention_reduce (attention.metal:103-216): causal GQA over the cache, times
 * sigmoid(gate). partials: scratch of infdev_attention_scratch_bytes(rows, maxSplits) bytes. */
int infdev_attention(infdev_ctx* ctx, const float* q, const float* qg, const void* cacheK, const void* cacheV, const infdev_query* queries,
                     int queryCount, int64_t rows, const int32_t* table, int32_t tableStride, int32_t blockTokens, uint32_t maxSplits,
                     float* partials, float* out);
size_t infdev_attention_scratch_bytes(int64_t rows, uint32_t maxSplits);
/* No counterpart in the reference. The same attention as infdev_attention for callers that cannot allocate device
 * memory at all (a server that handed every free byte to its K/V pool at start-up, or a decode loop that must not
 * make a device-synchronising allocation call): the split-K partials live in an array built into the library
 * (about 2 MiB per GPU, held until the process exits) instead of a caller buffer, and the call performs no
 * cudaMalloc / cudaFree. Limits: at most 8 packed rows (one decode step of 8 sequences) and 16 splits per row;
 * more rows are refused with INFDEV_E_ARGUMENT. The first call on a device looks up the array's device address;
 * make that call before starting any stream capture. All calls share the one array, so two calls that overlap on
 * the GPU (different streams or contexts of one process) race; calls on one stream are safe. */
int infdev_attention_static(infdev_ctx* ctx, const float* q, const float* qg, const void* cacheK, const void* cacheV, const infdev_query* queries,
                            int queryCount, int64_t rows, const int32_t* table, int32_t tableStride, int32_t blockTokens, float* out);

/* mtp_fuse (native_ops.metal:43-87): y [rows,8192] = [rmsnorm(embedding) * enorm | rmsnorm(h) * hnorm]; h is
 * the slot's stored seed, the previous row's hidden or the same row's hidden by mode (2, 1, 0); mode 1 also
 * stores the next seed. seedOffset: byte offset of the seed (fp32 [4096]) inside a state record. */
int infdev_mtp_fuse(infdev_ctx* ctx, const float* embedding, const float* hidden, const infdev_query* queries, int queryCount, const float* enorm,
                    const float* hnorm, int64_t rows, uint32_t mode, uint64_t seedOffset, uint64_t stateBytes, float* y);

/* ---- sampling, packing, verification ---- */
/* sample_logits (native_ops.metal:122-224): logits fp32 [count,vocab]; mode 0 target, 1 MTP drafting. */
int infdev_sample(infdev_ctx* ctx, const float* logits, int64_t vocab, infdev_query* queries, int queryCount, int64_t count, uint32_t mode,
                  int32_t* tokens);
/* The packing loop of forward() (forward.cpp:171-191) on the device. in[i].samples carries the slot's
 * requested-token count. meta[4] receives rows, logit rows, flags (1 sequential, 2 prefill), packed count. At most 32
 * queries (one lane each). */
int infdev_pack_queries(infdev_ctx* ctx, const infdev_query* in, int count, int drafting, uint32_t draftWidth, const uint64_t* statePrevious,
                        const uint64_t* stateNext, uint64_t candidateBase, uint64_t stateBytes, infdev_query* out, uint32_t* meta);
/* The acceptance loop of Engine::schedule (engine.cpp:205-216) on the device, for every query of a target pass:
 * sampled[query.logit + s] is emitted; a stop token ends the query after it; a speculative query continues while the
 * sampled token equals proposed[(s + 1) * 8 + query.state / query.count] and s < draftWidth. stops[slot * stopStride
 * .. + stopCounts[slot]) are the slot's stop tokens. verdict[3 i], [3 i + 1], [3 i + 2] = accepted proposals, emitted
 * tokens, stopped (0 / 1) of query i. */
int infdev_verify_drafts(infdev_ctx* ctx, const infdev_query* queries, int count, const int32_t* sampled, const int32_t* proposed,
                         uint32_t draftWidth, const int32_t* stops, uint32_t stopStride, const uint32_t* stopCounts, uint32_t* verdict);
/* Copies each speculative query's candidate state row number verdict[3 i] (the row after the last accepted proposal) to
 * the slot's next state record, stateNext[slot] (engine.cpp:217-218). */
int infdev_commit_states(infdev_ctx* ctx, const infdev_query* queries, int count, const uint32_t* verdict, const uint64_t* stateNext,
                         uint64_t candidateBase, uint64_t stateBytes);

#ifdef __cplusplus
}
#endif
#endif
