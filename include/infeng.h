/* infeng: the outward C ABI of the engine, binary-compatible with the reference's libinfeng
 * (runtime/engine.cpp:245-303, bound from Python in runtime/inference.py:26-38). A client of the reference
 * only has to load this library instead of libinfeng.dylib.
 *
 * Threading: every entry point may be called from any thread; all of them take the engine mutex, and
 * infeng_sequence_read blocks on the engine's condition variable until the scheduler thread has produced
 * the token. Tokens are copied in; the engine owns all device memory; no exception crosses this boundary.
 */
#ifndef INFENG_H
#define INFENG_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct infeng_engine infeng_engine;
typedef struct infeng_sequence infeng_sequence;

/* engine.cpp:247-249. weights: GGUF path; draftWeights: nullable GGUF path of a file that carries the MTP
 * block (blk.N.nextn.*) and then replaces `weights`; kernels: accepted for compatibility and ignored (the
 * Metal build compiles shader sources from that directory); context in (0, 65536]; error: >= 1024 bytes that
 * receive the message when the call returns NULL. Environment: INFENG_DEVICE (GPU index, default LOCAL_RANK or
 * 0), INFENG_KV_BLOCKS (physical 128-token K/V blocks, default ceil(context/128) as engine.cpp:86),
 * INFENG_DRAFT_WIDTH (MTP proposals per step, default 2 as forward.cpp:139), INFENG_SEED (base of the sampling
 * keys: sequence number i of an engine draws from a Philox stream keyed by (seed, i); default the clock), INFENG_CHECKPOINTS (entries of the prefix-checkpoint cache, default 8 as qwen35.hpp:24; each holds one state record),
 * INFENG_BLOCK_TOKENS, INFENG_COMMIT_TIMEOUT_MS, INFENG_GRAPHS (0 disables CUDA-graph replay of decode passes),
 * INFENG_BATCH_INVARIANT (1: every row goes through kernels that treat it on its own, the GEMV kernels for any row
 * count and the token-by-token delta rule, so a sequence's tokens are the same bits whatever shares its passes and
 * however the scheduler cut its prompt; prefill is several times slower). */
infeng_engine* infeng_engine_create(const char* weights, const char* draftWeights, const char* kernels, uint32_t context, char* error);
/* engine.cpp:251-254: drops one reference; the engine dies with its last sequence. */
void infeng_engine_release(infeng_engine* engine);
/* engine.cpp:256-259: takes the first free of 8 slots; NULL + "maximum live sequence count reached" when none. */
infeng_sequence* infeng_sequence_create(infeng_engine* engine, const int32_t* stops, uint32_t stopCount, float temperature, float topP, int32_t topK,
                                        uint32_t speculative, char* error);
/* No counterpart in the reference (its generator is seeded from the clock, engine.cpp:96-99). Gives the sequence a
 * sampling key of the client's choice instead of the one derived from the engine's base seed and the creation order:
 * with the same key, prompt and sampling parameters a sequence emits the same tokens whatever slot it holds and
 * whatever else is batched with it (the variate of its i-th token is Philox(key, i)). To be called before the first
 * append; returns 0, or -3 once the sequence has started generating. */
int32_t infeng_sequence_seed(infeng_sequence* sequence, uint64_t seed);
/* engine.cpp:261-265: waits for the in-flight pass of the sequence, frees its slot and K/V references. */
void infeng_sequence_release(infeng_sequence* sequence);
/* engine.cpp:267-284: appends prompt tokens and starts generation; returns the new token count (the first
 * cursor to read). count == UINT32_MAX cancels (returns 0). -3: still generating. -4: nothing to do, the
 * context would overflow, or a token id lies outside the vocabulary (the reference trusts its tokenizer; here the
 * ids index the embedding table on the device, so they are checked). */
int32_t infeng_sequence_append(infeng_sequence* sequence, const int32_t* tokens, uint32_t count);
/* engine.cpp:286-292: blocks until token `cursor` exists or generation stopped. Token id >= 0; -1 finished;
 * -5 the pass failed (no evictable K/V block, or a device error). */
int32_t infeng_sequence_read(infeng_sequence* sequence, uint32_t cursor);
/* engine.cpp:294-297: 0 parameter count, 1 weight bytes, 2 K/V bytes ever bound, 3 drafter (0 none, 1 MTP),
 * 4 draft width. Additions for throughput accounting: 5 passes run, 6 rows processed, 7 microseconds spent in
 * passes (host clock, commit included), 8 decoder layers, 9 vocabulary size, 10 nanoseconds of device time of
 * the passes (CUDA events on the stream), 11 kernels launched, 12 to 14 microseconds the scheduler spent outside
 * the passes: building batches, waiting for the engine lock after a pass, handing sampled tokens over, 15 rows of
 * prompt chunks among the rows of field 6 (prompt tokens restored from the prefix-checkpoint cache are not computed
 * and do not count). */
uint64_t infeng_engine_info(infeng_engine* engine, uint32_t field);
/* engine.cpp:299-303: 0 drafted tokens, 1 accepted tokens, 2 tokens held in the K/V cache. Additions: 3 position of
 * the anchor token of the sequence's latest speculative step, 4 .. 4 + draft width - 1 the drafter's proposals of
 * that step. */
uint64_t infeng_sequence_info(infeng_sequence* sequence, uint32_t field);
/* No counterpart in the reference (its state records are only reachable from the GPU). Copies `bytes` at `offset` of
 * the sequence's current state record to `out`: per gated-delta-rule layer the convolution taps fp32 [8192][4] and
 * the recurrent state fp32 [32][128][128], then the MTP seed fp32 [4096] (the target's final hidden state of the last
 * committed position, kept when a drafter is loaded). For persisting a conversation and for checking the state
 * against another implementation. Returns the bytes copied, -3 while the sequence is generating, -4 when the range
 * lies outside the record. field 0 of the call with bytes == 0 returns the record size. */
int64_t infeng_sequence_state(infeng_sequence* sequence, uint64_t offset, void* out, uint64_t bytes);

/* The header index of a GGUF file as the engine reads it (the role of ggml's gguf_init_from_buffer and its tensor
 * getters in loadWeights, forward.cpp:12-23; ggml is not a dependency of this build). Writes one text line per
 * tensor, "name<TAB>ggml type<TAB>absolute file offset of the data<TAB>bytes (0 = type not loadable)<TAB>ne0,ne1,...",
 * preceded by a line "gguf<TAB>version<TAB>alignment<TAB>data offset<TAB>tensor count", into `out` (capacity bytes,
 * NUL-terminated). Needs no GPU. Returns the length of the text, or -1 with the message in `error` (>= 1024 bytes)
 * when the file cannot be parsed or the text does not fit. */
int64_t infeng_gguf_describe(const char* path, char* out, uint64_t capacity, char* error);

#ifdef __cplusplus
}
#endif
#endif
