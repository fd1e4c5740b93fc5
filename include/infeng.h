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
 * INFENG_DRAFT_WIDTH (MTP proposals per step, default 2 as forward.cpp:139), INFENG_SEED (base of the per-slot
 * sampling seeds, default the clock), INFENG_BLOCK_TOKENS, INFENG_COMMIT_TIMEOUT_MS, INFENG_GRAPHS (0 disables CUDA-graph replay of decode passes). */
infeng_engine* infeng_engine_create(const char* weights, const char* draftWeights, const char* kernels, uint32_t context, char* error);
/* engine.cpp:251-254: drops one reference; the engine dies with its last sequence. */
void infeng_engine_release(infeng_engine* engine);
/* engine.cpp:256-259: takes the first free of 8 slots; NULL + "maximum live sequence count reached" when none. */
infeng_sequence* infeng_sequence_create(infeng_engine* engine, const int32_t* stops, uint32_t stopCount, float temperature, float topP, int32_t topK,
                                        uint32_t speculative, char* error);
/* engine.cpp:261-265: waits for the in-flight pass of the sequence, frees its slot and K/V references. */
void infeng_sequence_release(infeng_sequence* sequence);
/* engine.cpp:267-284: appends prompt tokens and starts generation; returns the new token count (the first
 * cursor to read). count == UINT32_MAX cancels (returns 0). -3: still generating. -4: nothing to do or the
 * context would overflow. */
int32_t infeng_sequence_append(infeng_sequence* sequence, const int32_t* tokens, uint32_t count);
/* engine.cpp:286-292: blocks until token `cursor` exists or generation stopped. Token id >= 0; -1 finished;
 * -5 the pass failed (no evictable K/V block, or a device error). */
int32_t infeng_sequence_read(infeng_sequence* sequence, uint32_t cursor);
/* engine.cpp:294-297: 0 parameter count, 1 weight bytes, 2 K/V bytes ever bound, 3 drafter (0 none, 1 MTP),
 * 4 draft width. Additions for throughput accounting: 5 passes run, 6 rows processed, 7 microseconds spent in
 * passes (host clock, commit included), 8 decoder layers, 9 vocabulary size, 10 nanoseconds of device time of
 * the passes (CUDA events on the stream), 11 kernels launched, 12 to 14 microseconds the scheduler spent outside
 * the passes: building batches, waiting for the engine lock after a pass, handing sampled tokens over. */
uint64_t infeng_engine_info(infeng_engine* engine, uint32_t field);
/* engine.cpp:299-303: 0 drafted tokens, 1 accepted tokens, 2 tokens held in the K/V cache. */
uint64_t infeng_sequence_info(infeng_sequence* sequence, uint32_t field);

#ifdef __cplusplus
}
#endif
#endif
