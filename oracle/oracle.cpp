// CPU oracle: a scalar restatement of the MTLQwen forward-step math.
//
// TEST INFRASTRUCTURE ONLY. Nothing in the product path may link, import or call this file;
// it exists so the CUDA kernels can be checked against an independent implementation, and so a
// CPU baseline can be timed beside them.
//
// Every function cites the reference source (paths relative to the MTLQwen tree) it follows.
// Parity status: the Q4_K / Q6_K dequantisers are pinned bit-for-bit against gguf-py's
// `gguf.quants.dequantize` through committed fixtures (tests/golden). The reference's own tests hold
// only end-to-end token ids that need the real 5.5 GB GGUF files and an Apple GPU, so every other
// function here is "parity unpinned" against the Metal kernels: it follows the kernel sources line
// by line but has never been compared with their output.
//
// Precision policy: activations are fp32 (the reference stores fp16 at every kernel boundary);
// dot products accumulate per 256-element block in fp32 and across blocks in double; the K/V cache is
// fp16 as in the reference. Built with -ffp-contract=off so the dequantisers match numpy exactly.
#include <omp.h>
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

namespace {

typedef _Float16 half_t;

inline float h16(const uint8_t* p) {  // quant_linear.metal:7-10
  uint16_t bits = uint16_t(p[0]) | (uint16_t(p[1]) << 8);
  half_t h;
  std::memcpy(&h, &bits, 2);
  return float(h);
}

inline float half_round(float v) { return float(half_t(v)); }

// quant_linear.metal:12-20
inline void scale_min_k4(unsigned j, const uint8_t* q, uint8_t& d, uint8_t& m) {
  if (j < 4) {
    d = q[j] & 63;
    m = q[j + 4] & 63;
  } else {
    d = (q[j + 4] & 15) | ((q[j - 4] >> 6) << 4);
    m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

// One 144-byte Q4_K super-block -> 256 floats. quant_linear.metal:32-48 (tile form) and :585-590.
void dequant_block_q4k(const uint8_t* b, float* out) {
  float d = h16(b), dm = h16(b + 2);
  for (unsigned t = 0; t < 4; ++t) {
    uint8_t sc0, mn0, sc1, mn1;
    scale_min_k4(2 * t, b + 4, sc0, mn0);
    scale_min_k4(2 * t + 1, b + 4, sc1, mn1);
    float d0 = d * float(sc0), m0 = dm * float(mn0), d1 = d * float(sc1), m1 = dm * float(mn1);
    for (unsigned l = 0; l < 32; ++l) {
      uint8_t q = b[16 + t * 32 + l];
      out[t * 64 + l] = d0 * float(q & 15) - m0;
      out[t * 64 + 32 + l] = d1 * float(q >> 4) - m1;
    }
  }
}

// One 210-byte Q6_K super-block -> 256 floats. quant_linear.metal:69-85.
void dequant_block_q6k(const uint8_t* b, float* out) {
  float d = h16(b + 208);
  for (unsigned h = 0; h < 2; ++h)
    for (unsigned s = 0; s < 4; ++s)
      for (unsigned l = 0; l < 32; ++l) {
        unsigned rr = s * 32 + l, qlo = h * 64 + ((rr & 32) ? 32 : 0) + l, r = h * 128 + rr;
        uint8_t q = b[qlo], lo = (rr & 64) ? (q >> 4) : (q & 15);
        uint8_t hi = (b[128 + h * 32 + l] >> (2 * s)) & 3;
        int8_t sc = int8_t(b[192 + h * 8 + (rr >> 4)]);
        out[r] = d * float(sc) * (float((hi << 4) | lo) - 32.0f);
      }
}

// One 34-byte Q8_0 block -> 32 floats: fp16 d, then 32 int8. quant_linear.metal:87-97.
void dequant_block_q8_0(const uint8_t* b, float* out) {
  float d = h16(b);
  for (unsigned l = 0; l < 32; ++l)
    out[l] = d * float(int8_t(b[2 + l]));
}

// One 176-byte Q5_K super-block -> 256 floats: fp16 d, fp16 dmin, 12 B of 6-bit scales / mins as in Q4_K, 32 B of
// high bits (bit j of byte l belongs to element 32 j + l), 128 B of low nibbles laid out as in Q4_K.
// quant_linear.metal:50-67.
void dequant_block_q5k(const uint8_t* b, float* out) {
  float d = h16(b), dm = h16(b + 2);
  for (unsigned t = 0; t < 4; ++t) {
    uint8_t sc0, mn0, sc1, mn1;
    scale_min_k4(2 * t, b + 4, sc0, mn0);
    scale_min_k4(2 * t + 1, b + 4, sc1, mn1);
    float d0 = d * float(sc0), m0 = dm * float(mn0), d1 = d * float(sc1), m1 = dm * float(mn1);
    for (unsigned l = 0; l < 32; ++l) {
      uint8_t q = b[48 + t * 32 + l], hm = b[16 + l];
      out[t * 64 + l] = d0 * float((q & 15) + ((hm & (1u << (2 * t))) ? 16 : 0)) - m0;
      out[t * 64 + 32 + l] = d1 * float((q >> 4) + ((hm & (1u << (2 * t + 1))) ? 16 : 0)) - m1;
    }
  }
}

// The 16 code points of the IQ4 non-linear 4-bit grid (quant_linear.metal:5).
const float kIq4nl[16] = {-127.0f, -104.0f, -83.0f, -65.0f, -49.0f, -35.0f, -22.0f, -10.0f, 1.0f, 13.0f, 25.0f, 38.0f, 53.0f, 69.0f, 89.0f, 113.0f};

// One 136-byte IQ4_XS super-block -> 256 floats: fp16 d, u16 of 2-bit scale highs, 4 B of 4-bit scale lows, 128 B of
// 4-bit code indices (16 bytes per 32-value sub-block: low nibbles are its first 16 values, high nibbles the last 16).
// quant_linear.metal:99-115.
void dequant_block_iq4xs(const uint8_t* b, float* out) {
  float d = h16(b);
  unsigned sh = unsigned(b[2]) | (unsigned(b[3]) << 8);
  for (unsigned j = 0; j < 8; ++j) {
    int ls = int((b[4 + (j >> 1)] >> (4 * (j & 1))) & 15) | int(((sh >> (2 * j)) & 3) << 4);
    float dl = d * float(ls - 32);
    for (unsigned l = 0; l < 32; ++l) {
      uint8_t q = b[8 + j * 16 + (l & 15)];
      out[j * 32 + l] = dl * kIq4nl[(l & 16) ? (q >> 4) : (q & 15)];
    }
  }
}

enum { TYPE_F32 = 0, TYPE_F16 = 1, TYPE_Q8_0 = 8, TYPE_Q4_K = 12, TYPE_Q5_K = 13, TYPE_Q6_K = 14, TYPE_IQ4_XS = 23 };

// Bytes and values of one block of a quantised type.
inline size_t block_bytes(int type) {
  return type == TYPE_Q4_K ? 144 : type == TYPE_Q6_K ? 210 : type == TYPE_Q5_K ? 176 : type == TYPE_IQ4_XS ? 136 : type == TYPE_Q8_0 ? 34 : 0;
}
inline int64_t block_values(int type) { return type == TYPE_Q8_0 ? 32 : 256; }

inline void dequant_block(int type, const uint8_t* b, float* out) {
  switch (type) {
    case TYPE_Q4_K: return dequant_block_q4k(b, out);
    case TYPE_Q6_K: return dequant_block_q6k(b, out);
    case TYPE_Q5_K: return dequant_block_q5k(b, out);
    case TYPE_IQ4_XS: return dequant_block_iq4xs(b, out);
    case TYPE_Q8_0: return dequant_block_q8_0(b, out);
  }
}

void dequant_row(const uint8_t* w, int type, int64_t n, int64_t k, float* out) {
  if (type == TYPE_F32) {
    std::memcpy(out, w + size_t(n) * k * 4, size_t(k) * 4);
    return;
  }
  if (type == TYPE_F16) {
    const half_t* p = reinterpret_cast<const half_t*>(w) + size_t(n) * k;
    for (int64_t i = 0; i < k; ++i)
      out[i] = float(p[i]);
    return;
  }
  const size_t bb = block_bytes(type);
  const int64_t values = block_values(type);
  const uint8_t* row = w + size_t(n) * (k / values) * bb;
  for (int64_t b = 0; b < k / values; ++b)
    dequant_block(type, row + b * bb, out + b * values);
}

inline double dot(const float* a, const float* b, int64_t k) {
  double total = 0.0;
  int64_t i = 0;
  for (; i + 256 <= k; i += 256) {
    float p[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < 256; j += 8)
      for (int l = 0; l < 8; ++l)
        p[l] += a[i + j + l] * b[i + j + l];
    total += double(((p[0] + p[1]) + (p[2] + p[3])) + ((p[4] + p[5]) + (p[6] + p[7])));
  }
  for (; i < k; ++i)
    total += double(a[i]) * double(b[i]);
  return total;
}

inline float silu(float v) { return v / (1.0f + std::exp(-v)); }
inline float sigmoid(float v) { return 1.0f / (1.0f + std::exp(-v)); }

}  // namespace

extern "C" {

// Threads the parallel loops below use from now on (for timing the oracle single-threaded and on all cores).
void orc_set_threads(int threads) { omp_set_num_threads(threads > 0 ? threads : 1); }

// ---- quant formats ---------------------------------------------------------------------------
void orc_dequant_q4k(const uint8_t* blocks, int64_t count, float* out) {
#pragma omp parallel for
  for (int64_t i = 0; i < count; ++i)
    dequant_block_q4k(blocks + i * 144, out + i * 256);
}

void orc_dequant_q6k(const uint8_t* blocks, int64_t count, float* out) {
#pragma omp parallel for
  for (int64_t i = 0; i < count; ++i)
    dequant_block_q6k(blocks + i * 210, out + i * 256);
}

// Any block type: `count` blocks -> count * (32 or 256) floats.
void orc_dequant(int type, const uint8_t* blocks, int64_t count, float* out) {
  const int64_t bytes = int64_t(block_bytes(type)), values = block_values(type);
#pragma omp parallel for
  for (int64_t i = 0; i < count; ++i)
    dequant_block(type, blocks + i * bytes, out + i * values);
}

// ---- linear ----------------------------------------------------------------------------------
// y[m,n] = sum_k x[m,k] * deq(W[n,k]) (+ residual[m,n]).
// quant_linear.metal:245-327 (Q4_K decode), :436-512 (Q6_K decode), :151-233 (prefill GEMM);
// epilogue `post` 0/1 as linear_decode_store :237-243. W is row-major by n, k/256 super-blocks per row.
void orc_linear(const uint8_t* w, int type, int64_t n, int64_t k, const float* x, int64_t m, float* y, const float* residual) {
  // Activation rows are taken 32 at a time so that a block of them stays in cache while the weight rows stream by;
  // every (row, column) dot product is computed independently, so the blocking does not change a single bit.
  for (int64_t r0 = 0; r0 < m; r0 += 32) {
    const int64_t r1 = std::min<int64_t>(m, r0 + 32);
#pragma omp parallel
    {
      std::vector<float> row(k);
#pragma omp for schedule(static)
      for (int64_t i = 0; i < n; ++i) {
        dequant_row(w, type, i, k, row.data());
        for (int64_t r = r0; r < r1; ++r) {
          float v = float(dot(x + r * k, row.data(), k));
          y[r * n + i] = residual ? v + residual[r * n + i] : v;
        }
      }
    }
  }
}

// y[m,n] = silu(x.Wg[n]) * (x.Wu[n]). fused_kernels.metal:48-78 (decode) and the `post == 2` epilogue of
// quant_linear.metal:224-232 (prefill).
void orc_gate_up(const uint8_t* wg, const uint8_t* wu, int type, int typeUp, int64_t n, int64_t k, const float* x, int64_t m, float* y) {
  for (int64_t r0 = 0; r0 < m; r0 += 32) {
    const int64_t r1 = std::min<int64_t>(m, r0 + 32);
#pragma omp parallel
    {
      std::vector<float> g(k), u(k);
#pragma omp for schedule(static)
      for (int64_t i = 0; i < n; ++i) {
        dequant_row(wg, type, i, k, g.data());
        dequant_row(wu, typeUp, i, k, u.data());
        for (int64_t r = r0; r < r1; ++r)
          y[r * n + i] = silu(float(dot(x + r * k, g.data(), k))) * float(dot(x + r * k, u.data(), k));
      }
    }
  }
}

// Row gather + dequantise. quant_linear.metal:572-591 (Q4_K); the Q6_K table follows :69-85.
void orc_embedding(const uint8_t* w, int type, int64_t k, const int32_t* ids, int64_t rows, float* y) {
  for (int64_t r = 0; r < rows; ++r)
    dequant_row(w, type, ids[r], k, y + r * k);
}

// ---- norms -----------------------------------------------------------------------------------
// native_ops.metal:16-34: y = x * rsqrt(mean(x^2) + eps) * w.
void orc_rms_norm(const float* x, const float* w, int64_t rows, int64_t dim, float eps, float* y) {
  for (int64_t r = 0; r < rows; ++r) {
    double ss = 0.0;
    for (int64_t d = 0; d < dim; ++d)
      ss += double(x[r * dim + d]) * x[r * dim + d];
    float scale = 1.0f / std::sqrt(float(ss / double(dim)) + eps);
    for (int64_t d = 0; d < dim; ++d)
      y[r * dim + d] = x[r * dim + d] * scale * w[d];
  }
}

// fused_kernels.metal:234-254: per (row, head) y = rmsnorm_128(o) * w * silu(z).
void orc_gated_rms_norm(const float* o, const float* z, const float* w, int64_t rowHeads, float* y) {
  for (int64_t r = 0; r < rowHeads; ++r) {
    double ss = 0.0;
    for (int d = 0; d < 128; ++d)
      ss += double(o[r * 128 + d]) * o[r * 128 + d];
    float scale = 1.0f / std::sqrt(float(ss / 128.0) + 1.0e-6f);
    for (int d = 0; d < 128; ++d)
      y[r * 128 + d] = o[r * 128 + d] * scale * w[d] * silu(z[r * 128 + d]);
  }
}

// ---- gated delta rule ------------------------------------------------------------------------
// native_ops.metal:89-113: beta = sigmoid(x.Wb), g = A * log(1 + exp(x.Wa + dt)); Wb, Wa are [32,4096] f32.
void orc_gdn_ba(const float* x, const float* wb, const float* wa, const float* A, const float* dt, int64_t rows, float* beta, float* g) {
  for (int64_t r = 0; r < rows; ++r)
    for (int h = 0; h < 32; ++h) {
      float b = float(dot(x + r * 4096, wb + h * 4096, 4096)), a = float(dot(x + r * 4096, wa + h * 4096, 4096)) + dt[h];
      beta[r * 32 + h] = sigmoid(b);
      g[r * 32 + h] = A[h] * std::log(1.0f + std::exp(a));
    }
}

// fused_kernels.metal:202-232 for one query of `rows` tokens: depthwise causal conv (4 taps) + SiLU over
// 8192 channels of `mixed` [rows,8192]; the three inputs before the chunk come from stateIn
// [8192][4] (null = fresh sequence = zeros). Writes q,k [rows,16,128] (the reference stores each q/k head
// twice, :221-224; here consumers index head % 16), v [rows,32,128], and the carried state after every
// token into states[rows][8192][4] when `everyToken`, else only the last token's into states[0].
void orc_gdn_conv(const float* mixed, const float* w, const float* stateIn, int64_t rows, float* q, float* k, float* v, float* states,
                  int everyToken) {
  for (int64_t p = 0; p < rows; ++p)
    for (int64_t c = 0; c < 8192; ++c) {
      float context[4], acc = 0.0f;
      for (int64_t r = 0; r < 4; ++r) {
        int64_t position = p - 3 + r;
        context[r] = position >= 0 ? mixed[position * 8192 + c] : stateIn ? stateIn[c * 4 + position + 4] : 0.0f;
        acc = std::fma(context[r], w[c * 4 + r], acc);
      }
      float value = silu(acc);
      if (c < 2048)
        q[p * 2048 + c] = value;
      else if (c < 4096)
        k[p * 2048 + c - 2048] = value;
      else
        v[p * 4096 + c - 4096] = value;
      if (everyToken || p + 1 == rows)
        std::memcpy(states + ((everyToken ? p : 0) * 8192 + c) * 4, context, 16);
    }
}

// delta_rule.metal:274-362, the sequential form, which is also the ground truth for the chunked
// prefill kernel (:73-253). q,k [T,16,128], v [T,32,128], g,beta [T,32]; S [32][128 k][128 v] fp32 is
// updated in place; out [T,32,128]. When `snapshots` is non-null the state after token t is copied to
// snapshots[t] (one selectable candidate row per token, :255).
void orc_delta_rule(const float* q, const float* k, const float* v, const float* g, const float* beta, int64_t T, float* S, float* out,
                    float* snapshots) {
  for (int64_t t = 0; t < T; ++t) {
#pragma omp parallel for
    for (int h = 0; h < 32; ++h) {
      const float *qh = q + (t * 16 + h % 16) * 128, *kh = k + (t * 16 + h % 16) * 128, *vh = v + (t * 32 + h) * 128;
      float* s = S + size_t(h) * 128 * 128;
      float qs = 0.0f, ks = 0.0f;
      for (int d = 0; d < 128; ++d) {
        qs += qh[d] * qh[d];
        ks += kh[d] * kh[d];
      }
      float qn = 1.0f / std::sqrt(qs + 1.0e-6f) * 0.08838834764831845f, kn = 1.0f / std::sqrt(ks + 1.0e-6f);
      float qv[128], kv[128], qk = 0.0f;
      for (int d = 0; d < 128; ++d) {
        qv[d] = qh[d] * qn;
        kv[d] = kh[d] * kn;
        qk += qv[d] * kv[d];
      }
      float decay = std::exp(g[t * 32 + h]), b = beta[t * 32 + h];
      float pred[128] = {0}, qstate[128] = {0};
      for (int kk = 0; kk < 128; ++kk)
        for (int vv = 0; vv < 128; ++vv) {
          float sv = s[kk * 128 + vv] * decay;
          s[kk * 128 + vv] = sv;
          pred[vv] += sv * kv[kk];
          qstate[vv] += sv * qv[kk];
        }
      float delta[128];
      for (int vv = 0; vv < 128; ++vv) {
        delta[vv] = (vh[vv] - pred[vv]) * b;
        out[(t * 32 + h) * 128 + vv] = qstate[vv] + delta[vv] * qk;
      }
      for (int kk = 0; kk < 128; ++kk)
        for (int vv = 0; vv < 128; ++vv)
          s[kk * 128 + vv] += kv[kk] * delta[vv];
    }
    if (snapshots)
      std::memcpy(snapshots + size_t(t) * 32 * 128 * 128, S, size_t(32) * 128 * 128 * 4);
  }
}

// ---- attention -------------------------------------------------------------------------------
// native_ops.metal:115-120 with theta = 1e7 and 32 pairs (forward.cpp:158-162). The reference fills the
// table on the GPU in fp32 and stores fp16; here it is evaluated in double and stored fp32 [maxContext,32,2]
// so host and device use one bit-identical table.
void orc_rope_table(int64_t positions, float* table) {
  for (int64_t p = 0; p < positions; ++p)
    for (int d = 0; d < 32; ++d) {
      double angle = double(p) / std::pow(1.0e7, double(d) / 32.0);
      table[(p * 32 + d) * 2] = float(std::cos(angle));
      table[(p * 32 + d) * 2 + 1] = float(std::sin(angle));
    }
}

// attention.metal:21-49. qg [rows,16,512] (q | gate per head), rawK [rows,4,256]; per-head RMS norm with
// qNorm/kNorm [256], NeoX RoPE on dims 0..63 (pairs i, i+32) at positions[row]. q -> [rows,16,256],
// k -> [rows,4,256].
void orc_attention_prepare(const float* qg, const float* rawK, const float* qNorm, const float* kNorm, const float* rope,
                           const int32_t* positions, int64_t rows, float* q, float* k) {
  for (int64_t row = 0; row < rows; ++row)
    for (int head = 0; head < 20; ++head) {
      bool query = head < 16;
      const float* source = query ? qg + (row * 16 + head) * 512 : rawK + (row * 4 + head - 16) * 256;
      const float* weight = query ? qNorm : kNorm;
      float* output = query ? q + (row * 16 + head) * 256 : k + (row * 4 + head - 16) * 256;
      double ss = 0.0;
      for (int d = 0; d < 256; ++d)
        ss += double(source[d]) * source[d];
      float scale = 1.0f / std::sqrt(float(ss / 256.0) + 1.0e-6f);
      const float* cs = rope + int64_t(positions[row]) * 64;
      for (int d = 0; d < 256; ++d) {
        float normalized = source[d] * scale * weight[d];
        if (d < 64) {
          int other = d < 32 ? d + 32 : d - 32, pair = d & 31;
          float paired = source[other] * scale * weight[other];
          normalized = normalized * cs[pair * 2] + (d < 32 ? -paired : paired) * cs[pair * 2 + 1];
        }
        output[d] = normalized;
      }
    }
}

// attention.metal:103-216 collapsed to one exact softmax per (row, head): causal GQA over a paged fp16
// cache. keys/values: physical pool [block][4 kv heads][blockTokens][256] fp16; table[row*tableStride + i]
// = physical block of the row's i-th logical block; attended[row] = number of cache tokens the row may
// see (its own position + 1). q [rows,16,256]; gate read from qg [rows,16,512] at +256; out [rows,16,256]
// = softmax(q.K/16).V * sigmoid(gate) (:213-214).
void orc_attention(const float* q, const float* qg, const uint16_t* keys, const uint16_t* values, const int32_t* table, int64_t tableStride,
                   const int32_t* attended, int64_t rows, int64_t blockTokens, float* out) {
#pragma omp parallel for collapse(2)
  for (int64_t row = 0; row < rows; ++row)
    for (int head = 0; head < 16; ++head) {
      int kvHead = head / 4;
      int64_t n = attended[row];
      std::vector<float> score(n);
      const float* qv = q + (row * 16 + head) * 256;
      float maximum = -INFINITY;
      for (int64_t t = 0; t < n; ++t) {
        int64_t block = table[row * tableStride + t / blockTokens];
        const half_t* kp = reinterpret_cast<const half_t*>(keys) + ((block * 4 + kvHead) * blockTokens + t % blockTokens) * 256;
        float s = 0.0f;
        for (int d = 0; d < 256; ++d)
          s = std::fma(qv[d], float(kp[d]), s);
        score[t] = s * (1.0f / 16.0f);
        maximum = std::max(maximum, score[t]);
      }
      double norm = 0.0;
      std::vector<double> numerator(256, 0.0);
      for (int64_t t = 0; t < n; ++t) {
        int64_t block = table[row * tableStride + t / blockTokens];
        const half_t* vp = reinterpret_cast<const half_t*>(values) + ((block * 4 + kvHead) * blockTokens + t % blockTokens) * 256;
        double weight = std::exp(double(score[t] - maximum));
        norm += weight;
        for (int d = 0; d < 256; ++d)
          numerator[d] += weight * double(float(vp[d]));
      }
      for (int d = 0; d < 256; ++d) {
        float gate = qg[(row * 16 + head) * 512 + 256 + d];
        out[(row * 16 + head) * 256 + d] = float(numerator[d] / norm) * sigmoid(gate);
      }
    }
}

void orc_f32_to_f16(const float* x, int64_t count, uint16_t* y) {
  for (int64_t i = 0; i < count; ++i) {
    half_t h = half_t(x[i]);
    std::memcpy(y + i, &h, 2);
  }
}

// ---- sampling --------------------------------------------------------------------------------
// Philox4x32-10 (Salmon et al., SC'11). The reference uses xorshift64 seeded from the wall clock
// (native_ops.metal:160-168, engine.cpp:96-99); the build replaces it with a counter-based generator so
// the variate of a slot's i-th emitted token does not depend on batching or speculation.
void orc_philox(uint64_t key, uint64_t counter, uint32_t out[4]) {
  uint32_t c0 = uint32_t(counter), c1 = uint32_t(counter >> 32), c2 = 0, c3 = 0, k0 = uint32_t(key), k1 = uint32_t(key >> 32);
  for (int round = 0; round < 10; ++round) {
    uint64_t p0 = uint64_t(0xD2511F53u) * c0, p1 = uint64_t(0xCD9E8D57u) * c2;
    uint32_t n0 = uint32_t(p1 >> 32) ^ c1 ^ k0, n1 = uint32_t(p1), n2 = uint32_t(p0 >> 32) ^ c3 ^ k1, n3 = uint32_t(p0);
    c0 = n0, c1 = n1, c2 = n2, c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0, out[1] = c1, out[2] = c2, out[3] = c3;
}

float orc_uniform(uint64_t key, uint64_t counter) {
  uint32_t r[4];
  orc_philox(key, counter, r);
  return float(r[0] >> 8) * (1.0f / 16777216.0f);
}

// native_ops.metal:122-224 for one row of logits. temperature <= 0: first-index argmax (:137-158).
// top_k > 0: the min(top_k,64) largest logits/temperature in descending order, ties by ascending index
// (the insertion sort of :194-207 is stable and skips equal values), top-p inside that set (:208-215),
// inverse-CDF pick with `random` (:216-223). top_k == 0: plain temperature sampling over the vocabulary,
// top-p ignored (:172-188). `margin` (nullable) receives best - second best logit for greedy rows.
int32_t orc_sample(const float* logits, int64_t vocab, float temperature, float topP, int32_t topK, float random, float* margin) {
  if (temperature <= 0) {
    int64_t best = 0;
    float second = -INFINITY;
    for (int64_t j = 1; j < vocab; ++j)
      if (logits[j] > logits[best]) {
        second = logits[best];
        best = j;
      } else
        second = std::max(second, logits[j]);
    if (margin)
      *margin = logits[best] - second;
    return int32_t(best);
  }
  if (!topK) {
    float maximum = -INFINITY;
    for (int64_t j = 0; j < vocab; ++j)
      maximum = std::max(maximum, logits[j] / temperature);
    double total = 0.0;
    for (int64_t j = 0; j < vocab; ++j)
      total += double(std::exp(logits[j] / temperature - maximum));
    double target = double(random) * total, cumulative = 0.0;
    for (int64_t j = 0; j < vocab; ++j) {
      cumulative += double(std::exp(logits[j] / temperature - maximum));
      if (cumulative >= target)
        return int32_t(j);
    }
    return int32_t(vocab - 1);
  }
  float values[64];
  int64_t indices[64];
  int count = std::min(topK, 64);
  for (int j = 0; j < count; ++j) {
    values[j] = -INFINITY;
    indices[j] = 0;
  }
  for (int64_t j = 0; j < vocab; ++j) {
    float value = logits[j] / temperature;
    if (value <= values[count - 1])
      continue;
    int p = count - 1;
    while (p && value > values[p - 1]) {
      values[p] = values[p - 1];
      indices[p] = indices[p - 1];
      --p;
    }
    values[p] = value;
    indices[p] = j;
  }
  float total = 0.0f;
  for (int j = 0; j < count; ++j)
    total += std::exp(values[j] - values[0]);
  float limit = topP * total, nucleus = 0.0f;
  int keep = 0;
  do {
    nucleus += std::exp(values[keep] - values[0]);
    ++keep;
  } while (keep < count && nucleus < limit);
  float target = random * nucleus, cumulative = 0.0f;
  for (int j = 0; j < keep; ++j) {
    cumulative += std::exp(values[j] - values[0]);
    if (cumulative >= target)
      return int32_t(indices[j]);
  }
  return int32_t(indices[keep - 1]);
}

// ---- whole model -----------------------------------------------------------------------------
// T tokens of one sequence through the decoder stack, following Ops::decoder (forward.cpp:77-120) and the
// per-row math of the kernels above. All tensor pointers are filled by the test harness from a GGUF file;
// quantised projections carry their ggml type.
struct OrcLayer {
  const float *attnNorm, *postNorm;
  const uint8_t *gate, *up, *down;
  // full attention
  const uint8_t *wq, *wk, *wv, *wo;
  const float *qNorm, *kNorm;
  // gated delta net
  const uint8_t *wqkv, *wz, *wout;
  const float *wBeta, *wAlpha, *ssmA, *ssmDt, *conv, *ssmNorm;
  // ggml types of the quantised matrices above (the real files mix Q4_K, Q5_K, Q6_K, Q8_0 and IQ4_XS)
  int32_t gateType, upType, downType, wqType, wkType, wvType, woType, wqkvType, wzType, woutType;
};

struct OrcModel {
  int32_t layers, vocab, embdType, outType, mtpProjType, maxContext;
  const uint8_t *embd, *output;
  const float* outputNorm;
  const float* rope;  // [maxContext,32,2]
  OrcLayer layer[64];  // layer[layers] is the attention layer of the MTP block when the file carries one
  // MTP block blk.<layers>.nextn.* (forward.cpp:122-130, 210): input norms, 8192 -> 4096 projection, head norm
  const float *mtpEnorm, *mtpHnorm, *mtpHeadNorm;
  const uint8_t* mtpProj;
};

// Per-sequence state: conv [gdn layers][8192][4], S [gdn layers][32][128][128], K/V fp16
// [attention layers][maxContext][4][256] stored as floats already rounded through fp16; the MTP layer has a
// cache of its own [maxContext][4][256] (K/V layer index 8 of the reference, forward.cpp:228).
struct OrcState {
  float *conv, *S, *keys, *values;
  int32_t length;
  float *mtpKeys, *mtpValues;
};

}  // extern "C"

namespace {

// The per-sequence part of gated full attention (forward.cpp:89-95) for T rows at positions pos .. pos + T - 1:
// attention_prepare, cache append (attention.metal:126-133), causal softmax over the cache, sigmoid gate. qg [T,8192],
// k, v [T,1024] are the projections of the rows; o [T,4096]. keys / values: this layer's [maxContext][1024] cache.
void attention_core(const OrcModel* model, const OrcLayer& w, float* keys, float* values, int pos, int64_t T, const float* qg, const float* k,
                    const float* v, float* o) {
  std::vector<float> q(T * 4096), kr(T * 1024);
  std::vector<int32_t> positions(T);
  for (int64_t t = 0; t < T; ++t)
    positions[t] = pos + int32_t(t);
  orc_attention_prepare(qg, k, w.qNorm, w.kNorm, model->rope, positions.data(), T, q.data(), kr.data());
  for (int64_t t = 0; t < T; ++t)
    for (int i = 0; i < 1024; ++i) {
      keys[size_t(pos + t) * 1024 + i] = half_round(kr[t * 1024 + i]);
      values[size_t(pos + t) * 1024 + i] = half_round(v[t * 1024 + i]);
    }
#pragma omp parallel for collapse(2)
  for (int64_t t = 0; t < T; ++t)
    for (int head = 0; head < 16; ++head) {
      const int kvHead = head / 4, last = pos + int(t);
      const float* qv = q.data() + (t * 16 + head) * 256;
      std::vector<float> score(last + 1);
      float maximum = -INFINITY;
      for (int c = 0; c <= last; ++c) {
        float sum = 0.0f;
        for (int d = 0; d < 256; ++d)
          sum = std::fma(qv[d], keys[size_t(c) * 1024 + kvHead * 256 + d], sum);
        score[c] = sum * (1.0f / 16.0f);
        maximum = std::max(maximum, score[c]);
      }
      double norm = 0.0, numerator[256] = {0};
      for (int c = 0; c <= last; ++c) {
        double weight = std::exp(double(score[c] - maximum));
        norm += weight;
        for (int d = 0; d < 256; ++d)
          numerator[d] += weight * values[size_t(c) * 1024 + kvHead * 256 + d];
      }
      for (int d = 0; d < 256; ++d)
        o[(t * 16 + head) * 256 + d] = float(numerator[d] / norm) * sigmoid(qg[(t * 16 + head) * 512 + 256 + d]);
    }
}

// Gated full attention of Ops::decoder (forward.cpp:84-96) for T rows of one sequence: q/k/v projections, the
// per-sequence part above, output projection added to h.
void attention_rows(const OrcModel* model, const OrcLayer& w, float* keys, float* values, int pos, int64_t T, const float* x, float* h) {
  const int64_t H = 4096;
  std::vector<float> qg(T * 8192), k(T * 1024), v(T * 1024), o(T * 4096), y(T * H);
  orc_linear(w.wq, w.wqType, 8192, H, x, T, qg.data(), nullptr);
  orc_linear(w.wk, w.wkType, 1024, H, x, T, k.data(), nullptr);
  orc_linear(w.wv, w.wvType, 1024, H, x, T, v.data(), nullptr);
  attention_core(model, w, keys, values, pos, T, qg.data(), k.data(), v.data(), o.data());
  orc_linear(w.wo, w.woType, H, H, o.data(), T, y.data(), h);
  std::memcpy(h, y.data(), size_t(T) * H * 4);
}

// The per-sequence part of a gated delta network layer (forward.cpp:99-106) for T rows: beta / g, causal conv with the
// carried taps, the sequential delta rule, gated norm. x [T,4096] normalised hidden, mixed [T,8192], z [T,4096]
// projections; gated [T,4096] is what the output projection takes.
void gdn_core(const OrcLayer& w, float* convState, float* S, bool fresh, int64_t T, const float* x, const float* mixed, const float* z,
              float* gated) {
  std::vector<float> beta(T * 32), g(T * 32), q(T * 2048), k(T * 2048), v(T * 4096), o(T * 4096), conv(8192 * 4);
  orc_gdn_ba(x, w.wBeta, w.wAlpha, w.ssmA, w.ssmDt, T, beta.data(), g.data());
  orc_gdn_conv(mixed, w.conv, fresh ? nullptr : convState, T, q.data(), k.data(), v.data(), conv.data(), 0);
  std::memcpy(convState, conv.data(), conv.size() * 4);
  orc_delta_rule(q.data(), k.data(), v.data(), g.data(), beta.data(), T, S, o.data(), nullptr);
  orc_gated_rms_norm(o.data(), z, w.ssmNorm, T * 32, gated);
}

// Gated delta network of Ops::decoder (forward.cpp:97-107) for T rows of one sequence.
void gdn_rows(const OrcModel* model, const OrcLayer& w, float* convState, float* S, bool fresh, int64_t T, const float* x, float* h) {
  const int64_t H = 4096;
  std::vector<float> mixed(T * 8192), z(T * H), gated(T * 4096), y(T * H);
  orc_linear(w.wqkv, w.wqkvType, 8192, H, x, T, mixed.data(), nullptr);
  orc_linear(w.wz, w.wzType, H, H, x, T, z.data(), nullptr);
  gdn_core(w, convState, S, fresh, T, x, mixed.data(), z.data(), gated.data());
  orc_linear(w.wout, w.woutType, H, H, gated.data(), T, y.data(), h);
  std::memcpy(h, y.data(), size_t(T) * H * 4);
}

// SwiGLU block (forward.cpp:109-119): h += down(silu(gate(x)) * up(x)), x = rmsnorm(h; post_attention_norm).
void mlp_rows(const OrcModel* model, const OrcLayer& w, int64_t T, float* h) {
  const int64_t H = 4096, I = 12288;
  std::vector<float> x(T * H), t(T * I), y(T * H);
  orc_rms_norm(h, w.postNorm, T, H, 1.0e-6f, x.data());
  orc_gate_up(w.gate, w.up, w.gateType, w.upType, I, H, x.data(), T, t.data());
  orc_linear(w.down, w.downType, H, I, t.data(), T, y.data(), h);
  std::memcpy(h, y.data(), size_t(T) * H * 4);
}

}  // namespace

extern "C" {

// Appends T tokens to the sequence in one pass. hidden (nullable) receives the final hidden state (before
// output_norm) of every row [T][4096]; the last `logitRows` rows also get rmsnorm(hidden; output_norm) . output^T
// in logits[logitRows][vocab] (forward.cpp:72-75). Row t is computed with exactly the arithmetic of a one-token
// call at its position, so one pass of T tokens and T passes of one token give identical bits.
void orc_model_forward(const OrcModel* model, OrcState* state, const int32_t* tokens, int64_t T, float* hidden, int64_t logitRows,
                       float* logits) {
  const int64_t H = 4096;
  std::vector<float> h(T * H), x(T * H);
  const int pos = state->length;
  orc_embedding(model->embd, model->embdType, H, tokens, T, h.data());
  int gdn = 0, att = 0;
  for (int L = 0; L < model->layers; ++L) {
    const OrcLayer& w = model->layer[L];
    orc_rms_norm(h.data(), w.attnNorm, T, H, 1.0e-6f, x.data());
    if ((L + 1) % 4 == 0) {
      attention_rows(model, w, state->keys + size_t(att) * model->maxContext * 1024, state->values + size_t(att) * model->maxContext * 1024, pos,
                     T, x.data(), h.data());
      ++att;
    } else {
      gdn_rows(model, w, state->conv + size_t(gdn) * 8192 * 4, state->S + size_t(gdn) * 32 * 128 * 128, pos == 0, T, x.data(), h.data());
      ++gdn;
    }
    mlp_rows(model, w, T, h.data());
  }
  state->length = pos + int(T);
  if (hidden)
    std::memcpy(hidden, h.data(), size_t(T) * H * 4);
  if (logits && logitRows > 0) {
    const float* rows = h.data() + (T - logitRows) * H;
    orc_rms_norm(rows, model->outputNorm, logitRows, H, 1.0e-6f, x.data());
    orc_linear(model->output, model->outType, model->vocab, H, x.data(), logitRows, logits, nullptr);
  }
}

// One token (the decode step): orc_model_forward with T = 1.
void orc_model_step(const OrcModel* model, OrcState* state, int32_t token, float* hidden, float* logits) {
  orc_model_forward(model, state, &token, 1, hidden, logits ? 1 : 0, logits);
}

// One decode step of B sequences in one pass, the way the engine batches them: every projection runs once over the
// B stacked rows (so a weight row is dequantised once for all of them, as the GEMV kernels read it once), the
// recurrent and attention parts run per sequence. Row b gets the same bits as orc_model_step on states[b] alone.
// hidden (nullable) [B][4096], logits (nullable) [B][vocab].
void orc_model_decode_batch(const OrcModel* model, OrcState* const* states, const int32_t* tokens, int64_t B, float* hidden, float* logits) {
  const int64_t H = 4096;
  std::vector<float> h(B * H), x(B * H), y(B * H);
  orc_embedding(model->embd, model->embdType, H, tokens, B, h.data());
  int gdn = 0, att = 0;
  for (int L = 0; L < model->layers; ++L) {
    const OrcLayer& w = model->layer[L];
    orc_rms_norm(h.data(), w.attnNorm, B, H, 1.0e-6f, x.data());
    if ((L + 1) % 4 == 0) {
      std::vector<float> qg(B * 8192), k(B * 1024), v(B * 1024), o(B * 4096);
      orc_linear(w.wq, w.wqType, 8192, H, x.data(), B, qg.data(), nullptr);
      orc_linear(w.wk, w.wkType, 1024, H, x.data(), B, k.data(), nullptr);
      orc_linear(w.wv, w.wvType, 1024, H, x.data(), B, v.data(), nullptr);
      for (int64_t b = 0; b < B; ++b)
        attention_core(model, w, states[b]->keys + size_t(att) * model->maxContext * 1024, states[b]->values + size_t(att) * model->maxContext * 1024,
                       states[b]->length, 1, qg.data() + b * 8192, k.data() + b * 1024, v.data() + b * 1024, o.data() + b * 4096);
      orc_linear(w.wo, w.woType, H, H, o.data(), B, y.data(), h.data());
      ++att;
    } else {
      std::vector<float> mixed(B * 8192), z(B * H), gated(B * 4096);
      orc_linear(w.wqkv, w.wqkvType, 8192, H, x.data(), B, mixed.data(), nullptr);
      orc_linear(w.wz, w.wzType, H, H, x.data(), B, z.data(), nullptr);
      for (int64_t b = 0; b < B; ++b)
        gdn_core(w, states[b]->conv + size_t(gdn) * 8192 * 4, states[b]->S + size_t(gdn) * 32 * 128 * 128, states[b]->length == 0, 1, x.data() + b * H,
                 mixed.data() + b * 8192, z.data() + b * H, gated.data() + b * 4096);
      orc_linear(w.wout, w.woutType, H, H, gated.data(), B, y.data(), h.data());
      ++gdn;
    }
    h = y;
    mlp_rows(model, w, B, h.data());
  }
  for (int64_t b = 0; b < B; ++b)
    ++states[b]->length;
  if (hidden)
    std::memcpy(hidden, h.data(), size_t(B) * H * 4);
  if (logits) {
    orc_rms_norm(h.data(), model->outputNorm, B, H, 1.0e-6f, x.data());
    orc_linear(model->output, model->outType, model->vocab, H, x.data(), B, logits, nullptr);
  }
}

// ---- MTP drafter -----------------------------------------------------------------------------
// native_ops.metal:43-87 for one row: y[8192] = [rmsnorm(embedding) * enorm | rmsnorm(h) * hnorm]. h == null stands
// for the first row of a fresh sequence, which has no predecessor (`initial`, :57): that half is zero.
void orc_mtp_fuse(const float* embedding, const float* h, const float* enorm, const float* hnorm, float* y) {
  std::vector<float> zero(4096, 0.0f);
  orc_rms_norm(embedding, enorm, 1, 4096, 1.0e-6f, y);
  orc_rms_norm(h ? h : zero.data(), hnorm, 1, 4096, 1.0e-6f, y + 4096);
}

// One row of the MTP block at `position` of the sequence: Ops::mtpInput (forward.cpp:122-130: embedding of `token`,
// mtp_fuse with `previousHidden`, eh_proj 8192 -> 4096), then
//  * storeOnly != 0: the tail of a target pass (forward.cpp:218-232): attn_norm, K / V projections and mtp_store_kv
//    (attention.metal:53-100: K RMS norm + RoPE, fp16 store) into the MTP cache at `position`;
//  * storeOnly == 0: one drafting step (forward.cpp:197-217): the whole attention layer blk.<layers> over the MTP
//    cache (which it appends to at `position`), its MLP, and when logits is non-null shared_head_norm + lm_head.
// previousHidden is what the step fuses with: the target's hidden state of position - 1 for the tail and for the
// first drafting step (the stored seed), the MTP block's own previous output for later drafting steps (the
// reference passes the embedding a second time there, forward.cpp:125-128, 199; proposals only affect the
// acceptance rate, never the emitted tokens). hidden (nullable) receives the block's output.
void orc_mtp_step(const OrcModel* model, OrcState* state, int32_t token, const float* previousHidden, int32_t position, int32_t storeOnly,
                  float* hidden, float* logits) {
  const int64_t H = 4096;
  const OrcLayer& w = model->layer[model->layers];
  std::vector<float> embedding(H), fused(2 * H), h(H), x(H);
  orc_embedding(model->embd, model->embdType, H, &token, 1, embedding.data());
  orc_mtp_fuse(embedding.data(), previousHidden, model->mtpEnorm, model->mtpHnorm, fused.data());
  orc_linear(model->mtpProj, model->mtpProjType, H, 2 * H, fused.data(), 1, h.data(), nullptr);
  orc_rms_norm(h.data(), w.attnNorm, 1, H, 1.0e-6f, x.data());
  if (storeOnly) {
    std::vector<float> k(1024), v(1024), kr(1024), qg(8192, 0.0f), q(4096);
    orc_linear(w.wk, w.wkType, 1024, H, x.data(), 1, k.data(), nullptr);
    orc_linear(w.wv, w.wvType, 1024, H, x.data(), 1, v.data(), nullptr);
    orc_attention_prepare(qg.data(), k.data(), w.kNorm, w.kNorm, model->rope, &position, 1, q.data(), kr.data());
    for (int i = 0; i < 1024; ++i) {
      state->mtpKeys[size_t(position) * 1024 + i] = half_round(kr[i]);
      state->mtpValues[size_t(position) * 1024 + i] = half_round(v[i]);
    }
    return;
  }
  attention_rows(model, w, state->mtpKeys, state->mtpValues, position, 1, x.data(), h.data());
  mlp_rows(model, w, 1, h.data());
  if (hidden)
    std::memcpy(hidden, h.data(), H * 4);
  if (logits) {
    orc_rms_norm(h.data(), model->mtpHeadNorm, 1, H, 1.0e-6f, x.data());
    orc_linear(model->output, model->outType, model->vocab, H, x.data(), 1, logits, nullptr);
  }
}

// engine.cpp:9-16: chained 64-bit hash over one 512-token checkpoint block.
uint64_t orc_hash_checkpoint(uint64_t hash, const int32_t* tokens) {
  hash ^= 0x9e3779b97f4a7c15ull;
  for (uint32_t i = 0; i < 512; ++i) {
    hash ^= uint32_t(tokens[i]) + 0x9e3779b9u + (hash << 6) + (hash >> 2);
    hash *= 0x100000001b3ull;
  }
  return hash;
}

}  // extern "C"
