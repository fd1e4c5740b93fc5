"""ctypes binding of the infdev_* C ABI (include/infdev.h): buffers, stream and kernel launches.

This is the Python face of the device layer that the C++ engine drives directly; tests and benchmarks
use it to call single kernels with device-resident inputs. It never falls back to a CPU path: loading
fails loudly when the shared library is missing, and creating a Device fails without a B200.
"""
import ctypes

import numpy as np

from . import build as _build

F32, F16, Q8_0, Q4_K, Q5_K, Q6_K, IQ4_XS = 0, 1, 8, 12, 13, 14, 23
BLOCK_BYTES = {Q4_K: 144, Q6_K: 210, Q5_K: 176, IQ4_XS: 136, Q8_0: 34}
CONV_STATE_BYTES, RECURRENT_STATE_BYTES = 8192 * 4 * 4, 32 * 128 * 128 * 4
GDN_LAYER_STATE_BYTES = CONV_STATE_BYTES + RECURRENT_STATE_BYTES
UNBOUND = 0xffffffff


class Query(ctypes.Structure):
  """infdev_query (include/infdev.h), the CUDA form of GpuQuery (backend/metal/kernel/batch.hpp:11-16)."""
  _fields_ = [("previous", ctypes.c_uint64), ("next", ctypes.c_uint64), ("start", ctypes.c_uint32), ("count", ctypes.c_uint32),
              ("position", ctypes.c_uint32), ("slot", ctypes.c_uint32), ("state", ctypes.c_uint32), ("logit", ctypes.c_uint32),
              ("samples", ctypes.c_uint32), ("temperature", ctypes.c_float), ("topP", ctypes.c_float), ("topK", ctypes.c_int32),
              ("seed", ctypes.c_uint64)]


_lib = None


def library():
  """Loads (building first if stale) libinfeng.so and declares the infdev_* prototypes."""
  global _lib
  if _lib is not None:
    return _lib
  lib = ctypes.CDLL(str(_build.build()))
  vp, i64, i32, u32, f32p, u64 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint64
  proto = {
    "infdev_create": (vp, (i32, ctypes.c_char_p)),
    "infdev_destroy": (None, (vp, )),
    "infdev_error": (ctypes.c_char_p, (vp, )),
    "infdev_sm_count": (i32, (vp, )),
    "infdev_launch_count": (u64, (vp, )),
    "infdev_alloc": (vp, (vp, ctypes.c_size_t, i32)),
    "infdev_free": (None, (vp, vp)),
    "infdev_upload": (i32, (vp, vp, vp, ctypes.c_size_t)),
    "infdev_download": (i32, (vp, vp, vp, ctypes.c_size_t)),
    "infdev_peek": (i32, (vp, vp, vp, ctypes.c_size_t)),
    "infdev_copy": (i32, (vp, vp, vp, ctypes.c_size_t)),
    "infdev_fill": (i32, (vp, vp, i32, ctypes.c_size_t)),
    "infdev_commit": (i32, (vp, u32)),
    "infdev_check_abort_path": (i32, (vp, u32)),
    "infdev_event_create": (vp, (vp, )),
    "infdev_event_destroy": (None, (vp, vp)),
    "infdev_event_record": (i32, (vp, vp)),
    "infdev_event_elapsed_ms": (ctypes.c_float, (vp, vp, vp)),
    "infdev_set_xsplit": (i32, (vp, i32)),
    "infdev_set_integer_decode": (i32, (vp, i32)),
    "infdev_image_bytes": (ctypes.c_size_t, (i64, i64)),
    "infdev_quantize": (i32, (vp, vp, i64, i64, vp)),
    "infdev_image_capture": (i32, (vp, vp)),
    "infdev_image_supply": (i32, (vp, vp)),
    "infdev_set_umma": (i32, (vp, i32)),
    "infdev_graph_begin": (i32, (vp, )),
    "infdev_graph_end": (vp, (vp, )),
    "infdev_graph_launch": (i32, (vp, vp)),
    "infdev_graph_destroy": (None, (vp, vp)),
    "infdev_dequant": (i32, (vp, i32, vp, i64, f32p)),
    "infdev_linear": (i32, (vp, i32, vp, i64, i64, f32p, i64, f32p, f32p)),
    "infdev_linear_group": (i32, (vp, i32, i32, vp, vp, i64, f32p, i64, vp)),
    "infdev_gate_up": (i32, (vp, i32, vp, vp, i64, i64, f32p, i64, f32p)),
    "infdev_gather_tokens": (i32, (vp, vp, i32, vp, u32, vp, u32, vp)),
    "infdev_embedding": (i32, (vp, i32, vp, i64, vp, i64, f32p)),
    "infdev_rms_norm": (i32, (vp, f32p, f32p, i64, i64, f32p)),
    "infdev_rms_norm_gather": (i32, (vp, f32p, f32p, vp, i32, i64, f32p)),
    "infdev_gdn_prepare": (i32, (vp, f32p, f32p, f32p, f32p, f32p, f32p, f32p, vp, i32, i64, u64, u64, f32p, f32p, f32p, f32p, f32p)),
    "infdev_delta_rule": (i32, (vp, f32p, f32p, f32p, f32p, f32p, f32p, f32p, vp, i32, u64, u64, f32p)),
    "infdev_gdn_decode": (i32, (vp, f32p, f32p, f32p, f32p, f32p, f32p, f32p, f32p, f32p, vp, i32, u64, u64, u64, f32p)),
    "infdev_delta_rule_prefill": (i32, (vp, f32p, f32p, f32p, f32p, f32p, f32p, f32p, vp, i32, u64, u64, f32p)),
    "infdev_rope_table": (i32, (vp, i64, f32p)),
    "infdev_attention_prepare": (i32, (vp, f32p, f32p, f32p, f32p, f32p, f32p, vp, i32, i64, vp, i32, i32, f32p, vp, vp)),
    "infdev_attention": (i32, (vp, f32p, f32p, vp, vp, vp, i32, i64, vp, i32, i32, u32, f32p, f32p)),
    "infdev_attention_scratch_bytes": (ctypes.c_size_t, (i64, u32)),
    "infdev_attention_static": (i32, (vp, f32p, f32p, vp, vp, vp, i32, i64, vp, i32, i32, f32p)),
    "infdev_mtp_fuse": (i32, (vp, f32p, f32p, vp, i32, f32p, f32p, i64, u32, u64, u64, f32p)),
    "infdev_sample": (i32, (vp, f32p, i64, vp, i32, i64, u32, vp)),
    "infdev_pack_queries": (i32, (vp, vp, i32, i32, u32, vp, vp, u64, u64, vp, vp)),
    "infdev_verify_drafts": (i32, (vp, vp, i32, vp, vp, u32, vp, u32, vp, vp)),
    "infdev_commit_states": (i32, (vp, vp, i32, vp, vp, u64, u64)),
  }
  for name, (restype, argtypes) in proto.items():
    function = getattr(lib, name)
    function.restype, function.argtypes = restype, argtypes
  lib._infdev_symbols = tuple(proto)
  _lib = lib
  return lib


class Buffer:
  """A device (or host-visible) allocation with its element type and shape."""

  def __init__(self, device, shape, dtype, host_visible=False):
    self.device, self.shape, self.dtype = device, tuple(np.atleast_1d(shape).tolist()) if not isinstance(shape, tuple) else shape, np.dtype(dtype)
    self.nbytes = int(np.prod(self.shape)) * self.dtype.itemsize
    self.ptr = library().infdev_alloc(device.ctx, self.nbytes, int(host_visible))
    if not self.ptr:
      raise RuntimeError(device.error())

  def upload(self, array):
    array = np.ascontiguousarray(array, dtype=self.dtype)
    assert array.nbytes == self.nbytes, (array.nbytes, self.nbytes)
    self.device.check(library().infdev_upload(self.device.ctx, self.ptr, array.ctypes.data, self.nbytes))
    self.device.commit()  # the source array may be temporary
    return self

  def download(self):
    out = np.empty(self.shape, self.dtype)
    self.device.check(library().infdev_download(self.device.ctx, out.ctypes.data, self.ptr, self.nbytes))
    return out

  def free(self):
    if self.ptr:
      library().infdev_free(self.device.ctx, self.ptr)
      self.ptr = None


class Device:
  """One infdev context = one GPU, one stream (Device of backend/metal/device.hpp:39-78)."""

  def __init__(self, index=0):
    error = ctypes.create_string_buffer(1024)
    self.ctx = library().infdev_create(index, error)
    if not self.ctx:
      raise RuntimeError("infdev_create failed: " + error.value.decode())
    self.lib = library()

  def error(self):
    return self.lib.infdev_error(self.ctx).decode()

  def check(self, code):
    if code != 0:
      raise RuntimeError(f"infdev error {code}: {self.error()}")

  def close(self):
    if self.ctx:
      self.lib.infdev_destroy(self.ctx)
      self.ctx = None

  @property
  def sm_count(self):
    return self.lib.infdev_sm_count(self.ctx)

  @property
  def launch_count(self):
    return int(self.lib.infdev_launch_count(self.ctx))

  def commit(self, timeout_ms=60000):
    self.check(self.lib.infdev_commit(self.ctx, timeout_ms))

  def empty(self, shape, dtype=np.float32, host_visible=False):
    return Buffer(self, shape if isinstance(shape, tuple) else (int(shape), ), dtype, host_visible)

  def array(self, array, dtype=None):
    array = np.ascontiguousarray(array, dtype=dtype)
    return Buffer(self, array.shape, array.dtype).upload(array)

  def queries(self, records):
    """Uploads a list of Query records; returns the device buffer."""
    packed = (Query * max(len(records), 1))(*records)
    raw = np.frombuffer(bytes(packed), dtype=np.uint8)
    return self.array(raw)

  # ---- timing ----
  def event(self):
    return self.lib.infdev_event_create(self.ctx)

  def record(self, event):
    self.check(self.lib.infdev_event_record(self.ctx, event))

  def elapsed_ms(self, start, stop):
    return float(self.lib.infdev_event_elapsed_ms(self.ctx, start, stop))

  def set_umma(self, enabled):
    self.check(self.lib.infdev_set_umma(self.ctx, int(enabled)))

  def set_xsplit(self, xsplit):
    self.check(self.lib.infdev_set_xsplit(self.ctx, xsplit))

  def set_integer_decode(self, enabled):
    self.check(self.lib.infdev_set_integer_decode(self.ctx, int(enabled)))

  # ---- activation images ----
  def image_bytes(self, rows, k):
    return self.lib.infdev_image_bytes(rows, k)

  def quantize(self, x, rows, k, image):
    self.check(self.lib.infdev_quantize(self.ctx, x.ptr, rows, k, image.ptr))

  def image_capture(self, image):
    """The next producer call also writes the image of its result."""
    self.check(self.lib.infdev_image_capture(self.ctx, image.ptr))

  def image_supply(self, image):
    """The next linear call reads this image instead of quantising its activations."""
    self.check(self.lib.infdev_image_supply(self.ctx, image.ptr))

  # ---- kernels ----
  def dequant(self, qtype, blocks, count, out):
    self.check(self.lib.infdev_dequant(self.ctx, qtype, blocks.ptr, count, out.ptr))

  def linear(self, qtype, w, n, k, x, m, y, residual=None):
    self.check(self.lib.infdev_linear(self.ctx, qtype, w.ptr, n, k, x.ptr, m, y.ptr, residual.ptr if residual is not None else None))

  def linear_group(self, qtype, weights, ns, k, x, m, ys):
    count = len(weights)
    w = (ctypes.c_void_p * count)(*[b.ptr for b in weights])
    n = (ctypes.c_int64 * count)(*ns)
    y = (ctypes.c_void_p * count)(*[b.ptr for b in ys])
    self.check(self.lib.infdev_linear_group(self.ctx, qtype, count, w, n, k, x.ptr, m, y))

  def gate_up(self, qtype, wg, wu, n, k, x, m, y):
    self.check(self.lib.infdev_gate_up(self.ctx, qtype, wg.ptr, wu.ptr, n, k, x.ptr, m, y.ptr))

  def embedding(self, qtype, table, k, tokens, rows, out):
    self.check(self.lib.infdev_embedding(self.ctx, qtype, table.ptr, k, tokens.ptr, rows, out.ptr))

  def rms_norm(self, x, w, rows, dim, y):
    self.check(self.lib.infdev_rms_norm(self.ctx, x.ptr, w.ptr, rows, dim, y.ptr))

  def gdn_prepare(self, x, mixed, w_beta, w_alpha, ssm_a, ssm_dt, conv_w, queries, nq, rows, state_offset, state_bytes, q, k, v, beta, g):
    self.check(self.lib.infdev_gdn_prepare(self.ctx, x.ptr, mixed.ptr, w_beta.ptr, w_alpha.ptr, ssm_a.ptr, ssm_dt.ptr, conv_w.ptr, queries.ptr, nq,
                                           rows, state_offset, state_bytes, q.ptr, k.ptr, v.ptr, beta.ptr, g.ptr))

  def delta_rule(self, q, k, v, g, beta, z, norm_w, queries, nq, state_offset, state_bytes, out, prefill=False):
    """prefill: long non-speculative queries take the chunked kernel (infdev_delta_rule_prefill)."""
    call = self.lib.infdev_delta_rule_prefill if prefill else self.lib.infdev_delta_rule
    self.check(call(self.ctx, q.ptr, k.ptr, v.ptr, g.ptr, beta.ptr, z.ptr if z is not None else None,
                                          norm_w.ptr if norm_w is not None else None, queries.ptr, nq, state_offset, state_bytes, out.ptr))

  def gdn_decode(self, x, mixed, w_beta, w_alpha, ssm_a, ssm_dt, conv_w, z, norm_w, queries, nq, conv_offset, state_offset, state_bytes, out):
    """gdn_prepare + gated delta_rule in one launch (passes without prefill chunks)."""
    self.check(self.lib.infdev_gdn_decode(self.ctx, x.ptr, mixed.ptr, w_beta.ptr, w_alpha.ptr, ssm_a.ptr, ssm_dt.ptr, conv_w.ptr, z.ptr, norm_w.ptr,
                                          queries.ptr, nq, conv_offset, state_offset, state_bytes, out.ptr))

  def rope_table(self, positions):
    table = self.empty((positions, 32, 2))
    self.check(self.lib.infdev_rope_table(self.ctx, positions, table.ptr))
    return table

  def attention_prepare(self, qg, k, v, q_norm, k_norm, rope, queries, nq, rows, table, table_stride, block_tokens, q, cache_k, cache_v):
    self.check(self.lib.infdev_attention_prepare(self.ctx, qg.ptr, k.ptr, v.ptr, q_norm.ptr, k_norm.ptr, rope.ptr, queries.ptr, nq, rows, table.ptr,
                                                 table_stride, block_tokens, q.ptr, cache_k.ptr, cache_v.ptr))

  def attention(self, q, qg, cache_k, cache_v, queries, nq, rows, table, table_stride, block_tokens, max_splits, partials, out):
    self.check(self.lib.infdev_attention(self.ctx, q.ptr, qg.ptr, cache_k.ptr, cache_v.ptr, queries.ptr, nq, rows, table.ptr, table_stride,
                                         block_tokens, max_splits, partials.ptr, out.ptr))

  def attention_scratch_bytes(self, rows, max_splits):
    return int(self.lib.infdev_attention_scratch_bytes(rows, max_splits))

  def sample(self, logits, vocab, queries, nq, count, mode, tokens):
    self.check(self.lib.infdev_sample(self.ctx, logits.ptr, vocab, queries.ptr, nq, count, mode, tokens.ptr))

  def mtp_fuse(self, embedding, hidden, queries, nq, enorm, hnorm, rows, mode, seed_offset, state_bytes, y):
    self.check(self.lib.infdev_mtp_fuse(self.ctx, embedding.ptr, hidden.ptr, queries.ptr, nq, enorm.ptr, hnorm.ptr, rows, mode, seed_offset,
                                        state_bytes, y.ptr))

  def verify_drafts(self, queries, nq, sampled, proposed, draft_width, stops, stop_stride, stop_counts, verdict):
    self.check(self.lib.infdev_verify_drafts(self.ctx, queries.ptr, nq, sampled.ptr, proposed.ptr, draft_width, stops.ptr, stop_stride,
                                             stop_counts.ptr, verdict.ptr))

  def commit_states(self, queries, nq, verdict, state_next, candidate_base, state_bytes):
    self.check(self.lib.infdev_commit_states(self.ctx, queries.ptr, nq, verdict.ptr, state_next.ptr, candidate_base, state_bytes))
