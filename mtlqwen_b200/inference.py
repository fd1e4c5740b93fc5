"""Python boundary of the engine: `InferenceEngine` and `Sequence` with the interface of the reference's
runtime/inference.py (engine.sequence(stop_token_ids, temperature, top_p, top_k, speculative),
Sequence.append/read/cancel/length/speculative_counters/close), bound with ctypes to the infeng_* C ABI of
libinfeng.so (include/infeng.h). Python only moves token ids; the scheduler thread, the K/V pool, the prefix
cache and every kernel live in the shared library.
"""
import ctypes
from pathlib import Path

from . import build as _build

MAX_BATCH = 8


def bind(path):
  """Opens a library that exports the infeng_* C ABI and declares its prototypes."""
  lib = ctypes.CDLL(str(path))
  void = ctypes.c_void_p
  lib.infeng_engine_create.argtypes = (ctypes.c_char_p, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_uint32, ctypes.c_char_p)
  lib.infeng_engine_create.restype = void
  lib.infeng_engine_release.argtypes, lib.infeng_engine_release.restype = (void, ), None
  lib.infeng_sequence_create.argtypes = (void, ctypes.POINTER(ctypes.c_int32), ctypes.c_uint32, ctypes.c_float, ctypes.c_float, ctypes.c_int32,
                                         ctypes.c_uint32, ctypes.c_char_p)
  lib.infeng_sequence_create.restype = void
  lib.infeng_sequence_release.argtypes, lib.infeng_sequence_release.restype = (void, ), None
  lib.infeng_sequence_append.argtypes, lib.infeng_sequence_append.restype = (void, ctypes.POINTER(ctypes.c_int32), ctypes.c_uint32), ctypes.c_int32
  lib.infeng_sequence_read.argtypes, lib.infeng_sequence_read.restype = (void, ctypes.c_uint32), ctypes.c_int32
  lib.infeng_engine_info.argtypes, lib.infeng_engine_info.restype = (void, ctypes.c_uint32), ctypes.c_uint64
  lib.infeng_sequence_info.argtypes, lib.infeng_sequence_info.restype = (void, ctypes.c_uint32), ctypes.c_uint64
  lib.infeng_sequence_seed.argtypes, lib.infeng_sequence_seed.restype = (void, ctypes.c_uint64), ctypes.c_int32
  lib.infeng_sequence_state.argtypes, lib.infeng_sequence_state.restype = (void, ctypes.c_uint64, void, ctypes.c_uint64), ctypes.c_int64
  return lib


_LIB = None


def _lib():
  """The CUDA library of this package, built on first use."""
  global _LIB
  if _LIB is None:
    _LIB = bind(_build.build())
  return _LIB


# Error codes of the C ABI (runtime/inference.py:46-50).
def _check(value, error=None):
  errors = {-3: "sequence is still generating", -4: "completion has no available model context", -5: "KV block pool has no evictable capacity"}
  if value is None: raise RuntimeError((error.value or b"native CUDA operation failed").decode())
  if value in errors: raise RuntimeError(errors[value])
  return value


class Sequence:

  def __init__(self, engine, stop_token_ids, temperature, top_p, top_k, speculative, seed=None):
    self.engine, self.handle = engine, 0
    self.stop_token_ids, self.speculative = frozenset(stop_token_ids), bool(speculative and engine.draft_width)
    stops = (ctypes.c_int32 * len(stop_token_ids))(*stop_token_ids)
    error = ctypes.create_string_buffer(1024)
    self.handle = _check(self.engine.lib.infeng_sequence_create(engine.handle, stops, len(stops), temperature, top_p, top_k or 0, self.speculative, error),
                         error)
    if seed is not None:
      _check(self.engine.lib.infeng_sequence_seed(self.handle, seed))

  def append(self, tokens=()):
    ids = (ctypes.c_int32 * len(tokens))(*tokens)
    return _check(self.engine.lib.infeng_sequence_append(self.handle, ids, len(tokens)))

  def read(self, cursor):
    value = _check(self.engine.lib.infeng_sequence_read(self.handle, cursor))
    return None if value == -1 else value

  def cancel(self):
    if self.handle: self.engine.lib.infeng_sequence_append(self.handle, None, 0xffffffff)

  @property
  def length(self):
    return self.engine.lib.infeng_sequence_info(self.handle, 2)

  def speculative_counters(self):
    drafted = self.engine.lib.infeng_sequence_info(self.handle, 0)
    accepted = self.engine.lib.infeng_sequence_info(self.handle, 1)
    return {"drafted_tokens": drafted, "accepted_tokens": accepted, "acceptance_rate": accepted / drafted if drafted else None}

  def draft_step(self):
    """(position of the anchor token, proposals) of the latest speculative step of this sequence."""
    width = self.engine.draft_width
    return self.engine.lib.infeng_sequence_info(self.handle, 3), [int(self.engine.lib.infeng_sequence_info(self.handle, 4 + i)) for i in range(width)]

  def state(self, offset=0, count=None):
    """fp32 values of the sequence's state record from byte `offset` (all of it by default); the sequence must be idle."""
    import numpy as np
    total = self.engine.lib.infeng_sequence_state(self.handle, 0, None, 0)
    out = np.empty((total - offset) // 4 if count is None else count, np.float32)
    _check(self.engine.lib.infeng_sequence_state(self.handle, offset, out.ctypes.data, out.nbytes))
    return out

  def close(self):
    if self.handle: self.engine.lib.infeng_sequence_release(self.handle)
    self.handle = 0

  def __del__(self):
    self.close()


class InferenceEngine:

  def __init__(self, weights: str | Path, *, draft_weights: str | Path | None = None, max_context=65536, library=None):
    """library: an object returned by bind() for another build of the same C ABI; by default the package's own."""
    if not 0 < max_context <= 65536: raise ValueError(f"max_context must be between 1 and 65536, got {max_context}")
    self.lib = library or _lib()
    draft_path = str(draft_weights).encode() if draft_weights is not None else None
    error = ctypes.create_string_buffer(1024)
    self.handle = _check(self.lib.infeng_engine_create(str(weights).encode(), draft_path, b"", max_context, error), error)
    self.drafter = ("none", "mtp", "dflash")[self.lib.infeng_engine_info(self.handle, 3)]
    self.draft_width = self.lib.infeng_engine_info(self.handle, 4)
    self.max_context, self.max_batch_sequences = max_context, MAX_BATCH
    self.vocab_size = self.lib.infeng_engine_info(self.handle, 9)
    self.parameter_count = self.lib.infeng_engine_info(self.handle, 0)
    self.weight_bytes = self.lib.infeng_engine_info(self.handle, 1)

  def sequence(self, *, stop_token_ids=None, temperature=0.0, top_p=1.0, top_k=None, speculative=False, seed=None):
    """seed (an addition to the reference's signature): a sampling key of the caller's choice, for reproducible requests."""
    return Sequence(self, list(stop_token_ids or ()), temperature, top_p, top_k, speculative, seed)

  @property
  def mapped_bytes(self):
    return self.lib.infeng_engine_info(self.handle, 2)

  def step_counters(self):
    """Passes run, packed rows processed, host microseconds and device nanoseconds spent in passes, kernels launched,
    and the scheduler's host microseconds outside the passes (batch building, waiting for the engine lock, handing
    tokens over) since the engine started."""
    return {"passes": self.lib.infeng_engine_info(self.handle, 5), "rows": self.lib.infeng_engine_info(self.handle, 6),
            "micros": self.lib.infeng_engine_info(self.handle, 7), "device_ns": self.lib.infeng_engine_info(self.handle, 10),
            "launches": self.lib.infeng_engine_info(self.handle, 11), "build_micros": self.lib.infeng_engine_info(self.handle, 12),
            "lock_micros": self.lib.infeng_engine_info(self.handle, 13), "publish_micros": self.lib.infeng_engine_info(self.handle, 14),
            "prefill_rows": self.lib.infeng_engine_info(self.handle, 15)}

  def close(self):
    if getattr(self, "handle", 0): self.lib.infeng_engine_release(self.handle)
    self.handle = 0

  def __del__(self):
    self.close()
