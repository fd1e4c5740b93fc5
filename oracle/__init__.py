"""ctypes front end of the CPU oracle (oracle/oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by `__graft_entry__.smoke()` and by the CPU-baseline legs
of `bench.py`. The product package never imports it.
"""
import ctypes
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
LIB = ROOT / "_build" / "liboracle.so"
F32, F16, Q8_0, Q4_K, Q5_K, Q6_K, IQ4_XS = 0, 1, 8, 12, 13, 14, 23
BLOCK_BYTES = {Q4_K: 144, Q6_K: 210, Q5_K: 176, IQ4_XS: 136, Q8_0: 34}
BLOCK_VALUES = {Q4_K: 256, Q6_K: 256, Q5_K: 256, IQ4_XS: 256, Q8_0: 32}


def build(force=False):
  source = ROOT / "oracle.cpp"
  if force or not LIB.exists() or (source.exists() and source.stat().st_mtime > LIB.stat().st_mtime):
    subprocess.run(["make", "-C", str(ROOT)], check=True, capture_output=True)
  return LIB


_lib = None


def lib():
  global _lib
  if _lib is None:
    _lib = ctypes.CDLL(str(build()))
    _lib.orc_uniform.restype = ctypes.c_float
    _lib.orc_uniform.argtypes = (ctypes.c_uint64, ctypes.c_uint64)
    _lib.orc_sample.restype = ctypes.c_int32
    _lib.orc_hash_checkpoint.restype = ctypes.c_uint64
    _lib.orc_hash_checkpoint.argtypes = (ctypes.c_uint64, ctypes.c_void_p)
  return _lib


def _p(array):
  return ctypes.c_void_p(array.ctypes.data) if array is not None else None


def _f32(array):
  return np.ascontiguousarray(array, dtype=np.float32)


def _i64(value):
  return ctypes.c_int64(int(value))


def set_threads(threads):
  """OpenMP threads of the oracle's parallel loops from now on."""
  lib().orc_set_threads(ctypes.c_int(int(threads)))


def dequant(blocks, qtype):
  blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, BLOCK_BYTES[qtype])
  out = np.empty((blocks.shape[0], BLOCK_VALUES[qtype]), dtype=np.float32)
  lib().orc_dequant(ctypes.c_int(qtype), _p(blocks), _i64(blocks.shape[0]), _p(out))
  return out


def linear(w, qtype, n, k, x, residual=None):
  x = _f32(x).reshape(-1, k)
  y = np.empty((x.shape[0], n), dtype=np.float32)
  res = _f32(residual) if residual is not None else None
  lib().orc_linear(_p(w), ctypes.c_int(qtype), _i64(n), _i64(k), _p(x), _i64(x.shape[0]), _p(y), _p(res))
  return y


def gate_up(wg, wu, qtype, n, k, x):
  x = _f32(x).reshape(-1, k)
  y = np.empty((x.shape[0], n), dtype=np.float32)
  lib().orc_gate_up(_p(wg), _p(wu), ctypes.c_int(qtype), ctypes.c_int(qtype), _i64(n), _i64(k), _p(x), _i64(x.shape[0]), _p(y))
  return y


def embedding(w, qtype, k, ids):
  ids = np.ascontiguousarray(ids, dtype=np.int32)
  y = np.empty((ids.size, k), dtype=np.float32)
  lib().orc_embedding(_p(w), ctypes.c_int(qtype), _i64(k), _p(ids), _i64(ids.size), _p(y))
  return y


def rms_norm(x, w, eps=1.0e-6):
  x, w = _f32(x), _f32(w)
  y = np.empty_like(x)
  lib().orc_rms_norm(_p(x), _p(w), _i64(x.size // w.size), _i64(w.size), ctypes.c_float(eps), _p(y))
  return y


def gated_rms_norm(o, z, w):
  o, z, w = _f32(o), _f32(z), _f32(w)
  y = np.empty_like(o)
  lib().orc_gated_rms_norm(_p(o), _p(z), _p(w), _i64(o.size // 128), _p(y))
  return y


def gdn_ba(x, wb, wa, A, dt):
  x = _f32(x).reshape(-1, 4096)
  wb, wa, A, dt = _f32(wb), _f32(wa), _f32(A), _f32(dt)
  beta, g = np.empty((x.shape[0], 32), np.float32), np.empty((x.shape[0], 32), np.float32)
  lib().orc_gdn_ba(_p(x), _p(wb), _p(wa), _p(A), _p(dt), _i64(x.shape[0]), _p(beta), _p(g))
  return beta, g


def gdn_conv(mixed, w, state_in=None, every_token=False):
  mixed, w = _f32(mixed).reshape(-1, 8192), _f32(w)
  rows = mixed.shape[0]
  state = _f32(state_in) if state_in is not None else None
  q, k, v = (np.empty((rows, 16, 128), np.float32), np.empty((rows, 16, 128), np.float32), np.empty((rows, 32, 128), np.float32))
  states = np.empty((rows if every_token else 1, 8192, 4), np.float32)
  lib().orc_gdn_conv(_p(mixed), _p(w), _p(state), _i64(rows), _p(q), _p(k), _p(v), _p(states), ctypes.c_int(every_token))
  return q, k, v, states


def delta_rule(q, k, v, g, beta, S, snapshots=False):
  q, k, v, g, beta = _f32(q), _f32(k), _f32(v), _f32(g), _f32(beta)
  T = v.size // 4096
  S = np.array(S, dtype=np.float32, copy=True).reshape(32, 128, 128)
  out = np.empty((T, 32, 128), np.float32)
  snaps = np.empty((T, 32, 128, 128), np.float32) if snapshots else None
  lib().orc_delta_rule(_p(q), _p(k), _p(v), _p(g), _p(beta), _i64(T), _p(S), _p(out), _p(snaps))
  return out, S, snaps


def rope_table(positions):
  table = np.empty((positions, 32, 2), np.float32)
  lib().orc_rope_table(_i64(positions), _p(table))
  return table


def attention_prepare(qg, raw_k, q_norm, k_norm, rope, positions):
  qg, raw_k = _f32(qg).reshape(-1, 16, 512), _f32(raw_k).reshape(-1, 4, 256)
  positions = np.ascontiguousarray(positions, dtype=np.int32)
  rows = qg.shape[0]
  q, k = np.empty((rows, 16, 256), np.float32), np.empty((rows, 4, 256), np.float32)
  lib().orc_attention_prepare(_p(qg), _p(raw_k), _p(_f32(q_norm)), _p(_f32(k_norm)), _p(_f32(rope)), _p(positions), _i64(rows), _p(q), _p(k))
  return q, k


def attention(q, qg, keys, values, table, attended, block_tokens):
  q, qg = _f32(q).reshape(-1, 16, 256), _f32(qg).reshape(-1, 16, 512)
  table = np.ascontiguousarray(table, dtype=np.int32)
  attended = np.ascontiguousarray(attended, dtype=np.int32)
  rows = q.shape[0]
  out = np.empty((rows, 16, 256), np.float32)
  lib().orc_attention(_p(q), _p(qg), _p(keys), _p(values), _p(table), _i64(table.shape[1]), _p(attended), _i64(rows), _i64(block_tokens),
                      _p(out))
  return out


def f32_to_f16_bits(x):
  x = _f32(x)
  y = np.empty(x.shape, np.uint16)
  lib().orc_f32_to_f16(_p(x), _i64(x.size), _p(y))
  return y


def uniform(key, counter):
  return float(lib().orc_uniform(ctypes.c_uint64(key), ctypes.c_uint64(counter)))


def philox(key, counter):
  out = (ctypes.c_uint32 * 4)()
  lib().orc_philox(ctypes.c_uint64(key), ctypes.c_uint64(counter), out)
  return list(out)


def sample(logits, temperature=0.0, top_p=1.0, top_k=0, random=0.0):
  logits = _f32(logits)
  margin = ctypes.c_float(0)
  token = lib().orc_sample(_p(logits), _i64(logits.size), ctypes.c_float(temperature), ctypes.c_float(top_p), ctypes.c_int32(top_k),
                           ctypes.c_float(random), ctypes.byref(margin))
  return int(token), float(margin.value)


def hash_checkpoint(previous, tokens):
  tokens = np.ascontiguousarray(tokens, dtype=np.int32)
  assert tokens.size == 512
  return int(lib().orc_hash_checkpoint(ctypes.c_uint64(previous), _p(tokens)))


_QUANTISED = ("gate", "up", "down", "wq", "wk", "wv", "wo", "wqkv", "wz", "wout")


class _Layer(ctypes.Structure):
  _fields_ = [(name, ctypes.c_void_p) for name in ("attnNorm", "postNorm", "gate", "up", "down", "wq", "wk", "wv", "wo", "qNorm", "kNorm", "wqkv",
                                                   "wz", "wout", "wBeta", "wAlpha", "ssmA", "ssmDt", "conv", "ssmNorm")]
  _fields_ += [(name + "Type", ctypes.c_int32) for name in _QUANTISED]


class _Model(ctypes.Structure):
  _fields_ = [("layers", ctypes.c_int32), ("vocab", ctypes.c_int32), ("embdType", ctypes.c_int32), ("outType", ctypes.c_int32),
              ("mtpProjType", ctypes.c_int32), ("maxContext", ctypes.c_int32), ("embd", ctypes.c_void_p), ("output", ctypes.c_void_p),
              ("outputNorm", ctypes.c_void_p), ("rope", ctypes.c_void_p), ("layer", _Layer * 64), ("mtpEnorm", ctypes.c_void_p),
              ("mtpHnorm", ctypes.c_void_p), ("mtpHeadNorm", ctypes.c_void_p), ("mtpProj", ctypes.c_void_p)]


class _State(ctypes.Structure):
  _fields_ = [("conv", ctypes.c_void_p), ("S", ctypes.c_void_p), ("keys", ctypes.c_void_p), ("values", ctypes.c_void_p),
              ("length", ctypes.c_int32), ("mtpKeys", ctypes.c_void_p), ("mtpValues", ctypes.c_void_p)]


def mtp_fuse(embedding, hidden, enorm, hnorm):
  """One row of mtp_fuse; hidden None = the first row of a fresh sequence."""
  y = np.empty(8192, np.float32)
  lib().orc_mtp_fuse(_p(_f32(embedding)), _p(_f32(hidden)) if hidden is not None else None, _p(_f32(enorm)), _p(_f32(hnorm)), _p(y))
  return y


class Model:
  """Whole-decoder oracle over tensors read from a GGUF file: `tensors` maps reference tensor names to
  (numpy array, ggml type). One instance = one sequence's state; `step(token)` appends a token, `forward(tokens)`
  several in one pass. When the file carries an MTP block (blk.<layers>.nextn.*) the drafter is available too."""

  def __init__(self, tensors, layers, vocab, max_context):
    self._keep = tensors
    self.vocab, self.layers = vocab, layers
    m = _Model()
    m.layers, m.vocab, m.maxContext = layers, vocab, max_context
    m.embdType, m.outType = tensors["token_embd.weight"][1], tensors["output.weight"][1]
    # F16 tensors (ssm_beta / ssm_alpha of the real files) are handed to the C side as float32 copies
    self._converted = {name: np.ascontiguousarray(array.view(np.float16).astype(np.float32)) for name, (array, kind) in tensors.items() if kind == F16}
    ptr = lambda name: (self._converted[name] if name in self._converted else tensors[name][0]).ctypes.data
    m.embd, m.output, m.outputNorm = ptr("token_embd.weight"), ptr("output.weight"), ptr("output_norm.weight")
    self._rope = rope_table(max_context)
    m.rope = self._rope.ctypes.data
    names = {
      "attnNorm": "attn_norm.weight", "postNorm": "post_attention_norm.weight", "gate": "ffn_gate.weight", "up": "ffn_up.weight",
      "down": "ffn_down.weight", "wq": "attn_q.weight", "wk": "attn_k.weight", "wv": "attn_v.weight", "wo": "attn_output.weight",
      "qNorm": "attn_q_norm.weight", "kNorm": "attn_k_norm.weight", "wqkv": "attn_qkv.weight", "wz": "attn_gate.weight",
      "wout": "ssm_out.weight", "wBeta": "ssm_beta.weight", "wAlpha": "ssm_alpha.weight", "ssmA": "ssm_a", "ssmDt": "ssm_dt.bias",
      "conv": "ssm_conv1d.weight", "ssmNorm": "ssm_norm.weight"
    }
    self.has_mtp = f"blk.{layers}.nextn.eh_proj.weight" in tensors
    for L in range(layers + (1 if self.has_mtp else 0)):
      for field, name in names.items():
        key = f"blk.{L}.{name}"
        if key in tensors:
          setattr(m.layer[L], field, ptr(key))
          if field in _QUANTISED:
            setattr(m.layer[L], field + "Type", tensors[key][1])
    if self.has_mtp:
      nextn = f"blk.{layers}.nextn."
      m.mtpEnorm, m.mtpHnorm = ptr(nextn + "enorm.weight"), ptr(nextn + "hnorm.weight")
      m.mtpHeadNorm, m.mtpProj = ptr(nextn + "shared_head_norm.weight"), ptr(nextn + "eh_proj.weight")
      m.mtpProjType = tensors[nextn + "eh_proj.weight"][1]
    self._model = m
    gdn, att = layers - layers // 4, layers // 4
    self._conv = np.zeros((max(gdn, 1), 8192, 4), np.float32)
    self._S = np.zeros((max(gdn, 1), 32, 128, 128), np.float32)
    self._keys = np.zeros((max(att, 1), max_context, 1024), np.float32)
    self._values = np.zeros((max(att, 1), max_context, 1024), np.float32)
    self._mtp_keys = np.zeros((max_context if self.has_mtp else 1, 1024), np.float32)
    self._mtp_values = np.zeros_like(self._mtp_keys)
    s = _State()
    s.conv, s.S, s.keys, s.values, s.length = (self._conv.ctypes.data, self._S.ctypes.data, self._keys.ctypes.data, self._values.ctypes.data, 0)
    s.mtpKeys, s.mtpValues = self._mtp_keys.ctypes.data, self._mtp_values.ctypes.data
    self._state = s

  @property
  def length(self):
    return self._state.length

  def step(self, token, want_logits=True):
    hidden = np.empty(4096, np.float32)
    logits = np.empty(self.vocab, np.float32) if want_logits else None
    lib().orc_model_step(ctypes.byref(self._model), ctypes.byref(self._state), ctypes.c_int32(int(token)), _p(hidden), _p(logits))
    return hidden, logits

  def forward(self, tokens, logit_rows=1):
    """Appends `tokens` in one pass; returns (hidden [T,4096], logits of the last `logit_rows` rows)."""
    tokens = np.ascontiguousarray(tokens, dtype=np.int32)
    hidden = np.empty((tokens.size, 4096), np.float32)
    logits = np.empty((logit_rows, self.vocab), np.float32) if logit_rows else None
    lib().orc_model_forward(ctypes.byref(self._model), ctypes.byref(self._state), _p(tokens), _i64(tokens.size), _p(hidden), _i64(logit_rows),
                            _p(logits))
    return hidden, logits

  def mtp_step(self, token, previous_hidden, position, store_only=False, want_logits=True):
    """One row of the MTP block at `position` (orc_mtp_step): the K/V store of a target pass's tail, or a drafting
    step returning (block output, logits)."""
    assert self.has_mtp
    hidden = None if store_only else np.empty(4096, np.float32)
    logits = np.empty(self.vocab, np.float32) if want_logits and not store_only else None
    previous = _f32(previous_hidden) if previous_hidden is not None else None
    lib().orc_mtp_step(ctypes.byref(self._model), ctypes.byref(self._state), ctypes.c_int32(int(token)), _p(previous), ctypes.c_int32(int(position)),
                       ctypes.c_int32(int(store_only)), _p(hidden), _p(logits))
    return hidden, logits


def decode_batch(models, tokens, want_logits=True):
  """One decode step of several sequences of the same weights in one pass (orc_model_decode_batch): `models` are
  Model instances built from the same tensors; returns (hidden [B,4096], logits [B,vocab] or None)."""
  count = len(models)
  states = (ctypes.POINTER(_State) * count)(*[ctypes.pointer(m._state) for m in models])
  ids = np.ascontiguousarray(tokens, dtype=np.int32)
  hidden = np.empty((count, 4096), np.float32)
  logits = np.empty((count, models[0].vocab), np.float32) if want_logits else None
  lib().orc_model_decode_batch(ctypes.byref(models[0]._model), states, _p(ids), _i64(count), _p(hidden), _p(logits))
  return hidden, logits
