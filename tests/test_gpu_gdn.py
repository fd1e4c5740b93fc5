"""GPU: gated delta-rule layer (BASELINE config 2) against the sequential CPU oracle."""
import numpy as np
import pytest

import oracle
from mtlqwen_b200 import device as D
from mtlqwen_b200.testing import images

pytestmark = pytest.mark.gpu
TOL = 1e-3  # BASELINE: GDN outputs within 1e-3 relative error in fp32 accumulation
LAYER = D.GDN_LAYER_STATE_BYTES


def rel_err(got, want):
  want = want.astype(np.float64)
  return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


def layer_weights(rng):
  return dict(w_beta=(rng.standard_normal((32, 4096)) / 64).astype(np.float32), w_alpha=(rng.standard_normal((32, 4096)) / 64).astype(np.float32),
              ssm_a=(-rng.uniform(1, 16, 32)).astype(np.float32), ssm_dt=(0.1 * rng.standard_normal(32)).astype(np.float32),
              conv=(0.5 * rng.standard_normal((8192, 4))).astype(np.float32), norm=(1 + 0.01 * rng.standard_normal(128)).astype(np.float32))


def run_layer(dev, rng, lengths, fresh=(), speculative=(), prefill=False, fused=False, outputs=None):
  """One GDN layer over len(lengths) queries packed back to back. `fresh` queries start from no state,
  `speculative` ones write one candidate state row per token."""
  w = layer_weights(rng)
  rows, nq = int(sum(lengths)), len(lengths)
  x = rng.standard_normal((rows, 4096)).astype(np.float32)
  mixed = rng.standard_normal((rows, 8192)).astype(np.float32)
  z = rng.standard_normal((rows, 4096)).astype(np.float32)
  conv0 = rng.standard_normal((nq, 8192, 4)).astype(np.float32)
  S0 = (0.01 * rng.standard_normal((nq, 32, 128, 128))).astype(np.float32)
  records = np.concatenate([conv0.reshape(nq, -1), S0.reshape(nq, -1)], axis=1)
  previous = dev.array(records)
  next_ = dev.empty((nq, LAYER // 4))
  candidate_rows = int(sum(lengths[i] for i in speculative))
  candidates = dev.empty((max(candidate_rows, 1), LAYER // 4))
  queries, start, cand = [], 0, 0
  for i, count in enumerate(lengths):
    q = D.Query()
    q.previous = 0 if i in fresh else previous.ptr + i * LAYER
    q.next = candidates.ptr + cand * LAYER if i in speculative else next_.ptr + i * LAYER
    q.start, q.count, q.position, q.slot = start, count, 0 if i in fresh else 77, i
    q.state = cand if i in speculative else D.UNBOUND
    if i in speculative:
      cand += count
    queries.append(q)
    start += count
  dq = dev.queries(queries)
  bufs = {name: dev.array(value) for name, value in w.items()}
  q_out, k_out, v_out = dev.empty((rows, 16, 128)), dev.empty((rows, 16, 128)), dev.empty((rows, 32, 128))
  beta, g, out = dev.empty((rows, 32)), dev.empty((rows, 32)), dev.empty((rows, 32, 128))
  if not fused:
    dev.gdn_prepare(dev.array(x), dev.array(mixed), bufs["w_beta"], bufs["w_alpha"], bufs["ssm_a"], bufs["ssm_dt"], bufs["conv"], dq, nq, rows, 0,
                    LAYER, q_out, k_out, v_out, beta, g)
  # The kernel also writes the quantised image of its output when asked; it must equal the quantisation of `out`.
  image, want_image = dev.empty(dev.image_bytes(rows, 4096), np.uint8), dev.empty(dev.image_bytes(rows, 4096), np.uint8)
  capture = rows < 256 and not prefill  # the prefill variant writes no image
  if capture:
    dev.image_capture(image)
  if fused:  # preparation and recurrence in one launch
    dev.gdn_decode(dev.array(x), dev.array(mixed), bufs["w_beta"], bufs["w_alpha"], bufs["ssm_a"], bufs["ssm_dt"], bufs["conv"], dev.array(z),
                   bufs["norm"], dq, nq, 0, D.CONV_STATE_BYTES, LAYER, out)
  else:
    dev.delta_rule(q_out, k_out, v_out, g, beta, dev.array(z), bufs["norm"], dq, nq, D.CONV_STATE_BYTES, LAYER, out, prefill=prefill)
  dev.quantize(out, rows, 4096, want_image)
  dev.commit()
  if capture:
    for a, b in zip(images.decode(image.download(), rows, 4096), images.decode(want_image.download(), rows, 4096)):
      assert a.tobytes() == b.tobytes()
  got_out, got_next, got_cand = out.download(), next_.download(), candidates.download()
  if outputs is not None:
    outputs.extend([got_out, got_next, got_cand])
  worst, start, cand = 0.0, 0, 0
  for i, count in enumerate(lengths):
    rows_i = slice(start, start + count)
    b, gg = oracle.gdn_ba(x[rows_i], w["w_beta"], w["w_alpha"], w["ssm_a"], w["ssm_dt"])
    spec = i in speculative
    qo, ko, vo, states = oracle.gdn_conv(mixed[rows_i], w["conv"], None if i in fresh else conv0[i], every_token=spec)
    S_init = np.zeros((32, 128, 128), np.float32) if i in fresh else S0[i]
    o, S_final, snaps = oracle.delta_rule(qo, ko, vo, gg, b, S_init, snapshots=spec)
    y = oracle.gated_rms_norm(o, z[rows_i], w["norm"])
    worst = max(worst, rel_err(got_out[rows_i], y))
    if spec:
      for t in range(count):
        rec = got_cand[cand + t]
        worst = max(worst, rel_err(rec[:8192 * 4], states[t].reshape(-1)), rel_err(rec[8192 * 4:], snaps[t].reshape(-1)))
      cand += count
    else:
      rec = got_next[i]
      worst = max(worst, rel_err(rec[:8192 * 4], states[0].reshape(-1)), rel_err(rec[8192 * 4:], S_final.reshape(-1)))
    start += count
  return worst


def test_gdn_decode_eight_sequences(dev):
  assert run_layer(dev, np.random.default_rng(1), [1] * 8) < TOL


def test_gdn_ragged_prefill_config2(dev):
  """8 sequences, ragged chunk lengths uniform in [1, 512], state initialised from N(0, 0.01)."""
  rng = np.random.default_rng(2)
  lengths = [int(v) for v in rng.integers(1, 513, 8)]
  assert run_layer(dev, rng, lengths) < TOL


def test_gdn_mixed_pass_fresh_and_speculative(dev):
  rng = np.random.default_rng(3)
  assert run_layer(dev, rng, [1, 37, 5, 1, 128, 5, 2, 1], fresh=(1, 3), speculative=(2, 5)) < TOL


def test_gdn_single_query_edge_lengths(dev):
  rng = np.random.default_rng(4)
  for lengths in ([1], [2], [3], [4], [512]):
    assert run_layer(dev, rng, lengths, fresh=(0, )) < TOL


def test_gdn_chunked_prefill_config2(dev):
  """The same ragged lengths through infdev_delta_rule_prefill: queries of 16 tokens or more take the chunked kernel."""
  rng = np.random.default_rng(2)
  lengths = [int(v) for v in rng.integers(1, 513, 8)]
  assert run_layer(dev, rng, lengths, prefill=True) < TOL


def test_gdn_chunked_mixed_pass(dev):
  """Chunked, sequential (short or speculative) and fresh queries in one pass; lengths around the 16-token chunk."""
  rng = np.random.default_rng(5)
  assert run_layer(dev, rng, [16, 15, 17, 1, 128, 40, 33, 31], fresh=(0, 4), speculative=(5, ), prefill=True) < TOL


def test_gdn_chunked_agrees_with_sequential(dev):
  """Both forms are fp32 on the CUDA cores and must agree far inside the tolerance against the oracle."""
  a = run_layer(dev, np.random.default_rng(6), [100, 64], prefill=False)
  b = run_layer(dev, np.random.default_rng(6), [100, 64], prefill=True)
  assert a < TOL and b < TOL and abs(a - b) < 2e-4


def test_prefill_variant_refuses_an_image(dev):
  dev.image_capture(dev.empty(dev.image_bytes(8, 4096), np.uint8))
  with pytest.raises(RuntimeError, match="no image"):
    dev.delta_rule(dev.empty(1), dev.empty(1), dev.empty(1), dev.empty(1), dev.empty(1), None, None, dev.queries([D.Query()]), 1, 0, LAYER, dev.empty(1),
                   prefill=True)


def test_gdn_fused_decode_is_identical_to_the_two_launches(dev):
  """infdev_gdn_decode = infdev_gdn_prepare + infdev_delta_rule with the same arithmetic: outputs, recurrent states, conv
  taps and speculative candidate records must agree bit for bit, and with the oracle within the tolerance."""
  lengths, fresh, speculative = [1, 1, 5, 1, 3, 1, 1, 2], (1, ), (2, 4)
  a, b = [], []
  assert run_layer(dev, np.random.default_rng(7), lengths, fresh=fresh, speculative=speculative, outputs=a) < TOL
  assert run_layer(dev, np.random.default_rng(7), lengths, fresh=fresh, speculative=speculative, fused=True, outputs=b) < TOL
  for x, y in zip(a, b):
    assert x.tobytes() == y.tobytes()
