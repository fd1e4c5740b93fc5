"""GPU: the latency / throughput report in the reference benchmark's terms (TTFT, TPOT, MBU, MFU) runs on a reduced
model and its figures are consistent with each other."""
import pytest

from mtlqwen_b200 import benchmark
from mtlqwen_b200.inference import InferenceEngine
from mtlqwen_b200.testing import synth

pytestmark = pytest.mark.gpu


def test_report_figures_are_consistent(tmp_path):
  path = tmp_path / "tiny.gguf"
  synth.write_gguf(path, layers=4, vocab=4096, mtp=False, seed=8)
  model = InferenceEngine(path, max_context=512)
  try:
    tokens = [(7 * i + 3) % 4096 for i in range(96)]
    figures = benchmark.report(model, tokens, decode=16, batch=4, speculative=False, warmup=1, iters=2)
  finally:
    model.close()
  assert figures["TTFT_ms"] > 0 and figures["TPOT_ms"] > 0 and figures["mapped_kv_MiB"] > 0
  assert figures["TTL_s"] == pytest.approx(figures["TTFT_ms"] / 1e3 + figures["TPOT_ms"] * 16 / 1e3)
  assert figures["decode_aggregate_tok_s"] == pytest.approx(4 * figures["session_decode_tok_s"])
  assert figures["prefill_aggregate_tok_s"] == pytest.approx(4 * 96 / (figures["TTFT_ms"] / 1e3))
  assert 0 < figures["MBU_pct"] < 100 and 0 < figures["MFU_pct"] < 100 and figures["drafted"] == 0
