"""CPU: the GGUF header reader of the engine (csrc/gguf_reader.hpp, reached through infeng_gguf_describe) against
gguf-py, the reference implementation of the container format: a file written by gguf.GGUFWriter with scalar,
string, array and string-array metadata must index to the same names, types, shapes and data offsets as
gguf.GGUFReader sees, and so must the synthetic model files this repository writes itself."""
import ctypes

import numpy as np
import pytest

gguf = pytest.importorskip("gguf")

from mtlqwen_b200 import build
from mtlqwen_b200.testing import synth


def describe(path):
  lib = ctypes.CDLL(str(build.build()))
  lib.infeng_gguf_describe.restype = ctypes.c_int64
  lib.infeng_gguf_describe.argtypes = (ctypes.c_char_p, ctypes.c_char_p, ctypes.c_uint64, ctypes.c_char_p)
  out, error = ctypes.create_string_buffer(1 << 20), ctypes.create_string_buffer(1024)
  length = lib.infeng_gguf_describe(str(path).encode(), out, len(out), error)
  if length < 0:
    raise RuntimeError(error.value.decode())
  head, *lines = out.value.decode().strip().split("\n")
  _, version, alignment, data_offset, count = head.split("\t")
  tensors = {}
  for line in lines:
    name, kind, offset, size, shape = line.split("\t")
    tensors[name] = (int(kind), int(offset), int(size), tuple(int(d) for d in shape.split(",")))
  assert len(tensors) == int(count)
  return int(version), int(alignment), int(data_offset), tensors


def reference_index(path):
  reader = gguf.GGUFReader(str(path))
  return reader.data_offset, {t.name: (int(t.tensor_type), int(t.data_offset), int(t.n_bytes), tuple(int(d) for d in t.shape)) for t in reader.tensors}


def test_reader_agrees_with_gguf_py_on_a_file_written_by_gguf_py(tmp_path):
  path = tmp_path / "written-by-gguf-py.gguf"
  rng = np.random.default_rng(0)
  writer = gguf.GGUFWriter(str(path), "qwen35")
  writer.add_uint32("qwen35.block_count", 4)
  writer.add_float32("qwen35.rope.freq_base", 1.0e7)
  writer.add_bool("general.is_test", True)
  writer.add_string("general.name", "reader parity")
  writer.add_array("tokenizer.ggml.tokens", ["<pad>", "hello", "wor ld", ""])  # string array: each element is length-prefixed
  writer.add_array("tokenizer.ggml.token_type", [1, 1, 2, 3])  # scalar array
  writer.add_array("tokenizer.ggml.scores", [0.5, -1.25, 3.0])
  writer.add_uint64("general.file_bytes_hint", 1 << 40)
  writer.add_tensor("output_norm.weight", rng.standard_normal(4096).astype(np.float32))
  writer.add_tensor("blk.0.ssm_conv1d.weight", rng.standard_normal((8192, 4)).astype(np.float32))
  writer.add_tensor("blk.0.ssm_beta.weight", rng.standard_normal((32, 4096)).astype(np.float16))
  q4 = synth.q4k_blocks(8 * 4096 // 256, rng).reshape(8, -1)
  writer.add_tensor("blk.0.attn_k.weight", q4, raw_dtype=gguf.GGMLQuantizationType.Q4_K)
  q6 = synth.q6k_blocks(16 * 4096 // 256, rng).reshape(16, -1)
  writer.add_tensor("token_embd.weight", q6, raw_dtype=gguf.GGMLQuantizationType.Q6_K)
  q8 = np.frombuffer(rng.bytes(4 * 8192 // 32 * 34), np.uint8).reshape(4, -1)
  writer.add_tensor("blk.0.nextn.eh_proj.weight", q8, raw_dtype=gguf.GGMLQuantizationType.Q8_0)
  writer.write_header_to_file()
  writer.write_kv_data_to_file()
  writer.write_tensors_to_file()
  writer.close()

  version, alignment, data_offset, ours = describe(path)
  reference_offset, theirs = reference_index(path)
  assert version == 3 and alignment == 32 and data_offset == reference_offset
  assert ours == theirs
  assert ours["blk.0.attn_k.weight"][0] == 12 and ours["blk.0.attn_k.weight"][3] == (4096, 8)  # ne0 = k, ne1 = n
  assert ours["blk.0.nextn.eh_proj.weight"][0] == 8 and ours["blk.0.nextn.eh_proj.weight"][2] == 4 * 8192 // 32 * 34


def test_reader_and_gguf_py_agree_on_the_synthetic_model_files(tmp_path):
  path = tmp_path / "tiny.gguf"
  synth.write_gguf(path, layers=4, vocab=512, mtp=True, seed=3)
  _, _, data_offset, ours = describe(path)
  reference_offset, theirs = reference_index(path)
  assert data_offset == reference_offset and ours == theirs and len(ours) > 50
  # the test-side reader of the same files sees the same bytes
  tensors = synth.read_gguf(path)
  raw = np.memmap(path, dtype=np.uint8, mode="r")
  for name in ("token_embd.weight", "blk.3.attn_q.weight", "blk.4.nextn.eh_proj.weight"):
    kind, offset, size, _ = ours[name]
    assert tensors[name][1] == kind and np.array_equal(tensors[name][0].view(np.uint8).ravel(), raw[offset:offset + size])


def test_malformed_files_are_refused(tmp_path):
  bad = tmp_path / "bad.gguf"
  bad.write_bytes(b"GGUF" + np.uint32(3).tobytes() + np.uint64(1).tobytes() + np.uint64(0).tobytes())  # one tensor promised, none there
  with pytest.raises(RuntimeError, match="truncated"):
    describe(bad)
  bad.write_bytes(b"not a gguf file at all")
  with pytest.raises(RuntimeError, match="GGUF"):
    describe(bad)
  zero_alignment = tmp_path / "zero.gguf"
  header = b"GGUF" + np.uint32(3).tobytes() + np.uint64(0).tobytes() + np.uint64(1).tobytes()
  key = b"general.alignment"
  header += np.uint64(len(key)).tobytes() + key + np.uint32(4).tobytes() + np.uint32(0).tobytes()
  zero_alignment.write_bytes(header)
  with pytest.raises(RuntimeError, match="alignment"):
    describe(zero_alignment)
