// Minimal GGUF (v2/v3) header reader: tensor names, shapes, ggml types and data offsets.
//
// The reference obtains the same information from ggml's gguf_init_from_buffer (forward.cpp:12-23); ggml
// is not a dependency here, so the published container layout is parsed directly: magic "GGUF", u32
// version, u64 tensor count, u64 key/value count, the key/value section (skipped except
// general.alignment), one info record per tensor, padding to the alignment, then the tensor data.
#pragma once
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace infeng {

struct GgufTensor {
  std::string name;
  std::vector<uint64_t> shape;  // ne[0] is the innermost (contiguous) dimension
  uint32_t type = 0;
  uint64_t offset = 0, bytes = 0, elements = 0;  // offset is relative to dataOffset
};

struct GgufFile {
  uint32_t version = 0;
  uint64_t alignment = 32, dataOffset = 0;
  std::vector<GgufTensor> tensors;
};

class GgufCursor {
  const uint8_t* base;
  uint64_t size, at = 0;

 public:
  GgufCursor(const uint8_t* data, uint64_t bytes) : base(data), size(bytes) {}
  uint64_t position() const { return at; }

  template <class T> T read() {
    if (at + sizeof(T) > size)
      throw std::runtime_error("GGUF header is truncated");
    T value;
    std::memcpy(&value, base + at, sizeof(T));
    at += sizeof(T);
    return value;
  }

  std::string text() {
    const uint64_t length = read<uint64_t>();
    if (at + length > size)
      throw std::runtime_error("GGUF header is truncated");
    std::string value(reinterpret_cast<const char*>(base + at), length);
    at += length;
    return value;
  }

  void skip(uint64_t bytes) {
    if (at + bytes > size)
      throw std::runtime_error("GGUF header is truncated");
    at += bytes;
  }
};

inline uint64_t gguf_scalar_bytes(uint32_t valueType) {
  switch (valueType) {
    case 0: case 1: case 7: return 1;    // u8, i8, bool
    case 2: case 3: return 2;            // u16, i16
    case 4: case 5: case 6: return 4;    // u32, i32, f32
    case 10: case 11: case 12: return 8; // u64, i64, f64
    default: return 0;
  }
}

inline void gguf_skip_value(GgufCursor& cursor, uint32_t valueType) {
  if (valueType == 8) {  // string
    cursor.text();
  } else if (valueType == 9) {  // array: element type, count, elements
    const uint32_t inner = cursor.read<uint32_t>();
    const uint64_t count = cursor.read<uint64_t>();
    if (inner == 8 || inner == 9) {
      for (uint64_t i = 0; i < count; ++i)
        gguf_skip_value(cursor, inner);
    } else {
      const uint64_t width = gguf_scalar_bytes(inner);
      if (!width)
        throw std::runtime_error("GGUF metadata has an unknown array element type");
      cursor.skip(width * count);
    }
  } else {
    const uint64_t width = gguf_scalar_bytes(valueType);
    if (!width)
      throw std::runtime_error("GGUF metadata has an unknown value type");
    cursor.skip(width);
  }
}

// Bytes of a tensor of `elements` values of a ggml type; 0 for types this engine does not load.
inline uint64_t gguf_tensor_bytes(uint32_t type, uint64_t elements) {
  switch (type) {
    case 0: return elements * 4;            // F32
    case 1: return elements * 2;            // F16
    case 8: return elements / 32 * 34;      // Q8_0
    case 12: return elements / 256 * 144;   // Q4_K
    case 13: return elements / 256 * 176;   // Q5_K
    case 14: return elements / 256 * 210;   // Q6_K
    case 23: return elements / 256 * 136;   // IQ4_XS
    default: return 0;
  }
}

inline GgufFile gguf_parse(const uint8_t* data, uint64_t bytes) {
  GgufCursor cursor(data, bytes);
  if (cursor.read<uint32_t>() != 0x46554747u)
    throw std::runtime_error("not a GGUF file (bad magic)");
  GgufFile file;
  file.version = cursor.read<uint32_t>();
  if (file.version < 2 || file.version > 3)
    throw std::runtime_error("unsupported GGUF version " + std::to_string(file.version));
  const uint64_t tensorCount = cursor.read<uint64_t>(), pairCount = cursor.read<uint64_t>();
  for (uint64_t i = 0; i < pairCount; ++i) {
    const std::string key = cursor.text();
    const uint32_t valueType = cursor.read<uint32_t>();
    if (key == "general.alignment" && valueType == 4)
      file.alignment = cursor.read<uint32_t>();
    else
      gguf_skip_value(cursor, valueType);
  }
  file.tensors.resize(tensorCount);
  for (GgufTensor& tensor : file.tensors) {
    tensor.name = cursor.text();
    const uint32_t dims = cursor.read<uint32_t>();
    if (dims == 0 || dims > 4)
      throw std::runtime_error("GGUF tensor " + tensor.name + " has an unsupported rank");
    tensor.elements = 1;
    for (uint32_t d = 0; d < dims; ++d) {
      tensor.shape.push_back(cursor.read<uint64_t>());
      tensor.elements *= tensor.shape.back();
    }
    tensor.type = cursor.read<uint32_t>();
    tensor.offset = cursor.read<uint64_t>();
    tensor.bytes = gguf_tensor_bytes(tensor.type, tensor.elements);
  }
  if (!file.alignment || (file.alignment & (file.alignment - 1)))
    throw std::runtime_error("GGUF general.alignment must be a power of two, got " + std::to_string(file.alignment));
  file.dataOffset = (cursor.position() + file.alignment - 1) / file.alignment * file.alignment;
  if (file.dataOffset > bytes)
    throw std::runtime_error("GGUF header is truncated");
  for (const GgufTensor& tensor : file.tensors)
    if (tensor.bytes && (tensor.offset > bytes - file.dataOffset || tensor.bytes > bytes - file.dataOffset - tensor.offset))
      throw std::runtime_error("GGUF tensor " + tensor.name + " extends past the end of the file");
  return file;
}

}  // namespace infeng
