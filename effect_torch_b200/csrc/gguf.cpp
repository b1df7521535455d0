// GGUF v3 catalog parser and tensor loader of the C ABI.
//
// Follows crates/runtime/src/gguf.rs: strict, resource-limited, cancellable. The header (magic, version, metadata table,
// tensor catalog) is parsed without reading any payload (parse_gguf, :682-946); a tensor's payload is then read into a
// caller buffer with positioned reads (read_gguf_tensor_into, :948-990) or streamed into device memory through pinned
// staging. Limits, checks and message texts are the reference's; the only widening is that GGML type codes 2 (Q4_0) and
// 8 (Q8_0) are accepted next to 0 (F32) and 10..14 (K-quants), with 32-value blocks instead of 256.
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstring>
#include <string>
#include <unordered_set>
#include <vector>

#include "common.h"

namespace {

using namespace etc;

constexpr uint32_t kGgufMagicValue = 0x46554747;  // "GGUF"
constexpr uint32_t kVersion = 3;
constexpr uint32_t kQuantizationVersion = 2;
constexpr uint64_t kDefaultAlignment = 32;
constexpr uint64_t kJsSafeInteger = 9007199254740991ull;
constexpr size_t kReadChunkBytes = 8u << 20;
constexpr size_t kHeaderReadChunkBytes = 64u << 10;
constexpr uint64_t kMaxHeaderBytes = 64ull << 20;
constexpr uint64_t kMaxMetadataCount = 4096;
constexpr uint64_t kMaxTensorCount = 65536;
constexpr uint64_t kMaxMetadataKeyBytes = 65535;
constexpr uint64_t kMaxTensorNameBytes = 64;
constexpr uint64_t kMaxMetadataStringBytes = 16ull << 20;
constexpr uint64_t kMaxMetadataArrayElements = 1048576;
constexpr uint32_t kFileMagic = 0x45544346;

struct ParseError {
  etc_status status;
  std::string message;
};
ParseError invalid(const std::string& m) { return {ETC_INVALID_ARGUMENT, "gguf: " + m}; }
ParseError io_failed(const std::string& m) { return {ETC_TRANSFER, "gguf: I/O failed: " + m}; }
ParseError cancelled() { return {ETC_CANCELLED, "gguf: operation aborted"}; }

struct MetadataEntry {
  std::string key;
  uint32_t type = 0;          // GGUF value type code; 9 = array
  uint32_t element_type = 0;  // arrays: element type code
  uint64_t count = 0;         // arrays: number of elements
  uint64_t u = 0;             // integers and bool, two's complement for signed types
  double f = 0.0;             // f32 / f64
  std::string s;              // string
};

struct TensorEntry {
  std::string name;
  int codec = 0;
  std::vector<uint64_t> logical;  // row-major (GGUF dimensions reversed)
  uint64_t physical_rows = 0, physical_row_units = 0;  // F32: logical shape; quantized: [rows, encoded_row_bytes]
  uint64_t data_offset = 0, byte_len = 0;
};

const char* format_name(int code) {
  switch (code) {
    case 0: return "F32";
    case 2: return "Q4_0";
    case 8: return "Q8_0";
    case 10: return "Q2_K";
    case 11: return "Q3_K";
    case 12: return "Q4_K";
    case 13: return "Q5_K";
    case 14: return "Q6_K";
    default: return "?";
  }
}

struct Reader {
  int fd;
  uint64_t file_len;
  uint64_t position = 0;
  const volatile int* cancel;

  void check_cancelled() const {
    if (cancel && *cancel) throw cancelled();
  }
  void read_exact(void* out, size_t length) {
    check_cancelled();
    if (position + length < position) throw invalid("header position overflows");
    const uint64_t end = position + length;
    if (end > file_len) throw invalid("unexpected end of file in header");
    if (end > kMaxHeaderBytes) throw invalid("header exceeds the " + std::to_string(kMaxHeaderBytes) + "-byte resource limit");
    unsigned char* dst = static_cast<unsigned char*>(out);
    size_t done = 0;
    while (done < length) {
      check_cancelled();
      const size_t chunk = std::min(kHeaderReadChunkBytes, length - done);
      size_t got = 0;
      while (got < chunk) {
        const ssize_t n = pread(fd, dst + done + got, chunk - got, (off_t)(position + got));
        if (n < 0) {
          if (errno == EINTR) continue;
          throw io_failed(std::strerror(errno));
        }
        if (n == 0) throw io_failed("failed to fill whole buffer");
        got += (size_t)n;
      }
      done += chunk;
      position += chunk;
    }
  }
  template <typename T>
  T scalar() {
    T v;
    read_exact(&v, sizeof(T));  // little-endian host
    return v;
  }
  bool boolean() {
    const uint8_t v = scalar<uint8_t>();
    if (v > 1) throw invalid("invalid boolean metadata byte " + std::to_string(v));
    return v == 1;
  }
  // Validates a count against the hard maximum and against the bytes that remain, before anything is allocated.
  size_t count(uint64_t value, const std::string& what, uint64_t minimum_bytes, uint64_t maximum) const {
    if (value > maximum) throw invalid(what + " count " + std::to_string(value) + " exceeds the resource limit " + std::to_string(maximum));
    const uint64_t limit = std::min(file_len, kMaxHeaderBytes);
    const uint64_t remaining = limit > position ? limit - position : 0;
    if (minimum_bytes > 0 && value > remaining / minimum_bytes)
      throw invalid(what + " count " + std::to_string(value) + " exceeds the remaining file");
    return (size_t)value;
  }
  std::string string(const std::string& what, uint64_t maximum) {
    const uint64_t byte_len = scalar<uint64_t>();
    const size_t length = count(byte_len, what, 1, maximum);
    std::string bytes(length, '\0');
    if (length) read_exact(&bytes[0], length);
    // UTF-8 validation (strict: no overlongs, no surrogates, at most U+10FFFF)
    const unsigned char* p = reinterpret_cast<const unsigned char*>(bytes.data());
    size_t i = 0;
    while (i < length) {
      const unsigned char c = p[i];
      size_t n = 0;
      uint32_t cp = 0;
      if (c < 0x80) { ++i; continue; }
      if ((c & 0xE0) == 0xC0) { n = 1; cp = c & 0x1F; }
      else if ((c & 0xF0) == 0xE0) { n = 2; cp = c & 0x0F; }
      else if ((c & 0xF8) == 0xF0) { n = 3; cp = c & 0x07; }
      else throw invalid(what + " is not valid UTF-8");
      if (n > length - 1 - i) throw invalid(what + " is not valid UTF-8");  // continuation bytes missing
      for (size_t k = 1; k <= n; ++k) {
        if ((p[i + k] & 0xC0) != 0x80) throw invalid(what + " is not valid UTF-8");
        cp = (cp << 6) | (p[i + k] & 0x3F);
      }
      const bool overlong = (n == 1 && cp < 0x80) || (n == 2 && cp < 0x800) || (n == 3 && cp < 0x10000);
      if (overlong || cp > 0x10FFFF || (cp >= 0xD800 && cp <= 0xDFFF)) throw invalid(what + " is not valid UTF-8");
      i += n + 1;
    }
    return bytes;
  }
};

uint64_t checked_u64(uint64_t v, const char* what) {
  if (v > kJsSafeInteger) throw invalid(std::string(what) + " value " + std::to_string(v) + " is outside the JavaScript safe integer range");
  return v;
}
int64_t checked_i64(int64_t v, const char* what) {
  if (v < -(int64_t)kJsSafeInteger || v > (int64_t)kJsSafeInteger)
    throw invalid(std::string(what) + " value " + std::to_string(v) + " is outside the JavaScript safe integer range");
  return v;
}

// Reads (and validates) one scalar of GGUF type `type`; integer-like values land in e.u, floats in e.f, strings in e.s.
void read_scalar(Reader& r, uint32_t type, MetadataEntry& e, bool in_array) {
  switch (type) {
    case 0: e.u = r.scalar<uint8_t>(); break;
    case 1: e.u = (uint64_t)(int64_t)r.scalar<int8_t>(); break;
    case 2: e.u = r.scalar<uint16_t>(); break;
    case 3: e.u = (uint64_t)(int64_t)r.scalar<int16_t>(); break;
    case 4: e.u = r.scalar<uint32_t>(); break;
    case 5: e.u = (uint64_t)(int64_t)r.scalar<int32_t>(); break;
    case 6: e.f = r.scalar<float>(); break;
    case 7: e.u = r.boolean() ? 1 : 0; break;
    case 8: e.s = r.string(in_array ? "metadata array string" : "metadata string", kMaxMetadataStringBytes); break;
    case 10: e.u = checked_u64(r.scalar<uint64_t>(), in_array ? "metadata u64 array" : "metadata u64"); break;
    case 11: e.u = (uint64_t)checked_i64(r.scalar<int64_t>(), in_array ? "metadata i64 array" : "metadata i64"); break;
    case 12: e.f = r.scalar<double>(); break;
    default: throw invalid("unsupported metadata value type " + std::to_string(type));
  }
}

void read_array(Reader& r, MetadataEntry& e) {
  e.element_type = r.scalar<uint32_t>();
  if (e.element_type == 9) throw invalid("nested metadata arrays are not supported by this parser");
  const uint64_t n = r.scalar<uint64_t>();
  uint64_t minimum = 0;
  switch (e.element_type) {
    case 0: case 1: case 7: minimum = 1; break;
    case 2: case 3: minimum = 2; break;
    case 4: case 5: case 6: minimum = 4; break;
    case 8: case 10: case 11: case 12: minimum = 8; break;
    default: throw invalid("unsupported metadata array element type " + std::to_string(e.element_type));
  }
  e.count = r.count(n, "metadata array", minimum, kMaxMetadataArrayElements);
  MetadataEntry scratch;  // elements are validated, only the first string/number is kept for inspection
  for (uint64_t i = 0; i < e.count; ++i) {
    read_scalar(r, e.element_type, scratch, true);
    if (i == 0) { e.u = scratch.u; e.f = scratch.f; e.s = scratch.s; }
  }
}

int block_values(int codec) { return codec == 0 ? 0 : (codec == 2 || codec == 8 ? 32 : 256); }
int block_bytes(int codec) {
  switch (codec) {
    case 2: return 18;
    case 8: return 34;
    case 10: return 84;
    case 11: return 110;
    case 12: return 144;
    case 13: return 176;
    case 14: return 210;
    default: return 0;
  }
}

uint64_t checked_mul(uint64_t a, uint64_t b, const std::string& what) {
  if (a != 0 && b > UINT64_MAX / a) throw invalid(what);
  return a * b;
}

}  // namespace

struct etc_gguf {
  uint32_t magic = kFileMagic;
  int fd = -1;
  uint64_t file_len = 0;
  std::string architecture;
  std::vector<MetadataEntry> metadata;
  std::vector<TensorEntry> tensors;
};

namespace {

void parse(etc_gguf& g, const volatile int* cancel) {
  Reader r{g.fd, g.file_len, 0, cancel};
  r.check_cancelled();
  if (r.scalar<uint32_t>() != kGgufMagicValue) throw invalid("invalid magic");
  const uint32_t version = r.scalar<uint32_t>();
  if (version != kVersion) throw invalid("unsupported version " + std::to_string(version) + "; expected version " + std::to_string(kVersion));
  const uint64_t tensor_count_raw = r.scalar<uint64_t>();
  const uint64_t metadata_count_raw = r.scalar<uint64_t>();
  const size_t metadata_count = r.count(metadata_count_raw, "metadata", 13, kMaxMetadataCount);
  const size_t tensor_count = r.count(tensor_count_raw, "tensor", 32, kMaxTensorCount);

  std::unordered_set<std::string> keys;
  g.metadata.reserve(metadata_count);
  for (size_t i = 0; i < metadata_count; ++i) {
    MetadataEntry e;
    e.key = r.string("metadata key", kMaxMetadataKeyBytes);
    if (e.key.empty()) throw invalid("metadata key must not be empty");
    if (!keys.insert(e.key).second) throw invalid("duplicate metadata key \"" + e.key + "\"");
    e.type = r.scalar<uint32_t>();
    if (e.type == 9) read_array(r, e);
    else read_scalar(r, e.type, e, false);
    g.metadata.push_back(std::move(e));
  }
  auto find = [&](const char* key) -> const MetadataEntry* {
    for (const auto& e : g.metadata)
      if (e.key == key) return &e;
    return nullptr;
  };
  const MetadataEntry* arch = find("general.architecture");
  if (!arch) throw invalid("missing general.architecture metadata");
  if (arch->type != 8) throw invalid("general.architecture metadata must be a string");
  if (arch->s.empty()) throw invalid("general.architecture metadata must not be empty");
  g.architecture = arch->s;
  uint64_t alignment = kDefaultAlignment;
  if (const MetadataEntry* a = find("general.alignment")) {
    if (a->type != 4) throw invalid("general.alignment metadata must be u32");
    alignment = a->u;
  }
  if (alignment == 0 || (alignment & (alignment - 1)) != 0)
    throw invalid("general.alignment must be a positive power of two, got " + std::to_string(alignment));

  struct Raw { std::string name; std::vector<uint64_t> dims; int codec; uint64_t relative_offset; };
  std::vector<Raw> raws;
  raws.reserve(tensor_count);
  std::unordered_set<std::string> names;
  bool any_quantized = false;
  for (size_t i = 0; i < tensor_count; ++i) {
    Raw raw;
    raw.name = r.string("tensor name", kMaxTensorNameBytes);
    if (raw.name.empty()) throw invalid("tensor name must not be empty");
    if (!names.insert(raw.name).second) throw invalid("duplicate tensor name \"" + raw.name + "\"");
    const uint32_t rank = r.scalar<uint32_t>();
    if (rank < 1 || rank > 4) throw invalid("tensor \"" + raw.name + "\" rank must be in 1..=4, got " + std::to_string(rank));
    for (uint32_t d = 0; d < rank; ++d) {
      const uint64_t dim = r.scalar<uint64_t>();
      if (dim == 0 || dim > kJsSafeInteger) throw invalid("tensor \"" + raw.name + "\" has invalid dimension " + std::to_string(dim));
      raw.dims.push_back(dim);
    }
    const uint32_t code = r.scalar<uint32_t>();
    if (!(code == 0 || code == 2 || code == 8 || (code >= 10 && code <= 14)))
      throw invalid("unsupported GGML tensor type code " + std::to_string(code));
    raw.codec = (int)code;
    any_quantized |= code != 0;
    raw.relative_offset = r.scalar<uint64_t>();
    if (raw.relative_offset % alignment != 0)
      throw invalid("tensor \"" + raw.name + "\" offset " + std::to_string(raw.relative_offset) + " is not aligned to " + std::to_string(alignment));
    raws.push_back(std::move(raw));
  }
  if (any_quantized) {
    const MetadataEntry* q = find("general.quantization_version");
    if (!q) throw invalid("missing general.quantization_version metadata for quantized tensors");
    if (q->type != 4) throw invalid("general.quantization_version metadata must be u32");
    if (q->u != kQuantizationVersion)
      throw invalid("unsupported general.quantization_version " + std::to_string(q->u) + "; expected " + std::to_string(kQuantizationVersion));
  }
  if (r.position + (alignment - 1) < r.position) throw invalid("aligned offset overflows");
  const uint64_t data_start = (r.position + alignment - 1) / alignment * alignment;
  if (data_start > g.file_len) throw invalid("aligned tensor-data section starts beyond the file");

  for (auto& raw : raws) {
    TensorEntry t;
    t.name = raw.name;
    t.codec = raw.codec;
    t.logical.assign(raw.dims.rbegin(), raw.dims.rend());
    const std::string quoted = "tensor \"" + raw.name + "\"";
    if (raw.codec == 0) {
      uint64_t elements = 1;
      for (uint64_t d : t.logical) elements = checked_mul(elements, d, quoted + " size overflows");
      t.byte_len = checked_mul(elements, 4, quoted + " byte length overflows");
      t.physical_rows = 0;
      t.physical_row_units = 0;
    } else {
      const uint64_t columns = raw.dims[0];
      const uint64_t bv = (uint64_t)block_values(raw.codec);
      if (columns % bv != 0)
        throw invalid(quoted + " least-major dimension " + std::to_string(columns) + " is not divisible by " + std::to_string(bv) + " for " +
                      format_name(raw.codec));
      uint64_t rows = 1;
      for (size_t d = 1; d < raw.dims.size(); ++d) rows = checked_mul(rows, raw.dims[d], quoted + " row count size overflows");
      const uint64_t row_bytes = checked_mul(columns / bv, (uint64_t)block_bytes(raw.codec), quoted + " encoded row length overflows");
      t.byte_len = checked_mul(rows, row_bytes, quoted + " byte length overflows");
      t.physical_rows = rows;
      t.physical_row_units = row_bytes;
    }
    if (data_start + raw.relative_offset < data_start) throw invalid("absolute tensor offset overflows");
    t.data_offset = data_start + raw.relative_offset;
    if (t.data_offset + t.byte_len < t.data_offset) throw invalid("tensor range end overflows");
    const uint64_t end = t.data_offset + t.byte_len;
    if (end > g.file_len)
      throw invalid(quoted + " range [" + std::to_string(t.data_offset) + ", " + std::to_string(end) + ") exceeds file size " +
                    std::to_string(g.file_len));
    g.tensors.push_back(std::move(t));
  }
  std::vector<size_t> order(g.tensors.size());
  for (size_t i = 0; i < order.size(); ++i) order[i] = i;
  std::sort(order.begin(), order.end(), [&](size_t a, size_t b) { return g.tensors[a].data_offset < g.tensors[b].data_offset; });
  for (size_t i = 1; i < order.size(); ++i) {
    const TensorEntry& prev = g.tensors[order[i - 1]];
    const TensorEntry& next = g.tensors[order[i]];
    if (next.data_offset < prev.data_offset + prev.byte_len)
      throw invalid("tensor ranges for \"" + prev.name + "\" and \"" + next.name + "\" overlap");
  }
  r.check_cancelled();
}

bool valid_file(const etc_gguf* g) { return g && g->magic == kFileMagic; }

etc_status read_range(const etc_gguf* g, uint64_t offset, unsigned char* dst, size_t length) {
  size_t got = 0;
  while (got < length) {
    const ssize_t n = pread(g->fd, dst + got, length - got, (off_t)(offset + got));
    if (n < 0) {
      if (errno == EINTR) continue;
      return fail(ETC_TRANSFER, std::string("gguf: I/O failed: ") + std::strerror(errno));
    }
    if (n == 0) return fail(ETC_TRANSFER, "gguf: I/O failed: failed to fill whole buffer");
    got += (size_t)n;
  }
  return ETC_OK;
}

}  // namespace

extern "C" {

etc_status etc_gguf_open(const char* path, const volatile int* cancelled_flag, etc_gguf** out) {
  if (!path || !out) return fail(ETC_INVALID_ARGUMENT, "gguf: path and output handle are required");
  *out = nullptr;
  if (cancelled_flag && *cancelled_flag) return fail(ETC_CANCELLED, "gguf: operation aborted");
  const int fd = open(path, O_RDONLY | O_CLOEXEC);
  if (fd < 0) return fail(ETC_TRANSFER, std::string("gguf: I/O failed: ") + std::strerror(errno));
  struct stat st;
  if (fstat(fd, &st) != 0) {
    const std::string message = std::strerror(errno);
    close(fd);
    return fail(ETC_TRANSFER, "gguf: I/O failed: " + message);
  }
  etc_gguf* g = new etc_gguf();
  g->fd = fd;
  g->file_len = (uint64_t)st.st_size;
  try {
    parse(*g, cancelled_flag);
  } catch (const ParseError& e) {
    close(fd);
    delete g;
    return fail(e.status, e.message);
  } catch (const std::bad_alloc&) {
    close(fd);
    delete g;
    return fail(ETC_INVALID_ARGUMENT, "gguf: header is too large");
  }
  *out = g;
  return ETC_OK;
}

etc_status etc_gguf_close(etc_gguf* file) {
  if (!file) return ETC_OK;
  if (!valid_file(file)) return fail(ETC_INVALID_HANDLE, "gguf: handle is invalid or closed");
  close(file->fd);
  file->magic = 0;
  delete file;
  return ETC_OK;
}

etc_status etc_gguf_summary(const etc_gguf* file, const char** architecture, int64_t* metadata_count, int64_t* tensor_count) {
  if (!valid_file(file)) return fail(ETC_INVALID_HANDLE, "gguf: handle is invalid or closed");
  if (architecture) *architecture = file->architecture.c_str();
  if (metadata_count) *metadata_count = (int64_t)file->metadata.size();
  if (tensor_count) *tensor_count = (int64_t)file->tensors.size();
  return ETC_OK;
}

etc_status etc_gguf_metadata(const etc_gguf* file, int64_t index, const char** key, int* value_type, int* element_type,
                             int64_t* count, uint64_t* integer_bits, double* real, const char** string) {
  if (!valid_file(file)) return fail(ETC_INVALID_HANDLE, "gguf: handle is invalid or closed");
  if (index < 0 || (size_t)index >= file->metadata.size()) return fail(ETC_INVALID_ARGUMENT, "gguf: metadata index is out of range");
  const MetadataEntry& e = file->metadata[(size_t)index];
  if (key) *key = e.key.c_str();
  if (value_type) *value_type = (int)e.type;
  if (element_type) *element_type = (int)e.element_type;
  if (count) *count = (int64_t)e.count;
  if (integer_bits) *integer_bits = e.u;
  if (real) *real = e.f;
  if (string) *string = e.s.c_str();
  return ETC_OK;
}

etc_status etc_gguf_tensor(const etc_gguf* file, int64_t index, const char** name, etc_codec* codec, int* rank,
                           int64_t* logical_shape4, int64_t* physical_shape4, uint64_t* data_offset, uint64_t* byte_len) {
  if (!valid_file(file)) return fail(ETC_INVALID_HANDLE, "gguf: handle is invalid or closed");
  if (index < 0 || (size_t)index >= file->tensors.size()) return fail(ETC_INVALID_ARGUMENT, "gguf: tensor index is out of range");
  const TensorEntry& t = file->tensors[(size_t)index];
  if (name) *name = t.name.c_str();
  if (codec) *codec = (etc_codec)t.codec;
  if (rank) *rank = (int)t.logical.size();
  if (logical_shape4)
    for (size_t d = 0; d < 4; ++d) logical_shape4[d] = d < t.logical.size() ? (int64_t)t.logical[d] : 0;
  if (physical_shape4) {
    for (size_t d = 0; d < 4; ++d) physical_shape4[d] = 0;
    if (t.codec == 0) {
      for (size_t d = 0; d < t.logical.size(); ++d) physical_shape4[d] = (int64_t)t.logical[d];
    } else {
      physical_shape4[0] = (int64_t)t.physical_rows;
      physical_shape4[1] = (int64_t)t.physical_row_units;
    }
  }
  if (data_offset) *data_offset = t.data_offset;
  if (byte_len) *byte_len = t.byte_len;
  return ETC_OK;
}

etc_status etc_gguf_find_tensor(const etc_gguf* file, const char* name, int64_t* index) {
  if (!valid_file(file)) return fail(ETC_INVALID_HANDLE, "gguf: handle is invalid or closed");
  if (!name || !index) return fail(ETC_INVALID_ARGUMENT, "gguf: name and index are required");
  for (size_t i = 0; i < file->tensors.size(); ++i)
    if (file->tensors[i].name == name) {
      *index = (int64_t)i;
      return ETC_OK;
    }
  return fail(ETC_INVALID_ARGUMENT, std::string("gguf: no tensor named \"") + name + "\"");
}

etc_status etc_gguf_read_tensor_into(const etc_gguf* file, int64_t index, void* h_dst, uint64_t dst_bytes,
                                     const volatile int* cancelled_flag) {
  if (!valid_file(file)) return fail(ETC_INVALID_HANDLE, "gguf: handle is invalid or closed");
  if (index < 0 || (size_t)index >= file->tensors.size()) return fail(ETC_INVALID_ARGUMENT, "gguf: tensor index is out of range");
  const TensorEntry& t = file->tensors[(size_t)index];
  if (dst_bytes != t.byte_len)
    return fail(ETC_INVALID_ARGUMENT, "gguf: tensor \"" + t.name + "\" requires " + std::to_string(t.byte_len) + " destination bytes, got " +
                                          std::to_string(dst_bytes));
  unsigned char* dst = static_cast<unsigned char*>(h_dst);
  for (uint64_t done = 0; done < t.byte_len; done += kReadChunkBytes) {
    if (cancelled_flag && *cancelled_flag) return fail(ETC_CANCELLED, "gguf: operation aborted");
    ETC_TRY(read_range(file, t.data_offset + done, dst + done, (size_t)std::min<uint64_t>(kReadChunkBytes, t.byte_len - done)));
  }
  if (cancelled_flag && *cancelled_flag) return fail(ETC_CANCELLED, "gguf: operation aborted");
  return ETC_OK;
}

etc_status etc_gguf_load_tensor_device(etc_runtime* rt, const etc_gguf* file, int64_t index, void* d_dst, uint64_t dst_bytes,
                                       const volatile int* cancelled_flag) {
  ETC_TRY(activate(rt));
  if (!valid_file(file)) return fail(ETC_INVALID_HANDLE, "gguf: handle is invalid or closed");
  if (index < 0 || (size_t)index >= file->tensors.size()) return fail(ETC_INVALID_ARGUMENT, "gguf: tensor index is out of range");
  const TensorEntry& t = file->tensors[(size_t)index];
  if (dst_bytes != t.byte_len)
    return fail(ETC_INVALID_ARGUMENT, "gguf: tensor \"" + t.name + "\" requires " + std::to_string(t.byte_len) + " destination bytes, got " +
                                          std::to_string(dst_bytes));
  // two pinned staging buffers: the file read of one chunk overlaps the host-to-device copy of the previous one
  unsigned char* staging[2] = {nullptr, nullptr};
  cudaEvent_t landed[2] = {nullptr, nullptr};
  etc_status st = ETC_OK;
  for (int b = 0; b < 2 && st == ETC_OK; ++b) {
    if (cudaMallocHost((void**)&staging[b], kReadChunkBytes) != cudaSuccess || cudaEventCreateWithFlags(&landed[b], cudaEventDisableTiming) != cudaSuccess)
      st = fail(ETC_TRANSFER, "gguf: pinned staging allocation failed");
  }
  int slot = 0;
  for (uint64_t done = 0; st == ETC_OK && done < t.byte_len; done += kReadChunkBytes, slot ^= 1) {
    if (cancelled_flag && *cancelled_flag) { st = fail(ETC_CANCELLED, "gguf: operation aborted"); break; }
    const size_t chunk = (size_t)std::min<uint64_t>(kReadChunkBytes, t.byte_len - done);
    if (cudaEventSynchronize(landed[slot]) != cudaSuccess) { st = fail(ETC_TRANSFER, "gguf: device copy failed"); break; }
    st = read_range(file, t.data_offset + done, staging[slot], chunk);
    if (st != ETC_OK) break;
    if (cudaMemcpyAsync(static_cast<unsigned char*>(d_dst) + done, staging[slot], chunk, cudaMemcpyHostToDevice, rt->stream) != cudaSuccess ||
        cudaEventRecord(landed[slot], rt->stream) != cudaSuccess)
      st = fail(ETC_TRANSFER, "gguf: device copy failed");
  }
  // the message of a failure above is only kept when there was one (a stale text of an earlier call must not leak out)
  std::string message = st != ETC_OK ? last_error() : std::string();
  if (cudaStreamSynchronize(rt->stream) != cudaSuccess && st == ETC_OK) {
    st = ETC_TRANSFER;
    message = "gguf: device copy failed";
  }
  for (int b = 0; b < 2; ++b) {
    if (staging[b]) cudaFreeHost(staging[b]);
    if (landed[b]) cudaEventDestroy(landed[b]);
  }
  if (st != ETC_OK) return fail(st, message);
  if (st == ETC_OK && cancelled_flag && *cancelled_flag) return fail(ETC_CANCELLED, "gguf: operation aborted");
  return st;
}

}  // extern "C"
