// The GGUF container, host side: header, metadata and tensor table are parsed once, the tensor data
// stays on disk and is read (or uploaded to the GPU) tensor by tensor. Counterpart of the
// reference's GGUFFile (Sources/IshizukiKit/Config/GGUFFile.swift:179-397) and of the block geometry
// in GGMLType (GGUFFile.swift:13-121); same limits, same refusals.
#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <new>
#include <string>
#include <vector>

#include "../../include/ishizuki_cuda.h"

namespace {

struct TypeGeometry {
  int id, block, bytes;
  const char *name;
};
// GGMLType.blockSize / typeSize / name (GGUFFile.swift:44-113)
const TypeGeometry kTypes[] = {
    {0, 1, 4, "F32"},       {1, 1, 2, "F16"},       {2, 32, 18, "Q4_0"},     {3, 32, 20, "Q4_1"},     {6, 32, 22, "Q5_0"},
    {7, 32, 24, "Q5_1"},    {8, 32, 34, "Q8_0"},    {9, 32, 36, "Q8_1"},     {10, 256, 84, "Q2_K"},   {11, 256, 110, "Q3_K"},
    {12, 256, 144, "Q4_K"}, {13, 256, 176, "Q5_K"}, {14, 256, 210, "Q6_K"},  {15, 256, 292, "Q8_K"},  {16, 256, 66, "IQ2_XXS"},
    {17, 256, 74, "IQ2_XS"}, {18, 256, 98, "IQ3_XXS"}, {19, 256, 50, "IQ1_S"}, {20, 32, 18, "IQ4_NL"}, {21, 256, 110, "IQ3_S"},
    {22, 256, 82, "IQ2_S"}, {23, 256, 136, "IQ4_XS"}, {24, 1, 1, "I8"},      {25, 1, 2, "I16"},       {26, 1, 4, "I32"},
    {27, 1, 8, "I64"},      {28, 1, 8, "F64"},      {29, 256, 56, "IQ1_M"},  {30, 1, 2, "BF16"},
};

const TypeGeometry *geometry(uint32_t id) {
  for (const TypeGeometry &t : kTypes)
    if ((uint32_t)t.id == id) return &t;
  return nullptr;
}

enum ValueKind { kUint = 1, kInt = 2, kDouble = 3, kBool = 4, kString = 5, kArray = 6 };

struct Value {
  int kind = 0;
  uint64_t u = 0;
  int64_t i = 0;
  double d = 0;
  std::string s;
  std::vector<Value> items;
};

struct Tensor {
  std::string name;
  int rank = 0;
  int64_t shape[4] = {1, 1, 1, 1};  // row-major: the file's fastest-varying-first order reversed
  uint32_t type = 0;
  int64_t offset = 0, bytes = 0;
};

struct Failure {
  std::string text;
};

// sequential little-endian reader over the file with the reference's plausibility limits
struct Reader {
  int fd;
  int64_t pos = 0, size = 0;
  std::vector<uint8_t> buf;
  int64_t buf_at = 0;

  void need(int64_t count) {
    if (pos >= buf_at && pos + count <= buf_at + (int64_t)buf.size()) return;
    const int64_t want = std::max<int64_t>(count, 1 << 20);
    const int64_t take = std::min<int64_t>(want, size - pos);
    if (take < count) throw Failure{"GGUF header ends mid-field"};
    buf.resize((size_t)take);
    int64_t got = 0;
    while (got < take) {
      const ssize_t r = pread(fd, buf.data() + got, (size_t)(take - got), (off_t)(pos + got));
      if (r <= 0) throw Failure{"GGUF header ends mid-field"};
      got += r;
    }
    buf_at = pos;
  }
  template <class T>
  T scalar() {
    need(sizeof(T));
    T v;
    memcpy(&v, buf.data() + (pos - buf_at), sizeof(T));
    pos += sizeof(T);
    return v;  // x86-64 and aarch64 hosts are little-endian, as the file is
  }
  uint32_t u32() { return scalar<uint32_t>(); }
  uint64_t u64() { return scalar<uint64_t>(); }
  std::string string() {
    const uint64_t length = u64();
    if (length >= (1ull << 28)) throw Failure{"GGUF string length " + std::to_string(length) + " is implausible"};
    need((int64_t)length);
    std::string s(reinterpret_cast<const char *>(buf.data() + (pos - buf_at)), (size_t)length);
    pos += (int64_t)length;
    return s;
  }
  Value value(uint32_t type) {
    Value v;
    switch (type) {
      case 0: v.kind = kUint, v.u = scalar<uint8_t>(); break;
      case 1: v.kind = kInt, v.i = scalar<int8_t>(); break;
      case 2: v.kind = kUint, v.u = scalar<uint16_t>(); break;
      case 3: v.kind = kInt, v.i = scalar<int16_t>(); break;
      case 4: v.kind = kUint, v.u = u32(); break;
      case 5: v.kind = kInt, v.i = scalar<int32_t>(); break;
      case 6: v.kind = kDouble, v.d = (double)scalar<float>(); break;
      case 7: v.kind = kBool, v.u = scalar<uint8_t>() != 0; break;
      case 8: v.kind = kString, v.s = string(); break;
      case 9: {
        const uint32_t element = u32();
        const uint64_t count = u64();
        if (count >= (1ull << 26)) throw Failure{"GGUF array of " + std::to_string(count) + " is implausible"};
        v.kind = kArray;
        v.items.reserve((size_t)count);
        for (uint64_t k = 0; k < count; ++k) v.items.push_back(value(element));
        break;
      }
      case 10: v.kind = kUint, v.u = u64(); break;
      case 11: v.kind = kInt, v.i = (int64_t)u64(); break;
      case 12: v.kind = kDouble, v.d = scalar<double>(); break;
      default: throw Failure{"GGUF metadata type " + std::to_string(type) + " is unknown"};
    }
    return v;
  }
};

bool as_int(const Value &v, int64_t *out) {
  switch (v.kind) {
    case kUint: *out = (int64_t)v.u; return v.u <= (uint64_t)INT64_MAX;
    case kInt: *out = v.i; return true;
    case kDouble: *out = (int64_t)(v.d < 0 ? v.d - 0.5 : v.d + 0.5); return true;
    case kBool: *out = v.u ? 1 : 0; return true;
    default: return false;
  }
}

}  // namespace

struct ishi_gguf {
  int fd = -1;
  uint32_t version = 0;
  int64_t data_offset = 0, alignment = 32, file_size = 0;
  std::map<std::string, Value> metadata;
  std::vector<std::string> keys;  // in file order
  std::vector<Tensor> tensors;
  std::map<std::string, int64_t> index;
  std::string last_error;
};

namespace {

ishi_status gguf_fail(ishi_gguf *g, ishi_status s, const std::string &text) {
  if (g) g->last_error = text;
  return s;
}

const Value *lookup(const ishi_gguf *g, const char *key) {
  if (!g || !key) return nullptr;
  auto it = g->metadata.find(key);
  return it == g->metadata.end() ? nullptr : &it->second;
}

}  // namespace

extern "C" {

ishi_status ishi_gguf_open(const char *path, ishi_gguf **out, char *error_out, size_t error_len) {
  if (out) *out = nullptr;
  auto report = [&](ishi_status s, const std::string &text) {
    if (error_out && error_len) snprintf(error_out, error_len, "%s", text.c_str());
    return s;
  };
  if (!path || !out) return report(ISHI_E_INVALID, "null argument");
  std::unique_ptr<ishi_gguf> g(new (std::nothrow) ishi_gguf());
  if (!g) return report(ISHI_E_NOMEM, "out of memory");
  g->fd = open(path, O_RDONLY);
  if (g->fd < 0) return report(ISHI_E_INVALID, std::string("cannot open ") + path);
  struct stat st;
  if (fstat(g->fd, &st) != 0) {
    close(g->fd);
    return report(ISHI_E_INVALID, "cannot stat the file");
  }
  g->file_size = (int64_t)st.st_size;
  try {
    Reader r{g->fd};
    r.size = g->file_size;
    if (r.u32() != 0x46554747u) throw Failure{"not a GGUF file"};
    g->version = r.u32();
    if (g->version != 2 && g->version != 3) throw Failure{"GGUF version " + std::to_string(g->version) + " is not supported"};
    const uint64_t tensor_count = r.u64(), metadata_count = r.u64();
    if (tensor_count >= 1000000 || metadata_count >= 1000000) throw Failure{"GGUF header counts are implausible"};
    for (uint64_t k = 0; k < metadata_count; ++k) {
      std::string key = r.string();
      const uint32_t type = r.u32();
      Value v = r.value(type);
      if (!g->metadata.count(key)) g->keys.push_back(key);
      g->metadata[key] = std::move(v);
    }
    int64_t alignment = 32;
    if (const Value *a = lookup(g.get(), "general.alignment")) {
      if (!as_int(*a, &alignment)) alignment = 32;
    }
    if (alignment <= 0 || (alignment & (alignment - 1)) != 0)
      throw Failure{"GGUF alignment " + std::to_string(alignment) + " is not a power of two"};
    g->alignment = alignment;
    g->tensors.reserve((size_t)tensor_count);
    for (uint64_t k = 0; k < tensor_count; ++k) {
      Tensor t;
      t.name = r.string();
      const uint32_t rank = r.u32();
      if (rank < 1 || rank > 4) throw Failure{t.name + " has rank " + std::to_string(rank)};
      t.rank = (int)rank;
      int64_t dims[4] = {1, 1, 1, 1};
      int64_t elements = 1;
      for (uint32_t d = 0; d < rank; ++d) {
        const uint64_t extent = r.u64();
        if (extent > (1ull << 40) || (extent != 0 && elements > (int64_t)((1ull << 62) / extent)))
          throw Failure{t.name + " has an implausible shape"};
        dims[d] = (int64_t)extent;
        elements *= dims[d];
      }
      for (uint32_t d = 0; d < rank; ++d) t.shape[d] = dims[rank - 1 - d];
      t.type = r.u32();
      const TypeGeometry *geo = geometry(t.type);
      if (!geo) throw Failure{t.name + " has unknown GGML type " + std::to_string(t.type)};
      t.offset = (int64_t)r.u64();
      if (elements % geo->block != 0)
        throw Failure{t.name + " has " + std::to_string(elements) + " elements, not a multiple of " + geo->name + "'s " +
                      std::to_string(geo->block) + "-element block"};
      t.bytes = elements / geo->block * geo->bytes;
      g->index[t.name] = (int64_t)g->tensors.size();
      g->tensors.push_back(std::move(t));
    }
    g->data_offset = (r.pos + alignment - 1) / alignment * alignment;
  } catch (const Failure &f) {
    close(g->fd);
    return report(ISHI_E_UNSUPPORTED, f.text);
  } catch (const std::bad_alloc &) {
    close(g->fd);
    return report(ISHI_E_NOMEM, "out of memory while reading the header");
  }
  *out = g.release();
  return ISHI_OK;
}

void ishi_gguf_close(ishi_gguf *g) {
  if (!g) return;
  if (g->fd >= 0) close(g->fd);
  delete g;
}

const char *ishi_gguf_last_error(const ishi_gguf *g) { return g ? g->last_error.c_str() : "null file"; }
uint32_t ishi_gguf_version(const ishi_gguf *g) { return g ? g->version : 0; }
int64_t ishi_gguf_data_offset(const ishi_gguf *g) { return g ? g->data_offset : 0; }
int64_t ishi_gguf_alignment(const ishi_gguf *g) { return g ? g->alignment : 0; }
int64_t ishi_gguf_tensor_count(const ishi_gguf *g) { return g ? (int64_t)g->tensors.size() : 0; }
int64_t ishi_gguf_metadata_count(const ishi_gguf *g) { return g ? (int64_t)g->keys.size() : 0; }
const char *ishi_gguf_metadata_key(const ishi_gguf *g, int64_t i) {
  return (g && i >= 0 && i < (int64_t)g->keys.size()) ? g->keys[(size_t)i].c_str() : nullptr;
}

int64_t ishi_gguf_find_tensor(const ishi_gguf *g, const char *name) {
  if (!g || !name) return -1;
  auto it = g->index.find(name);
  return it == g->index.end() ? -1 : it->second;
}

ishi_status ishi_gguf_tensor(const ishi_gguf *g, int64_t i, ishi_gguf_tensor_info *out) {
  if (!g || !out || i < 0 || i >= (int64_t)g->tensors.size()) return ISHI_E_INVALID;
  const Tensor &t = g->tensors[(size_t)i];
  out->name = t.name.c_str();
  out->rank = t.rank;
  for (int d = 0; d < 4; ++d) out->shape[d] = t.shape[d];
  out->ggml_type = (int32_t)t.type;
  out->offset = t.offset;
  out->byte_count = t.bytes;
  return ISHI_OK;
}

int ishi_gguf_type_block_size(int ggml_type) {
  const TypeGeometry *geo = geometry((uint32_t)ggml_type);
  return geo ? geo->block : 0;
}
int ishi_gguf_type_size(int ggml_type) {
  const TypeGeometry *geo = geometry((uint32_t)ggml_type);
  return geo ? geo->bytes : 0;
}
const char *ishi_gguf_type_name(int ggml_type) {
  const TypeGeometry *geo = geometry((uint32_t)ggml_type);
  return geo ? geo->name : nullptr;
}

int ishi_gguf_metadata_kind(const ishi_gguf *g, const char *key) {
  const Value *v = lookup(g, key);
  return v ? v->kind : 0;
}
ishi_status ishi_gguf_metadata_int(const ishi_gguf *g, const char *key, int64_t *out) {
  const Value *v = lookup(g, key);
  if (!v || !out) return ISHI_E_INVALID;
  return as_int(*v, out) ? ISHI_OK : ISHI_E_SHAPE;
}
ishi_status ishi_gguf_metadata_float(const ishi_gguf *g, const char *key, double *out) {
  const Value *v = lookup(g, key);
  if (!v || !out) return ISHI_E_INVALID;
  switch (v->kind) {
    case kUint: *out = (double)v->u; return ISHI_OK;
    case kInt: *out = (double)v->i; return ISHI_OK;
    case kDouble: *out = v->d; return ISHI_OK;
    default: return ISHI_E_SHAPE;
  }
}
const char *ishi_gguf_metadata_string(const ishi_gguf *g, const char *key) {
  const Value *v = lookup(g, key);
  return (v && v->kind == kString) ? v->s.c_str() : nullptr;
}
int64_t ishi_gguf_metadata_array_length(const ishi_gguf *g, const char *key) {
  const Value *v = lookup(g, key);
  return (v && v->kind == kArray) ? (int64_t)v->items.size() : -1;
}
ishi_status ishi_gguf_metadata_array_int(const ishi_gguf *g, const char *key, int64_t i, int64_t *out) {
  const Value *v = lookup(g, key);
  if (!v || !out || v->kind != kArray || i < 0 || i >= (int64_t)v->items.size()) return ISHI_E_INVALID;
  return as_int(v->items[(size_t)i], out) ? ISHI_OK : ISHI_E_SHAPE;
}
const char *ishi_gguf_metadata_array_string(const ishi_gguf *g, const char *key, int64_t i) {
  const Value *v = lookup(g, key);
  if (!v || v->kind != kArray || i < 0 || i >= (int64_t)v->items.size()) return nullptr;
  return v->items[(size_t)i].kind == kString ? v->items[(size_t)i].s.c_str() : nullptr;
}

ishi_status ishi_gguf_read_tensor(ishi_gguf *g, int64_t i, void *dst_host, int64_t dst_bytes) {
  if (!g || !dst_host || i < 0 || i >= (int64_t)g->tensors.size()) return ISHI_E_INVALID;
  const Tensor &t = g->tensors[(size_t)i];
  if (dst_bytes < t.bytes) return gguf_fail(g, ISHI_E_SHAPE, t.name + " needs " + std::to_string(t.bytes) + " bytes");
  const int64_t at = g->data_offset + t.offset;
  if (t.offset < 0 || at + t.bytes > g->file_size) return gguf_fail(g, ISHI_E_SHAPE, t.name + " runs past the end of the file");
  int64_t got = 0;
  while (got < t.bytes) {
    const ssize_t r = pread(g->fd, static_cast<uint8_t *>(dst_host) + got, (size_t)(t.bytes - got), (off_t)(at + got));
    if (r <= 0) return gguf_fail(g, ISHI_E_SHAPE, t.name + " runs past the end of the file");
    got += r;
  }
  return ISHI_OK;
}

ishi_status ishi_gguf_upload_tensor(ishi_gguf *g, int64_t i, void *dst_dev, int64_t dst_bytes, void *stream) {
  if (!g || !dst_dev || i < 0 || i >= (int64_t)g->tensors.size()) return ISHI_E_INVALID;
  const Tensor &t = g->tensors[(size_t)i];
  if (dst_bytes < t.bytes) return gguf_fail(g, ISHI_E_SHAPE, t.name + " needs " + std::to_string(t.bytes) + " bytes");
  const int64_t at = g->data_offset + t.offset;
  if (t.offset < 0 || at + t.bytes > g->file_size) return gguf_fail(g, ISHI_E_SHAPE, t.name + " runs past the end of the file");
  // through two page-locked staging buffers, so that reading the file overlaps the copies
  constexpr int64_t kChunk = 8 << 20;
  void *stage[2] = {nullptr, nullptr};
  cudaEvent_t done[2] = {nullptr, nullptr};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ishi_status status = ISHI_OK;
  for (int b = 0; b < 2 && status == ISHI_OK; ++b) {
    if (cudaHostAlloc(&stage[b], (size_t)std::min(kChunk, std::max<int64_t>(t.bytes, 1)), cudaHostAllocDefault) != cudaSuccess ||
        cudaEventCreateWithFlags(&done[b], cudaEventDisableTiming) != cudaSuccess)
      status = gguf_fail(g, ISHI_E_NOMEM, "no page-locked staging memory");
  }
  int64_t moved = 0;
  for (int b = 0; status == ISHI_OK && moved < t.bytes; b ^= 1) {
    const int64_t take = std::min(kChunk, t.bytes - moved);
    if (cudaEventSynchronize(done[b]) != cudaSuccess) status = gguf_fail(g, ISHI_E_CUDA, "waiting for a staging buffer failed");
    int64_t got = 0;
    while (status == ISHI_OK && got < take) {
      const ssize_t r = pread(g->fd, static_cast<uint8_t *>(stage[b]) + got, (size_t)(take - got), (off_t)(at + moved + got));
      if (r <= 0) status = gguf_fail(g, ISHI_E_SHAPE, t.name + " runs past the end of the file");
      else got += r;
    }
    if (status != ISHI_OK) break;
    if (cudaMemcpyAsync(static_cast<uint8_t *>(dst_dev) + moved, stage[b], (size_t)take, cudaMemcpyHostToDevice, st) != cudaSuccess ||
        cudaEventRecord(done[b], st) != cudaSuccess)
      status = gguf_fail(g, ISHI_E_CUDA, "copying " + t.name + " to the device failed");
    moved += take;
  }
  for (int b = 0; b < 2; ++b) {
    if (done[b]) {
      cudaEventSynchronize(done[b]);
      cudaEventDestroy(done[b]);
    }
    if (stage[b]) cudaFreeHost(stage[b]);
  }
  return status;
}

}  // extern "C"
