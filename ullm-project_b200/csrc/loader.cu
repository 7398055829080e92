// Weights from a safetensors file, quantised on the device while they load.
//
// The reference plans safetensors as the weight source and conversion at load as the place where quantised
// encodings come from (docs/plans/main-plan.md:26, :76, :112); it has no loader yet.  This one reads the file in
// row chunks through the queue's pinned staging memory, widens F16 / BF16 to fp32 on the device and runs the same
// quantiser as ullm_cuda_quantize on every chunk, so that the packed bytes equal a one-piece quantisation.
// Format: 8-byte little-endian header length, a JSON object {name: {"dtype", "shape", "data_offsets": [begin, end]},
// "__metadata__": {...}}, then the tensor data; offsets are relative to the first byte after the header.
#include "internal.hpp"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdio>
#include <string>

namespace ullm {
namespace {

struct Found {
  uint32_t dtype = 0, rank = 0;
  uint64_t rows = 0, cols = 0, offset = 0, bytes = 0;
};

// A deliberately small JSON reader: just enough for the safetensors header (objects, arrays of integers, strings).
struct Cursor {
  const char *p, *end;
  void ws() {
    while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
  }
  bool eat(char c) {
    ws();
    if (p < end && *p == c) {
      ++p;
      return true;
    }
    return false;
  }
  bool string(std::string *out) {
    ws();
    if (p >= end || *p != '"') return false;
    ++p;
    out->clear();
    while (p < end && *p != '"') {
      if (*p == '\\') {
        if (++p >= end) return false;
        const char c = *p;
        out->push_back(c == 'n' ? '\n' : c == 't' ? '\t' : c);  // \" \\ \/ keep the character; \uXXXX is not expected in names
      } else {
        out->push_back(*p);
      }
      ++p;
    }
    if (p >= end) return false;
    ++p;
    return true;
  }
  bool integer(uint64_t *out) {
    ws();
    if (p >= end || *p < '0' || *p > '9') return false;
    uint64_t v = 0;
    while (p < end && *p >= '0' && *p <= '9') {
      if (v > (UINT64_MAX - 9) / 10) return false;
      v = v * 10 + (uint64_t)(*p - '0');
      ++p;
    }
    *out = v;
    return true;
  }
  // skips any value (used for "__metadata__" and unknown keys)
  bool skip() {
    ws();
    if (p >= end) return false;
    if (*p == '"') {
      std::string s;
      return string(&s);
    }
    if (*p == '{' || *p == '[') {
      const char open = *p, close = open == '{' ? '}' : ']';
      ++p;
      if (eat(close)) return true;
      for (;;) {
        if (open == '{') {
          std::string k;
          if (!string(&k) || !eat(':')) return false;
        }
        if (!skip()) return false;
        if (eat(',')) continue;
        return eat(close);
      }
    }
    while (p < end && *p != ',' && *p != '}' && *p != ']') ++p;  // number / true / false / null
    return true;
  }
};

ullm_status_t dtype_of(const std::string &name, uint32_t *out, sink_t *sink) {
  if (name == "F32") *out = ULLM_CUDA_DTYPE_F32;
  else if (name == "F16") *out = ULLM_CUDA_DTYPE_F16;
  else if (name == "BF16") *out = ULLM_CUDA_DTYPE_BF16;
  else
    return errorf(sink, ULLM_STATUS_UNSUPPORTED,
                  "safetensors dtype %s is not a source for on-load quantisation (F32, F16, BF16 are); 8-bit float payloads "
                  "are not reinterpreted: e4m3fn and e4m3fnuz codes differ", name.c_str());
  return ULLM_STATUS_OK;
}

ullm_status_t find_tensor(const char *path, const char *tensor_name, Found *out, sink_t *sink) {
  if (path == nullptr || tensor_name == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "path or tensor name is null");
  FILE *f = std::fopen(path, "rb");
  if (f == nullptr) return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "cannot open %s", path);
  uint8_t len8[8];
  uint64_t hlen = 0;
  bool ok = std::fread(len8, 1, 8, f) == 8;
  for (int i = 7; ok && i >= 0; --i) hlen = (hlen << 8) | len8[i];
  ok = ok && hlen >= 2 && hlen <= (uint64_t(100) << 20);  // the format caps the header at 100 MB
  std::string header;
  if (ok) {
    header.resize((size_t)hlen);
    ok = std::fread(&header[0], 1, (size_t)hlen, f) == (size_t)hlen;
  }
  long long file_size = -1;
  if (ok && std::fseek(f, 0, SEEK_END) == 0) file_size = std::ftell(f);
  std::fclose(f);
  if (!ok || file_size < 0) return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "%s is not a safetensors file (bad header length)", path);
  Cursor c{header.data(), header.data() + header.size()};
  if (!c.eat('{')) return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "%s: the header is not a JSON object", path);
  if (c.eat('}')) return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "%s holds no tensor named %s", path, tensor_name);
  for (;;) {
    std::string key;
    if (!c.string(&key) || !c.eat(':')) return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "%s: malformed header", path);
    if (key != tensor_name) {
      if (!c.skip()) return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "%s: malformed header", path);
    } else {
      if (!c.eat('{')) return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "%s: malformed entry for %s", path, tensor_name);
      std::string dtype;
      std::vector<uint64_t> shape;
      uint64_t begin = 0, end = 0;
      bool have_dtype = false, have_shape = false, have_off = false;
      for (;;) {
        std::string field;
        if (!c.string(&field) || !c.eat(':')) return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "%s: malformed entry for %s", path, tensor_name);
        bool good = true;
        if (field == "dtype") {
          good = c.string(&dtype);
          have_dtype = good;
        } else if (field == "shape") {
          good = c.eat('[');
          if (good && !c.eat(']')) {
            do {
              uint64_t v;
              good = c.integer(&v);
              shape.push_back(v);
            } while (good && c.eat(','));
            good = good && c.eat(']');
          }
          have_shape = good;
        } else if (field == "data_offsets") {
          good = c.eat('[') && c.integer(&begin) && c.eat(',') && c.integer(&end) && c.eat(']');
          have_off = good;
        } else {
          good = c.skip();
        }
        if (!good) return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "%s: malformed entry for %s", path, tensor_name);
        if (c.eat(',')) continue;
        if (!c.eat('}')) return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "%s: malformed entry for %s", path, tensor_name);
        break;
      }
      if (!have_dtype || !have_shape || !have_off)
        return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "%s: the entry for %s lacks dtype, shape or data_offsets", path, tensor_name);
      ullm_status_t st = dtype_of(dtype, &out->dtype, sink);
      if (st != ULLM_STATUS_OK) return st;
      if (shape.empty() || shape.size() > 2)
        return errorf(sink, ULLM_STATUS_UNSUPPORTED, "%s: tensor %s has rank %zu; a weight is rank 1 or 2", path, tensor_name, shape.size());
      out->rank = (uint32_t)shape.size();
      out->rows = shape.size() == 2 ? shape[0] : 1;
      out->cols = shape.back();
      uint64_t elems = 0, bytes = 0;
      if (__builtin_mul_overflow(out->rows, out->cols, &elems) || __builtin_mul_overflow(elems, dtype_bytes(out->dtype), &bytes) ||
          end < begin || end - begin != bytes || 8 + hlen + end > (uint64_t)file_size)
        return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "%s: data_offsets of %s do not match its shape or leave the file", path, tensor_name);
      out->offset = 8 + hlen + begin;
      out->bytes = bytes;
      return ULLM_STATUS_OK;
    }
    if (c.eat(',')) continue;
    break;
  }
  return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "%s holds no tensor named %s", path, tensor_name);
}

__global__ void widen_kernel(const void *src, uint32_t dtype, uint64_t count, float *dst) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x)
    dst[i] = dtype == ULLM_CUDA_DTYPE_BF16  ? __bfloat162float(static_cast<const __nv_bfloat16 *>(src)[i])
             : dtype == ULLM_CUDA_DTYPE_F16 ? __half2float(static_cast<const __half *>(src)[i])
                                            : static_cast<const float *>(src)[i];
}

}  // namespace
}  // namespace ullm

using namespace ullm;

extern "C" {

ullm_status_t ullm_cuda_safetensors_find(const char *path, const char *tensor_name,
                                         ullm_cuda_safetensors_info_t *info, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  st = validate_struct(info, sink, "safetensors info");
  if (st != ULLM_STATUS_OK) return st;
  Found f;
  st = find_tensor(path, tensor_name, &f, sink);
  if (st != ULLM_STATUS_OK) return st;
  info->dtype = f.dtype;
  info->rank = f.rank;
  info->rows = f.rows;
  info->cols = f.cols;
  info->data_offset = f.offset;
  info->data_bytes = f.bytes;
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("safetensors find")
}

ullm_status_t ullm_cuda_quantize_safetensors(ullm_cuda_queue_t *queue, const char *path, const char *tensor_name,
                                             const ullm_cuda_weight_t *weight, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (weight == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "weight descriptor is null");
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  if (q->capturing) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "a file cannot be loaded into a stream capture");
  WeightPtrs wp;
  st = resolve_weight(*weight, q->ctx, sink, &wp);
  if (st != ULLM_STATUS_OK) return st;
  if (wp.encoding == ULLM_CUDA_ENCODING_NVFP4)
    return write_error(sink, ULLM_STATUS_UNSUPPORTED,
                       "NVFP4's tensor scale depends on the whole tensor, which this chunked loader never holds: upload the "
                       "fp32 tensor and use ullm_cuda_quantize");
  Found f;
  st = find_tensor(path, tensor_name, &f, sink);
  if (st != ULLM_STATUS_OK) return st;
  if (f.rows != wp.n || f.cols != wp.k)
    return errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "tensor %s is [%llu, %llu] but the weight descriptor says [%llu, %llu]", tensor_name,
                  (unsigned long long)f.rows, (unsigned long long)f.cols, (unsigned long long)wp.n, (unsigned long long)wp.k);
  if (!submissions_open(sink, &st)) return st;
  const uint64_t eb = dtype_bytes(f.dtype), row_bytes = wp.k * eb;
  uint64_t rows_per_chunk = kStagingBytes / row_bytes;
  if (rows_per_chunk == 0) return write_error(sink, ULLM_STATUS_UNSUPPORTED, "one row of the tensor exceeds the staging area");
  if (rows_per_chunk > wp.n) rows_per_chunk = wp.n;
  // chunk-sized device scratch: the raw rows and their fp32 widening
  void *raw = nullptr;
  float *wide = nullptr;
  ULLM_CUDA_TRY(cudaMalloc(&raw, rows_per_chunk * row_bytes), "loader scratch");
  cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&wide), rows_per_chunk * wp.k * 4);
  if (e != cudaSuccess) {
    (void)cudaFree(raw);
    return cuda_error(sink, e, "loader scratch");
  }
  FILE *fp = std::fopen(path, "rb");
  ullm_status_t result = ULLM_STATUS_OK;
  if (fp == nullptr || std::fseek(fp, (long)f.offset, SEEK_SET) != 0) result = errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "cannot read %s", path);
  uint8_t *values = const_cast<uint8_t *>(wp.values);
  uint8_t *scales = static_cast<uint8_t *>(const_cast<void *>(wp.scales));
  const uint64_t vrow = wp.encoding == ULLM_CUDA_ENCODING_AQ4 ? wp.k / 2 : wp.k;
  const uint64_t srow = wp.encoding == ULLM_CUDA_ENCODING_AQ4 ? (wp.k / ULLM_CUDA_AQ4_GROUP) * 2 : 4;
  uint64_t kernels = 0, copies = 0;
  for (uint64_t row0 = 0; result == ULLM_STATUS_OK && row0 < wp.n; row0 += rows_per_chunk) {
    const uint64_t rows = wp.n - row0 < rows_per_chunk ? wp.n - row0 : rows_per_chunk;
    const size_t bytes = (size_t)(rows * row_bytes);
    if (std::fread(q->staging, 1, bytes, fp) != bytes) {
      result = errorf(sink, ULLM_STATUS_INVALID_ARGUMENT, "%s ends inside tensor %s", path, tensor_name);
      break;
    }
    e = cudaMemcpyAsync(raw, q->staging, bytes, cudaMemcpyHostToDevice, q->stream);
    if (e == cudaSuccess) {
      widen_kernel<<<256, 256, 0, q->stream>>>(raw, f.dtype, rows * wp.k, wide);
      launch_quantize(q->stream, wide, wp.encoding, rows, wp.k, values + row0 * vrow, scales + row0 * srow);
      e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(q->stream);  // the staging area is reused by the next chunk
    if (e != cudaSuccess) result = cuda_error(sink, e, "safetensors chunk");
    kernels += 2;
    copies += 1;
  }
  if (fp != nullptr) std::fclose(fp);
  (void)cudaFree(raw);
  (void)cudaFree(wide);
  if (result != ULLM_STATUS_OK) return result;
  std::lock_guard<std::mutex> g(q->mutex);
  q->dispatch_count += kernels;
  q->total_dispatch += kernels;
  q->copy_count += copies;
  return ULLM_STATUS_OK;
  ULLM_ENTRY_END("quantize safetensors")
}

}  // extern "C"
