// AQ4 / FP8 quantise, pack, unpack and dequantise kernels, the counter-based
// synthetic generator, and their C-ABI entry points.
//
// The reference only *describes* packed 4-bit storage (two values per U8 byte,
// ceil(n/2) bytes then one scale per block: crates/ullm-core/src/dtype.rs:56-122)
// and tags e4m3fn as a dtype (crates/ullm-core/src/dtype.rs:6-16); it has no
// quantiser.  The rules implemented here are:
//   AQ4  scale = f16_rne(min(amax/7, 65504)); q = clamp(rint(w / f32(scale)), -7, 7), 0 when scale == 0;
//        nibble u = q + 8; byte j = u[2j] | u[2j+1] << 4; dequant = f32(u-8) * f32(scale)   (exact)
//   FP8  scale[n] = amax_n / 448; code = e4m3fn_rne(clamp(w / scale, +-448)), 0 when scale == 0;
//        dequant = f32(code) * scale[n]
// All divisions are IEEE (__fdiv_rn) so that results are bit-identical to the CPU oracle.
// These kernels are HBM-bound elementwise passes; none of them is on the decode hot path.
#include "internal.hpp"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace ullm {

// ---- generator ---------------------------------------------------------------

__device__ __forceinline__ uint64_t splitmix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

static uint64_t host_splitmix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
static uint64_t stream_key(uint64_t seed, uint64_t tensor_id) { return host_splitmix64(host_splitmix64(seed) ^ tensor_id); }

// Irwin-Hall sum of twelve 16-bit uniforms, in integers: z = (2S - 12*65535) * 2^-17.
__device__ __forceinline__ float synth_one(uint64_t key, uint64_t i) {
  int s = 0;
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const uint64_t h = splitmix64(key + 3ull * i + (uint64_t)j);
    s += (int)(h & 0xffff) + (int)((h >> 16) & 0xffff) + (int)((h >> 32) & 0xffff) + (int)(h >> 48);
  }
  return (float)(2 * s - 12 * 65535) * 7.62939453125e-06f;
}

__global__ void synth_weights_kernel(uint64_t key, uint64_t first, uint64_t count, float std, float *out) {
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x)
    out[i] = synth_one(key, first + i) * std;
}

__global__ void synth_activations_kernel(uint64_t key, uint64_t first, uint64_t count, __nv_bfloat16 *out) {
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16_rn(synth_one(key, first + i));
}

__global__ void synth_weight_tile_kernel(uint64_t key, uint64_t full_k, uint64_t row0, uint64_t col0, uint64_t n,
                                         uint64_t k, float std, float *out) {
  const uint64_t total = n * k;
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t r = i / k, c = i - r * k;
    out[i] = synth_one(key, (row0 + r) * full_k + col0 + c) * std;
  }
}

static unsigned grid_for(uint64_t items, unsigned block) {
  uint64_t g = (items + block - 1) / block;
  const uint64_t cap = 148ull * 16ull;
  return (unsigned)(g < 1 ? 1 : (g > cap ? cap : g));
}

void launch_synth_weights(cudaStream_t s, uint64_t seed, uint64_t tensor_id, uint64_t first, uint64_t count,
                          float std, float *out) {
  synth_weights_kernel<<<grid_for(count, 256), 256, 0, s>>>(stream_key(seed, tensor_id), first, count, std, out);
}
void launch_synth_activations(cudaStream_t s, uint64_t seed, uint64_t tensor_id, uint64_t first, uint64_t count,
                              void *out_bf16) {
  synth_activations_kernel<<<grid_for(count, 256), 256, 0, s>>>(stream_key(seed, tensor_id), first, count,
                                                                static_cast<__nv_bfloat16 *>(out_bf16));
}
void launch_synth_weight_tile(cudaStream_t s, uint64_t seed, uint64_t tensor_id, uint64_t full_k, uint64_t row0,
                              uint64_t col0, uint64_t n, uint64_t k, float std, float *out) {
  synth_weight_tile_kernel<<<grid_for(n * k, 256), 256, 0, s>>>(stream_key(seed, tensor_id), full_k, row0, col0, n, k,
                                                                std, out);
}

// ---- AQ4 -----------------------------------------------------------------------

// One warp per (row, group of 128): each lane owns 4 consecutive elements.
__global__ void aq4_quantize_kernel(const float *__restrict__ w, uint64_t groups_total, uint8_t *__restrict__ packed,
                                    __half *__restrict__ scales) {
  const uint64_t warp = (blockIdx.x * (uint64_t)blockDim.x + threadIdx.x) >> 5;
  const uint64_t nwarps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (uint64_t g = warp; g < groups_total; g += nwarps) {
    const float4 v = reinterpret_cast<const float4 *>(w + g * 128)[lane];
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const __half hs = __float2half_rn(fminf(__fdiv_rn(amax, 7.0f), 65504.0f));
    const float sf = __half2float(hs);
    int q0 = 0, q1 = 0, q2 = 0, q3 = 0;
    if (sf != 0.0f) {
      q0 = (int)fminf(fmaxf(rintf(__fdiv_rn(v.x, sf)), -7.0f), 7.0f);
      q1 = (int)fminf(fmaxf(rintf(__fdiv_rn(v.y, sf)), -7.0f), 7.0f);
      q2 = (int)fminf(fmaxf(rintf(__fdiv_rn(v.z, sf)), -7.0f), 7.0f);
      q3 = (int)fminf(fmaxf(rintf(__fdiv_rn(v.w, sf)), -7.0f), 7.0f);
    }
    const uint16_t two = (uint16_t)((q0 + 8) | ((q1 + 8) << 4) | ((q2 + 8) << 8) | ((q3 + 8) << 12));
    reinterpret_cast<uint16_t *>(packed + g * 64)[lane] = two;
    if (lane == 0) scales[g] = hs;
  }
}

__global__ void aq4_unpack_kernel(const uint8_t *__restrict__ packed, uint64_t bytes, int8_t *__restrict__ q) {
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < bytes; i += (uint64_t)gridDim.x * blockDim.x) {
    const uint8_t b = packed[i];
    char2 o;
    o.x = (signed char)((int)(b & 0xf) - 8);
    o.y = (signed char)((int)(b >> 4) - 8);
    reinterpret_cast<char2 *>(q)[i] = o;
  }
}

__global__ void aq4_pack_kernel(const int8_t *__restrict__ q, uint64_t bytes, uint8_t *__restrict__ packed) {
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < bytes; i += (uint64_t)gridDim.x * blockDim.x) {
    const char2 v = reinterpret_cast<const char2 *>(q)[i];
    packed[i] = (uint8_t)((((int)v.x + 8) & 0xf) | ((((int)v.y + 8) & 0xf) << 4));
  }
}

template <typename Out>
__device__ __forceinline__ Out to_out(float v);
template <>
__device__ __forceinline__ float to_out<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

template <typename Out>
__global__ void aq4_dequantize_kernel(const uint8_t *__restrict__ packed, const __half *__restrict__ scales,
                                      uint64_t bytes, Out *__restrict__ out) {
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < bytes; i += (uint64_t)gridDim.x * blockDim.x) {
    const uint8_t b = packed[i];
    const float sf = __half2float(scales[i >> 6]);  // 64 bytes per group of 128
    out[2 * i] = to_out<Out>(__fmul_rn((float)((int)(b & 0xf) - 8), sf));
    out[2 * i + 1] = to_out<Out>(__fmul_rn((float)((int)(b >> 4) - 8), sf));
  }
}

// ---- FP8 -----------------------------------------------------------------------

__device__ __forceinline__ uint8_t encode_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

__device__ __forceinline__ float decode_e4m3(uint8_t c) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)c, __NV_E4M3);
  return __half2float(__half(h));
}

// One block per output channel: amax over the row, then encode.
__global__ void fp8_quantize_kernel(const float *__restrict__ w, uint64_t k, uint8_t *__restrict__ codes,
                                    float *__restrict__ scale) {
  __shared__ float red[32];
  const uint64_t row = blockIdx.x;
  const float *src = w + row * k;
  float amax = 0.0f;
  for (uint64_t i = threadIdx.x; i < k; i += blockDim.x) amax = fmaxf(amax, fabsf(src[i]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (threadIdx.x == 0) red[0] = v;
  }
  __syncthreads();
  amax = red[0];
  const float s = __fdiv_rn(amax, 448.0f);
  if (threadIdx.x == 0) scale[row] = s;
  for (uint64_t i = threadIdx.x; i < k; i += blockDim.x) {
    float v = 0.0f;
    if (s != 0.0f) v = fminf(fmaxf(__fdiv_rn(src[i], s), -448.0f), 448.0f);
    codes[row * k + i] = encode_e4m3(v);
  }
}

template <typename Out>
__global__ void fp8_dequantize_kernel(const uint8_t *__restrict__ codes, const float *__restrict__ scale, uint64_t n,
                                      uint64_t k, Out *__restrict__ out) {
  const uint64_t total = n * k;
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x)
    out[i] = to_out<Out>(__fmul_rn(decode_e4m3(codes[i]), scale[i / k]));
}

void launch_quantize(cudaStream_t s, const float *src, uint32_t encoding, uint64_t n, uint64_t k, uint8_t *values,
                     void *scales) {
  if (encoding == ULLM_CUDA_ENCODING_NVFP4) {
    launch_nvfp4_quantize(s, src, n, k, values, scales);
  } else if (encoding == ULLM_CUDA_ENCODING_AQ4) {
    const uint64_t groups = n * (k / 128);
    aq4_quantize_kernel<<<grid_for(groups * 32, 256), 256, 0, s>>>(src, groups, values, static_cast<__half *>(scales));
  } else {
    fp8_quantize_kernel<<<(unsigned)n, 256, 0, s>>>(src, k, values, static_cast<float *>(scales));
  }
}
void launch_aq4_unpack(cudaStream_t s, const uint8_t *values, uint64_t bytes, int8_t *out) {
  aq4_unpack_kernel<<<grid_for(bytes, 256), 256, 0, s>>>(values, bytes, out);
}
void launch_aq4_pack(cudaStream_t s, const int8_t *src, uint64_t bytes, uint8_t *values) {
  aq4_pack_kernel<<<grid_for(bytes, 256), 256, 0, s>>>(src, bytes, values);
}
void launch_dequantize(cudaStream_t s, uint32_t encoding, const uint8_t *values, const void *scales, uint64_t n,
                       uint64_t k, void *out, uint32_t out_dtype) {
  if (encoding == ULLM_CUDA_ENCODING_NVFP4) {
    launch_nvfp4_dequantize(s, values, scales, n, k, out, out_dtype);
  } else if (encoding == ULLM_CUDA_ENCODING_AQ4) {
    const uint64_t bytes = n * (k / 2);
    if (out_dtype == ULLM_CUDA_DTYPE_F32)
      aq4_dequantize_kernel<float><<<grid_for(bytes, 256), 256, 0, s>>>(values, static_cast<const __half *>(scales),
                                                                        bytes, static_cast<float *>(out));
    else
      aq4_dequantize_kernel<__nv_bfloat16><<<grid_for(bytes, 256), 256, 0, s>>>(
          values, static_cast<const __half *>(scales), bytes, static_cast<__nv_bfloat16 *>(out));
  } else {
    if (out_dtype == ULLM_CUDA_DTYPE_F32)
      fp8_dequantize_kernel<float><<<grid_for(n * k, 256), 256, 0, s>>>(values, static_cast<const float *>(scales), n,
                                                                        k, static_cast<float *>(out));
    else
      fp8_dequantize_kernel<__nv_bfloat16><<<grid_for(n * k, 256), 256, 0, s>>>(
          values, static_cast<const float *>(scales), n, k, static_cast<__nv_bfloat16 *>(out));
  }
}

}  // namespace ullm

using namespace ullm;

extern "C" {

ullm_status_t ullm_cuda_synth_weights(ullm_cuda_queue_t *queue, uint64_t seed, uint64_t tensor_id,
                                      uint64_t first_element, uint64_t count, float std,
                                      ullm_cuda_tensor_t out_f32, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  if (count == 0) return ULLM_STATUS_OK;
  if (count > (1ull << 40)) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "count is implausibly large");
  void *o = nullptr;
  st = resolve(out_f32, count * 4, 4, q->ctx, "synthetic weight output", sink, &o);
  if (st != ULLM_STATUS_OK) return st;
  launch_synth_weights(q->stream, seed, tensor_id, first_element, count, std, static_cast<float *>(o));
  return end_launch(q, sink, "synth_weights launch");
  ULLM_ENTRY_END("synth weights")
}

ullm_status_t ullm_cuda_synth_activations(ullm_cuda_queue_t *queue, uint64_t seed, uint64_t tensor_id,
                                          uint64_t first_element, uint64_t count, ullm_cuda_tensor_t out_bf16,
                                          ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  if (count == 0) return ULLM_STATUS_OK;
  if (count > (1ull << 40)) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "count is implausibly large");
  void *o = nullptr;
  st = resolve(out_bf16, count * 2, 2, q->ctx, "synthetic activation output", sink, &o);
  if (st != ULLM_STATUS_OK) return st;
  launch_synth_activations(q->stream, seed, tensor_id, first_element, count, o);
  return end_launch(q, sink, "synth_activations launch");
  ULLM_ENTRY_END("synth activations")
}

ullm_status_t ullm_cuda_quantize(ullm_cuda_queue_t *queue, ullm_cuda_tensor_t src_f32,
                                 const ullm_cuda_weight_t *weight, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (weight == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "weight descriptor is null");
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  WeightPtrs w;
  st = resolve_weight(*weight, q->ctx, sink, &w);
  if (st != ULLM_STATUS_OK) return st;
  void *src = nullptr;
  st = resolve(src_f32, w.n * w.k * 4, 16, q->ctx, "fp32 source", sink, &src);
  if (st != ULLM_STATUS_OK) return st;
  launch_quantize(q->stream, static_cast<const float *>(src), w.encoding, w.n, w.k, const_cast<uint8_t *>(w.values),
                  const_cast<void *>(w.scales));
  return end_launch(q, sink, "quantize launch");
  ULLM_ENTRY_END("quantize")
}

ullm_status_t ullm_cuda_aq4_unpack(ullm_cuda_queue_t *queue, const ullm_cuda_weight_t *weight,
                                   ullm_cuda_tensor_t out_i8, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (weight == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "weight descriptor is null");
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  WeightPtrs w;
  st = resolve_weight(*weight, q->ctx, sink, &w);
  if (st != ULLM_STATUS_OK) return st;
  if (w.encoding != ULLM_CUDA_ENCODING_AQ4) return write_error(sink, ULLM_STATUS_UNSUPPORTED, "unpack is AQ4 only");
  void *o = nullptr;
  st = resolve(out_i8, w.n * w.k, 2, q->ctx, "int8 output", sink, &o);
  if (st != ULLM_STATUS_OK) return st;
  launch_aq4_unpack(q->stream, w.values, w.n * (w.k / 2), static_cast<int8_t *>(o));
  return end_launch(q, sink, "aq4_unpack launch");
  ULLM_ENTRY_END("aq4 unpack")
}

ullm_status_t ullm_cuda_aq4_pack(ullm_cuda_queue_t *queue, ullm_cuda_tensor_t src_i8,
                                 const ullm_cuda_weight_t *weight, ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (weight == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "weight descriptor is null");
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  WeightPtrs w;
  st = resolve_weight(*weight, q->ctx, sink, &w);
  if (st != ULLM_STATUS_OK) return st;
  if (w.encoding != ULLM_CUDA_ENCODING_AQ4) return write_error(sink, ULLM_STATUS_UNSUPPORTED, "pack is AQ4 only");
  void *src = nullptr;
  st = resolve(src_i8, w.n * w.k, 2, q->ctx, "int8 source", sink, &src);
  if (st != ULLM_STATUS_OK) return st;
  launch_aq4_pack(q->stream, static_cast<const int8_t *>(src), w.n * (w.k / 2), const_cast<uint8_t *>(w.values));
  return end_launch(q, sink, "aq4_pack launch");
  ULLM_ENTRY_END("aq4 pack")
}

ullm_status_t ullm_cuda_dequantize(ullm_cuda_queue_t *queue, const ullm_cuda_weight_t *weight,
                                   ullm_cuda_tensor_t out, uint32_t out_dtype,
                                   ullm_cuda_error_sink_t *error_sink) {
  ULLM_ENTRY_BEGIN
  sink_t *sink = error_sink;
  ullm_status_t st = validate_sink(sink);
  if (st != ULLM_STATUS_OK) return st;
  if (weight == nullptr) return write_error(sink, ULLM_STATUS_INVALID_ARGUMENT, "weight descriptor is null");
  Queue *q = nullptr;
  st = begin_op(queue, sink, &q);
  if (st != ULLM_STATUS_OK) return st;
  WeightPtrs w;
  st = resolve_weight(*weight, q->ctx, sink, &w);
  if (st != ULLM_STATUS_OK) return st;
  if (out_dtype != ULLM_CUDA_DTYPE_F32 && out_dtype != ULLM_CUDA_DTYPE_BF16)
    return write_error(sink, ULLM_STATUS_UNSUPPORTED, "dequantise output must be F32 or BF16");
  void *o = nullptr;
  st = resolve(out, w.n * w.k * dtype_bytes(out_dtype), 4, q->ctx, "dequantised output", sink, &o);
  if (st != ULLM_STATUS_OK) return st;
  launch_dequantize(q->stream, w.encoding, w.values, w.scales, w.n, w.k, o, out_dtype);
  return end_launch(q, sink, "dequantize launch");
  ULLM_ENTRY_END("dequantize")
}

}  // extern "C"
