// NVFP4 weights: quantiser, dequantiser and the decode matvec (M <= 8).
//
// NVFP4 is the 4-bit format the reference already describes — packed 4-bit values in U8 storage with one scale
// per block, scale dtype in {bf16, f16, f32} (crates/ullm-core/src/dtype.rs:56-66, size rule :100-122) — and for
// which its plan adds a tensor scale to the tensor representation and the kernel contract
// (docs/plans/main-plan.md:102-114).  Nothing in the reference computes with it.  Here: e2m1 values, blocks of 16
// along K, f16 block scales, one f32 power-of-two tensor scale stored behind the block scales:
//     w' = e2m1(code) * f32(block_scale) * tensor_scale        (both products exact in fp32)
// The quantiser is bit-exact against the oracle (IEEE divisions, round to nearest with ties to the even code).
// The decode matvec multiplies the dequantised weights with bf16 activations exactly (fp32 FMA): one warp per weight
// row, 16-byte weight loads (32 weights = two blocks), activations staged once per block in shared memory.  The
// tensor-core paths do not serve this encoding: a 16-deep block scale cannot be drained per block from a 32-deep MMA,
// and the block-scaled MMA kinds take power-of-two (ue8m0) or e4m3 scales with BOTH operands in 4 / 6 / 8-bit float,
// i.e. they would also quantise the activations (a W4A4 mode with its own tolerance).
#include "internal.hpp"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>

namespace ullm {
namespace {

constexpr uint32_t kBlock = 16;

__device__ __forceinline__ uint32_t e2m1_rne(float x) {
  // thresholds are the midpoints of the grid {0, .5, 1, 1.5, 2, 3, 4, 6}; on a midpoint the even code wins
  const float a = fminf(fabsf(x), 6.0f);
  uint32_t c = 0;
  c = (a > 0.25f) ? 1u : c;
  c = (a >= 0.75f) ? 2u : c;
  c = (a > 1.25f) ? 3u : c;
  c = (a >= 1.75f) ? 4u : c;
  c = (a > 2.5f) ? 5u : c;
  c = (a >= 3.5f) ? 6u : c;
  c = (a > 5.0f) ? 7u : c;
  return (c != 0u && x < 0.0f) ? (c | 8u) : c;
}

__global__ void nvfp4_amax_kernel(const float *w, uint64_t count, uint32_t *amax_bits) {
  float m = 0.0f;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(w[i]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) atomicMax(amax_bits, __float_as_uint(m));  // non-negative floats order like their bits
}

// in place: the word holds the bits of the tensor's largest magnitude, and receives the tensor scale
__global__ void nvfp4_tensor_scale_kernel(uint32_t *word) {
  const float amax = __uint_as_float(*word);
  float ts = 1.0f;
  if (amax > 0.0f) {
    int e;
    (void)frexpf(__fdiv_rn(amax, 6.0f), &e);  // amax / 6 = m * 2^e, m in [0.5, 1)
    ts = ldexpf(1.0f, e - 1);
  }
  *reinterpret_cast<float *>(word) = ts;
}

// one thread per block of 16 weights
__global__ void nvfp4_quantize_kernel(const float *w, uint64_t blocks, const float *tensor_scale, uint8_t *values, __half *scales) {
  const float ts = *tensor_scale;
  for (uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; b < blocks; b += (uint64_t)gridDim.x * blockDim.x) {
    float v[16];
    const float4 *src = reinterpret_cast<const float4 *>(w + b * kBlock);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 f = src[i];
      v[4 * i] = f.x, v[4 * i + 1] = f.y, v[4 * i + 2] = f.z, v[4 * i + 3] = f.w;
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const __half sb = __float2half_rn(__fdiv_rn(__fdiv_rn(amax, 6.0f), ts));
    const float step = __half2float(sb) * ts;  // exact: an f16 times a power of two
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t c = step > 0.0f ? e2m1_rne(__fdiv_rn(v[i], step)) : 0u;
      if (i < 8)
        lo |= c << (4 * i);
      else
        hi |= c << (4 * (i - 8));
    }
    reinterpret_cast<uint2 *>(values)[b] = make_uint2(lo, hi);
    scales[b] = sb;
  }
}

__device__ __forceinline__ float e2m1_value(uint32_t c) {
  const float mag = (c & 7u) < 2u ? 0.5f * (float)(c & 7u) : __uint_as_float(((((c & 7u) >> 1) + 126u) << 23) | ((c & 1u) << 22));
  return (c & 8u) ? -mag : mag;
}

template <typename OUT>
__global__ void nvfp4_dequantize_kernel(const uint8_t *values, const __half *scales, const float *tensor_scale, uint64_t blocks, OUT *out) {
  const float ts = *tensor_scale;
  for (uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; b < blocks; b += (uint64_t)gridDim.x * blockDim.x) {
    const uint2 pk = reinterpret_cast<const uint2 *>(values)[b];
    const float sb = __half2float(scales[b]);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t c = ((i < 8 ? pk.x : pk.y) >> (4 * (i & 7))) & 15u;
      const float f = e2m1_value(c) * sb * ts;
      if constexpr (sizeof(OUT) == 4)
        out[b * kBlock + i] = f;
      else
        out[b * kBlock + i] = __float2bfloat16_rn(f);
    }
  }
}

struct MvParams {
  const void *x;
  void *y;
  const uint8_t *w;
  const __half *scales;
  const float *tensor_scale;
  const float *residual;
  uint64_t x_stride, y_stride, res_stride;
  uint32_t n, k, k_pad, x_dtype, y_dtype;
};

// One warp per weight row; a lane takes 32 consecutive weights (16 bytes, two scale blocks) per iteration of 1024.
// Activations: fp32 in shared memory as [iteration][j][lane] float4 (j = 0..7: the lane's 32 values), conflict-free.
template <int M>
__global__ void __launch_bounds__(512, 1) nvfp4_matvec_kernel(const MvParams p) {
  extern __shared__ __align__(16) float xs[];  // [M][k_pad]
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t iters = p.k_pad / 1024;
  for (uint32_t c = threadIdx.x; c < p.k_pad / 4; c += blockDim.x) {  // c = float4 index along k
    const uint32_t it = c >> 8, ln = (c >> 3) & 31, j = c & 7;
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c * 4 < p.k) {  // K % 32 == 0: a float4 never straddles the end
        if (p.x_dtype == ULLM_CUDA_DTYPE_F32) {
          const float *s = static_cast<const float *>(p.x) + (uint64_t)m * p.x_stride + c * 4;
          v = make_float4(__bfloat162float(__float2bfloat16_rn(s[0])), __bfloat162float(__float2bfloat16_rn(s[1])),
                          __bfloat162float(__float2bfloat16_rn(s[2])), __bfloat162float(__float2bfloat16_rn(s[3])));
        } else {
          const __nv_bfloat16 *s = static_cast<const __nv_bfloat16 *>(p.x) + (uint64_t)m * p.x_stride + c * 4;
          v = make_float4(__bfloat162float(s[0]), __bfloat162float(s[1]), __bfloat162float(s[2]), __bfloat162float(s[3]));
        }
      }
      reinterpret_cast<float4 *>(xs)[(uint64_t)m * (p.k_pad / 4) + (it * 8 + j) * 32 + ln] = v;
    }
  }
  __syncthreads();
  const float ts = *p.tensor_scale;
  const uint32_t gwarp = blockIdx.x * (blockDim.x / 32) + warp, nwarps = gridDim.x * (blockDim.x / 32);
  for (uint32_t row = gwarp; row < p.n; row += nwarps) {
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.0f;
    for (uint32_t it = 0; it < iters; ++it) {
      const uint32_t k0 = it * 1024 + lane * 32;
      if (k0 >= p.k) continue;
      const uint4 wq = *reinterpret_cast<const uint4 *>(p.w + (uint64_t)row * (p.k / 2) + k0 / 2);
      const uint32_t sc2 = *reinterpret_cast<const uint32_t *>(p.scales + (uint64_t)row * (p.k / kBlock) + k0 / kBlock);
      const float s0 = __half2float(__ushort_as_half((unsigned short)(sc2 & 0xffffu)));
      const float s1 = __half2float(__ushort_as_half((unsigned short)(sc2 >> 16)));
      const uint32_t words[4] = {wq.x, wq.y, wq.z, wq.w};
      float part[M][2];
#pragma unroll
      for (int m = 0; m < M; ++m) part[m][0] = part[m][1] = 0.0f;
#pragma unroll
      for (int wi = 0; wi < 4; ++wi) {   // 8 weights per word; words 0,1 = block 0, words 2,3 = block 1
        float wv[8];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)((words[wi] >> (8 * b)) & 0xffu), __NV_E2M1);
          const float2 f = __half22float2(__half2(h));
          wv[2 * b] = f.x, wv[2 * b + 1] = f.y;
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const float4 *xb = reinterpret_cast<const float4 *>(xs) + (uint64_t)m * (p.k_pad / 4) + (it * 8 + wi * 2) * 32 + lane;
          const float4 a = xb[0], b4 = xb[32];
          float t = part[m][wi >> 1];
          t = fmaf(wv[0], a.x, t), t = fmaf(wv[1], a.y, t), t = fmaf(wv[2], a.z, t), t = fmaf(wv[3], a.w, t);
          t = fmaf(wv[4], b4.x, t), t = fmaf(wv[5], b4.y, t), t = fmaf(wv[6], b4.z, t), t = fmaf(wv[7], b4.w, t);
          part[m][wi >> 1] = t;
        }
      }
#pragma unroll
      for (int m = 0; m < M; ++m) acc[m] = fmaf(part[m][0], s0, fmaf(part[m][1], s1, acc[m]));
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float v = acc[m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) {
        v *= ts;
        if (p.residual != nullptr) v += p.residual[(uint64_t)m * p.res_stride + row];
        if (p.y_dtype == ULLM_CUDA_DTYPE_F32)
          static_cast<float *>(p.y)[(uint64_t)m * p.y_stride + row] = v;
        else
          static_cast<__nv_bfloat16 *>(p.y)[(uint64_t)m * p.y_stride + row] = __float2bfloat16_rn(v);
      }
    }
  }
}

unsigned grid_of(uint64_t work, unsigned threads) {
  const uint64_t g = (work + threads - 1) / threads;
  return (unsigned)(g < 1 ? 1 : (g > 4096 ? 4096 : g));
}

template <int M>
cudaError_t launch_mv(const Context *ctx, cudaStream_t s, const MvParams &p) {
  const size_t smem = (size_t)M * p.k_pad * 4;
  static std::mutex mu;
  static size_t granted[kMaxDevices] = {};
  {
    std::lock_guard<std::mutex> g(mu);
    if (smem > granted[ctx->device]) {
      cudaError_t e = cudaFuncSetAttribute(nvfp4_matvec_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      granted[ctx->device] = smem;
    }
  }
  unsigned grid = (unsigned)ctx->sm_count;
  const unsigned needed = (p.n + 15) / 16;
  if (grid > needed) grid = needed;
  nvfp4_matvec_kernel<M><<<grid, 512, smem, s>>>(p);
  return cudaGetLastError();
}

}  // namespace

uint64_t nvfp4_scale_bytes(uint64_t n, uint64_t k) { return (n * (k / kBlock) * 2 + 15) / 16 * 16 + 4; }
static const float *tensor_scale_of(const void *scales, uint64_t n, uint64_t k) {
  return reinterpret_cast<const float *>(static_cast<const uint8_t *>(scales) + (n * (k / kBlock) * 2 + 15) / 16 * 16);
}

void launch_nvfp4_quantize(cudaStream_t s, const float *src, uint64_t n, uint64_t k, uint8_t *values, void *scales) {
  float *ts = const_cast<float *>(tensor_scale_of(scales, n, k));
  (void)cudaMemsetAsync(ts, 0, 4, s);
  nvfp4_amax_kernel<<<grid_of(n * k, 256), 256, 0, s>>>(src, n * k, reinterpret_cast<uint32_t *>(ts));
  nvfp4_tensor_scale_kernel<<<1, 1, 0, s>>>(reinterpret_cast<uint32_t *>(ts));
  nvfp4_quantize_kernel<<<grid_of(n * k / kBlock, 256), 256, 0, s>>>(src, n * k / kBlock, ts, values, static_cast<__half *>(scales));
}

void launch_nvfp4_dequantize(cudaStream_t s, const uint8_t *values, const void *scales, uint64_t n, uint64_t k, void *out,
                             uint32_t out_dtype) {
  const float *ts = tensor_scale_of(scales, n, k);
  if (out_dtype == ULLM_CUDA_DTYPE_F32)
    nvfp4_dequantize_kernel<float><<<grid_of(n * k / kBlock, 256), 256, 0, s>>>(values, static_cast<const __half *>(scales), ts,
                                                                                n * k / kBlock, static_cast<float *>(out));
  else
    nvfp4_dequantize_kernel<__nv_bfloat16><<<grid_of(n * k / kBlock, 256), 256, 0, s>>>(
        values, static_cast<const __half *>(scales), ts, n * k / kBlock, static_cast<__nv_bfloat16 *>(out));
}

bool nvfp4_matvec_supports(const LinearArgs &a, const char **why) {
  if (a.m < 1 || a.m > 8) {
    *why = "NVFP4 weights are served by the decode kernel only (1 <= M <= 8); the tensor-core kernels do not take this encoding";
    return false;
  }
  if (a.prologue != ULLM_CUDA_PROLOGUE_NONE || a.epilogue != ULLM_CUDA_EPILOGUE_NONE) {
    *why = "the NVFP4 decode kernel offers no prologue or epilogue";
    return false;
  }
  if ((size_t)a.m * ((a.k + 1023) / 1024 * 1024) * 4 > 224u * 1024u) {
    *why = "M*K activations do not fit the NVFP4 decode kernel's shared-memory staging";
    return false;
  }
  return true;
}

int launch_matvec_nvfp4(const Context *ctx, cudaStream_t stream, const LinearArgs &a, cudaError_t *err) {
  MvParams p{};
  p.x = a.x;
  p.y = a.y;
  p.w = a.w;
  p.scales = static_cast<const __half *>(a.scales);
  p.tensor_scale = tensor_scale_of(a.scales, a.n, a.k);
  p.residual = a.residual;
  p.x_stride = a.x_stride;
  p.y_stride = a.y_stride;
  p.res_stride = a.res_stride;
  p.n = a.n;
  p.k = a.k;
  p.k_pad = (a.k + 1023) / 1024 * 1024;
  p.x_dtype = a.x_dtype;
  p.y_dtype = a.y_dtype;
  switch (a.m) {
    case 1: *err = launch_mv<1>(ctx, stream, p); break;
    case 2: *err = launch_mv<2>(ctx, stream, p); break;
    case 3: *err = launch_mv<3>(ctx, stream, p); break;
    case 4: *err = launch_mv<4>(ctx, stream, p); break;
    case 5: *err = launch_mv<5>(ctx, stream, p); break;
    case 6: *err = launch_mv<6>(ctx, stream, p); break;
    case 7: *err = launch_mv<7>(ctx, stream, p); break;
    case 8: *err = launch_mv<8>(ctx, stream, p); break;
    default: *err = cudaErrorInvalidValue; break;
  }
  return *err == cudaSuccess ? 1 : -1;
}

}  // namespace ullm
