// Decode matvec: y[M,N] = prologue(x)[M,K] . W'[N,K]^T for M <= 8, with the AQ4 /
// FP8 dequantisation fused into the weight stream.  CUDA cores only (no tensor
// cores): the op is bound by HBM reads of the packed weights.
//
// The reference has no numeric kernel; this file fills the quantised-linear slot
// that its runtime design describes (kernel chosen by op, dtype, encoding, shape:
// docs/architecture/runtime.md:83-91) behind the Backend::execute boundary
// (crates/ullm-core/src/backend.rs:5-11).
//
// Shape of the kernel
//   * persistent grid: (#SMs x CTAs/SM) CTAs of 256 threads; every CTA stages the
//     activations once into shared memory (optionally applying RMSNorm or SwiGLU
//     while it does so), then its warps walk over groups of R output rows;
//   * a lane streams 16-byte pieces of R weight rows straight from global memory
//     (ld.global.nc, no L1 allocation), U pieces per row in flight;
//   * FP8: cvt.e4m3x2 -> f16x2 -> f32, FFMA into fp32 accumulators, one multiply by
//     the per-channel scale at the end;
//   * AQ4: a nibble is dropped into the mantissa of 0.5f with one PRMT
//     (0x3f000000 | u << 16 = 0.5 + u/256), so that  sum x*q = 256*sum(x*f) - 136*sum(x)
//     with sum(x) per 32-element piece precomputed at staging time; the fp16 group
//     scale multiplies the fp32 partial sum of each piece (a piece never straddles a
//     group of 128);
//   * the activations sit in shared memory in [iteration][quad][lane][4] order so
//     that a warp's 16-byte shared loads are conflict-free;
//   * K is reduced across the lanes of one warp with shuffles.
// Algorithmic bytes per launch: N*K (FP8) or N*K/2 + N*K/64 (AQ4) weight bytes
// + scales + M*K*2 in + M*N*2 out.
#include "internal.hpp"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace ullm {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

__device__ __forceinline__ uint4 ldg_stream(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ float bf16_round_f32(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// elements one lane consumes per 16-byte weight load
template <uint32_t ENC>
struct Piece {
  static constexpr int kElems = ENC == ULLM_CUDA_ENCODING_AQ4 ? 32 : 16;
  static constexpr int kQuads = kElems / 4;        // float4 reads of x per piece
};

// Position of activation element k inside the staged [iteration][quad][lane][4] layout.
template <uint32_t ENC>
__device__ __forceinline__ uint32_t x_slot(uint32_t k) {
  constexpr int E = Piece<ENC>::kElems;
  const uint32_t it = k / (E * 32), rem = k % (E * 32);
  const uint32_t lane = rem / E, p = rem % E;
  uint32_t quad, e;
  if (ENC == ULLM_CUDA_ENCODING_AQ4) {
    // word j = p/8 holds 8 nibbles; even nibbles form quad 2j, odd nibbles quad 2j+1
    const uint32_t j = p >> 3, q = p & 7;
    quad = 2 * j + (q & 1);
    e = q >> 1;
  } else {
    quad = p >> 2;
    e = p & 3;
  }
  return ((it * Piece<ENC>::kQuads + quad) * 32 + lane) * 4 + e;
}

struct Params {
  const void *x;
  void *y;
  const uint8_t *w;
  const void *scales;
  uint32_t n, k;
  uint64_t x_stride, y_stride;
  uint32_t x_dtype, y_dtype, prologue;
  float rms_eps;
  uint32_t k_pad;  // K rounded up to a whole warp iteration
};

__device__ __forceinline__ float load_x(const Params &p, uint32_t m, uint32_t k) {
  if (p.x_dtype == ULLM_CUDA_DTYPE_F32)
    return bf16_round_f32(static_cast<const float *>(p.x)[(uint64_t)m * p.x_stride + k]);
  return __bfloat162float(static_cast<const __nv_bfloat16 *>(p.x)[(uint64_t)m * p.x_stride + k]);
}

// Stages prologue(x) for all M rows into shared memory as fp32 values that are
// exactly representable in bf16, zero-padded up to k_pad; for AQ4 also the sum of
// each 32-element piece.
template <int M, uint32_t ENC>
__device__ void stage_activations(const Params &p, float *xs, float *xsum, float *red) {
  const uint32_t tid = threadIdx.x;
  float inv[M];
#pragma unroll
  for (int m = 0; m < M; ++m) inv[m] = 1.0f;
  if (p.prologue == ULLM_CUDA_PROLOGUE_RMSNORM) {
    float ss[M];
#pragma unroll
    for (int m = 0; m < M; ++m) ss[m] = 0.0f;
    for (uint32_t k = tid; k < p.k; k += kThreads)
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const float v = load_x(p, m, k);
        ss[m] = fmaf(v, v, ss[m]);
      }
#pragma unroll
    for (int m = 0; m < M; ++m) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss[m] += __shfl_xor_sync(0xffffffffu, ss[m], o);
      if ((tid & 31) == 0) red[m * kWarps + (tid >> 5)] = ss[m];
    }
    __syncthreads();
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float t = 0.0f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) t += red[m * kWarps + w];
      inv[m] = 1.0f / sqrtf(t / (float)p.k + p.rms_eps);
    }
  }
  for (uint32_t k = tid; k < p.k_pad; k += kThreads) {
    const uint32_t slot = x_slot<ENC>(k);
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float v = 0.0f;
      if (k < p.k) {
        if (p.prologue == ULLM_CUDA_PROLOGUE_SWIGLU) {
          // input row is [gate(K) | up(K)]
          const float g = load_x(p, m, k), u = load_x(p, m, p.k + k);
          v = bf16_round_f32(g / (1.0f + expf(-g)) * u);
        } else if (p.prologue == ULLM_CUDA_PROLOGUE_RMSNORM) {
          v = bf16_round_f32(load_x(p, m, k) * inv[m]);
        } else {
          v = load_x(p, m, k);
        }
      }
      xs[(uint64_t)m * p.k_pad + slot] = v;
    }
  }
  __syncthreads();
  if (ENC == ULLM_CUDA_ENCODING_AQ4) {
    // piece index = (iteration, lane); its 8 quads are 32 lanes apart
    const uint32_t pieces = p.k_pad / 32;
    for (uint32_t i = tid; i < pieces * M; i += kThreads) {
      const uint32_t m = i / pieces, pc = i % pieces;
      const uint32_t it = pc / 32, lane = pc % 32;
      const float4 *base = reinterpret_cast<const float4 *>(xs + (uint64_t)m * p.k_pad) + (it * 8) * 32 + lane;
      float s = 0.0f;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float4 v = base[q * 32];
        s += (v.x + v.y) + (v.z + v.w);
      }
      xsum[m * pieces + pc] = s;
    }
    __syncthreads();
  }
}

__device__ __forceinline__ void store_out(const Params &p, uint32_t m, uint32_t row, float v) {
  if (p.y_dtype == ULLM_CUDA_DTYPE_F32)
    static_cast<float *>(p.y)[(uint64_t)m * p.y_stride + row] = v;
  else
    static_cast<__nv_bfloat16 *>(p.y)[(uint64_t)m * p.y_stride + row] = __float2bfloat16_rn(v);
}

// M activations rows, R weight rows per warp pass, U 16-byte loads per row in flight.
template <int M, int R, int U, uint32_t ENC>
__global__ void __launch_bounds__(kThreads, 1) matvec_kernel(const Params p) {
  extern __shared__ __align__(16) float smem[];
  constexpr int E = Piece<ENC>::kElems;
  constexpr int Q = Piece<ENC>::kQuads;
  float *xs = smem;                                  // [M][k_pad]
  float *xsum = xs + (uint64_t)M * p.k_pad;          // AQ4: [M][k_pad/32]
  float *red = xsum + (ENC == ULLM_CUDA_ENCODING_AQ4 ? (uint64_t)M * (p.k_pad / 32) : 0);  // [M][kWarps]

  stage_activations<M, ENC>(p, xs, xsum, red);

  const uint32_t lane = threadIdx.x & 31;
  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t gwarp = blockIdx.x * kWarps + warp;
  const uint32_t nwarps = gridDim.x * kWarps;
  const uint32_t groups = (p.n + R - 1) / R;
  const uint32_t iters = p.k_pad / (E * 32);
  const uint64_t row_bytes = ENC == ULLM_CUDA_ENCODING_AQ4 ? p.k / 2 : p.k;
  const float4 *xs4 = reinterpret_cast<const float4 *>(xs);
  const uint32_t xrow4 = p.k_pad / 4;  // float4 per activation row

  for (uint32_t g = gwarp; g < groups; g += nwarps) {
    const uint32_t row0 = g * R;
    float acc[R][M];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < M; ++m) acc[r][m] = 0.0f;

    for (uint32_t it0 = 0; it0 < iters; it0 += U) {
      uint4 wv[U][R];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t k0 = (it0 + u) * (E * 32) + lane * E;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const uint32_t row = row0 + r;
          if (it0 + u < iters && k0 < p.k && row < p.n)
            wv[u][r] = ldg_stream(p.w + (uint64_t)row * row_bytes + (ENC == ULLM_CUDA_ENCODING_AQ4 ? k0 / 2 : k0));
          else
            wv[u][r] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (it0 + u >= iters) break;
        const uint32_t it = it0 + u;
        const float4 *xb = xs4 + (it * Q) * 32 + lane;
        if (ENC == ULLM_CUDA_ENCODING_FP8_CHANNEL) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float4 xv[M];
#pragma unroll
            for (int m = 0; m < M; ++m) xv[m] = xb[m * xrow4 + j * 32];
#pragma unroll
            for (int r = 0; r < R; ++r) {
              const uint32_t word = j == 0 ? wv[u][r].x : j == 1 ? wv[u][r].y : j == 2 ? wv[u][r].z : wv[u][r].w;
              const __half2_raw h01 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(word & 0xffffu), __NV_E4M3);
              const __half2_raw h23 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(word >> 16), __NV_E4M3);
              const float2 f01 = __half22float2(__half2(h01));
              const float2 f23 = __half22float2(__half2(h23));
#pragma unroll
              for (int m = 0; m < M; ++m) {
                float a = acc[r][m];
                a = fmaf(f01.x, xv[m].x, a);
                a = fmaf(f01.y, xv[m].y, a);
                a = fmaf(f23.x, xv[m].z, a);
                a = fmaf(f23.y, xv[m].w, a);
                acc[r][m] = a;
              }
            }
          }
        } else {
          // AQ4: one piece = 32 weights of one scale group
          float d[R][M];
#pragma unroll
          for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < M; ++m) d[r][m] = 0.0f;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float4 xe[M], xo[M];
#pragma unroll
            for (int m = 0; m < M; ++m) {
              xe[m] = xb[m * xrow4 + (2 * j) * 32];
              xo[m] = xb[m * xrow4 + (2 * j + 1) * 32];
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
              const uint32_t word = j == 0 ? wv[u][r].x : j == 1 ? wv[u][r].y : j == 2 ? wv[u][r].z : wv[u][r].w;
              const uint32_t lo = word & 0x0f0f0f0fu;         // elements 0,2,4,6 of the word
              const uint32_t hi = (word >> 4) & 0x0f0f0f0fu;  // elements 1,3,5,7
              const float e0 = __uint_as_float(__byte_perm(lo, 0x3f000000u, 0x7044));
              const float e1 = __uint_as_float(__byte_perm(lo, 0x3f000000u, 0x7144));
              const float e2 = __uint_as_float(__byte_perm(lo, 0x3f000000u, 0x7244));
              const float e3 = __uint_as_float(__byte_perm(lo, 0x3f000000u, 0x7344));
              const float o0 = __uint_as_float(__byte_perm(hi, 0x3f000000u, 0x7044));
              const float o1 = __uint_as_float(__byte_perm(hi, 0x3f000000u, 0x7144));
              const float o2 = __uint_as_float(__byte_perm(hi, 0x3f000000u, 0x7244));
              const float o3 = __uint_as_float(__byte_perm(hi, 0x3f000000u, 0x7344));
#pragma unroll
              for (int m = 0; m < M; ++m) {
                float a = d[r][m];
                a = fmaf(e0, xe[m].x, a);
                a = fmaf(e1, xe[m].y, a);
                a = fmaf(e2, xe[m].z, a);
                a = fmaf(e3, xe[m].w, a);
                a = fmaf(o0, xo[m].x, a);
                a = fmaf(o1, xo[m].y, a);
                a = fmaf(o2, xo[m].z, a);
                a = fmaf(o3, xo[m].w, a);
                d[r][m] = a;
              }
            }
          }
          const uint32_t k0 = it * (E * 32) + lane * E;
          const uint32_t pieces = p.k_pad / 32;
          const uint32_t pc = it * 32 + lane;
          float xsm[M];
#pragma unroll
          for (int m = 0; m < M; ++m) xsm[m] = xsum[m * pieces + pc];
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const uint32_t row = row0 + r;
            float s = 0.0f;
            if (k0 < p.k && row < p.n)
              s = __half2float(static_cast<const __half *>(p.scales)[(uint64_t)row * (p.k / 128) + k0 / 128]);
#pragma unroll
            for (int m = 0; m < M; ++m) acc[r][m] = fmaf(s, fmaf(256.0f, d[r][m], -136.0f * xsm[m]), acc[r][m]);
          }
        }
      }
    }

#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float v = acc[r][m];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        acc[r][m] = v;
      }
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const uint32_t row = row0 + r;
        if (row < p.n) {
          float sc = 1.0f;
          if (ENC == ULLM_CUDA_ENCODING_FP8_CHANNEL) sc = static_cast<const float *>(p.scales)[row];
#pragma unroll
          for (int m = 0; m < M; ++m) store_out(p, m, row, acc[r][m] * sc);
        }
      }
    }
  }
}

size_t smem_bytes(uint32_t m, uint32_t k_pad, uint32_t enc) {
  size_t floats = (size_t)m * k_pad + (size_t)m * kWarps;
  if (enc == ULLM_CUDA_ENCODING_AQ4) floats += (size_t)m * (k_pad / 32);
  return floats * sizeof(float);
}

uint32_t pad_k(uint32_t k, uint32_t enc) {
  const uint32_t it = enc == ULLM_CUDA_ENCODING_AQ4 ? 1024u : 512u;
  return (k + it - 1) / it * it;
}

template <int M, int R, int U, uint32_t ENC>
cudaError_t launch_one(const Context *ctx, cudaStream_t stream, const Params &p) {
  const size_t smem = smem_bytes(M, p.k_pad, ENC);
  auto kern = matvec_kernel<M, R, U, ENC>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, smem);
  if (e != cudaSuccess) return e;
  if (per_sm < 1) return cudaErrorLaunchOutOfResources;
  const uint32_t groups = (p.n + R - 1) / R;
  uint32_t grid = (uint32_t)ctx->sm_count * (uint32_t)per_sm;
  const uint32_t needed = (groups + kWarps - 1) / kWarps;
  if (grid > needed) grid = needed;
  kern<<<grid, kThreads, smem, stream>>>(p);
  return cudaGetLastError();
}

template <int M, uint32_t ENC>
cudaError_t launch_m(const Context *ctx, cudaStream_t stream, const Params &p) {
  // Enough row groups to give every SM ~24 warps; otherwise fewer rows per warp.
  const uint32_t want = (uint32_t)ctx->sm_count * 24u;
  const uint32_t iters = p.k_pad / (Piece<ENC>::kElems * 32);
  if (M <= 2) {
    if (p.n / 4 >= want) return iters >= 2 ? launch_one<M, 4, 2, ENC>(ctx, stream, p) : launch_one<M, 4, 1, ENC>(ctx, stream, p);
    if (p.n / 2 >= want) return iters >= 4 ? launch_one<M, 2, 4, ENC>(ctx, stream, p) : launch_one<M, 2, 2, ENC>(ctx, stream, p);
    return iters >= 4 ? launch_one<M, 1, 4, ENC>(ctx, stream, p) : launch_one<M, 1, 2, ENC>(ctx, stream, p);
  }
  if (p.n / 2 >= want) return launch_one<M, 2, 2, ENC>(ctx, stream, p);
  return iters >= 4 ? launch_one<M, 1, 4, ENC>(ctx, stream, p) : launch_one<M, 1, 2, ENC>(ctx, stream, p);
}

template <uint32_t ENC>
cudaError_t launch_enc(const Context *ctx, cudaStream_t stream, const Params &p, uint32_t m) {
  switch (m) {
    case 1: return launch_m<1, ENC>(ctx, stream, p);
    case 2: return launch_m<2, ENC>(ctx, stream, p);
    case 3: return launch_m<3, ENC>(ctx, stream, p);
    case 4: return launch_m<4, ENC>(ctx, stream, p);
    case 5: return launch_m<5, ENC>(ctx, stream, p);
    case 6: return launch_m<6, ENC>(ctx, stream, p);
    case 7: return launch_m<7, ENC>(ctx, stream, p);
    case 8: return launch_m<8, ENC>(ctx, stream, p);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

bool matvec_supports(const LinearArgs &a, const char **why) {
  if (a.m < 1 || a.m > 8) {
    *why = "the matvec kernel serves 1 <= M <= 8";
    return false;
  }
  const uint32_t kp = pad_k(a.k, a.encoding);
  if (smem_bytes(a.m, kp, a.encoding) > 200u * 1024u) {
    *why = "M*K activations do not fit the matvec kernel's shared-memory staging";
    return false;
  }
  return true;
}

int launch_matvec(const Context *ctx, cudaStream_t stream, const LinearArgs &a, cudaError_t *err) {
  Params p;
  p.x = a.x;
  p.y = a.y;
  p.w = a.w;
  p.scales = a.scales;
  p.n = a.n;
  p.k = a.k;
  p.x_stride = a.x_stride;
  p.y_stride = a.y_stride;
  p.x_dtype = a.x_dtype;
  p.y_dtype = a.y_dtype;
  p.prologue = a.prologue;
  p.rms_eps = a.rms_eps;
  p.k_pad = pad_k(a.k, a.encoding);
  cudaError_t e = a.encoding == ULLM_CUDA_ENCODING_AQ4 ? launch_enc<ULLM_CUDA_ENCODING_AQ4>(ctx, stream, p, a.m)
                                                       : launch_enc<ULLM_CUDA_ENCODING_FP8_CHANNEL>(ctx, stream, p, a.m);
  *err = e;
  return e == cudaSuccess ? 1 : -1;
}

}  // namespace ullm
