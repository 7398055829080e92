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
//   * persistent grid: one CTA per SM (768 threads for the common one-row case).  A CTA
//     first starts the weight loads of its first row groups (registers + an L2 prefetch),
//     THEN waits for the previous kernel in the stream (programmatic dependent launch),
//     stages the activations once into shared memory (applying RMSNorm or SwiGLU while it
//     does so), and then its warps walk over groups of R output rows.  So the launch
//     latency, the tail of the previous kernel and the first HBM round trip overlap
//     instead of adding up.
//   * optional SwiGLU epilogue: a warp computes gate row j and up row N/2 + j together and
//     writes bf16(silu(bf16 g) * bf16 u), so that the following down projection reads
//     activations that are already combined.
//   * a lane streams 16-byte pieces of R weight rows straight from global memory into
//     registers (ld.global.nc, no L1 allocation), U pieces per row in flight.  The kernel
//     spends ~3.5 instructions per FP8 weight, i.e. ~60 % of the issue slots at full HBM
//     rate: routing the weights through shared memory (cp.async or bulk-copy rings were
//     measured) costs more issue slots than the registers it frees are worth.
//   * FP8: activations are staged as fp32 in [iteration][quad][lane][4] order (conflict-free
//     16-byte shared loads); weights go cvt.e4m3x2 -> f16x2 -> f32, FFMA into fp32
//     accumulators, one multiply by the per-channel scale at the end.
//   * AQ4: activations are staged as block fixed point — per 32-element piece a common
//     power-of-two factor and a signed 23-bit integer per element (exact for every bf16
//     value within 2^-14 of the piece maximum, i.e. fp32-accumulate accuracy), split into
//     three byte planes.  Nibbles are isolated with two LOP3 per 8 weights and multiplied
//     with DP4A (4 MACs per instruction):  sum x*q = sum x*u - 8*sum x, all in int32; one
//     I2F and one FFMA per piece apply 2^-shift * fp16 group scale.  A piece never
//     straddles a scale group of 128.
//   * K is reduced across the lanes of one warp with shuffles.  For matrices with too few rows to give
//     every warp a row group, a row's K range is cut into S slices handled by S consecutive warps whose
//     partial sums meet in shared memory (named barrier per warp set, fixed summation order).
//   * RMSNorm takes an optional bf16 weight vector; an optional f32 residual is added to the result.
// Algorithmic bytes per launch: N*K (FP8) or N*K/2 + N*K/64 (AQ4) weight bytes
// + scales + M*K*2 in + M*N*2 out.
#pragma once
#include "internal.hpp"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstdlib>

namespace ullm {

namespace matvec_impl {

constexpr int kMaxWarps = 32;
constexpr int kMaxClusterBlocks = 16;  // largest cluster the gather is laid out for
// Kernel flavours: plain, input = sum of the ranks' slots, output = push into every rank's slot.
// kModePushInCluster: as kModePushIn, but the blocks of a thread-block cluster each sum a share of the slots and
// hand it to the others through distributed shared memory.
constexpr int kModePlain = 0, kModePushIn = 1, kModePushOut = 2, kModePushInCluster = 3;
constexpr uint32_t kFlagMatvecWait = 4u;
constexpr uint32_t AQ4 = ULLM_CUDA_ENCODING_AQ4;
constexpr uint32_t FP8 = ULLM_CUDA_ENCODING_FP8_CHANNEL;

__device__ __forceinline__ uint4 ldg_stream(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Programmatic dependent launch: let the next kernel in the stream begin its own
// prologue, and wait for the previous kernel's results to be visible.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float bf16_round_f32(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// elements one lane consumes per 16-byte weight load
template <uint32_t ENC>
struct Piece {
  static constexpr int kElems = ENC == AQ4 ? 32 : 16;
};

struct Params {
  const void *x;
  void *y;
  const uint8_t *w;
  const void *scales;
  uint32_t n, k;
  uint64_t x_stride, y_stride;
  uint32_t x_dtype, y_dtype, prologue, epilogue;
  float rms_eps;
  uint32_t k_pad;   // K rounded up to a whole warp iteration
  uint32_t vec_ok;  // activation rows allow 16-byte loads
  uint32_t tail_slices;  // > 1: the row groups left after the whole rounds are cut into this many K slices
  const void *norm_weight;  // bf16 gamma[K] of the RMSNorm prologue, or null
  const float *residual;    // f32 [M, res_stride] added to the result, or null
  uint64_t res_stride;
  PushOut po;       // tp != 0: the fp32 output goes into every rank's slot (fused all-reduce, producer half)
  PushIn pi;        // tp != 0: the input is the sum of the ranks' slots (consumer half)
  uint32_t *flags;  // device view of the context's error words
  uint32_t *abort_word;  // device-resident: non-zero once any wait of the context has given up
  uint64_t wait_ns;      // limit of a wait for a peer's data
};

// Reads N 16-byte words of {value, tag, value, tag} until every tag equals `want`.  Time-bounded: when the
// limit runs out the context is flagged, the device-resident abort word is set and whatever was read is used
// (the host reports the results as invalid).  A wait that finds the abort word already set gives up at once, so
// all the work queued behind an expired wait unwinds in about one limit.
template <int N>
__device__ __forceinline__ void poll_pairs(const Params &p, const uint4 *src, uint32_t want, uint4 (&q)[N]) {
  if (p.abort_word != nullptr && *reinterpret_cast<volatile uint32_t *>(p.abort_word) != 0u) return;
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
#pragma unroll
    for (int i = 0; i < N; ++i)
      asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(q[i].x), "=r"(q[i].y), "=r"(q[i].z), "=r"(q[i].w)
                   : "l"(src + i)
                   : "memory");
    bool ok = true;
#pragma unroll
    for (int i = 0; i < N; ++i) ok = ok && q[i].y == want && q[i].w == want;
    if (ok) return;
    if ((spin & 0x3fu) == 0x3fu) {
      uint64_t now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      const bool aborted = p.abort_word != nullptr && *reinterpret_cast<volatile uint32_t *>(p.abort_word) != 0u;
      if (aborted || now - t0 > p.wait_ns) {
        if (p.abort_word != nullptr) atomicOr(p.abort_word, 1u);
        if (p.flags != nullptr) atomicOr(p.flags, kFlagMatvecWait);
        return;
      }
    }
  }
}

// ---- thread-block cluster helpers (distributed shared memory) ----------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
// the shared::cluster address of `smem_addr` (a shared::cta address of this block) in block `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_block(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_u32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
// every thread of every block of the cluster; the stores above are visible to all blocks afterwards
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// x[m][k .. k+8) (k % 8 == 0, k + 8 <= row length) as eight packed bf16 values; fp32
// inputs are rounded to bf16 here (the op is defined on bf16 activations).
template <int MODE, bool PAIR = false>
__device__ __forceinline__ uint4 load8_packed(const Params &p, uint32_t m, uint32_t k, const uint32_t *gathered = nullptr) {
  uint32_t w[4];
  if (MODE == kModePushInCluster) {
    // the cluster has gathered the summed rows as packed bf16 [M][K] in this block's shared memory
    return *reinterpret_cast<const uint4 *>(gathered + ((uint64_t)m * p.k + k) / 2);
  } else if (MODE == kModePushIn) {
    // fused all-reduce, consumer half: sum the ranks' slots, {value, tag} pairs, in rank order (deterministic).
    // With PAIR (kernels that have the registers: 640 threads or fewer) two ranks' words are requested together,
    // so a unit costs tp/2 round trips to L2 rather than tp; a word whose tag is not there yet is polled on its own.
    const uint32_t use_global = *p.pi.step_counter * p.pi.uses_per_step + p.pi.use;
    const uint32_t want = use_global + 1u;
    const uint8_t *base = p.pi.local_base + p.pi.slot_off[use_global & 1u] + ((uint64_t)m * p.k + k) * 8;
    float v[8];
    if (p.pi.residual != nullptr) {  // residual first, then the ranks in rank order
      const float4 *rs = reinterpret_cast<const float4 *>(p.pi.residual + (uint64_t)m * p.k + k);
      const float4 a = rs[0], b = rs[1];
      v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    }
#pragma unroll
    for (uint32_t r = 0; r < (uint32_t)kMaxPeers; r += PAIR ? 2 : 1) {
      if (r < p.pi.tp) {
        const uint4 *s0 = reinterpret_cast<const uint4 *>(base + (uint64_t)r * p.pi.slot_stride);
        const bool two = PAIR && r + 1 < p.pi.tp;
        const uint4 *s1 = reinterpret_cast<const uint4 *>(base + (uint64_t)(two ? r + 1 : r) * p.pi.slot_stride);
        uint4 q0[4], q1[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(q0[i].x), "=r"(q0[i].y), "=r"(q0[i].z), "=r"(q0[i].w)
                       : "l"(s0 + i)
                       : "memory");
        if (PAIR) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(q1[i].x), "=r"(q1[i].y), "=r"(q1[i].z), "=r"(q1[i].w)
                         : "l"(s1 + i)
                         : "memory");
        }
        bool ok0 = true, ok1 = true;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          ok0 = ok0 && q0[i].y == want && q0[i].w == want;
          if (PAIR) ok1 = ok1 && q1[i].y == want && q1[i].w == want;
        }
        if (!ok0) poll_pairs<4>(p, s0, want, q0);
        if (PAIR && !ok1) poll_pairs<4>(p, s1, want, q1);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          v[2 * i] += __uint_as_float(q0[i].x);
          v[2 * i + 1] += __uint_as_float(q0[i].z);
        }
        if (two) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            v[2 * i] += __uint_as_float(q1[i].x);
            v[2 * i + 1] += __uint_as_float(q1[i].z);
          }
        }
      }
    }
    if (p.pi.reduced_out != nullptr && blockIdx.x == 0) {
      float4 *dst = reinterpret_cast<float4 *>(p.pi.reduced_out + (uint64_t)m * p.k + k);
      dst[0] = make_float4(v[0], v[1], v[2], v[3]);
      dst[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t *>(&h);
    }
  } else if (p.x_dtype == ULLM_CUDA_DTYPE_F32) {
    const float *src = static_cast<const float *>(p.x) + (uint64_t)m * p.x_stride + k;
    float v[8];
    if (p.vec_ok) {
      const float4 a = reinterpret_cast<const float4 *>(src)[0], b = reinterpret_cast<const float4 *>(src)[1];
      v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = src[i];
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t *>(&h);
    }
  } else {
    const __nv_bfloat16 *src = static_cast<const __nv_bfloat16 *>(p.x) + (uint64_t)m * p.x_stride + k;
    if (p.vec_ok) {
      const uint4 a = *reinterpret_cast<const uint4 *>(src);
      return a;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
      w[i] = (uint32_t)__bfloat16_as_ushort(src[2 * i]) | ((uint32_t)__bfloat16_as_ushort(src[2 * i + 1]) << 16);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ void unpack8(const uint4 pk, float (&v)[8]) {
  const uint32_t w[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ float sumsq8(const uint4 pk) {
  float v[8], s = 0.0f;
  unpack8(pk, v);
#pragma unroll
  for (int i = 0; i < 8; ++i) s = fmaf(v[i], v[i], s);
  return s;
}

// Final staged values of one chunk: prologue applied, bf16-representable fp32.
template <int MODE>
__device__ __forceinline__ void finish8(const Params &p, uint32_t m, uint32_t k, const uint4 pk, float inv,
                                        float (&v)[8]) {
  unpack8(pk, v);
  if (p.prologue == ULLM_CUDA_PROLOGUE_SWIGLU) {  // the row is [gate(K) | up(K)]
    if (MODE != kModePushInCluster) {             // (never combined with the cluster gather)
      float u[8];
      unpack8(load8_packed<MODE>(p, m, p.k + k), u);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = bf16_round_f32(v[i] / (1.0f + expf(-v[i])) * u[i]);
    }
  } else if (p.prologue == ULLM_CUDA_PROLOGUE_RMSNORM) {
    if (p.norm_weight != nullptr) {  // one rounding: bf16((x * inv) * gamma)
      float g[8];
      unpack8(*reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(p.norm_weight) + k), g);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = bf16_round_f32(v[i] * inv * g[i]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = bf16_round_f32(v[i] * inv);
    }
  }
}

struct Aq4Smem {
  uint32_t *planes;  // [M][iters][6][32][4]
  float *pf;         // [M][pieces]  2^-shift of the piece
  int *xsum;         // [M][pieces]  sum of the piece's integers
};

// FP8: fp32 activations in [iteration][quad][lane][4] order.  Chunk c (8 consecutive k) is half
// of lane (c/2)%32's piece: quads 2h and 2h+1.
__device__ __forceinline__ void emit_fp8(const Params &p, float *xs, uint32_t m, uint32_t c, const float (&v)[8]) {
  const uint32_t it = c >> 6, lane = (c >> 1) & 31, h = c & 1;
  float4 *dst = reinterpret_cast<float4 *>(xs) + (uint64_t)m * (p.k_pad / 4) + ((it * 4 + 2 * h) * 32 + lane);
  dst[0] = make_float4(v[0], v[1], v[2], v[3]);
  dst[32] = make_float4(v[4], v[5], v[6], v[7]);
}

// AQ4: block fixed point.  Chunk c is word j = c%4 of piece c/4; the four threads of a piece are
// adjacent lanes (every lane of the warp must call this).  Per piece 24 words ordered
// t = (j*2 + parity)*3 + plane, word (j, parity, plane) = plane bytes of elements 8j + parity + {0,2,4,6},
// stored as 6 uint4 chunks in [iteration][chunk][lane] order.
__device__ __forceinline__ void emit_aq4(const Params &p, const Aq4Smem &s, uint32_t m, uint32_t c,
                                         const float (&v)[8]) {
  const uint32_t pieces = p.k_pad / 32;
  const uint32_t pc = c >> 2, j = c & 3;
  const uint32_t it = pc >> 5, lane = pc & 31;
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  // shift so that amax * 2^shift lies in [2^21, 2^22); zero, subnormal or huge pieces clamp
  const int e = (int)((__float_as_uint(amax) >> 23) & 0xff) - 127;
  int shift = 21 - e;
  shift = shift > 126 ? 126 : (shift < -100 ? -100 : shift);
  const float up = __uint_as_float((uint32_t)(shift + 127) << 23);    // 2^shift
  const float down = __uint_as_float((uint32_t)(127 - shift) << 23);  // 2^-shift
  int xi[8], sum = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    xi[i] = __float2int_rn(v[i] * up);
    sum += xi[i];
  }
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  sum += __shfl_xor_sync(0xffffffffu, sum, 2);
  uint32_t *base = s.planes + (uint64_t)m * pieces * 24;
#pragma unroll
  for (int par = 0; par < 2; ++par)
#pragma unroll
    for (int pl = 0; pl < 3; ++pl) {
      const int sh = 8 * pl;
      const uint32_t word = ((uint32_t)(xi[par] >> sh) & 0xffu) | (((uint32_t)(xi[par + 2] >> sh) & 0xffu) << 8) |
                            (((uint32_t)(xi[par + 4] >> sh) & 0xffu) << 16) |
                            (((uint32_t)(xi[par + 6] >> sh) & 0xffu) << 24);
      const uint32_t t = (j * 2 + par) * 3 + pl;
      base[((it * 6 + (t >> 2)) * 32 + lane) * 4 + (t & 3)] = word;
    }
  if (j == 0) {
    s.pf[m * pieces + pc] = amax > 0.0f ? down : 0.0f;
    s.xsum[m * pieces + pc] = sum;
  }
}

// Cluster gather (consumer half of the fused all-reduce, one reading of the slots per cluster): block c of a
// cluster of C blocks sums, for every row, the 16-byte units [c*per, (c+1)*per) of the ranks' slots (a unit =
// two {value, tag} pairs), adds the residual, and stores the two bf16-rounded sums into the `gathered` array
// of EVERY block of the cluster through distributed shared memory, together with its share of the sum of
// squares.  After the cluster barrier every block holds all M rows as packed bf16 and the C partial sums of
// squares (added in block order, so that all blocks compute the same RMSNorm factor).  The first cluster also
// writes the fp32 sums to reduced_out.  Every thread of every block reaches the barrier whatever its waits did.
template <int M, int T>
__device__ void gather_cluster(const Params &p, uint32_t *gathered, float *ss_parts, float *red) {
  const uint32_t C = cluster_nctarank(), cr = cluster_ctarank();
  const uint32_t use_global = *p.pi.step_counter * p.pi.uses_per_step + p.pi.use;
  const uint32_t want = use_global + 1u;
  const uint8_t *base = p.pi.local_base + p.pi.slot_off[use_global & 1u];
  const uint32_t units_row = p.k / 2;
  const uint32_t per = (units_row + C - 1) / C;
  const uint32_t u0 = cr * per;
  const uint32_t u1 = u0 + per < units_row ? u0 + per : units_row;
  const bool writer = cluster_id_x() == 0 && p.pi.reduced_out != nullptr;
  const uint32_t g_addr = (uint32_t)__cvta_generic_to_shared(gathered);
  const uint32_t s_addr = (uint32_t)__cvta_generic_to_shared(ss_parts);
  float ss[M];
#pragma unroll
  for (int m = 0; m < M; ++m) ss[m] = 0.0f;
  for (uint32_t i = threadIdx.x; i < (uint32_t)M * per; i += T) {
    const uint32_t m = i / per, u = u0 + i % per;
    if (u >= u1) continue;
    const uint64_t e = (uint64_t)m * p.k + 2ull * u;  // first of the unit's two elements
    float a = 0.0f, b = 0.0f;
    if (p.pi.residual != nullptr) {
      const float2 r = *reinterpret_cast<const float2 *>(p.pi.residual + e);
      a = r.x, b = r.y;
    }
    const uint8_t *src = base + e * 8;
    uint4 q[kMaxPeers];
#pragma unroll
    for (uint32_t r = 0; r < (uint32_t)kMaxPeers; ++r)
      if (r < p.pi.tp)
        asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(q[r].x), "=r"(q[r].y), "=r"(q[r].z), "=r"(q[r].w)
                     : "l"(src + (uint64_t)r * p.pi.slot_stride)
                     : "memory");
#pragma unroll
    for (uint32_t r = 0; r < (uint32_t)kMaxPeers; ++r)
      if (r < p.pi.tp) {
        if (q[r].y != want || q[r].w != want) {
          uint4 one[1] = {q[r]};
          poll_pairs<1>(p, reinterpret_cast<const uint4 *>(src + (uint64_t)r * p.pi.slot_stride), want, one);
          q[r] = one[0];
        }
        a += __uint_as_float(q[r].x);
        b += __uint_as_float(q[r].z);
      }
    if (writer) *reinterpret_cast<float2 *>(p.pi.reduced_out + e) = make_float2(a, b);
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    const uint32_t w = *reinterpret_cast<const uint32_t *>(&h);
    const float fa = __uint_as_float(w << 16), fb = __uint_as_float(w & 0xffff0000u);
#pragma unroll
    for (int mm = 0; mm < M; ++mm)
      if ((uint32_t)mm == m) ss[mm] = fmaf(fa, fa, fmaf(fb, fb, ss[mm]));
    const uint32_t dst = g_addr + (uint32_t)(e / 2) * 4u;
    for (uint32_t c = 0; c < C; ++c) st_cluster_u32(map_to_block(dst, c), w);
  }
#pragma unroll
  for (int m = 0; m < M; ++m) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss[m] += __shfl_xor_sync(0xffffffffu, ss[m], o);
    if ((threadIdx.x & 31) == 0) red[m * kMaxWarps + (threadIdx.x >> 5)] = ss[m];
  }
  __syncthreads();
  if (threadIdx.x < (uint32_t)M) {
    float t = 0.0f;
    for (int w = 0; w < T / 32; ++w) t += red[threadIdx.x * kMaxWarps + w];
    const uint32_t dst = s_addr + (threadIdx.x * kMaxClusterBlocks + cr) * 4u;
    for (uint32_t c = 0; c < C; ++c) st_cluster_u32(map_to_block(dst, c), __float_as_uint(t));
  }
  cluster_sync_all();
}

// Stages prologue(x) for all M rows.  With RMSNorm the raw chunks are kept in registers
// (packed bf16) between the sum-of-squares pass and the scaling pass whenever they fit, so x
// is read from global memory once.
template <int M, int T, int CACHE, uint32_t ENC, int MODE>
__device__ void stage_activations(const Params &p, float *xs, const Aq4Smem &aq, float *red, uint32_t *gathered,
                                  float *ss_parts) {
  const uint32_t tid = threadIdx.x;
  const uint32_t nchunks = p.k / 8, padded = p.k_pad / 8;
  const bool rms = p.prologue == ULLM_CUDA_PROLOGUE_RMSNORM;
  constexpr bool CLUSTER = MODE == kModePushInCluster;
  const bool cached = !CLUSTER && rms && nchunks <= (uint32_t)(CACHE * T);
  uint4 cache[M][CLUSTER ? 1 : CACHE];
  float inv[M];
#pragma unroll
  for (int m = 0; m < M; ++m) inv[m] = 1.0f;
  if (CLUSTER) {
    gather_cluster<M, T>(p, gathered, ss_parts, red);
    if (rms) {
      const uint32_t C = cluster_nctarank();
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float t = 0.0f;
        for (uint32_t c = 0; c < C; ++c) t += ss_parts[m * kMaxClusterBlocks + c];
        inv[m] = 1.0f / sqrtf(t / (float)p.k + p.rms_eps);
      }
    }
  } else if (rms) {
    float ss[M];
#pragma unroll
    for (int m = 0; m < M; ++m) ss[m] = 0.0f;
    if (cached) {
#pragma unroll
      for (int i = 0; i < CACHE; ++i) {
        const uint32_t c = tid + i * T;
#pragma unroll
        for (int m = 0; m < M; ++m) {
          cache[m][i] = c < nchunks ? load8_packed<MODE, (T <= 640)>(p, m, c * 8) : make_uint4(0u, 0u, 0u, 0u);
          ss[m] += sumsq8(cache[m][i]);
        }
      }
    } else {
      for (uint32_t c = tid; c < nchunks; c += T)
#pragma unroll
        for (int m = 0; m < M; ++m) ss[m] += sumsq8(load8_packed<MODE, (T <= 640)>(p, m, c * 8));
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss[m] += __shfl_xor_sync(0xffffffffu, ss[m], o);
      if ((tid & 31) == 0) red[m * kMaxWarps + (tid >> 5)] = ss[m];
    }
    __syncthreads();
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float t = 0.0f;
#pragma unroll
      for (int w = 0; w < T / 32; ++w) t += red[m * kMaxWarps + w];
      inv[m] = 1.0f / sqrtf(t / (float)p.k + p.rms_eps);
    }
  }
  auto emit = [&](uint32_t c, int m, const uint4 pk) {
    float v[8];
    if (c < nchunks) {
      finish8<MODE>(p, m, c * 8, pk, inv[m], v);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    }
    if (ENC == AQ4)
      emit_aq4(p, aq, m, c, v);
    else
      emit_fp8(p, xs, m, c, v);
  };
  // `padded` is a multiple of 64, T a multiple of 32: the bound below is uniform per warp
  if (cached) {
#pragma unroll
    for (int i = 0; i < CACHE; ++i) {
      const uint32_t c = tid + i * T;
      if (c < padded) {
#pragma unroll
        for (int m = 0; m < M; ++m) emit(c, m, cache[m][i]);
      }
    }
  } else {
    for (uint32_t c = tid; c < padded; c += T) {
#pragma unroll
      for (int m = 0; m < M; ++m)
        emit(c, m, c < nchunks ? load8_packed<MODE, (T <= 640)>(p, m, c * 8, gathered) : make_uint4(0u, 0u, 0u, 0u));
    }
  }
  __syncthreads();
}

__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) { return __dp4a((int)a, (int)b, c); }
__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c) { return (int)__dp4a(a, b, (uint32_t)c); }

template <int MODE>
__device__ __forceinline__ void store_out(const Params &p, uint32_t m, uint32_t col, float v) {
  if (MODE == kModePushOut) {
    // fused all-reduce, producer half: {value, tag} goes into this rank's slot on every rank as one
    // 8-byte store (the tag makes the value self-announcing: no fence or flag follows)
    const uint32_t use_global = *p.po.step_counter * p.po.uses_per_step + p.po.use;
    const uint64_t off = p.po.slot_off[use_global & 1u] + (uint64_t)p.po.rank * p.po.slot_stride +
                         ((uint64_t)m * p.n + col) * 8;
#pragma unroll
    for (uint32_t r = 0; r < (uint32_t)kMaxPeers; ++r)  // static indices keep the pointer table in the parameter bank
      if (r < p.po.tp)
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p.po.peer_base[r] + off), "r"(__float_as_uint(v)),
                     "r"(use_global + 1u)
                     : "memory");
    return;
  }
  if (p.residual != nullptr) v += p.residual[(uint64_t)m * p.res_stride + col];
  if (p.y_dtype == ULLM_CUDA_DTYPE_F32)
    static_cast<float *>(p.y)[(uint64_t)m * p.y_stride + col] = v;
  else
    static_cast<__nv_bfloat16 *>(p.y)[(uint64_t)m * p.y_stride + col] = __float2bfloat16_rn(v);
}

// M activation rows, R weight rows per warp pass, U 16-byte loads per row in flight, T threads.
// With the SwiGLU epilogue (R even) a pass takes R/2 gate rows and the R/2 matching up rows.
// S > 1: the K range of a row group is cut into S slices, taken by S consecutive warps of one block.
template <int M, int R, int U, uint32_t ENC, int T, int MODE, int S = 1>
__global__ void __launch_bounds__(T, 1) matvec_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  static_assert(S == 1 || (ENC == FP8 && (T / 32) % S == 0 && (T / 32) / S <= 15), "K slices: FP8 only, one named barrier per warp set");
  // S == 1, FP8: the row groups that do not fill a whole round over all warps may be cut into K slices at run time
  constexpr bool kTail = S == 1 && ENC == FP8;
  constexpr int E = Piece<ENC>::kElems;
  constexpr int CACHE = M <= 2 ? 4 : 2;
  constexpr bool IN = MODE == kModePushIn || MODE == kModePushInCluster;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t warp = threadIdx.x >> 5;
  // a warp set (S consecutive warps) works on one row group at a time
  // set w of block b takes row groups w * gridDim.x + b, + nwarps, ...: with fewer groups than warp sets every SM
  // still streams its share (8192 rows in two-row groups fill 27 or 28 of the 32 warps of all 148 blocks, not all 32
  // warps of 128 blocks)
  const uint32_t gwarp = (warp / S) * gridDim.x + blockIdx.x;
  const uint32_t nwarps = gridDim.x * (T / 32) / S;
  const uint32_t slice = S > 1 ? warp % S : 0u;
  const bool pair = p.epilogue == ULLM_CUDA_EPILOGUE_SWIGLU;
  const uint32_t half_n = p.n / 2;
  const uint32_t groups = pair ? (half_n + R / 2 - 1) / (R / 2 > 0 ? R / 2 : 1) : (p.n + R - 1) / R;
  const uint32_t iters = p.k_pad / (E * 32);
  const uint32_t it_per = (iters + S - 1) / S;
  uint32_t slice_cur = slice, slices_cur = S;  // of the row group in hand
  uint32_t it_begin = slice * it_per;
  uint32_t it_end = it_begin + it_per < iters ? it_begin + it_per : iters;
  const uint32_t pieces = p.k_pad / 32;
  const uint64_t row_bytes = ENC == AQ4 ? p.k / 2 : p.k;
  // weight row of slot r in group g (>= n when out of range)
  auto row_of = [&](uint32_t g, int r) -> uint32_t {
    if (!pair) return g * R + r;
    const uint32_t j = g * (R / 2) + (uint32_t)(r % (R / 2 > 0 ? R / 2 : 1));
    return j < half_n ? (r < R / 2 ? j : half_n + j) : p.n;
  };

  pdl_launch_dependents();

  uint4 wv[U][R];
  // AQ4 group scales: lane l keeps the scale of group 32*block + l of each row, one block =
  // 4096 elements = 4 iterations; a piece fetches its own with one shuffle.
  constexpr int SB = ENC == AQ4 ? (U + 3) / 4 : 1;
  __half screg[SB][R];
  auto load_step = [&](uint32_t g, uint32_t it0) {
    if (ENC == AQ4 && (it0 & 3u) == 0u) {
#pragma unroll
      for (int b = 0; b < SB; ++b)
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const uint32_t row = row_of(g, r);
          const uint32_t grp = (it0 / 4 + b) * 32 + lane;
          screg[b][r] = (row < p.n && grp < p.k / 128)
                            ? static_cast<const __half *>(p.scales)[(uint64_t)row * (p.k / 128) + grp]
                            : __float2half(0.0f);
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t k0 = (it0 + u) * (E * 32) + lane * E;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const uint32_t row = row_of(g, r);
        if (it0 + u < it_end && k0 < p.k && row < p.n)
          wv[u][r] = ldg_stream(p.w + (uint64_t)row * row_bytes + (ENC == AQ4 ? k0 / 2 : k0));
        else
          wv[u][r] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };
  // Weights do not depend on the previous kernel: start streaming before waiting for it.
  // Registers take the first step; the rest of the first group (up to 8 KiB per warp) is
  // pulled into L2 so that it is there when the activations have been staged.
  if (gwarp < groups) {
    load_step(gwarp, it_begin);
    if (lane < R) {
      const uint32_t row = row_of(gwarp, (int)lane);
      const uint32_t first = it_begin * (E * 32) / (ENC == AQ4 ? 2 : 1);  // byte offset of this warp's slice
      uint32_t bytes = (uint32_t)row_bytes > first ? (uint32_t)row_bytes - first : 0u;
      const uint32_t cap = (8192u / R) & ~15u;
      bytes = bytes < cap ? bytes : cap;
      if (S > 1) bytes = bytes < it_per * E * 32 ? bytes : it_per * E * 32;
      bytes &= ~15u;
      if (row < p.n && bytes >= 16)
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.w + (uint64_t)row * row_bytes + first), "r"(bytes)
                     : "memory");
    }
  }
  pdl_wait();

  float *xs = nullptr;
  Aq4Smem aq{};
  float *red;
  if (ENC == AQ4) {
    aq.planes = reinterpret_cast<uint32_t *>(smem_raw);
    aq.pf = reinterpret_cast<float *>(aq.planes + (uint64_t)M * pieces * 24);
    aq.xsum = reinterpret_cast<int *>(aq.pf + (uint64_t)M * pieces);
    red = reinterpret_cast<float *>(aq.xsum + (uint64_t)M * pieces);
  } else {
    xs = reinterpret_cast<float *>(smem_raw);
    red = xs + (uint64_t)M * p.k_pad;
  }
  // after the block-reduction words: partial sums of the K slices, then the cluster gather's arrays
  float *slice_part = red + M * kMaxWarps;                                  // [2][T/32][R*M] when S > 1
  float *ss_parts = slice_part + (S > 1 || kTail ? 2 * (T / 32) * R * M : 0);  // [M][kMaxClusterBlocks]
  uint32_t *gathered = reinterpret_cast<uint32_t *>(ss_parts + M * kMaxClusterBlocks);  // packed bf16 [M][K], 16-byte aligned
  (void)IN;
  stage_activations<M, T, CACHE, ENC, MODE>(p, xs, aq, red, gathered, ss_parts);

  bool prefetched = true;
  uint32_t parity = 0;
  // Whole rounds: one row group per warp (set) and round.  What is left over (fewer groups than warps) would
  // keep a few warps streaming whole rows while the others idle; with tail_slices > 1 each left-over group is
  // taken by that many consecutive warps, spread over all blocks, each with a slice of K.
  const uint32_t tail = kTail ? p.tail_slices : 1u;
  const uint32_t whole = tail > 1u ? groups / nwarps * nwarps : groups;
  bool in_tail = false;
  for (uint32_t g = gwarp;; g += nwarps) {
    if (g >= whole) {
      if (!kTail || tail <= 1u || in_tail) break;
      in_tail = true;
      const uint32_t li = (warp / tail) * gridDim.x + blockIdx.x;
      if (li >= groups - whole) break;  // the same answer in every warp of a set
      g = whole + li;
      slices_cur = tail;
      slice_cur = warp % tail;
      const uint32_t per = (iters + tail - 1) / tail;
      it_begin = slice_cur * per;
      it_end = it_begin + per < iters ? it_begin + per : iters;
      if (it_begin > it_end) it_begin = it_end;
    }
    float acc[R][M];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < M; ++m) acc[r][m] = 0.0f;

    for (uint32_t it0 = it_begin; it0 < it_end; it0 += U) {
      if (!prefetched) load_step(g, it0);
      prefetched = false;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (it0 + u >= it_end) break;
        const uint32_t it = it0 + u;
        if (ENC == FP8) {
          const float4 *xb = reinterpret_cast<const float4 *>(xs) + (it * 4) * 32 + lane;
          const uint32_t xrow4 = p.k_pad / 4;
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
          // one piece = 32 weights of one scale group; integer dot products per byte plane
          int s0[R][M], s1[R][M], s2[R][M];
#pragma unroll
          for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < M; ++m) s0[r][m] = s1[r][m] = s2[r][m] = 0;
          const uint32_t pc = it * 32 + lane;
          // 24 words per activation row: word t = (j*2 + parity)*3 + plane
          uint32_t xw[M][24];
#pragma unroll
          for (int m = 0; m < M; ++m)
#pragma unroll
            for (int c = 0; c < 6; ++c) {
              const uint4 v4 =
                  reinterpret_cast<const uint4 *>(aq.planes + (uint64_t)m * pieces * 24)[(it * 6 + c) * 32 + lane];
              xw[m][4 * c] = v4.x, xw[m][4 * c + 1] = v4.y, xw[m][4 * c + 2] = v4.z, xw[m][4 * c + 3] = v4.w;
            }
#pragma unroll
          for (int jp = 0; jp < 8; ++jp) {
            const int j = jp >> 1, par = jp & 1;
#pragma unroll
            for (int r = 0; r < R; ++r) {
              const uint32_t word = j == 0 ? wv[u][r].x : j == 1 ? wv[u][r].y : j == 2 ? wv[u][r].z : wv[u][r].w;
              const uint32_t nib = (par == 0 ? word : (word >> 4)) & 0x0f0f0f0fu;
#pragma unroll
              for (int m = 0; m < M; ++m) {
                s0[r][m] = dp4a_uu(xw[m][jp * 3], nib, s0[r][m]);
                s1[r][m] = dp4a_uu(xw[m][jp * 3 + 1], nib, s1[r][m]);
                s2[r][m] = dp4a_ss(xw[m][jp * 3 + 2], nib, s2[r][m]);
              }
            }
          }
          float pfm[M];
          int xsm[M];
#pragma unroll
          for (int m = 0; m < M; ++m) {
            pfm[m] = aq.pf[m * pieces + pc];
            xsm[m] = aq.xsum[m * pieces + pc];
          }
          const int sb = U >= 4 ? u / 4 : 0;
          const int src_lane = (int)((it & 3u) * 8u + (lane >> 2));  // group of this piece within the block
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const float sc = __shfl_sync(0xffffffffu, __half2float(screg[sb][r]), src_lane);
#pragma unroll
            for (int m = 0; m < M; ++m) {
              // sum x*(u-8) as an integer (|.| < 2^30); wrap-around in the partial terms cancels
              const int d = (int)(((uint32_t)s2[r][m] << 16) + ((uint32_t)s1[r][m] << 8) + (uint32_t)s0[r][m] -
                                  ((uint32_t)xsm[m] << 3));
              acc[r][m] = fmaf((float)d, sc * pfm[m], acc[r][m]);
            }
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
    if (S > 1 || (kTail && slices_cur > 1u)) {
      // the slices of this row group meet in shared memory; slice 0 adds them in slice order.  The buffers
      // alternate, so a warp that runs ahead writes the other buffer and then stops at the next barrier.
      float *mine = slice_part + ((uint64_t)parity * (T / 32) + warp) * (R * M);
      if (lane == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
          for (int m = 0; m < M; ++m) mine[r * M + m] = acc[r][m];
      }
      asm volatile("bar.sync %0, %1;" ::"r"(1u + warp / slices_cur), "r"(slices_cur * 32u) : "memory");
      if (slice_cur == 0 && lane == 0) {
        for (uint32_t sl = 1; sl < slices_cur; ++sl)
#pragma unroll
          for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < M; ++m) acc[r][m] += mine[sl * (R * M) + r * M + m];
      }
      parity ^= 1u;
    }
    if (lane == 0 && slice_cur == 0) {
      if (ENC == FP8) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const uint32_t row = row_of(g, r);
          const float sc = row < p.n ? static_cast<const float *>(p.scales)[row] : 0.0f;
#pragma unroll
          for (int m = 0; m < M; ++m) acc[r][m] *= sc;
        }
      }
      if (pair) {
        if constexpr (R >= 2) {
#pragma unroll
          for (int r = 0; r < R / 2; ++r) {
            const uint32_t j = g * (R / 2) + r;
            if (j < half_n) {
#pragma unroll
              for (int m = 0; m < M; ++m) {
                const float gt = bf16_round_f32(acc[r][m]), up = bf16_round_f32(acc[r + R / 2][m]);
                store_out<MODE>(p, m, j, gt / (1.0f + expf(-gt)) * up);
              }
            }
          }
        }
      } else {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const uint32_t row = g * R + r;
          if (row < p.n) {
#pragma unroll
            for (int m = 0; m < M; ++m) store_out<MODE>(p, m, row, acc[r][m]);
          }
        }
      }
    }
  }
}

// Shared memory of one block: staged activations, block-reduction words, K-slice partials (`slice_floats`)
// and, for the cluster gather, the partial sums of squares and the gathered bf16 rows.
inline size_t smem_bytes(uint32_t m, uint32_t k_pad, uint32_t enc, uint32_t k = 0, bool cluster = false,
                         size_t slice_floats = 0) {
  size_t bytes = (size_t)m * kMaxWarps * 4 + slice_floats * 4;
  if (enc == AQ4)
    bytes += (size_t)m * (k_pad / 32) * (24 * 4 + 4 + 4);
  else
    bytes += (size_t)m * k_pad * 4;
  if (cluster) bytes += (size_t)m * kMaxClusterBlocks * 4 + (size_t)m * k * 2;
  return bytes;
}

constexpr size_t kSmemBudget = 224u * 1024u;  // of the 227 KiB a CTA may opt into

inline uint32_t pad_k(uint32_t k, uint32_t enc) {
  const uint32_t it = enc == AQ4 ? 1024u : 512u;
  return (k + it - 1) / it * it;
}

// Blocks per cluster for the cluster gather on this device: the largest of 8, 4, 2 whose co-resident clusters
// keep at least 80 % of the blocks the best cluster size keeps.  A larger cluster divides the gather (about 25 k
// warp instructions and 8 x 64 KiB of L2 reads per row at eight ranks, measured) among more blocks, but leaves
// SMs idle where a GPC's SM count is not a multiple of it: on B200 clusters of 8 or 4 keep 128 of 148 SMs.  The
// gather is only used where the kernels are far from bandwidth-bound (tensor-parallel shards), so the idle SMs
// cost less than the shared gather saves.  0 = no cluster launch possible.
template <typename Kern>
int pick_cluster(Kern kern, int sm_count, int threads, size_t smem, int *blocks_out) {
  int blocks_of[3] = {0, 0, 0};
  const int sizes[3] = {8, 4, 2};
  int most = 0;
  for (int i = 0; i < 3; ++i) {
    const int c = sizes[i];
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(sm_count / c * c));
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)c;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess) {
      (void)cudaGetLastError();
      continue;
    }
    int blocks = clusters * c;
    if (blocks > sm_count / c * c) blocks = sm_count / c * c;
    blocks_of[i] = blocks;
    if (blocks > most) most = blocks;
  }
  for (int i = 0; i < 3; ++i)
    if (blocks_of[i] > 0 && blocks_of[i] * 100 >= most * 80) {
      *blocks_out = blocks_of[i];
      return sizes[i];
    }
  *blocks_out = 0;
  return 0;
}

// K slices for the row groups left after the whole rounds (1 = none): the largest of 8, 4, 2 that divides the
// warps of a block, leaves at most 15 warp sets per block (one named barrier each) and finds a warp set for every
// left-over group.
inline uint32_t tail_slices(uint32_t groups, uint32_t warps, uint32_t warps_per_block) {
  if (warps == 0 || groups < warps) return 1u;
  const uint32_t left = groups % warps;
  if (left == 0) return 1u;
  for (uint32_t s = 8; s >= 2; s /= 2)
    if (warps_per_block % s == 0 && warps_per_block / s <= 15 && (uint64_t)left * s <= warps) return s;
  return 1u;
}

template <int M, int R, int U, uint32_t ENC, int T, int S = 1>
cudaError_t launch_one(const Context *ctx, cudaStream_t stream, const Params &p_in) {
  Params p = p_in;
  const bool want_cluster = p.pi.tp != 0 && p.pi.cluster != 0;
  constexpr size_t slice_floats = S > 1 || (S == 1 && ENC == FP8) ? (size_t)2 * (T / 32) * R * M : 0;
  const int mode = p.pi.tp != 0 ? (want_cluster ? kModePushInCluster : kModePushIn) : (p.po.tp != 0 ? kModePushOut : kModePlain);
  const size_t smem = smem_bytes(M, p.k_pad, ENC, p.k, mode == kModePushInCluster, slice_floats);
  if (mode == kModePushInCluster && (smem > kSmemBudget || p.prologue == ULLM_CUDA_PROLOGUE_SWIGLU || p.k % 8 != 0)) {
    p.pi.cluster = 0;  // the gathered rows do not fit beside the staged ones: every block gathers for itself
    return launch_one<M, R, U, ENC, T, S>(ctx, stream, p);
  }
  auto kern = mode == kModePushIn           ? matvec_kernel<M, R, U, ENC, T, kModePushIn, S>
              : mode == kModePushInCluster ? matvec_kernel<M, R, U, ENC, T, kModePushInCluster, S>
              : mode == kModePushOut       ? matvec_kernel<M, R, U, ENC, T, kModePushOut, S>
                                           : matvec_kernel<M, R, U, ENC, T, kModePlain, S>;
  // Function attributes are per device: the shared-memory limit is raised once per (device, kernel, size) and the
  // cluster shape is asked once per (device, kernel).  One block per SM by design.
  static std::mutex mu;
  static size_t granted[kMaxDevices][4] = {};
  static int cluster_size[kMaxDevices] = {}, cluster_blocks[kMaxDevices] = {};
  const int dev = ctx->device;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  int csize = 0, cblocks = 0;
  {
    std::lock_guard<std::mutex> g(mu);
    if (smem > granted[dev][mode]) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      granted[dev][mode] = smem;
      if (mode == kModePushInCluster) cluster_size[dev] = 0;  // ask again with the new size
    }
    if (mode == kModePushInCluster) {
      if (cluster_size[dev] == 0) {
        cluster_size[dev] = pick_cluster(kern, ctx->sm_count, T, smem, &cluster_blocks[dev]);
        if (cluster_size[dev] == 0) cluster_size[dev] = -1;
      }
      csize = cluster_size[dev];
      cblocks = cluster_blocks[dev];
    }
  }
  const bool pair = p.epilogue == ULLM_CUDA_EPILOGUE_SWIGLU;
  const uint32_t groups = pair ? (p.n / 2 + R / 2 - 1) / (R / 2 > 0 ? R / 2 : 1) : (p.n + R - 1) / R;
  uint32_t grid = (uint32_t)ctx->sm_count;
  if (grid > groups) grid = groups;  // at least one row group per block
  cudaLaunchConfig_t cfg{};
  cfg.blockDim = dim3(T);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (mode == kModePushInCluster) {
    if (csize < 2) {  // no cluster shape fits this device: every block gathers for itself
      p.pi.cluster = 0;
      return launch_one<M, R, U, ENC, T, S>(ctx, stream, p);
    }
    if (p.pi.cluster >= 2 && p.pi.cluster <= 8 && (p.pi.cluster & (p.pi.cluster - 1)) == 0 && (int)p.pi.cluster < csize)
      csize = (int)p.pi.cluster;  // an explicitly smaller cluster was asked for
    // whole clusters only, all of them co-resident: every block takes part in the gather whether or not it has rows
    uint32_t blocks = (uint32_t)cblocks / (uint32_t)csize * (uint32_t)csize;
    if (grid < blocks) blocks = (grid + (uint32_t)csize - 1) / (uint32_t)csize * (uint32_t)csize;
    grid = blocks;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = (unsigned)csize;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  p.tail_slices = S == 1 && ENC == FP8 ? tail_slices(groups, grid * (uint32_t)(T / 32), T / 32) : 1u;
  cfg.gridDim = dim3(grid);
  return cudaLaunchKernelEx(&cfg, kern, p);
}

// Share of the last round of row groups that is filled: 1.0 = every warp gets the same work.
inline double balance(uint32_t units, uint32_t warps, uint32_t warps_per_block = 0) {
  const uint32_t rounds = (units + warps - 1) / warps;
  if (rounds == 0) return 0.0;
  double cost = (double)rounds;
  if (warps_per_block != 0) {  // the last round may be cut into K slices
    const uint32_t s = tail_slices(units, warps, warps_per_block);
    if (s > 1) cost = (double)(units / warps) + 1.0 / s;
  }
  return (double)units / (cost * warps);
}

#ifdef ULLM_CUDA_TUNING
// Tuning builds only (-DULLM_CUDA_TUNING): ULLM_CUDA_MATVEC_VARIANT=<n> forces variant n of the M == 1
// table below (read once).  The shipped library reads no environment variable.
inline int forced_variant() {
  static const int v = [] {
    const char *e = std::getenv("ULLM_CUDA_MATVEC_VARIANT");
    return e ? std::atoi(e) : -1;
  }();
  return v;
}
#else
inline int forced_variant() { return -1; }
#endif

template <uint32_t ENC>
cudaError_t launch_m1(const Context *ctx, cudaStream_t stream, const Params &p) {
  const bool pair = p.epilogue == ULLM_CUDA_EPILOGUE_SWIGLU;
  const uint32_t rows = pair ? p.n / 2 : p.n;
  int v = forced_variant();
  if (v < 0) {
    // Measured on B200 (HBM GB/s over 7 decode shapes and a whole stack): the two best
    // configurations are 4 rows x 2 loads on 640 threads and 2 rows x 4 loads on 1024 threads;
    // which one wins on a shape follows from how evenly the row groups divide among the warps.
    const uint32_t tb = ENC == FP8 ? 1u : 0u;  // FP8 cuts the last round into K slices
    const double b4 = balance(pair ? (rows + 1) / 2 : (rows + 3) / 4, (uint32_t)ctx->sm_count * 20u, 20u * tb);
    const double b2 = balance(pair ? rows : (rows + 1) / 2, (uint32_t)ctx->sm_count * 32u, 32u * tb);
    const double b1 = pair ? 0.0 : balance(rows, (uint32_t)ctx->sm_count * 32u, 32u * tb);
    v = b2 >= b4 ? 8 : 9;
    if (b1 > (b2 > b4 ? b2 : b4) + 0.25) v = 4;  // few, long rows: one row per pass
    if (ENC == FP8 && !pair && p.k >= 2048u) {
      // Too few rows for one round of two-row groups over all warps (tensor-parallel shards): cut K four ways,
      // so four times as many warps stream the weights.  One row per warp set when even that leaves warps idle.
      const uint32_t warps = (uint32_t)ctx->sm_count * 32u;
      const uint32_t units2 = (rows + 1) / 2;
      if ((uint64_t)units2 * 10u < (uint64_t)warps * 7u) v = (uint64_t)units2 * 4u * 10u < (uint64_t)warps * 7u ? 14 : 18;
    }
    if (ENC == AQ4) {
      // AQ4 holds more state per row (three integer accumulators): 1024 threads would spill.
      // Measured best: 4 rows x 2 loads (768 threads) for very tall matrices, else 2 rows x 4 loads.
      v = rows >= 65536u ? 0 : (p.k >= 8192u ? 11 : 2);
    }
  }
  if (ENC == AQ4 && v != 0 && v != 2 && v != 11) v = 2;  // an unknown forced index falls back to a valid one
  if (ENC == FP8 && v != 4 && v != 8 && v != 9 && v != 14 && v != 18) v = 8;
  if (pair && (v == 4 || v == 14 || v == 18)) v = 8;  // the SwiGLU epilogue needs an even number of rows per pass
  if constexpr (ENC == FP8) {
    switch (v) {
      case 4: return launch_one<1, 1, 4, ENC, 1024>(ctx, stream, p);
      case 8: return launch_one<1, 2, 4, ENC, 1024>(ctx, stream, p);
      case 9: return launch_one<1, 4, 2, ENC, 640>(ctx, stream, p);
      case 14: return launch_one<1, 1, 4, ENC, 1024, 4>(ctx, stream, p);
      case 18: return launch_one<1, 2, 4, ENC, 1024, 4>(ctx, stream, p);
      default: return cudaErrorInvalidValue;
    }
  } else {
    switch (v) {
      case 0: return launch_one<1, 4, 2, ENC, 768>(ctx, stream, p);
      case 2: return launch_one<1, 2, 4, ENC, 768>(ctx, stream, p);
      case 11: return launch_one<1, 2, 4, ENC, 512>(ctx, stream, p);
      default: return cudaErrorInvalidValue;
    }
  }
}

template <int M, uint32_t ENC>
cudaError_t launch_m(const Context *ctx, cudaStream_t stream, const Params &p) {
  if constexpr (M == 1) {
    return launch_m1<ENC>(ctx, stream, p);
  } else {
    // 512 threads, up to 128 registers each
    constexpr int T = 512;
    const bool pair = p.epilogue == ULLM_CUDA_EPILOGUE_SWIGLU;
    const uint32_t rows = pair ? p.n / 2 : p.n;
    const uint32_t warps = (uint32_t)ctx->sm_count * (T / 32);
    const uint32_t tb = ENC == FP8 ? (uint32_t)(T / 32) : 0u;
    const double b2 = balance(pair ? rows : (rows + 1) / 2, warps, tb);
    const double b1 = pair ? 0.0 : balance(rows, warps, tb);
    if (b2 >= b1 - 0.05) return launch_one<M, 2, 2, ENC, T>(ctx, stream, p);
    return launch_one<M, 1, 4, ENC, T>(ctx, stream, p);
  }
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

}  // namespace matvec_impl

// One translation unit per encoding (matvec_fp8.cu, matvec_aq4.cu) instantiates these.
struct MatvecLaunch {
  matvec_impl::Params p;
  uint32_t m;
};
cudaError_t launch_matvec_fp8(const Context *ctx, cudaStream_t stream, const MatvecLaunch &l);
cudaError_t launch_matvec_aq4(const Context *ctx, cudaStream_t stream, const MatvecLaunch &l);

}  // namespace ullm
