// Prefill / batched-decode GEMM: y[M,N] = prologue(x)[M,K] . W'[N,K]^T with the AQ4 / FP8
// dequantisation fused into the main loop, on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory).
//
// The reference has no GEMM (hipBLASLt appears only as a planned dependency,
// docs/compatibility/amd-gpu.md:96-102); this is the tensor-core half of the quantised
// linear op selected by shape (docs/architecture/runtime.md:83-91).
//
// Orientation ("swap AB"): the WEIGHT rows are the 128-row M side of the MMA and the TOKENS
// are its N side (tile of TT <= 256 tokens).  Consequences:
//   * a weight element is dequantised once per (128 rows x TT tokens) tile, i.e. M/TT times;
//   * the per-output-channel (FP8) or per-group (AQ4) scale is a per-LANE scalar of the
//     accumulator, so the epilogue thread that owns lane n applies it without any lookup;
//   * small token counts (batched decode) simply use a narrow N.
// One CTA per SM computes one 128 x TT tile; warp roles:
//   warp 0      TMA: activation tiles [TT x 64] bf16, 128-byte swizzle, completion on an mbarrier
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (kind::f16, bf16 x bf16 -> f32)
//   warps 2-9   weight producers: two threads per row n0 + r stream it from global memory (16-byte
//               loads, four to eight k-tiles ahead), convert to EXACT bf16 (e4m3 -> bf16; 4-bit q -> bf16
//               integer) and write the K-major, 128-byte-swizzled A tile the MMA reads
//   warps 10-17 epilogue: tcgen05.ld, scale, convert, store
// FP8: all of K accumulates in one tensor-memory buffer; scale[n] is applied once at the end.
// AQ4: products of bf16 activations with integers -7..7 are exact, so a 128-deep group is
// accumulated unscaled, drained, and added into fp32 registers as scale[n,g] * partial; two
// accumulator buffers ping-pong so that draining overlaps the next group's MMAs.
// Every mbarrier wait is bounded in time; on expiry the kernel flags the context and unwinds
// (tensor memory is always released).
#include "internal.hpp"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace ullm {

namespace {

constexpr uint32_t AQ4 = ULLM_CUDA_ENCODING_AQ4;
constexpr uint32_t FP8 = ULLM_CUDA_ENCODING_FP8_CHANNEL;
constexpr int BM = 128;  // weight rows per tile (MMA M)
constexpr int BK = 64;   // k per stage: 64 bf16 = one 128-byte swizzle row
constexpr int kProducerWarps = 8;
constexpr int kProducerWarp0 = 2, kEpilogueWarp0 = kProducerWarp0 + kProducerWarps;
constexpr int kThreads = (kEpilogueWarp0 + 8) * 32;
constexpr uint32_t kFlagGemmWait = 2u;
constexpr uint64_t kWaitLimitNs = 20ull * 1000ull * 1000ull * 1000ull;

struct GemmParams {
  const uint8_t *w;
  const void *scales;
  void *y;
  uint32_t m, n, k;
  uint64_t y_stride;
  uint32_t y_dtype;
  uint32_t stages;
  uint32_t *flags;
};

// ---- PTX wrappers ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: false = the CTA gives up (this thread timed out, or another one did).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                          uint32_t *device_flags) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 0x3fu) == 0u) {
      if (*abort_flag != 0u) return false;
      if (global_timer_ns() - t0 > kWaitLimitNs) {
        *abort_flag = 1u;
        if (device_flags != nullptr) atomicOr(device_flags, kFlagGemmWait);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// arrives on the mbarrier once every MMA issued so far by this thread has completed
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread l of the warp receives lane (quarter*32 + l)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint4 ldg_stream(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// K-major, 128-byte-swizzled operand tile (rows of 64 bf16, 8-row groups 1024 bytes apart):
// start address >> 4, leading byte offset 1 (unused with a swizzle), stride byte offset 1024 >> 4,
// descriptor version 1 (Blackwell), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  const uint32_t lo = ((smem_addr >> 4) & 0x3fffu) | (1u << 16);
  const uint32_t hi = 64u | (1u << 14) | (2u << 29);
  return ((uint64_t)hi << 32) | lo;
}

// instruction descriptor: D = f32, A = B = bf16, both K-major, M = 128, N = tt
__host__ __device__ constexpr uint32_t instr_desc_bf16(int tt) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(tt >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// ---- weight conversion to exact bf16 ----------------------------------------------------------
// four e4m3 codes (one word) -> two words of two bf16 each
__device__ __forceinline__ void fp8x4_to_bf16x4(uint32_t w, uint32_t &lo, uint32_t &hi) {
  const float2 f01 = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w & 0xffffu), __NV_E4M3)));
  const float2 f23 = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w >> 16), __NV_E4M3)));
  // an e4m3 value has 4 significant bits: the upper half of its fp32 pattern is its exact bf16
  lo = __byte_perm(__float_as_uint(f01.x), __float_as_uint(f01.y), 0x7632);
  hi = __byte_perm(__float_as_uint(f23.x), __float_as_uint(f23.y), 0x7632);
}
// eight nibbles (one word, element 2i in the low nibble of byte i) -> four words of two bf16 integers q = u - 8
__device__ __forceinline__ void aq4x8_to_bf16x8(uint32_t w, uint32_t (&out)[4]) {
  const __nv_bfloat162 bias = __floats2bfloat162_rn(136.0f, 136.0f);
  const uint32_t lo = w & 0x0f0f0f0fu;         // u of elements 0,2,4,6, one per byte
  const uint32_t hi = (w >> 4) & 0x0f0f0f0fu;  // u of elements 1,3,5,7
  const uint32_t t03 = __byte_perm(lo, hi, 0x5140);  // bytes u0,u1,u2,u3
  const uint32_t t47 = __byte_perm(lo, hi, 0x7362);  // bytes u4,u5,u6,u7
  // 0x4300 | u is the bf16 number 128 + u (exact for u < 128): widen each byte with a 0x43 high byte
  uint32_t v[4];
  v[0] = __byte_perm(t03, 0x43434343u, 0x4140);
  v[1] = __byte_perm(t03, 0x43434343u, 0x4342);
  v[2] = __byte_perm(t47, 0x43434343u, 0x4140);
  v[3] = __byte_perm(t47, 0x43434343u, 0x4342);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 q = __hsub2(*reinterpret_cast<const __nv_bfloat162 *>(&v[i]), bias);
    out[i] = *reinterpret_cast<const uint32_t *>(&q);
  }
}

template <uint32_t ENC, int TT>
__global__ void __launch_bounds__(kThreads, 1) gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
  extern __shared__ uint8_t smem_dyn[];
  constexpr uint32_t A_BYTES = BM * BK * 2;           // 16 KiB
  constexpr uint32_t B_BYTES = (uint32_t)TT * BK * 2;  // TT x 128 B
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t RAW16 = ENC == AQ4 ? 1 : 2;  // 16-byte loads of half a row per k-tile
  constexpr int ACC_BUFS = ENC == AQ4 ? 2 : 1;
  constexpr uint32_t TMEM_COLS = (uint32_t)(TT * ACC_BUFS) < 32u ? 32u : (uint32_t)(TT * ACC_BUFS);
  constexpr int MAX_STAGES = 8;
  __shared__ __align__(8) uint64_t bars[3 * MAX_STAGES + 4];
  __shared__ uint32_t tmem_base_slot;
  __shared__ uint32_t abort_flag;

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t n0 = blockIdx.x * BM, m0 = blockIdx.y * TT;
  const uint32_t NS = p.stages;
  const uint32_t ktiles = p.k / BK;
  // tiles must start on a 1024-byte boundary for the 128-byte swizzle
  const uint32_t smem0 = ((uint32_t)__cvta_generic_to_shared(smem_dyn) + 1023u) & ~1023u;
  const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(bars);
  auto full_a = [&](uint32_t s) { return bar0 + s * 8u; };
  auto full_b = [&](uint32_t s) { return bar0 + (MAX_STAGES + s) * 8u; };
  auto empty = [&](uint32_t s) { return bar0 + (2 * MAX_STAGES + s) * 8u; };
  auto acc_full = [&](uint32_t b) { return bar0 + (3 * MAX_STAGES + b) * 8u; };
  auto acc_empty = [&](uint32_t b) { return bar0 + (3 * MAX_STAGES + 2 + b) * 8u; };

  if (threadIdx.x == 0) {
    abort_flag = 0u;
    for (uint32_t s = 0; s < NS; ++s) {
      mbar_init(full_a(s), (uint32_t)kProducerWarps);  // one arrival per producer warp
      mbar_init(full_b(s), 1u);  // the TMA thread's expect_tx
      mbar_init(empty(s), 1u);   // tcgen05.commit
    }
    for (uint32_t b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1u);   // tcgen05.commit
      mbar_init(acc_empty(b), 8u);  // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc((uint32_t)__cvta_generic_to_shared(&tmem_base_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ---- TMA: activation tiles --------------------------------------------------------
    if (lane == 0) {
      uint32_t slot = 0, round = 0;
      for (uint32_t kt = 0; kt < ktiles; ++kt) {
        if (round > 0 && !mbar_wait(empty(slot), (round - 1) & 1u, &abort_flag, p.flags)) break;
        mbar_expect_tx(full_b(slot), B_BYTES);
        tma_load_2d(smem0 + slot * STAGE_BYTES + A_BYTES, &tmap_x, (int)(kt * BK), (int)m0, full_b(slot));
        if (++slot == NS) {
          slot = 0;
          ++round;
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issue ----------------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_bf16(TT);
      uint32_t slot = 0, round = 0;
      bool ok = true;
      for (uint32_t kt = 0; kt < ktiles && ok; ++kt) {
        uint32_t acc_col = 0, first = kt == 0 ? 1u : 0u;
        if (ENC == AQ4) {
          const uint32_t g = kt >> 1, buf = g & 1u;  // two k-tiles per scale group of 128
          acc_col = buf * TT;
          first = (kt & 1u) == 0u ? 1u : 0u;
          if (first && g >= 2) ok = mbar_wait(acc_empty(buf), ((g >> 1) - 1) & 1u, &abort_flag, p.flags);
        }
        ok = ok && mbar_wait(full_a(slot), round & 1u, &abort_flag, p.flags);
        ok = ok && mbar_wait(full_b(slot), round & 1u, &abort_flag, p.flags);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem0 + slot * STAGE_BYTES, b_addr = a_addr + A_BYTES;
#pragma unroll
        for (int k4 = 0; k4 < BK / 16; ++k4) {
          // 16 bf16 along K = 32 bytes inside the swizzled row: advance the start address only
          tc_mma_bf16(tmem_base + acc_col, smem_desc_sw128(a_addr + k4 * 32), smem_desc_sw128(b_addr + k4 * 32), idesc,
                      (first && k4 == 0) ? 0u : 1u);
        }
        tc_commit(empty(slot));  // the stage may be refilled when these MMAs are done
        if (ENC == AQ4) {
          if ((kt & 1u) == 1u) tc_commit(acc_full((kt >> 1) & 1u));
        } else if (kt + 1 == ktiles) {
          tc_commit(acc_full(0));
        }
        if (++slot == NS) {
          slot = 0;
          ++round;
        }
      }
    }
  } else if (warp < kEpilogueWarp0) {
    // ---- weight producers: threads 2r and 2r+1 own the two halves of row n0 + r of the tile -----
    const uint32_t pt = threadIdx.x - kProducerWarp0 * 32;
    const uint32_t r = pt >> 1, hf = pt & 1u;
    const uint32_t row = n0 + r;
    const bool valid = row < p.n;
    const uint32_t row_bytes = ENC == AQ4 ? p.k / 2 : p.k;
    const uint8_t *src = p.w + (uint64_t)(valid ? row : 0) * row_bytes + hf * (RAW16 * 16);
    constexpr int PF = ENC == AQ4 ? 8 : 4;  // k-tiles of raw bytes kept in registers ahead of the one being converted
    uint4 raw[PF][RAW16];
    auto fetch = [&](uint32_t kt, int j) {
#pragma unroll
      for (uint32_t i = 0; i < RAW16; ++i)
        raw[j][i] = (valid && kt < ktiles) ? ldg_stream(src + (uint64_t)kt * (2 * RAW16 * 16) + i * 16) : make_uint4(0, 0, 0, 0);
    };
#pragma unroll
    for (int j = 0; j < PF; ++j) fetch((uint32_t)j, j);
    uint32_t slot = 0, round = 0;
    for (uint32_t kt = 0; kt < ktiles; kt += PF) {
#pragma unroll
      for (int j = 0; j < PF; ++j) {
        if (kt + j >= ktiles) break;
        if (round > 0 && !mbar_wait(empty(slot), (round - 1) & 1u, &abort_flag, p.flags)) goto done;
        const uint32_t a_row = smem0 + slot * STAGE_BYTES + r * 128u;
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // chunk c = k 8c..8c+7 of this k-tile; this thread owns c = 4*hf + i
          const uint32_t c = 4u * hf + (uint32_t)i;
          uint32_t o[4];
          if (ENC == FP8) {  // 8 raw bytes = 2 words
            const uint4 q = raw[j][i >> 1];
            const uint32_t w0 = (i & 1) ? q.z : q.x, w1 = (i & 1) ? q.w : q.y;
            fp8x4_to_bf16x4(w0, o[0], o[1]);
            fp8x4_to_bf16x4(w1, o[2], o[3]);
          } else {  // 8 nibbles = 1 word
            const uint4 q = raw[j][0];
            const uint32_t w = i == 0 ? q.x : i == 1 ? q.y : i == 2 ? q.z : q.w;
            aq4x8_to_bf16x8(w, o);
          }
          asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a_row + ((c ^ (r & 7u)) << 4)), "r"(o[0]),
                       "r"(o[1]), "r"(o[2]), "r"(o[3])
                       : "memory");
        }
        fetch(kt + j + PF, j);  // refill the register slot just consumed
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the MMA
        __syncwarp();
        if (lane == 0) mbar_arrive(full_a(slot));
        if (++slot == NS) {
          slot = 0;
          ++round;
        }
      }
    }
  } else {
    // ---- epilogue: warp e covers TMEM lanes 32*(warp % 4) .. +31 and half of the token columns ----
    const uint32_t e = warp - kEpilogueWarp0;
    const uint32_t quarter = warp & 3u, half = e >> 2;
    constexpr int COLS = TT / 2 < 32 ? 32 : TT / 2;  // token columns of this warp (tcgen05.ld moves 32 at a time)
    const uint32_t row = n0 + quarter * 32 + lane;
    const uint32_t col0 = half * COLS;
    const bool active = col0 < (uint32_t)TT;  // TT == 32: the second half has nothing to do
    const uint32_t lane_addr = tmem_base + ((quarter * 32u) << 16);
    auto store_chunk = [&](uint32_t c, const float (&v)[32]) {
      // thread = output channel `row`; 32 lanes write 32 consecutive channels of one token
      if (row >= p.n) return;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const uint32_t tok = m0 + c + i;
        if (tok < p.m) {
          if (p.y_dtype == ULLM_CUDA_DTYPE_F32)
            static_cast<float *>(p.y)[(uint64_t)tok * p.y_stride + row] = v[i];
          else
            static_cast<__nv_bfloat16 *>(p.y)[(uint64_t)tok * p.y_stride + row] = __float2bfloat16_rn(v[i]);
        }
      }
    };
    if (ENC == FP8) {
      if (active && mbar_wait(acc_full(0), 0u, &abort_flag, p.flags)) {
        tc_fence_after();
        const float sc = row < p.n ? static_cast<const float *>(p.scales)[row] : 0.0f;
#pragma unroll 1
        for (int c = 0; c < COLS; c += 32) {
          uint32_t v[32];
          tmem_ld32(lane_addr + col0 + c, v);
          tmem_ld_wait();
          float f[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]) * sc;
          store_chunk(col0 + c, f);
        }
      }
    } else {
      float acc[COLS];
#pragma unroll
      for (int i = 0; i < COLS; ++i) acc[i] = 0.0f;
      const uint32_t groups = p.k / 128;
      const __half *srow = static_cast<const __half *>(p.scales) + (uint64_t)(row < p.n ? row : 0) * groups;
      float sc_next = row < p.n ? __half2float(srow[0]) : 0.0f;
      bool ok = true;
      for (uint32_t g = 0; g < groups && ok; ++g) {
        const uint32_t buf = g & 1u;
        const float sc = sc_next;
        if (g + 1 < groups && row < p.n) sc_next = __half2float(srow[g + 1]);
        ok = mbar_wait(acc_full(buf), (g >> 1) & 1u, &abort_flag, p.flags);
        if (!ok) break;
        tc_fence_after();
        if (active) {
#pragma unroll
          for (int c = 0; c < COLS; c += 32) {
            uint32_t v[32];
            tmem_ld32(lane_addr + buf * TT + col0 + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[c + i] = fmaf(sc, __uint_as_float(v[i]), acc[c + i]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty(buf));  // this buffer may take the group after next
      }
      if (ok && active) {
#pragma unroll
        for (int c = 0; c < COLS; c += 32) {
          float f[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = acc[c + i];
          store_chunk(col0 + c, f);
        }
      }
    }
  }
done:
  tc_fence_before();
  __syncthreads();
  if (abort_flag != 0u) {
    // a wait gave up: let copies that may still be in flight land before shared memory is released
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- elementwise helpers around the GEMM ------------------------------------------------------

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// out[m][k] = bf16( prologue(x)[m][k] ), one block per row
__global__ void prologue_kernel(const void *x, uint32_t x_dtype, uint64_t x_stride, uint32_t k, uint32_t prologue,
                                float eps, __nv_bfloat16 *out) {
  __shared__ float red[32];
  const uint32_t m = blockIdx.x;
  auto ld = [&](uint32_t i) -> float {
    return x_dtype == ULLM_CUDA_DTYPE_F32 ? bf16r(static_cast<const float *>(x)[(uint64_t)m * x_stride + i])
                                          : __bfloat162float(static_cast<const __nv_bfloat16 *>(x)[(uint64_t)m * x_stride + i]);
  };
  float inv = 1.0f;
  if (prologue == ULLM_CUDA_PROLOGUE_RMSNORM) {
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) {
      const float v = ld(i);
      ss = fmaf(v, v, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float t = 0.0f;
    for (uint32_t w = 0; w < blockDim.x / 32; ++w) t += red[w];
    inv = 1.0f / sqrtf(t / (float)k + eps);
  }
  for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) {
    float v = ld(i);
    if (prologue == ULLM_CUDA_PROLOGUE_SWIGLU) {
      const float u = ld(k + i);
      v = v / (1.0f + expf(-v)) * u;
    } else if (prologue == ULLM_CUDA_PROLOGUE_RMSNORM) {
      v = v * inv;
    }
    out[(uint64_t)m * k + i] = __float2bfloat16_rn(v);
  }
}

// y[m][j] = bf16( silu(g[m][j]) * g[m][f + j] ) for a bf16 [M, 2F] gate|up matrix
__global__ void swiglu_kernel(const __nv_bfloat16 *gu, uint32_t f, __nv_bfloat16 *y, uint64_t y_stride) {
  const uint32_t m = blockIdx.y;
  for (uint32_t j = blockIdx.x * blockDim.x + threadIdx.x; j < f; j += gridDim.x * blockDim.x) {
    const float g = __bfloat162float(gu[(uint64_t)m * 2 * f + j]), u = __bfloat162float(gu[(uint64_t)m * 2 * f + f + j]);
    y[(uint64_t)m * y_stride + j] = __float2bfloat16_rn(g / (1.0f + expf(-g)) * u);
  }
}

// ---- host side --------------------------------------------------------------------------------

using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
  static EncodeTiled fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiled>(p);
  }();
  return fn;
}

// bf16 activations [m][k] with a row pitch: box = 64 (k) x tt (rows), 128-byte swizzle, zero fill outside
bool make_x_map(CUtensorMap *map, const void *x, uint32_t m, uint32_t k, uint64_t stride_elems, uint32_t tt) {
  EncodeTiled enc = encode_tiled();
  if (enc == nullptr) return false;
  const cuuint64_t dims[2] = {k, m};
  const cuuint64_t strides[1] = {stride_elems * 2};
  const cuuint32_t box[2] = {BK, tt};
  const cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(x), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <uint32_t ENC, int TT>
cudaError_t launch_tile(cudaStream_t stream, const CUtensorMap &map, GemmParams p) {
  constexpr size_t stage = (size_t)BM * BK * 2 + (size_t)TT * BK * 2;
  size_t ns = (220u * 1024u - 1024u) / stage;
  if (ns > 8) ns = 8;
  p.stages = (uint32_t)ns;
  const size_t smem = ns * stage + 1024;
  auto kern = gemm_kernel<ENC, TT>;
  static std::mutex mu;
  static bool configured = false;
  {
    std::lock_guard<std::mutex> g(mu);
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      configured = true;
    }
  }
  dim3 grid((p.n + BM - 1) / BM, (p.m + TT - 1) / TT);
  kern<<<grid, kThreads, smem, stream>>>(map, p);
  return cudaGetLastError();
}

int tile_tokens(uint32_t m, uint32_t enc) {
  const int cap = enc == AQ4 ? 128 : 256;  // AQ4 keeps TT/2 accumulators per epilogue thread in registers
  int tt = 32;
  while (tt < cap && (uint32_t)tt < m) tt *= 2;
  return tt;
}

}  // namespace

bool gemm_supports(const Context *, const LinearArgs &a, const char **why) {
  if (a.k % 128 != 0) {
    *why = "the GEMM kernel needs K to be a multiple of 128";
    return false;
  }
  if (encode_tiled() == nullptr) {
    *why = "cuTensorMapEncodeTiled is not available from this driver";
    return false;
  }
  return true;
}

// Scratch owned by the context: grows on demand, reused by every GEMM on that context.
static cudaError_t ensure_scratch(const Context *cctx, size_t bytes, void **out) {
  Context *ctx = const_cast<Context *>(cctx);
  std::lock_guard<std::mutex> g(ctx->mutex);
  if (ctx->scratch_bytes < bytes) {
    if (ctx->scratch != nullptr) {
      cudaError_t e = cudaFree(ctx->scratch);
      if (e != cudaSuccess) return e;
      ctx->scratch = nullptr;
      ctx->scratch_bytes = 0;
    }
    cudaError_t e = cudaMalloc(&ctx->scratch, bytes);
    if (e != cudaSuccess) return e;
    ctx->scratch_bytes = bytes;
  }
  *out = ctx->scratch;
  return cudaSuccess;
}

cudaError_t gemm_reserve_scratch(const Context *ctx, size_t bytes) {
  void *unused = nullptr;
  return bytes == 0 ? cudaSuccess : ensure_scratch(ctx, bytes, &unused);
}

size_t gemm_scratch_bytes(const LinearArgs &a) {
  size_t bytes = 0;
  const bool needs_x = a.prologue != ULLM_CUDA_PROLOGUE_NONE || a.x_dtype != ULLM_CUDA_DTYPE_BF16 ||
                       reinterpret_cast<uintptr_t>(a.x) % 16 != 0 || (a.x_stride * 2) % 16 != 0;
  if (needs_x) bytes += ((size_t)a.m * a.k * 2 + 255) & ~size_t(255);
  if (a.epilogue == ULLM_CUDA_EPILOGUE_SWIGLU) bytes += (size_t)a.m * a.n * 2;
  return bytes;
}

// ---- allocation-free variant ---------------------------------------------------------------------
// Staging area of the allocation-free entry point.  `g_static_scratch` names a host-side shadow in
// host code, never a device address: the address is looked up once per device below.
static __device__ __align__(256) uint8_t g_static_scratch[ULLM_CUDA_STATIC_SCRATCH_BYTES];

static cudaError_t static_scratch_address(int device, uint8_t **out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static uint8_t *address[kMaxDevices] = {};
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> g(mu);
  if (address[device] == nullptr) {
    // the caller has made `device` current (begin_op); the symbol resolves per device
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return e;
    address[device] = static_cast<uint8_t *>(p);
  }
  *out = address[device];
  return cudaSuccess;
}

int launch_gemm_static_scratch(const Context *ctx, cudaStream_t stream, const LinearArgs &a, cudaError_t *err) {
  *err = cudaSuccess;
  if (a.epilogue != ULLM_CUDA_EPILOGUE_NONE) return -2;
  const bool needs_x = a.prologue != ULLM_CUDA_PROLOGUE_NONE || a.x_dtype != ULLM_CUDA_DTYPE_BF16 ||
                       reinterpret_cast<uintptr_t>(a.x) % 16 != 0 || (a.x_stride * 2) % 16 != 0;
  if (needs_x && (uint64_t)a.m * a.k * 2 > ULLM_CUDA_STATIC_SCRATCH_BYTES) return -2;
  int launches = 0;
  const void *x = a.x;
  uint64_t x_stride = a.x_stride;
  if (needs_x) {
    uint8_t *scratch = nullptr;
    *err = static_scratch_address(ctx->device, &scratch);
    if (*err != cudaSuccess) return -1;
    __nv_bfloat16 *xb = reinterpret_cast<__nv_bfloat16 *>(scratch);
    prologue_kernel<<<a.m, 256, 0, stream>>>(a.x, a.x_dtype, a.x_stride, a.k, a.prologue, a.rms_eps, xb);
    *err = cudaGetLastError();
    if (*err != cudaSuccess) return -1;
    ++launches;
    x = xb;
    x_stride = a.k;
  }
  GemmParams p{};
  p.w = a.w;
  p.scales = a.scales;
  p.m = a.m;
  p.n = a.n;
  p.k = a.k;
  p.flags = ctx->device_flags;
  p.y = a.y;
  p.y_stride = a.y_stride;
  p.y_dtype = a.y_dtype;
  const int tt = tile_tokens(a.m, a.encoding);
  CUtensorMap map;
  if (!make_x_map(&map, x, a.m, a.k, x_stride, (uint32_t)tt)) {
    *err = cudaErrorInvalidValue;
    return -1;
  }
  if (a.encoding == AQ4) {
    *err = tt == 32 ? launch_tile<AQ4, 32>(stream, map, p) : tt == 64 ? launch_tile<AQ4, 64>(stream, map, p)
                                                                      : launch_tile<AQ4, 128>(stream, map, p);
  } else {
    *err = tt == 32    ? launch_tile<FP8, 32>(stream, map, p)
           : tt == 64  ? launch_tile<FP8, 64>(stream, map, p)
           : tt == 128 ? launch_tile<FP8, 128>(stream, map, p)
                       : launch_tile<FP8, 256>(stream, map, p);
  }
  if (*err != cudaSuccess) return -1;
  return launches + 1;
}

int launch_gemm(const Context *ctx, cudaStream_t stream, const LinearArgs &a, cudaError_t *err) {
  int launches = 0;
  const bool needs_x = a.prologue != ULLM_CUDA_PROLOGUE_NONE || a.x_dtype != ULLM_CUDA_DTYPE_BF16 ||
                       reinterpret_cast<uintptr_t>(a.x) % 16 != 0 || (a.x_stride * 2) % 16 != 0;
  const bool pair = a.epilogue == ULLM_CUDA_EPILOGUE_SWIGLU;
  uint8_t *scratch = nullptr;
  const size_t need = gemm_scratch_bytes(a);
  if (need != 0) {
    void *s = nullptr;
    *err = ensure_scratch(ctx, need, &s);
    if (*err != cudaSuccess) return -1;
    scratch = static_cast<uint8_t *>(s);
  }
  const void *x = a.x;
  uint64_t x_stride = a.x_stride;
  size_t off = 0;
  if (needs_x) {
    __nv_bfloat16 *xb = reinterpret_cast<__nv_bfloat16 *>(scratch);
    prologue_kernel<<<a.m, 256, 0, stream>>>(a.x, a.x_dtype, a.x_stride, a.k, a.prologue, a.rms_eps, xb);
    *err = cudaGetLastError();
    if (*err != cudaSuccess) return -1;
    ++launches;
    x = xb;
    x_stride = a.k;
    off = ((size_t)a.m * a.k * 2 + 255) & ~size_t(255);
  }
  GemmParams p{};
  p.w = a.w;
  p.scales = a.scales;
  p.m = a.m;
  p.n = a.n;
  p.k = a.k;
  p.flags = ctx->device_flags;
  if (pair) {  // gate|up to scratch as bf16, combined afterwards
    p.y = scratch + off;
    p.y_stride = a.n;
    p.y_dtype = ULLM_CUDA_DTYPE_BF16;
  } else {
    p.y = a.y;
    p.y_stride = a.y_stride;
    p.y_dtype = a.y_dtype;
  }
  const int tt = tile_tokens(a.m, a.encoding);
  CUtensorMap map;
  if (!make_x_map(&map, x, a.m, a.k, x_stride, (uint32_t)tt)) {
    *err = cudaErrorInvalidValue;
    return -1;
  }
  cudaError_t e;
  if (a.encoding == AQ4) {
    e = tt == 32 ? launch_tile<AQ4, 32>(stream, map, p) : tt == 64 ? launch_tile<AQ4, 64>(stream, map, p)
                                                                   : launch_tile<AQ4, 128>(stream, map, p);
  } else {
    e = tt == 32    ? launch_tile<FP8, 32>(stream, map, p)
        : tt == 64  ? launch_tile<FP8, 64>(stream, map, p)
        : tt == 128 ? launch_tile<FP8, 128>(stream, map, p)
                    : launch_tile<FP8, 256>(stream, map, p);
  }
  *err = e;
  if (e != cudaSuccess) return -1;
  ++launches;
  if (pair) {
    dim3 grid((a.n / 2 + 255) / 256 > 64 ? 64 : (a.n / 2 + 255) / 256, a.m);
    swiglu_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16 *>(scratch + off), a.n / 2,
                                           static_cast<__nv_bfloat16 *>(a.y), a.y_stride);
    *err = cudaGetLastError();
    if (*err != cudaSuccess) return -1;
    ++launches;
  }
  return launches;
}

}  // namespace ullm
