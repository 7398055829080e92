// Prefill / batched-decode GEMM: y[M,N] = prologue(x)[M,K] . W'[N,K]^T with the AQ4 / FP8
// weights fed to the 5th-generation tensor cores AS STORED (tcgen05.mma kind::f8f6f4, e4m3 x e4m3
// -> f32 accumulators in tensor memory).
//
// The reference has no GEMM (hipBLASLt appears only as a planned dependency,
// docs/compatibility/amd-gpu.md:96-102); this is the tensor-core half of the quantised
// linear op selected by shape (docs/architecture/runtime.md:83-91).
//
// Number formats.  The tensor core multiplies e4m3 by e4m3 exactly and adds in fp32, so both
// operands are brought to e4m3 without losing bits:
//   * FP8 weights are e4m3 already: TMA moves the stored bytes straight into the swizzled operand
//     tile, no thread touches them.  scale[n] is applied once to the finished accumulator.
//   * An AQ4 weight q = u - 8 (-8..7) becomes the e4m3 byte sign | |q|, which IS the number
//     q * 2^-9 (the subnormals and the first binade of e4m3 are one linear ramp): about 1.6 integer
//     instructions per weight, shared memory to shared memory.
//   * A bf16 activation has 8 significant bits, e4m3 has 4: x * 2^p = hi + lo, p chosen per token so
//     that the row's largest magnitude lands in [128, 256).  hi = e4m3(x * 2^p) (round to nearest even)
//     leaves a signed rest of at most 8 units of the element's last bf16 bit: three significant bits.
//     Wide tiles store lo = e5m2(rest) and issue the second MMA with an e5m2 B operand (the instruction
//     takes the two operand formats independently) into the SAME accumulator; narrow tiles (up to 64
//     tokens), whose two planes form one B operand with separate accumulator columns, store
//     lo = e4m3(16 * rest) and the epilogue adds hi + lo / 16.  Either way the pair is EXACT for every
//     element whose scaled magnitude is at least 2^-6 (hi in e4m3's normal range), i.e. within a
//     factor 2^14 of the row's largest magnitude; smaller elements are off by at most 2^-14 scaled
//     units, 2^-22 of the row maximum (a row whose largest element is more than 2^14 times the typical
//     one therefore loses one bit of the typical elements per further factor of two).
//     Two MMAs per k-slice at twice the bf16 rate.
//
// Orientation ("swap AB"): the WEIGHT rows are the 128-row M side of the MMA and the TOKENS are
// its N side (tile of TT = 16..256 tokens), so the per-channel / per-group scale is a per-LANE
// scalar of the accumulator and a small token count just uses a narrow N.
// CTAs are persistent (one per SM) and walk a share of all (tile, k-block) work; a tile is 128 or 256
// weight rows x TT tokens, a k-block 128 k.  Warp roles:
//   warp 0      TMA: per k-block the FP8 weight tile [128 x 128 B] and the two activation planes
//               [TT x 128 B] each, 128-byte swizzle, completion on an mbarrier
//   warp 1      owns tensor memory; one lane issues tcgen05.mma
//   warp 2      AQ4 only, TMA: packed nibble tiles [128 x 64 B] into a ring of their own
//   warps 4-7   AQ4 only: nibble tile -> e4m3 operand tile (shared memory to shared memory)
//   warps 8-15  epilogue: tcgen05.ld, scales, store (or split-K partial + last-arriver sum)
// FP8: all k-blocks accumulate in one tensor-memory buffer.  AQ4: one buffer per 128-deep scale
// group, handed to the epilogue in batches, drained into fp32 registers as scale[n,g] * partial.
// Accumulators are double-buffered in tensor memory, so the epilogue of one tile overlaps the MMAs of
// the next.  A tile whose k-blocks fall into several CTAs' shares is finished by the CTA that arrives
// last at the tile's counter, adding the fp32 partials in a fixed order (deterministic).
// Wide FP8 tiles (more than 128 tokens) run on PAIRS of CTAs (clusters of two, tcgen05 cta_group::2): 256
// weight rows x 256 tokens per pair, each CTA loading its own weight rows and half of the token rows, one
// thread of the pair issuing the MMAs for both SMs; see the comment above the kernel.  bf16 results of tiles
// of 128 tokens or more leave through shared memory and TMA stores, one 32 x 32 piece per epilogue warp.
// Measured on B200 (tuning build, operations switched off one at a time): a barrier round trip between
// the single-thread roles costs about 0.2 us per stage and does not overlap the MMAs of that stage, and
// per-element result stores cost 42 us of a 243 us kernel; hence whole-k-block stages where they fit
// (pairs), bulk stores, and whole tiles instead of a k-split tail for wide tiles.
// Every mbarrier wait is bounded in time; on expiry the kernel flags the context and unwinds
// (tensor memory is always released).
#include "internal.hpp"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstdio>
#include <cstdlib>

namespace ullm {

namespace {

constexpr uint32_t AQ4 = ULLM_CUDA_ENCODING_AQ4;
constexpr uint32_t FP8 = ULLM_CUDA_ENCODING_FP8_CHANNEL;
constexpr int BM = 128;   // weight rows per tile (MMA M)
constexpr int BKB = 128;  // k per k-block: 128 e4m3 bytes = one 128-byte swizzle row = one AQ4 scale group
constexpr int kConvWarp0 = 4, kConvWarps = 4, kEpiWarp0 = 8, kEpiWarps = 8;
constexpr int kThreads = (kEpiWarp0 + kEpiWarps) * 32;
constexpr uint32_t A_BYTES = BM * BKB;        // e4m3 operand tile
constexpr uint32_t RAW_BYTES = BM * BKB / 2;  // packed nibble tile
constexpr int MAX_STAGES = 8, MAX_RAW = 8;
constexpr uint32_t kFlagGemmWait = 2u;
constexpr uint32_t kMaxCounterTiles = 1024;  // phase-2 tiles: fewer than the SM count

struct GemmParams {
  const void *scales;      // FP8: float[n]; AQ4: half[n][k/128]
  const float *tok_scale;  // [m] 2^-p of each token's activation planes
  void *y;
  uint64_t y_stride;
  uint32_t y_dtype;
  uint32_t m, n, k;
  uint32_t stages, raw_stages;
  uint32_t whole_rounds;    // phase 1: rounds of whole tiles, tile = round * gridDim.x + CTA, below sk_tile0
  uint32_t sk_tile0;        // phase 2: tiles sk_tile0 .. are cut into sk_ctas ranges of k-blocks
  uint32_t sk_ctas;
  uint32_t m_fastest;       // tile order, see tile_origin
  float *partial;           // [range][head, tail][row block][TT][128] fp32
  uint32_t *tile_counters;  // one per phase-2 tile, zero between launches
  uint32_t *flags;
  uint32_t *abort_word;     // device-resident: non-zero once any wait of the context has given up
  uint64_t wait_ns;         // limit of one barrier wait
  const float *residual;    // f32 [m, res_stride] added to the result, or null
  uint64_t res_stride;
  uint32_t out_bufs;        // > 0: bf16 results leave through shared memory and TMA stores, this many 2 KiB slots per epilogue warp
#ifdef ULLM_CUDA_TUNING
  unsigned long long *stats;  // tuning builds: clocks the single-thread roles spent waiting, summed over CTAs
  uint32_t dbg;               // timing experiments (results are wrong): 1 = rest plane read as e4m3, 2 = rest plane skipped,
                              // 4 = activation planes not loaded, 8 = no MMA issued, 16 = weights not loaded,
                              // 32 = nothing stored, 64 = accumulators not read, 128 = plain arrive instead of commit,
                              // 256 = AQ4 converters only pass their barriers, 512 = AQ4 epilogue skips the per-group drain
#endif
};

#ifdef ULLM_CUDA_TUNING
#define GEMM_STAT_DECL unsigned long long st_wait_a = 0, st_wait_b = 0, st_wait_c = 0; const long long st_t0 = clock64();
#define GEMM_STAT_WAIT(var, expr) do { const long long t_ = clock64(); expr; var += (unsigned long long)(clock64() - t_); } while (0)
#define GEMM_STAT_FLUSH(base) do { if (p.stats != nullptr) { atomicAdd(p.stats + (base), (unsigned long long)(clock64() - st_t0)); \
  atomicAdd(p.stats + (base) + 1, st_wait_a); atomicAdd(p.stats + (base) + 2, st_wait_b); } } while (0)
#else
#define GEMM_STAT_DECL
#define GEMM_STAT_WAIT(var, expr) do { expr; } while (0)
#define GEMM_STAT_FLUSH(base) do { } while (0)
#endif

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
// Bounded wait: false = the CTA gives up (this thread timed out, or another one did, or an earlier kernel of
// the context did: the device-resident abort word makes everything queued behind an expired wait unwind at once).
struct WaitCtl {
  volatile uint32_t *abort_flag;  // this CTA
  uint32_t *device_flags;         // host-visible
  volatile uint32_t *abort_word;  // the context's, in device memory
  uint64_t limit_ns;
};
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtl &w) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 0x3fu) == 0u) {
      if (*w.abort_flag != 0u) return false;
      const bool aborted = w.abort_word != nullptr && *w.abort_word != 0u;
      if (aborted || global_timer_ns() - t0 > w.limit_ns) {
        *w.abort_flag = 1u;
        if (w.abort_word != nullptr) atomicOr(const_cast<uint32_t *>(w.abort_word), 1u);
        if (w.device_flags != nullptr) atomicOr(w.device_flags, kFlagGemmWait);
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
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tc_mma_e4m3(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// 32 lanes x N consecutive fp32 columns: thread l of the warp receives lane (quarter*32 + l)
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&v)[32]) {
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
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
// TMA store of a [rows x tokens] box from shared memory; bulk-group bookkeeping of the issuing thread
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(src), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {  // at most N groups still read their shared-memory source
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---- CTA pairs (clusters of two, tcgen05 cta_group::2): rank 0 issues the MMAs for both ----
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the shared::cluster address of `addr` (a shared::cta address of this CTA) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// TMA into this CTA's shared memory, completion on a barrier that may be the pair's other CTA's
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(map), "r"(cluster_bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(map), "r"(cluster_bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// executed by the same warp of both CTAs of the pair
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// arrives on one barrier (of either CTA) once every MMA issued so far by this thread has completed in both CTAs
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
// M = 256 over the pair: each CTA supplies its 128 weight rows and its half of the token rows at the same
// shared-memory offsets, and receives its 128 accumulator lanes of all token columns
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, %0;" ::"n"(kEpiWarps * 32) : "memory"); }

// K-major swizzled operand tile whose rows are KS = 128 or 64 bytes (the swizzle span) and whose 8-row groups
// are 8 * KS bytes apart: start address >> 4, leading byte offset 1 (unused with a swizzle), stride byte offset
// (8 * KS) >> 4, descriptor version 1 (Blackwell), layout type 2 (SWIZZLE_128B) or 4 (SWIZZLE_64B).
template <int KS>
__device__ __forceinline__ uint64_t smem_desc(uint32_t smem_addr) {
  static_assert(KS == 128 || KS == 64, "swizzle span");
  const uint32_t lo = ((smem_addr >> 4) & 0x3fffu) | (1u << 16);
  const uint32_t hi = (uint32_t)(8 * KS / 16) | (1u << 14) | ((KS == 128 ? 2u : 4u) << 29);
  return ((uint64_t)hi << 32) | lo;
}

// instruction descriptor: D = f32, A = B = e4m3 (format 0), both K-major, M = 128, N = tt
__host__ __device__ constexpr uint32_t instr_desc_e4m3(int tt, int rows = BM) {
  return (1u << 4) | ((uint32_t)(tt >> 3) << 17) | ((uint32_t)(rows >> 4) << 24);
}

__host__ __device__ constexpr uint32_t tmem_cols(uint32_t want) {
  uint32_t c = 32;
  while (c < want) c *= 2;
  return c;
}

// Work distribution.  Phase 1: whole tiles, dealt round-robin (tile = round * gridDim.x + CTA) for
// `whole_rounds` rounds: CTAs that share operands run in step, and nothing needs fixing up.  Phase 2
// ("stream K") balances what is left: the k-blocks of the remaining tiles form one sequence, tile after
// tile, cut into `sk_ctas` equal ranges.  A CTA walks its range segment by segment (a segment =
// consecutive k-blocks of one tile).  A tile inside one range is stored directly; otherwise every
// contributor writes an fp32 partial and the one arriving last at the tile's counter adds them in range
// order (deterministic).  A CTA has at most two partial segments: a "head" (the tile began in an
// earlier range) and a "tail".
struct Segment {
  uint32_t tile, kb0, nkb, first_owner, contributors;
  bool head;
};

struct Walker {
  uint32_t round = 0, rounds, tiles, kb_all, sk_tile0, sk_ctas;
  uint64_t cur = 0, end = 0, units = 0;
  uint32_t me, workers;  // a worker is a CTA, or a CTA pair (both CTAs walk the same sequence)
  __device__ Walker(const GemmParams &p, uint32_t tiles_, uint32_t me_, uint32_t workers_) {
    me = me_;
    workers = workers_;
    kb_all = p.k / BKB;
    tiles = tiles_;
    rounds = p.whole_rounds;
    sk_tile0 = p.sk_tile0;
    sk_ctas = p.sk_ctas;
    if (me < sk_ctas) {
      units = (uint64_t)(tiles - sk_tile0) * kb_all;
      cur = start(me);
      end = start(me + 1);
    }
  }
  __device__ uint64_t start(uint32_t c) const { return (uint64_t)c * units / sk_ctas; }
  // the range that holds unit u: the largest c with floor(c * units / sk_ctas) <= u
  __device__ uint32_t owner(uint64_t u) const { return (uint32_t)(((u + 1) * sk_ctas - 1) / units); }
  __device__ bool next(Segment *s) {
    while (round < rounds) {
      const uint32_t t = round++ * workers + me;
      if (t < sk_tile0) {
        *s = Segment{t, 0u, kb_all, me, 1u, false};
        return true;
      }
    }
    if (cur >= end) return false;
    s->tile = sk_tile0 + (uint32_t)(cur / kb_all);
    s->kb0 = (uint32_t)(cur % kb_all);
    const uint64_t left = end - cur;
    s->nkb = kb_all - s->kb0 < left ? kb_all - s->kb0 : (uint32_t)left;
    if (s->nkb == kb_all) {
      s->first_owner = me;
      s->contributors = 1;
      s->head = false;
    } else {
      const uint64_t t0 = (cur / kb_all) * kb_all;
      s->first_owner = owner(t0);
      s->contributors = owner(t0 + kb_all - 1) - s->first_owner + 1;
      s->head = me > s->first_owner;
    }
    cur += s->nkb;
    return true;
  }
};

// Four bytes, each holding a nibble u = q + 8 (0..15): each becomes the e4m3 byte of q * 2^-9, that is
// |q| with the sign in bit 7 (|q| <= 8 sits in the linear part of e4m3, where the byte value is the magnitude).
__device__ __forceinline__ uint32_t nibble_bytes_to_e4m3(uint32_t b) {
  const uint32_t m = (~b >> 3) & 0x01010101u;     // 1 in every byte with u < 8 (negative q)
  const uint32_t r0 = b ^ 0x08080808u ^ (m * 15u);  // u - 8 where positive, 7 - u where negative
  return r0 + m * 129u;                             // negative: + 1 -> 8 - u, and bit 7
}

// k-blocks per pipeline stage.  A barrier round trip between the TMA thread and the MMA thread costs about as much as
// the MMAs of a narrow k-block, so the narrow FP8 tiles of batched decode move two k-blocks per stage.
template <uint32_t ENC, int TT, int KS, bool PAIR>
__host__ __device__ constexpr uint32_t kps_of() {
  return (ENC == FP8 && !PAIR && KS == BKB && TT <= 64) ? 2u : 1u;
}

// PAIR: the kernel is launched in clusters of two CTAs that share every tile: 256 weight rows (128 per CTA) x TT
// tokens, each CTA loading its own weight rows and HALF of the token rows; rank 0 issues tcgen05.mma.cta_group::2
// for both, so each SM's tensor core reads half of the activation tile from its own shared memory and the other
// half from its partner's.  Per flop that is a third less shared-memory traffic than two independent CTAs, which
// is what bounds the wide FP8 tiles.  No multicast load anywhere: every TMA copy is issued by the CTA it lands in.
template <uint32_t ENC, int TT, int RT, int KS, bool PAIR = false>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                const __grid_constant__ CUtensorMap tmap_y, const GemmParams p) {
  extern __shared__ uint8_t smem_dyn[];
  static_assert(!PAIR || (ENC == FP8 && RT == 1 && TT >= 128), "CTA pairs: wide FP8 tiles, one row block per CTA");
  // a stage holds KS bytes of k: a whole k-block, or half of one where the tiles are too large for more
  // than two whole-k-block stages (the loads of a 96 KB stage take longer than its MMAs)
  static_assert(KS == BKB || ENC == FP8, "the AQ4 converters write whole k-blocks");
  constexpr uint32_t SUBS = BKB / KS;                   // stages per k-block
  constexpr uint32_t A_STAGE = (uint32_t)BM * KS;       // one row block of the stage
  constexpr uint32_t B_TOK = PAIR ? TT / 2 : TT;        // token rows this CTA loads
  constexpr uint32_t B_BYTES = B_TOK * KS;              // one activation plane of the stage
  constexpr uint32_t KPS = kps_of<ENC, TT, KS, PAIR>();  // k-blocks per stage
  constexpr uint32_t SUB_BYTES = RT * A_STAGE + 2 * B_BYTES;  // operands of one k-block (or half of one)
  constexpr uint32_t STAGE_BYTES = KPS * SUB_BYTES;
  // Up to 64 tokens the two activation planes, adjacent in shared memory, are ONE operand of 2*TT rows: a
  // single MMA per k-slice leaves A.hi in columns [0,TT) and A.lo in [TT,2TT) and the epilogue adds them.
  // A narrow MMA costs the tensor pipe about as much as a wide one, so this halves the pipe time where
  // the weight stream should set the pace.
  constexpr bool NCAT = TT <= 64;
  constexpr uint32_t MMA_N = NCAT ? 2u * TT : (uint32_t)TT;
  constexpr uint32_t ACC_COLS = RT * MMA_N;  // one accumulator set: RT row blocks side by side
  // Accumulator sets in tensor memory.  FP8: one per segment, two in rotation when they fit.  AQ4: one per
  // 128-deep scale group; GB consecutive groups form a batch that is handed to the epilogue with one
  // barrier round trip, two batches in rotation.
  // (Wide tiles keep one group per batch and four in rotation: measured 0.63 vs 0.57 PFLOP/s at 2048 tokens.)
  constexpr uint32_t GB = (ENC == AQ4 && ACC_COLS < 128) ? 256u / ACC_COLS : 1u;  // groups per batch
  constexpr int NB = ENC == AQ4 ? (GB > 1 ? 2 : 4) : (ACC_COLS > 256 ? 1 : 2);
  constexpr uint32_t BUF_COLS = GB * ACC_COLS;
  constexpr uint32_t TMEM_COLS = tmem_cols(BUF_COLS * NB);
  static_assert(BUF_COLS * NB <= 512, "tensor memory has 512 columns");
  __shared__ __align__(8) uint64_t bars[3 * MAX_STAGES + 2 * MAX_RAW + 8];
  __shared__ uint32_t tmem_base_slot;
  __shared__ uint32_t abort_flag;
  __shared__ uint32_t last_flag;

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t NS = p.stages, RS = p.raw_stages;
  const uint32_t crank = PAIR ? cluster_rank() : 0u;  // 0 issues the pair's MMAs
  constexpr uint32_t TILE_ROWS = (PAIR ? 2 : RT) * BM;
  const uint32_t tiles_n = (p.n + TILE_ROWS - 1) / TILE_ROWS, tiles_m = (p.m + TT - 1) / TT;
  // first weight row of THIS CTA and first token of the tile
  auto tile_origin = [&](uint32_t tile, uint32_t *n0, uint32_t *m0) {
    // m fastest: consecutive tiles share the weight rows (read from HBM once); n fastest: they share the tokens
    const uint32_t tn = p.m_fastest ? tile / tiles_m : tile % tiles_n, tm = p.m_fastest ? tile % tiles_m : tile / tiles_n;
    *n0 = tn * TILE_ROWS + crank * BM;
    *m0 = tm * TT;
  };
  // tiles must start on a 1024-byte boundary for the 128-byte swizzle
  const uint32_t smem0 = ((uint32_t)__cvta_generic_to_shared(smem_dyn) + 1023u) & ~1023u;
  const uint32_t raw0 = smem0 + NS * STAGE_BYTES;
  const uint32_t out0 = raw0 + RS * RT * RAW_BYTES;  // epilogue staging: [warp][slot][32 tokens][32 rows] bf16
  const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(bars);
  auto full = [&](uint32_t s) { return bar0 + s * 8u; };                          // TMA bytes of the stage landed
  auto a_full = [&](uint32_t s) { return bar0 + (MAX_STAGES + s) * 8u; };         // AQ4: operand tile converted
  auto empty = [&](uint32_t s) { return bar0 + (2 * MAX_STAGES + s) * 8u; };      // the stage's MMAs are done
  auto raw_full = [&](uint32_t s) { return bar0 + (3 * MAX_STAGES + s) * 8u; };
  auto raw_empty = [&](uint32_t s) { return bar0 + (3 * MAX_STAGES + MAX_RAW + s) * 8u; };
  auto acc_full = [&](uint32_t b) { return bar0 + (3 * MAX_STAGES + 2 * MAX_RAW + b) * 8u; };
  auto acc_empty = [&](uint32_t b) { return bar0 + (3 * MAX_STAGES + 2 * MAX_RAW + 4 + b) * 8u; };

  if (threadIdx.x == 0) {
    abort_flag = 0u;
    last_flag = 0u;
    for (uint32_t s = 0; s < NS; ++s) {
      mbar_init(full(s), 1u);                       // the TMA thread's expect_tx
      mbar_init(a_full(s), (uint32_t)kConvWarps);   // one arrival per converter warp
      mbar_init(empty(s), 1u);                      // tcgen05.commit
    }
    for (uint32_t s = 0; s < RS; ++s) {
      mbar_init(raw_full(s), 1u);
      mbar_init(raw_empty(s), (uint32_t)kConvWarps);
    }
    for (uint32_t b = 0; b < 4; ++b) {
      mbar_init(acc_full(b), 1u);                     // tcgen05.commit
      mbar_init(acc_empty(b), (uint32_t)kEpiWarps * (PAIR ? 2u : 1u));  // one arrival per epilogue warp (of both CTAs)
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  // whatever is launched behind this kernel as a programmatic dependent may take SMs as this grid's blocks leave
  // them; it waits for this grid before it touches anything this grid reads or writes
  if (threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (PAIR) {
    // the partner's barriers must exist before anything signals them, and both CTAs allocate together
    __syncthreads();
    cluster_sync_all();
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair((uint32_t)__cvta_generic_to_shared(&tmem_base_slot), TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc((uint32_t)__cvta_generic_to_shared(&tmem_base_slot), TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const WaitCtl wctl{&abort_flag, p.flags, p.abort_word, p.wait_ns};
  Walker walk(p, tiles_n * tiles_m, PAIR ? blockIdx.x >> 1 : blockIdx.x, PAIR ? gridDim.x >> 1 : gridDim.x);
  Segment sg;

  if (warp == 0) {
    // ---- TMA: operand tiles -----------------------------------------------------------------
    if (lane == 0) {
      // everything before this point overlapped the kernel that wrote the activation planes
      asm volatile("griddepcontrol.wait;" ::: "memory");
      uint32_t slot = 0, round = 0;
      bool ok = true;
      GEMM_STAT_DECL
      while (ok && walk.next(&sg)) {
        uint32_t n0, m0;
        tile_origin(sg.tile, &n0, &m0);
        for (uint32_t i = 0; i < sg.nkb * SUBS; i += KPS) {
          const uint32_t cnt = sg.nkb * SUBS - i < KPS ? sg.nkb * SUBS - i : KPS;  // k-blocks in this stage
          bool got = true;
          if (round > 0) GEMM_STAT_WAIT(st_wait_a, got = mbar_wait(empty(slot), (round - 1) & 1u, wctl));
          if (!got) {
            ok = false;
            break;
          }
          const uint32_t a_addr = smem0 + slot * STAGE_BYTES;
          const int kx = (int)(sg.kb0 * BKB + i * KS);
          if (PAIR) {
            // both CTAs' bytes complete on rank 0's barrier, which its MMA thread waits for
            const uint32_t fb = map_to_cta(full(slot), 0u);
            const int tok0 = (int)(m0 + crank * B_TOK);
#ifdef ULLM_CUDA_TUNING
            const bool no_x = (p.dbg & 4u) != 0u, no_w = (p.dbg & 16u) != 0u;
#else
            constexpr bool no_x = false, no_w = false;
#endif
            if (crank == 0) mbar_expect_tx(full(slot), 2u * ((no_w ? 0u : A_STAGE) + (no_x ? 0u : 2 * B_BYTES)));
            if (!no_w) tma_load_2d_pair(a_addr, &tmap_w, kx, (int)n0, fb);
            if (!no_x) {
              tma_load_3d_pair(a_addr + A_STAGE, &tmap_x, kx, tok0, 0, fb);
              tma_load_3d_pair(a_addr + A_STAGE + B_BYTES, &tmap_x, kx, tok0, 1, fb);
            }
          } else {
#ifdef ULLM_CUDA_TUNING
            const bool no_x = (p.dbg & 4u) != 0u, no_w = (p.dbg & 16u) != 0u;
#else
            constexpr bool no_x = false, no_w = false;
#endif
            mbar_expect_tx(full(slot), cnt * (((ENC == FP8 && !no_w) ? RT * A_STAGE : 0u) + (no_x ? 0u : 2 * B_BYTES)));
            for (uint32_t j = 0; j < cnt; ++j) {
              const uint32_t sa = a_addr + j * SUB_BYTES;
              const int kj = kx + (int)(j * KS);
              if (ENC == FP8 && !no_w) {
#pragma unroll
                for (int r = 0; r < RT; ++r) tma_load_2d(sa + r * A_STAGE, &tmap_w, kj, (int)(n0 + r * BM), full(slot));
              }
              if (!no_x) {
                tma_load_3d(sa + RT * A_STAGE, &tmap_x, kj, (int)m0, 0, full(slot));
                tma_load_3d(sa + RT * A_STAGE + B_BYTES, &tmap_x, kj, (int)m0, 1, full(slot));
              }
            }
          }
          if (++slot == NS) {
            slot = 0;
            ++round;
          }
        }
      }
      GEMM_STAT_FLUSH(0);
    }
  } else if (warp == 1) {
    // ---- MMA issue ------------------------------------------------------------------------
    if (lane == 0 && crank == 0) {
      constexpr uint32_t idesc = instr_desc_e4m3((int)MMA_N, PAIR ? 2 * BM : BM);
      constexpr uint32_t idesc_lo = idesc | (1u << 10);  // B operand read as e5m2 (the rest plane of wide tiles)
      uint32_t slot = 0, round = 0, seg = 0, batch = 0, in_batch = 0;
      bool ok = true;
#ifdef ULLM_CUDA_TUNING
      unsigned long long sq_fence = 0, sq_issue = 0, sq_commit = 0;
      const uint32_t id_lo = (p.dbg & 1u) ? idesc : idesc_lo;
      const bool skip_lo = (p.dbg & 2u) != 0u, skip_mma = (p.dbg & 8u) != 0u;
#else
      constexpr uint32_t id_lo = idesc_lo;
      constexpr bool skip_lo = false, skip_mma = false;
#endif
      GEMM_STAT_DECL
      while (ok && walk.next(&sg)) {
        uint32_t buf = 0;
        if (ENC == FP8) {
          buf = seg % NB;
          const uint32_t use = seg / NB;
          if (use >= 1) GEMM_STAT_WAIT(st_wait_b, ok = mbar_wait(acc_empty(buf), (use - 1) & 1u, wctl));
        }
        for (uint32_t i = 0; i < sg.nkb * SUBS && ok; i += KPS) {
          const uint32_t cnt = sg.nkb * SUBS - i < KPS ? sg.nkb * SUBS - i : KPS;  // k-blocks in this stage
          uint32_t fresh = i == 0 ? 1u : 0u;
          if (ENC == AQ4) {
            buf = batch % NB;
            const uint32_t use = batch / NB;
            fresh = 1u;
            if (in_batch == 0 && use >= 1) GEMM_STAT_WAIT(st_wait_b, ok = mbar_wait(acc_empty(buf), (use - 1) & 1u, wctl));
            GEMM_STAT_WAIT(st_wait_c, ok = ok && mbar_wait(a_full(slot), round & 1u, wctl));
          }
          GEMM_STAT_WAIT(st_wait_a, ok = ok && mbar_wait(full(slot), round & 1u, wctl));
          if (!ok) break;
#ifdef ULLM_CUDA_TUNING
          const long long tq0 = clock64();
#endif
          tc_fence_after();
#ifdef ULLM_CUDA_TUNING
          const long long tq1 = clock64();
#endif
          for (uint32_t j = 0; j < cnt; ++j) {
            const uint32_t a_addr = smem0 + slot * STAGE_BYTES + j * SUB_BYTES, hi_addr = a_addr + RT * A_STAGE,
                           lo_addr = hi_addr + B_BYTES;
#pragma unroll
            for (int r = 0; r < RT; ++r) {
              const uint32_t d = tmem_base + buf * BUF_COLS + in_batch * ACC_COLS + r * MMA_N;
#pragma unroll
              for (int k4 = 0; k4 < KS / 32; ++k4) {
                // 32 e4m3 along K = 32 bytes inside the swizzled row: advance the start address only
                const uint64_t adesc = smem_desc<KS>(a_addr + r * A_STAGE + k4 * 32);
                const uint32_t acc = (fresh && j == 0 && k4 == 0) ? 0u : 1u;
                if (skip_mma) continue;
                if (PAIR) {
                  tc_mma_pair(d, adesc, smem_desc<KS>(hi_addr + k4 * 32), idesc, acc);
                  if (!skip_lo) tc_mma_pair(d, adesc, smem_desc<KS>(lo_addr + k4 * 32), id_lo, 1u);
                } else {
                  tc_mma_e4m3(d, adesc, smem_desc<KS>(hi_addr + k4 * 32), idesc, acc);
                  if (!NCAT && !skip_lo) tc_mma_e4m3(d, adesc, smem_desc<KS>(lo_addr + k4 * 32), id_lo, 1u);
                }
              }
            }
          }
#ifdef ULLM_CUDA_TUNING
          const long long tq2 = clock64();
#endif
          // the stage may be refilled when these MMAs are done (in both CTAs of a pair)
#ifdef ULLM_CUDA_TUNING
          if ((p.dbg & 128u) != 0u && !PAIR) {
            mbar_arrive(empty(slot));
          } else
#endif
          if (PAIR) {
            tc_commit_pair(empty(slot));
            tc_commit_pair(map_to_cta(empty(slot), 1u));
          } else {
            tc_commit(empty(slot));
          }
          if (ENC == AQ4) {
            if (++in_batch == GB || i + 1 == sg.nkb) {  // a batch does not span tiles
              tc_commit(acc_full(buf));
              ++batch;
              in_batch = 0;
            }
          } else if (i + cnt == sg.nkb * SUBS) {
            if (PAIR) {
              tc_commit_pair(acc_full(buf));
              tc_commit_pair(map_to_cta(acc_full(buf), 1u));
            } else {
              tc_commit(acc_full(buf));
            }
          }
#ifdef ULLM_CUDA_TUNING
          const long long tq3 = clock64();
          sq_fence += (unsigned long long)(tq1 - tq0);
          sq_issue += (unsigned long long)(tq2 - tq1);
          sq_commit += (unsigned long long)(tq3 - tq2);
#endif
          if (++slot == NS) {
            slot = 0;
            ++round;
          }
        }
        ++seg;
      }
#ifdef ULLM_CUDA_TUNING
      if (p.stats != nullptr) {
        atomicAdd(p.stats + 13, sq_fence);
        atomicAdd(p.stats + 14, sq_issue);
        atomicAdd(p.stats + 15, sq_commit);
      }
#endif
      GEMM_STAT_FLUSH(3);
#ifdef ULLM_CUDA_TUNING
      if (p.stats != nullptr) atomicAdd(p.stats + 12, st_wait_c);
#endif
    }
  } else if (warp == 2) {
    // ---- AQ4: TMA of the packed nibble tiles (weights: nothing to wait for) ------------------
    if (ENC == AQ4 && lane == 0) {
      uint32_t slot = 0, round = 0;
      bool ok = true;
      while (ok && walk.next(&sg)) {
        uint32_t n0, m0;
        tile_origin(sg.tile, &n0, &m0);
        for (uint32_t i = 0; i < sg.nkb; ++i) {
          if (round > 0 && !mbar_wait(raw_empty(slot), (round - 1) & 1u, wctl)) {
            ok = false;
            break;
          }
          mbar_expect_tx(raw_full(slot), RT * RAW_BYTES);
#pragma unroll
          for (int r = 0; r < RT; ++r)
            tma_load_2d(raw0 + (slot * RT + r) * RAW_BYTES, &tmap_w, (int)((sg.kb0 + i) * (BKB / 2)), (int)(n0 + r * BM),
                        raw_full(slot));
          if (++slot == RS) {
            slot = 0;
            ++round;
          }
        }
      }
    }
  } else if (warp >= kConvWarp0 && warp < kConvWarp0 + kConvWarps) {
    // ---- AQ4: nibble tile -> e4m3 operand tile ------------------------------------------------
    // The four converter warps share every k-block: thread t takes items t, t+128, t+256, t+384 of the 512
    // (row, 16-byte chunk) items, so a warp's loads are 512 contiguous bytes and its stores hit every bank once.
    // Item (row, c): the 16 bytes c of the row's 64 = k 32c .. 32c+31; the even elements of those 32 go to
    // operand chunk 2c, the odd ones to chunk 2c+1 (the activation planes use the same order).
    if (ENC == AQ4) {
      const uint32_t ct = threadIdx.x - kConvWarp0 * 32;
      uint32_t slot = 0, round = 0, rslot = 0, rround = 0;
      bool ok = true;
      GEMM_STAT_DECL
      while (ok && walk.next(&sg)) {
        for (uint32_t i = 0; i < sg.nkb; ++i) {
          bool got = true;
          GEMM_STAT_WAIT(st_wait_a, got = mbar_wait(raw_full(rslot), rround & 1u, wctl));
          if (!got) {
            ok = false;
            break;
          }
          // the nibbles are requested before the wait for a free operand tile, so that wait hides their latency
          uint4 q[RT][4];
#pragma unroll
          for (int r = 0; r < RT; ++r) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t addr = raw0 + (rslot * RT + r) * RAW_BYTES + (ct + 128u * j) * 16u;
              asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(q[r][j].x), "=r"(q[r][j].y), "=r"(q[r][j].z), "=r"(q[r][j].w)
                           : "r"(addr));
            }
          }
          if (round > 0) GEMM_STAT_WAIT(st_wait_b, got = mbar_wait(empty(slot), (round - 1) & 1u, wctl));
          if (!got) {
            ok = false;
            break;
          }
#ifdef ULLM_CUDA_TUNING
          if ((p.dbg & 256u) == 0u)
#endif
#pragma unroll
          for (int r = 0; r < RT; ++r) {
            const uint32_t a_addr = smem0 + slot * STAGE_BYTES + r * A_BYTES;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t row = (ct >> 2) + 32u * j, c = ct & 3u;
              const uint32_t a_row = a_addr + row * 128u;
              const uint32_t w[4] = {q[r][j].x, q[r][j].y, q[r][j].z, q[r][j].w};
              uint32_t ev[4], od[4];
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                ev[t] = nibble_bytes_to_e4m3(w[t] & 0x0f0f0f0fu);
                od[t] = nibble_bytes_to_e4m3((w[t] >> 4) & 0x0f0f0f0fu);
              }
              asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a_row + (((2u * c) ^ (row & 7u)) << 4)),
                           "r"(ev[0]), "r"(ev[1]), "r"(ev[2]), "r"(ev[3])
                           : "memory");
              asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a_row + (((2u * c + 1u) ^ (row & 7u)) << 4)),
                           "r"(od[0]), "r"(od[1]), "r"(od[2]), "r"(od[3])
                           : "memory");
            }
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the MMA
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(a_full(slot));
            mbar_arrive(raw_empty(rslot));
          }
          if (++slot == NS) {
            slot = 0;
            ++round;
          }
          if (++rslot == RS) {
            rslot = 0;
            ++rround;
          }
        }
      }
#ifdef ULLM_CUDA_TUNING
      if (ct == 0) GEMM_STAT_FLUSH(9);
#endif
    }
  } else if (warp >= kEpiWarp0) {
    // ---- epilogue: warp e covers TMEM lanes 32*(warp % 4) .. +31 and half of the token columns ----
    asm volatile("griddepcontrol.wait;" ::: "memory");  // token scales, group sums, the output
    const uint32_t e = warp - kEpiWarp0;
    const uint32_t quarter = warp & 3u, half = e >> 2;
    constexpr int CH = TT < 32 ? TT : 32;              // columns per tcgen05.ld when storing
    constexpr int COLS = TT / 2 < CH ? CH : TT / 2;     // token columns of this warp
    const uint32_t col0 = half * COLS;
    const bool active = col0 < (uint32_t)TT;  // narrow tiles: the second half has nothing to do
    const uint32_t lane_addr = tmem_base + ((quarter * 32u) << 16);
    const uint32_t row_in_tile = quarter * 32 + lane;
    const float mult = ENC == AQ4 ? 512.0f : 1.0f;  // 2^9: the nibble bytes were read as u * 2^-9
    constexpr uint64_t PART = (uint64_t)RT * TT * BM;  // floats of one partial tile
    uint32_t seg = 0, batch = 0, out_n = 0;
    bool ok = true;
    GEMM_STAT_DECL
    while (walk.next(&sg)) {
      uint32_t n0, m0;
      tile_origin(sg.tile, &n0, &m0);
      const bool direct = sg.contributors == 1;
      // a worker's partials: one pair of slots per CTA (PAIR: the two CTAs of worker w are CTAs 2w and 2w + 1)
      auto cta_of = [&](uint32_t worker) { return PAIR ? worker * 2u + crank : worker; };
      float *part = direct ? nullptr : p.partial + ((uint64_t)blockIdx.x * 2 + (sg.head ? 0 : 1)) * PART;
      // finished columns c .. c+CH-1 of row block r: final store, or this range's partial
      auto emit = [&](int r, uint32_t c, const float (&v)[CH], bool final_pass) {
        if (!final_pass) {
#pragma unroll
          for (int i = 0; i < CH; ++i) part[((uint64_t)r * TT + c + i) * BM + row_in_tile] = v[i];
          return;
        }
        const uint32_t row = n0 + r * BM + row_in_tile;
        if (row >= p.n) return;
#ifdef ULLM_CUDA_TUNING
        if ((p.dbg & 32u) != 0u && v[0] != 1234.5f) return;
#endif
#pragma unroll
        for (int i = 0; i < CH; ++i) {
          const uint32_t tok = m0 + c + i;
          if (tok < p.m) {
            float f = v[i] * (mult * __ldg(p.tok_scale + tok));
            if (p.residual != nullptr) f += p.residual[(uint64_t)tok * p.res_stride + row];
            if (p.y_dtype == ULLM_CUDA_DTYPE_F32)
              static_cast<float *>(p.y)[(uint64_t)tok * p.y_stride + row] = f;
            else
              static_cast<__nv_bfloat16 *>(p.y)[(uint64_t)tok * p.y_stride + row] = __float2bfloat16_rn(f);
          }
        }
      };
      // bf16 results (whole tiles): this warp's 32 rows x 32 tokens go to its own shared-memory slot and leave by one
      // TMA store (clipped at the matrix edges), so the stores cost the warp 32 shared-memory writes
      auto stage_out = [&](int r, uint32_t c, const float (&v)[CH]) {
        if constexpr (CH == 32) {
          const uint32_t slot_addr = out0 + ((e * p.out_bufs + (out_n % p.out_bufs)) << 11);
          const uint32_t row = n0 + r * BM + row_in_tile;
          if (lane == 0) {
            if (p.out_bufs > 1u)
              bulk_wait_read<1>();
            else
              bulk_wait_read<0>();
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < CH; ++i) {
            const uint32_t tok = m0 + c + i;
            float o = v[i] * (mult * __ldg(p.tok_scale + (tok < p.m ? tok : 0u)));
            if (p.residual != nullptr && tok < p.m && row < p.n) o += p.residual[(uint64_t)tok * p.res_stride + row];
            const __nv_bfloat16 h = __float2bfloat16_rn(o);
            asm volatile("st.shared.b16 [%0], %1;" ::"r"(slot_addr + (uint32_t)i * 64u + lane * 2u),
                         "h"(*reinterpret_cast<const unsigned short *>(&h))
                         : "memory");
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmap_y, slot_addr, (int)(n0 + r * BM + quarter * 32u), (int)(m0 + c));
            bulk_commit();
          }
          ++out_n;
        }
      };
      if (ENC == FP8) {
        const uint32_t buf = seg % NB, use = seg / NB;
        GEMM_STAT_WAIT(st_wait_a, ok = ok && mbar_wait(acc_full(buf), use & 1u, wctl));
        if (ok) {
          tc_fence_after();
#ifdef ULLM_CUDA_TUNING
          const bool skip_read = (p.dbg & 64u) != 0u;
#else
          constexpr bool skip_read = false;
#endif
          if (active && !skip_read) {
#pragma unroll 1
            for (int r = 0; r < RT; ++r) {
              const uint32_t row = n0 + r * BM + row_in_tile;
              const float sc = row < p.n ? static_cast<const float *>(p.scales)[row] : 0.0f;
#pragma unroll 1
              for (int c = 0; c < COLS; c += CH) {
                uint32_t v[CH], v2[CH];
                tmem_ld(lane_addr + buf * BUF_COLS + r * MMA_N + col0 + c, v);
                if (NCAT) tmem_ld(lane_addr + buf * BUF_COLS + r * MMA_N + TT + col0 + c, v2);
                tmem_ld_wait();
                float f[CH];
#pragma unroll
                for (int i = 0; i < CH; ++i)
                  f[i] = (NCAT ? fmaf(__uint_as_float(v2[i]), 0.0625f, __uint_as_float(v[i])) : __uint_as_float(v[i])) * sc;
                if (CH == 32 && p.out_bufs != 0u && direct)
                  stage_out(r, col0 + c, f);
                else
                  emit(r, col0 + c, f, direct);
              }
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {  // the accumulator may take the segment after next
            if (PAIR)
              mbar_arrive_cluster(map_to_cta(acc_empty(buf), 0u));
            else
              mbar_arrive(acc_empty(buf));
          }
        }
      } else {
        static_assert(ENC != AQ4 || RT == 1, "the AQ4 epilogue keeps one row block's running sums in registers");
        float acc[COLS];
#pragma unroll
        for (int i = 0; i < COLS; ++i) acc[i] = 0.0f;
        const uint32_t groups = p.k / 128;
        const uint32_t row = n0 + row_in_tile;
        const __half *srow = static_cast<const __half *>(p.scales) + (uint64_t)(row < p.n ? row : 0) * groups + sg.kb0;
        // the scales of a batch are requested one batch ahead, so their latency is off the drain's critical path
        if constexpr (GB == 1) {
          // one group per hand-off: the next group's scale is requested while this one is drained
          float sc_next = row < p.n ? __half2float(srow[0]) : 0.0f;
          for (uint32_t g = 0; g < sg.nkb && ok; ++g, ++batch) {
            const uint32_t buf = batch % NB, use = batch / NB;
            const float sc = sc_next;
            if (g + 1 < sg.nkb && row < p.n) sc_next = __half2float(srow[g + 1]);
            GEMM_STAT_WAIT(st_wait_a, ok = mbar_wait(acc_full(buf), use & 1u, wctl));
            if (!ok) break;
            tc_fence_after();
#ifdef ULLM_CUDA_TUNING
            if (active && (p.dbg & 512u) == 0u) {
#else
            if (active) {
#endif
#pragma unroll
              for (int c = 0; c < COLS; c += CH) {
                uint32_t v[CH], v2[CH];
                tmem_ld(lane_addr + buf * BUF_COLS + col0 + c, v);
                if (NCAT) tmem_ld(lane_addr + buf * BUF_COLS + TT + col0 + c, v2);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < CH; ++i)
                  acc[c + i] = fmaf(sc, NCAT ? fmaf(__uint_as_float(v2[i]), 0.0625f, __uint_as_float(v[i])) : __uint_as_float(v[i]), acc[c + i]);
              }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(buf));  // this buffer may take a later group
          }
        } else {
          // a batch of GB groups per hand-off (narrow tiles); the scales of a batch are requested one batch ahead
          float sc_next[GB];
#pragma unroll
          for (uint32_t j = 0; j < GB; ++j) sc_next[j] = (j < sg.nkb && row < p.n) ? __half2float(srow[j]) : 0.0f;
          for (uint32_t g = 0; g < sg.nkb && ok; ++batch) {
            const uint32_t cnt = sg.nkb - g < GB ? sg.nkb - g : GB;  // groups in this batch
            const uint32_t buf = batch % NB, use = batch / NB;
            float sc[GB];
#pragma unroll
            for (uint32_t j = 0; j < GB; ++j) {
              sc[j] = sc_next[j];
              sc_next[j] = (g + GB + j < sg.nkb && row < p.n) ? __half2float(srow[g + GB + j]) : 0.0f;
            }
            ok = mbar_wait(acc_full(buf), use & 1u, wctl);
            if (!ok) break;
            tc_fence_after();
            if (active) {
#pragma unroll
              for (uint32_t j = 0; j < GB; ++j) {
                if (j < cnt) {
#pragma unroll
                  for (int c = 0; c < COLS; c += CH) {
                    uint32_t v[CH], v2[CH];
                    tmem_ld(lane_addr + buf * BUF_COLS + j * ACC_COLS + col0 + c, v);
                    if (NCAT) tmem_ld(lane_addr + buf * BUF_COLS + j * ACC_COLS + TT + col0 + c, v2);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < CH; ++i)
                      acc[c + i] = fmaf(sc[j], NCAT ? fmaf(__uint_as_float(v2[i]), 0.0625f, __uint_as_float(v[i])) : __uint_as_float(v[i]),
                                        acc[c + i]);
                  }
                }
              }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(buf));  // this buffer may take the batch after next
            g += cnt;
          }
        }
        if (ok && active) {
#pragma unroll
          for (int c = 0; c < COLS; c += CH) {
            float f[CH];
#pragma unroll
            for (int i = 0; i < CH; ++i) f[i] = acc[c + i];
            if (CH == 32 && p.out_bufs != 0u && direct)
              stage_out(0, col0 + c, f);
            else
              emit(0, col0 + c, f, direct);
          }
        }
      }
      if (!direct) {
        // the partial is in global memory; whoever arrives last at the tile's counter adds the partials in
        // range order and stores.  All eight warps pass both barriers, also after a failed wait.
        __threadfence();
        epi_bar();
        if (threadIdx.x == kEpiWarp0 * 32) {
          uint32_t last = 0u;
          if (ok) {
            const uint32_t ci = PAIR ? (sg.tile - p.sk_tile0) * 2u + crank : sg.tile - p.sk_tile0;
            const uint32_t prev = atomicAdd(p.tile_counters + ci, 1u);
            if (prev + 1 == sg.contributors) {
              p.tile_counters[ci] = 0u;  // ready for the next launch
              last = 1u;
            }
          }
          last_flag = last;
        }
        epi_bar();
        if (last_flag != 0u && active) {
          __threadfence();
#pragma unroll 1
          for (int r = 0; r < RT; ++r) {
#pragma unroll 1
            for (int c = 0; c < COLS; c += CH) {
              float f[CH];
#pragma unroll
              for (int i = 0; i < CH; ++i) f[i] = 0.0f;
              for (uint32_t j = 0; j < sg.contributors; ++j) {
                // contributor j is range first_owner + j: its tail segment if it began the tile, else its head
                const float *src = p.partial + ((uint64_t)cta_of(sg.first_owner + j) * 2 + (j == 0 ? 1 : 0)) * PART +
                                   ((uint64_t)r * TT + col0 + c) * BM + row_in_tile;
#pragma unroll
                for (int i = 0; i < CH; ++i) f[i] += __ldcg(src + (uint64_t)i * BM);
              }
              emit(r, col0 + c, f, true);
            }
          }
        }
        epi_bar();  // last_flag is rewritten by the next partial segment
      }
      ++seg;
    }
    if (lane == 0 && p.out_bufs != 0u) bulk_wait_all();  // the stores have read their slots and are on their way
#ifdef ULLM_CUDA_TUNING
    if (threadIdx.x == kEpiWarp0 * 32) GEMM_STAT_FLUSH(6);
#endif
  }
  tc_fence_before();
  __syncthreads();
  if (abort_flag != 0u) {
    // a wait gave up: let copies that may still be in flight land before shared memory is released
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  // the partner's MMAs read this CTA's shared memory and signal its barriers: leave together
  if (PAIR) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    if (PAIR)
      tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else
      tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- activations -> two e4m3 planes ------------------------------------------------------------

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// One block per token row m.  value[i] = bf16( prologue(x)[m][i] ) exactly as the matvec path stages it;
// then planes[0][m][pos(i)] = hi = e4m3(value * 2^p) and planes[1][m][pos(i)] = the rest value * 2^p - hi, stored
// as e5m2(rest) (LO16 false: wide tiles, read as an e5m2 operand) or as e4m3(16 * rest) (LO16 true: narrow
// tiles, whose epilogue divides by 16); tok_scale[m] = 2^-p.
// PERM (AQ4): inside every 32 consecutive k the even elements come first, then the odd ones, which is
// the order the nibble conversion produces.
template <bool PERM, bool LO16>
__global__ void __launch_bounds__(256) act_planes_kernel(const void *x, uint32_t x_dtype, uint64_t x_stride, uint32_t k,
                                                         uint32_t prologue, float eps, const __nv_bfloat16 *gamma,
                                                         uint8_t *planes, uint64_t plane_stride, float *tok_scale) {
  __shared__ float red_ss[8], red_mx[8];
  // the GEMM launched behind this kernel may set itself up now; it waits for this grid before reading.  This grid
  // itself is launched as a programmatic dependent of whatever wrote x: nothing is read or written before the wait.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint32_t m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t groups = k / 128;
  auto ld = [&](uint32_t i) -> float {
    return x_dtype == ULLM_CUDA_DTYPE_F32 ? bf16r(static_cast<const float *>(x)[(uint64_t)m * x_stride + i])
                                          : __bfloat162float(static_cast<const __nv_bfloat16 *>(x)[(uint64_t)m * x_stride + i]);
  };
  auto pre = [&](uint32_t i) -> float {
    float v = ld(i);
    if (prologue == ULLM_CUDA_PROLOGUE_SWIGLU) {
      const float u = ld(k + i);
      v = v / (1.0f + expf(-v)) * u;
    }
    return v;
  };
  const bool weighted = prologue == ULLM_CUDA_PROLOGUE_RMSNORM && gamma != nullptr;
  // pass 1: sum of squares (RMSNorm) and the largest magnitude (of x * gamma when there is a weight vector:
  // the positive factor 1/rms and the final rounding are monotone, so this finds the largest staged magnitude)
  float ss = 0.0f, mx = 0.0f;
  for (uint32_t g = warp; g < groups; g += 8) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t i = g * 128 + lane * 4 + j;
      const float v = pre(i);
      ss = fmaf(v, v, ss);
      mx = fmaxf(mx, weighted ? fabsf(v * __bfloat162float(gamma[i])) : fabsf(v));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ss += __shfl_xor_sync(0xffffffffu, ss, o);
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if (lane == 0) {
    red_ss[warp] = ss;
    red_mx[warp] = mx;
  }
  __syncthreads();
  float tot = 0.0f, amax = 0.0f;
  for (int w = 0; w < 8; ++w) {
    tot += red_ss[w];
    amax = fmaxf(amax, red_mx[w]);
  }
  const float inv = prologue == ULLM_CUDA_PROLOGUE_RMSNORM ? 1.0f / sqrtf(tot / (float)k + eps) : 1.0f;
  // an upper bound of the largest staged magnitude (the staged value rounds (v * inv) * gamma, this rounds
  // (v * gamma) * inv: at most a few ulp apart, and the top of the range below leaves a factor 1.75 of room)
  amax = bf16r(amax * inv);
  int p = 0;
  if (amax > 0.0f && amax <= 3.0e38f) {
    int e;
    (void)frexpf(amax, &e);  // amax = f * 2^e, f in [0.5, 1)
    p = 8 - e;               // amax * 2^p in [128, 256); e4m3 reaches 448
    p = p > 126 ? 126 : (p < -126 ? -126 : p);
  }
  const float up = ldexpf(1.0f, p);
  if (threadIdx.x == 0) tok_scale[m] = ldexpf(1.0f, -p);
  // pass 2
  uint8_t *hi_row = planes + (uint64_t)m * k, *lo_row = hi_row + plane_stride;
  for (uint32_t g = warp; g < groups; g += 8) {
    float xs[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t i = g * 128 + lane * 4 + j;
      const float v = pre(i) * inv;
      xs[j] = bf16r(weighted ? v * __bfloat162float(gamma[i]) : v) * up;
    }
    const uint32_t h01 = __nv_cvt_float2_to_fp8x2(make_float2(xs[0], xs[1]), __NV_SATFINITE, __NV_E4M3);
    const uint32_t h23 = __nv_cvt_float2_to_fp8x2(make_float2(xs[2], xs[3]), __NV_SATFINITE, __NV_E4M3);
    const float2 hf01 = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)h01, __NV_E4M3)));
    const float2 hf23 = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)h23, __NV_E4M3)));
    const float ls = LO16 ? 16.0f : 1.0f;
    const float2 r01 = make_float2((xs[0] - hf01.x) * ls, (xs[1] - hf01.y) * ls);
    const float2 r23 = make_float2((xs[2] - hf23.x) * ls, (xs[3] - hf23.y) * ls);
    const uint32_t l01 = __nv_cvt_float2_to_fp8x2(r01, __NV_SATFINITE, LO16 ? __NV_E4M3 : __NV_E5M2);
    const uint32_t l23 = __nv_cvt_float2_to_fp8x2(r23, __NV_SATFINITE, LO16 ? __NV_E4M3 : __NV_E5M2);
    if (PERM) {
      // elements 4j..4j+3 of a 32-chunk (j = lane % 8): 4j and 4j+2 are even elements 2j, 2j+1 -> positions 2j, 2j+1;
      // 4j+1 and 4j+3 are odd elements 2j, 2j+1 -> positions 16+2j, 16+2j+1
      const uint32_t base = g * 128 + (lane >> 3) * 32 + (lane & 7u) * 2;
      const uint16_t h_even = (uint16_t)((h01 & 0xffu) | ((h23 & 0xffu) << 8)), h_odd = (uint16_t)((h01 >> 8) | (h23 & 0xff00u));
      const uint16_t l_even = (uint16_t)((l01 & 0xffu) | ((l23 & 0xffu) << 8)), l_odd = (uint16_t)((l01 >> 8) | (l23 & 0xff00u));
      *reinterpret_cast<uint16_t *>(hi_row + base) = h_even;
      *reinterpret_cast<uint16_t *>(hi_row + base + 16) = h_odd;
      *reinterpret_cast<uint16_t *>(lo_row + base) = l_even;
      *reinterpret_cast<uint16_t *>(lo_row + base + 16) = l_odd;
    } else {
      *reinterpret_cast<uint32_t *>(hi_row + g * 128 + lane * 4) = (h01 & 0xffffu) | (h23 << 16);
      *reinterpret_cast<uint32_t *>(lo_row + g * 128 + lane * 4) = (l01 & 0xffffu) | (l23 << 16);
    }
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

// activation planes [2][m][k] bytes: box = 128 (k) x tt (tokens) x 1 (plane), 128-byte swizzle, zero fill outside
bool make_x_map(CUtensorMap *map, const void *planes, uint32_t m, uint32_t k, uint32_t tt, uint32_t ks) {
  EncodeTiled enc = encode_tiled();
  if (enc == nullptr) return false;
  const cuuint64_t dims[3] = {k, m, 2};
  const cuuint64_t strides[2] = {k, (cuuint64_t)m * k};
  const cuuint32_t box[3] = {ks, tt, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(planes), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, ks == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// stored weight bytes [n][row_bytes]: FP8 box 128 B x 128 rows with the 128-byte swizzle (the operand tile
// itself); AQ4 box 64 B x 128 rows, unswizzled (read back by the converter warps)
bool make_w_map(CUtensorMap *map, const void *w, uint32_t n, uint32_t k, uint32_t enc_id, uint32_t ks) {
  EncodeTiled enc = encode_tiled();
  if (enc == nullptr) return false;
  const uint32_t row_bytes = enc_id == AQ4 ? k / 2 : k;
  const cuuint64_t dims[2] = {row_bytes, n};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {enc_id == AQ4 ? BKB / 2u : ks, BM};
  const cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(w), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE,
             enc_id == AQ4 ? CU_TENSOR_MAP_SWIZZLE_NONE : (ks == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B),
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// bf16 output [m][y_stride]: box = 32 channels x 32 tokens (one epilogue warp's piece), no swizzle, clipped at the edges
bool make_y_map(CUtensorMap *map, const void *y, uint32_t m, uint32_t n, uint64_t y_stride) {
  EncodeTiled enc = encode_tiled();
  if (enc == nullptr) return false;
  const cuuint64_t dims[2] = {n, m};
  const cuuint64_t strides[1] = {y_stride * 2};
  const cuuint32_t box[2] = {32, 32};
  const cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(y), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <uint32_t ENC, int TT, int RT, int KS = BKB, bool PAIR = false>
cudaError_t launch_tile(cudaStream_t stream, const CUtensorMap &wmap, const CUtensorMap &xmap, const CUtensorMap *ymap,
                        GemmParams p, uint32_t grid) {
  constexpr size_t stage = kps_of<ENC, TT, KS, PAIR>() * ((size_t)RT * BM * KS + 2 * (size_t)(PAIR ? TT / 2 : TT) * KS);
  constexpr size_t raw_stage = (size_t)RT * RAW_BYTES;
  constexpr size_t budget = 227u * 1024u - 2048u;  // the opt-in maximum less alignment slack and static shared memory
  size_t ns = 0, rs = 0;
  constexpr size_t out_one = (size_t)kEpiWarps * 2048;  // one staging slot per epilogue warp
  if (ENC == AQ4) {
    // the epilogue's staging slots come out of the nibble ring's share
    const size_t out_aq4 = (TT >= 128 && ymap != nullptr) ? out_one : 0;
    ns = (budget - out_aq4 - 3 * raw_stage) / stage;
    if (ns > MAX_STAGES) ns = MAX_STAGES;
    rs = (budget - out_aq4 - ns * stage) / raw_stage;
    if (rs > MAX_RAW) rs = MAX_RAW;
  } else {
    ns = budget / stage;
    if (ns > MAX_STAGES) ns = MAX_STAGES;
  }
  // staging for the TMA stores of the epilogue (wide FP8 tiles, bf16 output): two 2 KiB slots per epilogue warp
  // if they fit beside the stages, else one; a stage is given up only if not even that fits
  size_t out_bytes = 0;
  p.out_bufs = 0;
  if (ENC == AQ4 && TT >= 128 && ymap != nullptr) {
    p.out_bufs = 1;
    out_bytes = out_one;
  }
  if (ENC == FP8 && TT >= 128 && ymap != nullptr) {
    constexpr size_t one = out_one;
    if (ns * stage + 2 * one <= budget) {
      p.out_bufs = 2;
    } else if (ns * stage + one <= budget) {
      p.out_bufs = 1;
    } else if (ns > 2) {
      --ns;
      p.out_bufs = ns * stage + 2 * one <= budget ? 2 : 1;
    }
    out_bytes = p.out_bufs * one;
  }
  p.stages = (uint32_t)ns;
  p.raw_stages = (uint32_t)rs;
  const size_t smem = ns * stage + rs * raw_stage + out_bytes + 1024;
  auto kern = gemm_kernel<ENC, TT, RT, KS, PAIR>;
  // function attributes are per device: raised once per (device, kernel)
  static std::mutex mu;
  static bool configured[kMaxDevices] = {};
  {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> g(mu);
    if (!configured[dev]) {  // the largest size any launch of this instantiation asks for
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(budget + 1024));
      if (e != cudaSuccess) return e;
      configured[dev] = true;
    }
  }
  // programmatic dependent launch: barrier setup and tensor-memory allocation overlap the kernel that
  // writes the activation planes; the roles that read its output wait for it (griddepcontrol.wait)
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (PAIR) {
    if (grid % 2 != 0) return cudaErrorInvalidValue;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  return cudaLaunchKernelEx(&cfg, kern, wmap, xmap, ymap != nullptr ? *ymap : xmap, p);
}

#ifdef ULLM_CUDA_TUNING
// Tuning builds only (-DULLM_CUDA_TUNING): ULLM_CUDA_GEMM_TOKENS / _ROWS / _WHOLE / _STAGE_K override the tile
// choices below.  The shipped library reads no environment variable.
int env_int(const char *name) {
  const char *s = std::getenv(name);
  return s ? std::atoi(s) : 0;
}
#else
constexpr int env_int(const char *) { return 0; }
#endif

// CTA pairs for wide FP8 tiles unless a tuning build says otherwise
constexpr bool kPairsByDefault = true;

int tile_tokens(uint32_t m, uint32_t enc) {
  static const int forced = env_int("ULLM_CUDA_GEMM_TOKENS");
  const int cap = enc == AQ4 ? 128 : 256;  // AQ4 keeps TT/2 running sums per epilogue thread in registers
  if (forced >= 16 && forced <= cap && (forced & (forced - 1)) == 0) return forced;
  int tt = 16;
  while (tt < cap && (uint32_t)tt < m) tt *= 2;
  return tt;
}

inline size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

// Where everything lives in the scratch area, and how the problem is cut up.
struct Plan {
  int tt = 0, rt = 1;
  bool cta_pairs = false;  // clusters of two CTAs share 256-row tiles (tcgen05 cta_group::2)
  uint32_t tiles = 0, grid = 0, whole_rounds = 0, sk_tile0 = 0, sk_ctas = 0;
  bool m_fastest = false;
  size_t off_planes = 0, off_tok = 0, off_pair = 0, off_partial = 0, bytes = 0;
};

Plan make_plan(const Context *ctx, const LinearArgs &a, bool allow_partials) {
  Plan pl;
  const uint32_t sms = ctx != nullptr && ctx->sm_count > 0 ? (uint32_t)ctx->sm_count : 148u;
  pl.tt = tile_tokens(a.m, a.encoding);
  // 256 weight rows per tile (two row blocks sharing the activation tile) once there is enough work for
  // every SM: fewer activation bytes per FLOP through the L2 -> shared memory path
  static const int forced_rows = env_int("ULLM_CUDA_GEMM_ROWS");
  const uint32_t tiles_m = (a.m + pl.tt - 1) / pl.tt;
  if (a.encoding == FP8 && pl.tt == 256) {
    // Measured (PFLOP/s, 128 vs 256 rows): 1.06 / 0.89 at 2048 x 14336 x 4096, 1.03 / 1.17 at 2048 x 4096 x 14336,
    // 1.16 / 1.27 at 4096 x 57344 x 8192.  The 256-row accumulators fill tensor memory, so that tile's epilogue
    // does not overlap the next tile's MMAs: it pays off once K is long enough to amortise it.
    const uint32_t tiles2 = ((a.n + 2 * BM - 1) / (2 * BM)) * tiles_m;
    pl.rt = (a.k >= 8192 && tiles2 >= sms) ? 2 : 1;
    if (forced_rows == 128) pl.rt = 1;
    if (forced_rows == 256) pl.rt = 2;
    // CTA pairs wherever the second CTA of a pair has rows of its own
    static const int forced_pairs = env_int("ULLM_CUDA_GEMM_PAIRS");
    pl.cta_pairs = kPairsByDefault && sms % 2 == 0 && a.n > (uint32_t)BM;
    if (forced_pairs == 1) pl.cta_pairs = sms % 2 == 0;
    if (forced_pairs == 2) pl.cta_pairs = false;
    if (pl.cta_pairs) pl.rt = 1;
  }
  // workers walk the tiles: CTAs, or CTA pairs with 256-row tiles
  const uint32_t per_worker = pl.cta_pairs ? 2u : 1u;
  const uint32_t workers = sms / per_worker;
  const uint32_t tile_rows = (pl.cta_pairs ? 2 : pl.rt) * BM;
  const uint32_t tiles_n = (a.n + tile_rows - 1) / tile_rows;
  const uint32_t kb = a.k / BKB;
  pl.tiles = tiles_n * tiles_m;
  uint32_t grid = pl.tiles < workers ? pl.tiles : workers;
  // Whole tiles only: ceil(tiles / grid) rounds.  Hybrid: the full rounds whole, the remaining tiles cut
  // along K over the workers, which costs each CTA up to two partial tiles (written, fenced, read back).
  // Costs in k-block times.
  static const int forced_whole = env_int("ULLM_CUDA_GEMM_WHOLE");
  const uint32_t full = pl.tiles / workers, rem = pl.tiles % workers;
  // Measured on B200 (whole tiles against hybrid over 15 shapes per encoding): a kernel with partial tiles pays
  // about 40 us at 256 tokens per tile, 10 us at 128, a few us below, whatever the matrix size.
  double part = (pl.tt >= 256 ? 24.0 : pl.tt >= 128 ? 12.0 : 8.0) * pl.rt;
  if (a.encoding == AQ4) part /= 2.5;  // its k-blocks take 2.5 times as long
  const double cost_whole = (double)((pl.tiles + workers - 1) / workers) * kb;
  const double cost_hybrid = (double)full * kb + (rem ? (double)rem * kb / workers + 2.0 * part : 0.0);
  const bool hybrid = allow_partials && rem != 0 && (uint64_t)rem * kb >= 8 && forced_whole != 1 &&
                      (forced_whole == 2 || cost_hybrid < cost_whole);
  if (hybrid) {
    grid = workers;
    pl.whole_rounds = full;
    pl.sk_tile0 = full * workers;
    uint64_t ranges = (uint64_t)rem * kb / 4;  // at least four k-blocks per range
    pl.sk_ctas = (uint32_t)(ranges > workers ? workers : ranges);
  } else {
    pl.whole_rounds = (pl.tiles + grid - 1) / grid;
    pl.sk_tile0 = pl.tiles;
    pl.sk_ctas = 0;
  }
  pl.grid = grid * per_worker;
  pl.m_fastest = (uint64_t)2 * a.m * a.k <= (uint64_t)96 << 20;  // the activation planes stay in L2
  size_t off = 0;
  pl.off_planes = off;
  off += align256((size_t)2 * a.m * a.k);
  pl.off_tok = off;
  off += align256((size_t)a.m * 4);
  pl.off_pair = off;
  if (a.epilogue == ULLM_CUDA_EPILOGUE_SWIGLU) off += align256((size_t)a.m * a.n * 2);
  pl.off_partial = off;
  if (pl.sk_ctas != 0) off += align256((size_t)pl.sk_ctas * per_worker * 2 * pl.rt * pl.tt * BM * 4);
  pl.bytes = off;
  return pl;
}

// the planes and token scales of at most this many bytes of bf16 activations fit the static array
constexpr size_t kStaticExtra = ULLM_CUDA_STATIC_SCRATCH_BYTES / 32 + 1024;

cudaError_t run_plan(const Context *ctx, cudaStream_t stream, const LinearArgs &a, const Plan &pl, uint8_t *scratch,
                     uint32_t *tile_counters, int *launches) {
  if (encode_tiled() == nullptr) return cudaErrorNotSupported;  // the driver does not offer cuTensorMapEncodeTiled
  uint8_t *planes = scratch + pl.off_planes;
  float *tok = reinterpret_cast<float *>(scratch + pl.off_tok);
  const __nv_bfloat16 *gamma = static_cast<const __nv_bfloat16 *>(a.norm_weight);
  const bool lo16 = pl.tt <= 64;  // narrow tiles: the two planes are one operand, the rest plane is e4m3(16 * rest)
  const uint64_t pstride = (uint64_t)a.m * a.k;
  {
    using PlanesKernel = void (*)(const void *, uint32_t, uint64_t, uint32_t, uint32_t, float, const __nv_bfloat16 *, uint8_t *,
                                  uint64_t, float *);
    const PlanesKernel kern = a.encoding == AQ4 ? (lo16 ? act_planes_kernel<true, true> : act_planes_kernel<true, false>)
                                                : (lo16 ? act_planes_kernel<false, true> : act_planes_kernel<false, false>);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(a.m);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t le = cudaLaunchKernelEx(&cfg, kern, a.x, a.x_dtype, a.x_stride, a.k, a.prologue, a.rms_eps, gamma, planes, pstride, tok);
    if (le != cudaSuccess) return le;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  ++*launches;
  const bool pair = a.epilogue == ULLM_CUDA_EPILOGUE_SWIGLU;
  GemmParams p{};
  p.scales = a.scales;
  p.tok_scale = tok;
  p.m = a.m;
  p.n = a.n;
  p.k = a.k;
  p.whole_rounds = pl.whole_rounds;
  p.sk_tile0 = pl.sk_tile0;
  p.sk_ctas = pl.sk_ctas;
  p.m_fastest = pl.m_fastest ? 1u : 0u;
  p.partial = pl.sk_ctas == 0 ? nullptr : reinterpret_cast<float *>(scratch + pl.off_partial);
  p.tile_counters = tile_counters;
  p.flags = ctx->device_flags;
  p.abort_word = a.abort_word != nullptr ? a.abort_word : ctx->abort_word;
  p.wait_ns = (uint64_t)(a.wait_limit_ms != 0 ? a.wait_limit_ms : kDefaultWaitLimitMs) * 1000000ull;
  p.residual = pair ? nullptr : a.residual;
  p.res_stride = a.res_stride;
#ifdef ULLM_CUDA_TUNING
  p.stats = nullptr;
  p.dbg = (uint32_t)env_int("ULLM_CUDA_GEMM_DBG");
  static const bool want_stats = env_int("ULLM_CUDA_GEMM_STATS") == 1;
  if (want_stats) {
    static unsigned long long *buf = nullptr;
    if (buf == nullptr && cudaMalloc(reinterpret_cast<void **>(&buf), 16 * sizeof(unsigned long long)) != cudaSuccess) buf = nullptr;
    if (buf != nullptr && cudaMemsetAsync(buf, 0, 16 * sizeof(unsigned long long), stream) == cudaSuccess) p.stats = buf;
  }
#endif
  if (pair) {  // gate|up to scratch as bf16, combined afterwards
    p.y = scratch + pl.off_pair;
    p.y_stride = a.n;
    p.y_dtype = ULLM_CUDA_DTYPE_BF16;
  } else {
    p.y = a.y;
    p.y_stride = a.y_stride;
    p.y_dtype = a.y_dtype;
  }
  CUtensorMap wmap, xmap;
  // k per stage of the widest FP8 tiles: CTA pairs hold half the tokens each, so four whole k-blocks fit and every
  // barrier round trip covers twice the work (measured 1.12 vs 0.98 PFLOP/s at 2048 x 14336 x 4096); a single CTA's
  // 256-token stages are too large for more than two whole k-blocks, it takes half k-blocks
  static const int forced_stage_k = env_int("ULLM_CUDA_GEMM_STAGE_K");
  uint32_t ks = 128u;
  if (a.encoding == FP8 && pl.tt == 256) {
    ks = pl.cta_pairs ? 128u : 64u;
    if (forced_stage_k == 64 || forced_stage_k == 128) ks = (uint32_t)forced_stage_k;
  }
  // bf16 results of wide FP8 tiles leave by TMA stores when the output allows it (16-byte aligned rows)
  CUtensorMap ymap_store;
  const CUtensorMap *ymap = nullptr;
  if (pl.tt >= 128 && p.y_dtype == ULLM_CUDA_DTYPE_BF16 && (reinterpret_cast<uintptr_t>(p.y) & 15u) == 0 &&
      (p.y_stride * 2) % 16 == 0 && make_y_map(&ymap_store, p.y, a.m, a.n, p.y_stride))
    ymap = &ymap_store;
  // a CTA of a pair loads half of the tile's tokens
  if (!make_w_map(&wmap, a.w, a.n, a.k, a.encoding, ks) ||
      !make_x_map(&xmap, planes, a.m, a.k, (uint32_t)(pl.cta_pairs ? pl.tt / 2 : pl.tt), ks))
    return cudaErrorInvalidValue;
  if (a.encoding == AQ4) {
    switch (pl.tt) {
      case 16: e = launch_tile<AQ4, 16, 1>(stream, wmap, xmap, ymap, p, pl.grid); break;
      case 32: e = launch_tile<AQ4, 32, 1>(stream, wmap, xmap, ymap, p, pl.grid); break;
      case 64: e = launch_tile<AQ4, 64, 1>(stream, wmap, xmap, ymap, p, pl.grid); break;
      default: e = launch_tile<AQ4, 128, 1>(stream, wmap, xmap, ymap, p, pl.grid); break;
    }
  } else {
    switch (pl.tt) {
      case 16: e = launch_tile<FP8, 16, 1>(stream, wmap, xmap, ymap, p, pl.grid); break;
      case 32: e = launch_tile<FP8, 32, 1>(stream, wmap, xmap, ymap, p, pl.grid); break;
      case 64: e = launch_tile<FP8, 64, 1>(stream, wmap, xmap, ymap, p, pl.grid); break;
      case 128: e = launch_tile<FP8, 128, 1>(stream, wmap, xmap, ymap, p, pl.grid); break;
      default:
        if (pl.cta_pairs)
          e = ks == 64 ? launch_tile<FP8, 256, 1, 64, true>(stream, wmap, xmap, ymap, p, pl.grid)
                       : launch_tile<FP8, 256, 1, BKB, true>(stream, wmap, xmap, ymap, p, pl.grid);
        else if (ks == 64)
          e = pl.rt == 2 ? launch_tile<FP8, 256, 2, 64>(stream, wmap, xmap, ymap, p, pl.grid)
                         : launch_tile<FP8, 256, 1, 64>(stream, wmap, xmap, ymap, p, pl.grid);
        else
          e = pl.rt == 2 ? launch_tile<FP8, 256, 2>(stream, wmap, xmap, ymap, p, pl.grid)
                         : launch_tile<FP8, 256, 1>(stream, wmap, xmap, ymap, p, pl.grid);
        break;
    }
  }
  if (e != cudaSuccess) return e;
  ++*launches;
#ifdef ULLM_CUDA_TUNING
  if (p.stats != nullptr) {  // ULLM_CUDA_GEMM_STATS=1: share of the time each single-thread role spent waiting
    unsigned long long h[16];
    if (cudaStreamSynchronize(stream) == cudaSuccess && cudaMemcpy(h, p.stats, sizeof(h), cudaMemcpyDeviceToHost) == cudaSuccess) {
      auto pct = [](unsigned long long a, unsigned long long b) { return b ? 100.0 * (double)a / (double)b : 0.0; };
      std::fprintf(stderr, "gemm stats m=%u n=%u k=%u pairs=%d tt=%d rt=%d: TMA waits empty %.1f%% | MMA waits full %.1f%% acc_empty %.1f%% | epilogue waits acc_full %.1f%% (clocks/CTA %.0f)\n",
                   a.m, a.n, a.k, (int)pl.cta_pairs, pl.tt, pl.rt, pct(h[1], h[0]), pct(h[4], h[3]), pct(h[5], h[3]), pct(h[7], h[6]),
                   (double)h[6] / (double)pl.grid);
      std::fprintf(stderr, "  MMA thread: fence %.1f%% issue %.1f%% commits %.1f%% of its %.0f clocks\n", pct(h[13], h[3]), pct(h[14], h[3]),
                   pct(h[15], h[3]), (double)h[3] / (double)(pl.cta_pairs ? pl.grid / 2 : pl.grid));
      if (a.encoding == AQ4)
        std::fprintf(stderr, "  AQ4: MMA waits converted tile %.1f%% | converter waits nibbles %.1f%% free tile %.1f%% (clocks/CTA %.0f)\n",
                     pct(h[12], h[3]), pct(h[10], h[9]), pct(h[11], h[9]), (double)h[9] / (double)pl.grid);
    }
  }
#endif
  if (pair) {
    dim3 g2((a.n / 2 + 255) / 256 > 64 ? 64 : (a.n / 2 + 255) / 256, a.m);
    swiglu_kernel<<<g2, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16 *>(scratch + pl.off_pair), a.n / 2,
                                          static_cast<__nv_bfloat16 *>(a.y), a.y_stride);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    ++*launches;
  }
  return cudaSuccess;
}

}  // namespace

// A shape-only answer: no handle, driver or device is consulted (the weight span is 16-byte aligned by the
// buffer rules; a driver without cuTensorMapEncodeTiled is reported when the op is enqueued).
bool gemm_supports(const LinearArgs &a, const char **why) {
  if (a.k % 128 != 0) {
    *why = "the GEMM kernel needs K to be a multiple of 128";
    return false;
  }
  return true;
}

// Scratch owned by a queue: grows on demand, reused by every GEMM enqueued on that queue (which orders them).
static cudaError_t ensure_scratch(GemmScratch *sc, cudaStream_t stream, size_t bytes, void **out) {
  std::lock_guard<std::mutex> g(sc->mutex);
  if ((sc->tile_counters == nullptr || sc->bytes < bytes) && stream != nullptr) {
    // an allocation would invalidate a stream capture in progress: refuse instead (run the same linear once
    // outside the capture, or create the stack, which reserves its scratch, before capturing)
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    cudaError_t e = cudaStreamIsCapturing(stream, &cs);
    if (e != cudaSuccess) return e;
    if (cs != cudaStreamCaptureStatusNone) return cudaErrorStreamCaptureUnsupported;
  }
  if (sc->tile_counters == nullptr) {
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&sc->tile_counters), kMaxCounterTiles * sizeof(uint32_t));
    if (e != cudaSuccess) return e;
    e = cudaMemset(sc->tile_counters, 0, kMaxCounterTiles * sizeof(uint32_t));
    if (e != cudaSuccess) return e;
  }
  if (sc->bytes < bytes) {
    if (sc->ptr != nullptr) {
      // earlier GEMMs of this queue may still be reading the old area: it is released behind them
      void *old = sc->ptr;
      sc->ptr = nullptr;
      sc->bytes = 0;
      int dev = 0;
      (void)cudaGetDevice(&dev);
      if (stream != nullptr)
        (void)retire_behind(dev, stream, [old] { (void)cudaFree(old); });
      else
        (void)cudaFree(old);
    }
    cudaError_t e = cudaMalloc(&sc->ptr, bytes);
    if (e != cudaSuccess) return e;
    sc->bytes = bytes;
  }
  *out = sc->ptr;
  return cudaSuccess;
}

cudaError_t gemm_reserve_scratch(GemmScratch *sc, size_t bytes) {
  void *unused = nullptr;
  return ensure_scratch(sc, nullptr, bytes, &unused);
}

size_t gemm_scratch_bytes(const Context *ctx, const LinearArgs &a) { return make_plan(ctx, a, true).bytes; }

// ---- allocation-free variant ---------------------------------------------------------------------
// Staging area of the allocation-free entry point.  `g_static_scratch` names a host-side shadow in
// host code, never a device address: the address is looked up once per device below.
static __device__ __align__(256) uint8_t g_static_scratch[ULLM_CUDA_STATIC_SCRATCH_BYTES + kStaticExtra];

static cudaError_t static_scratch_address(int device, uint8_t **out) {
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
  if ((uint64_t)a.m * a.k * 2 > ULLM_CUDA_STATIC_SCRATCH_BYTES) return -2;
  const Plan pl = make_plan(ctx, a, false);  // whole tiles per CTA: partial tiles would need an allocation
  if (pl.bytes > sizeof(g_static_scratch)) return -2;
  uint8_t *scratch = nullptr;
  *err = static_scratch_address(ctx->device, &scratch);
  if (*err != cudaSuccess) return -1;
  int launches = 0;
  *err = run_plan(ctx, stream, a, pl, scratch, nullptr, &launches);  // whole tiles only: no arrival counters
  return *err == cudaSuccess ? launches : -1;
}

int launch_gemm(const Context *ctx, GemmScratch *scratch, cudaStream_t stream, const LinearArgs &a, cudaError_t *err) {
  const Plan pl = make_plan(ctx, a, true);
  void *s = nullptr;
  *err = ensure_scratch(scratch, stream, pl.bytes, &s);
  if (*err != cudaSuccess) return -1;
  int launches = 0;
  *err = run_plan(ctx, stream, a, pl, static_cast<uint8_t *>(s), scratch->tile_counters, &launches);
  return *err == cudaSuccess ? launches : -1;
}

}  // namespace ullm
