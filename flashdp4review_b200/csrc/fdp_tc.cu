// Tensor-core path for bf16 / fp16: one persistent, warp-specialised GEMM kernel template built
// on TMA (cp.async.bulk.tensor, 128-byte swizzle) -> shared-memory ring -> tcgen05.mma with fp32
// accumulators in TMEM -> tcgen05.ld epilogue.  Instances (A major, B major, epilogue, CTAs per tile):
//   wgrad   MN, MN, STORE_SCALED, 2   dW = scale * sum_b c_b G_b^T X_b + noise; every sample's K segment has
//                                     its own TMEM accumulator, added times c_b into registers
//           MN, MN, STORE, 2          same from a pre-scaled copy of G (T not a multiple of 64, or short T)
//   direct  MN, MN, SUMSQ, 1          per-sample ||G_b^T X_b||_F^2: tile squared in the epilogue, never stored
//   gram    K,  K,  GRAM, 1           sum_{t,s} (G_b G_b^T)_{ts} (X_b X_b^T)_{ts}, two accumulators in TMEM
//   dgrad   K,  MN or K, STORE, 2     dX = G W
//   forward K,  K or MN, STORE, 2     Y = X W^T + bias
// Roles in a CTA: warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 2-5 (2-9 for the
// store epilogues) = epilogue, each on the TMEM lane quarter warp % 4.  With two CTAs per tile the
// even CTA of a 2-CTA cluster issues tcgen05.mma.cta_group::2 for both.  Every mbarrier wait is
// bounded: when one runs out the CTA records a code in the status word, drains and leaves.
// No TMA load here uses cluster multicast.
#include <cuda.h>
#include <atomic>
#include <cstdlib>
#include <mutex>

#include "fdp_async.cuh"
#include "fdp_gram_units.h"
#include "fdp_kernels.h"

namespace fdp {
namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int BAR_BYTES = 256;
// EPI_STORE_SCALED keeps the clip factors of up to MAX_SMEM_FACTORS samples in shared memory
constexpr int MAX_SMEM_FACTORS = 4096;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + BAR_BYTES;
constexpr int SMEM_BYTES_SCALED = SMEM_BYTES + MAX_SMEM_FACTORS * 4;
constexpr int TMEM_COLS = 512;
constexpr int MAX_SMS = 148;           // workers the split-K parking area is sized for

// EPI_STORE_SCALED: the accumulator of each sample (K segment) is drained on its own and added, times
// that sample's clip factor, to fp32 registers of eight epilogue warps; G needs no scaled copy.
enum { EPI_STORE = 0, EPI_SUMSQ = 1, EPI_GRAM = 2, EPI_STORE_SCALED = 3 };
// eight epilogue warps (two per TMEM lane quarter, 128 columns each) for the store epilogues, four for the norms
#ifndef FDP_EPI_STORE_WARPS
#define FDP_EPI_STORE_WARPS 8
#endif
__host__ __device__ constexpr int epi_warps_for(int epi) { return epi == EPI_STORE_SCALED ? 8 : (epi == EPI_STORE ? FDP_EPI_STORE_WARPS : 4); }
constexpr int threads_for(int epi) { return 64 + 32 * epi_warps_for(epi); }
constexpr int smem_for(int epi) { return epi == EPI_STORE_SCALED ? SMEM_BYTES_SCALED : SMEM_BYTES; }

struct TcArgs {
  int M, N;             // extents of the output space of one batch (masks)
  int tiles_m, tiles_n; // tile grid of one batch
  int tiles_per_batch;
  int n_fastest;        // tile order: 1 = consecutive tiles walk along N (keeps the B operand in L2), 0 = along M
  int batch;
  int k_stages, k_stages2;  // K loop of operand pair 1 (and pair 2 for EPI_GRAM)
  int batch_rows;           // rows of one batch along the row coordinate of the tensor maps
  void* out; int out_dt; long long ld_out; float scale; NoiseKey nk;
  float* partials;      // norm passes: one partial per (work unit, epilogue warp)
  int T;
  int* status;          // status word of the call (workspace)
  int zero_status;      // this launch is the first of its call: its first thread clears the status word
  int dependent;        // host side: launch as a programmatic dependent of the kernel before it in the stream
  int sub_stages;       // EPI_STORE_SCALED: K stages per accumulator hand-off (<= seg_stages; chains of fp32 tensor mode)
  int norm_mode;        // EPI_STORE_SCALED: 1 = no store, sum of squares of the unit's accumulated tile -> partials;
                        // 2 = plain product (factor = scale for every segment), stored as usual
  int* sticky;          // this device's slot of the host-visible status array, or null
  uint32_t idesc;
  // split-K (store epilogues): work units [0, units_full) are whole tiles; each later tile is cut into
  // `split` K-stage ranges whose fp32 accumulators are parked in split_ws[slot][BM][BN]; the fix-up
  // kernel adds the parts in index order, adds the noise and stores the tile.  Nobody waits.
  // (Tried: the part that finishes last -- a ticket per tile -- sums the parts inside this kernel.
  // At B=16, T=1024, 1024->3072 that took 0.19 ms against 0.10 ms with the separate launch: the
  // sums then sit on the critical path of a few warps instead of spreading over the whole GPU.)
  int units_full, split;
  float* split_ws;
  // EPI_STORE_SCALED: K is `segs` segments (samples) of `seg_stages` stages; every segment has its own
  // accumulator, scaled by that sample's clip factor when it is drained.  The factors come either from
  // `factors` (global, computed by an earlier kernel) or, when norm_partials != null, from the norm
  // pass's partial sums: the epilogue warps reduce them into shared memory while the first main loop
  // runs, and the first CTA also writes the norms and factors out.
  const float* factors;
  int segs, seg_stages;
  const float* norm_partials; int norm_nparts; float C, clamp;
  float* norms_ws; float* factors_ws; float* norms_out; float* factors_out;
  // EPI_GRAM: the T x T plane of a sample is cut into 128 x 128 blocks; only blocks (i, j) with j >= i
  // are computed (weight 2, the diagonal ones weight 1).  A work unit is one t-block i against TWO
  // s-blocks j1, j2 (an N = 256 MMA whose B stage is filled by two 128-row copies), see gram_decode;
  // at most one unit per sample has a single block (N = 128, idesc_half).  Units are numbered sample
  // by sample and all cost the same, so round-robin dealing is balanced.
  int gram_nb;          // 128-row blocks per sample
  uint32_t idesc_half;
  // store epilogue: optional bias[N] (same 16-bit type as the operands) added to every row
  const void* bias; int bias_dt;
  // fp32 inputs as three bf16 products.  Both operand matrices are then [rows, 2n]: the high bf16
  // halves of the n columns, then the low halves (x = hi + lo up to 2^-18 |x|).  With terms = 3 the K
  // loop visits every K range three times -- hi*hi, hi*lo, lo*hi -- into the same accumulator (lo*lo,
  // 2^-18 of the product, is dropped).  term_stages: K stages of one term before the next term of the
  // same range begins (a sample's rows for the per-sample kernels; pair 2 of EPI_GRAM: term_stages2).
  // plane_*: columns of one half of the A / B matrix, i.e. the column offset of its low halves.
  int terms, term_stages, term_stages2;
  int plane_a, plane_b, plane_a2, plane_b2;
  // store GEMMs: tiles are walked in groups of m_group tile rows (0 = plain order), so that the CTAs
  // running together cover a squarer patch of the output and re-read less of the operands
  int m_group;
};

// ---- PTX wrappers (mbarrier helpers live in fdp_async.cuh) --------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
// ---- CTA-pair (cta_group::2) helpers: the even CTA of a 2-CTA cluster issues one 256-row MMA for both;
// loads are per CTA (no multicast), completion is signalled on the leader's mbarrier ------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(leader_bar) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t r[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// shared-memory matrix descriptor (sm_100 format): start address, leading / stride byte offsets in
// 16-byte units, version 1, 128-byte swizzle
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;  // descriptor version of sm_100
  d |= static_cast<uint64_t>(2) << 61;  // SWIZZLE_128B
  return d;
}
// Descriptor of the k16-th UMMA_K slice of an operand stage.
//  MN-major: 64-element (128 B) MN chunks of BK rows each, chunk stride BK*128 B (leading offset),
//            8-row groups 1024 B apart (stride offset); a K=16 slice is 16 rows = 2048 B further.
//  K-major : rows of 128 B (64 K elements), 8-row groups 1024 B apart; a K=16 slice is 32 B further.
template <bool MN_MAJOR>
__device__ __forceinline__ uint64_t operand_desc(uint32_t stage_base, int k16) {
  if (MN_MAJOR) return make_desc(stage_base + k16 * (UMMA_K * 128), BK * 128, 1024);
  return make_desc(stage_base + k16 * (UMMA_K * 2), 0, 1024);
}

// The Gaussian noise of 32 adjacent output elements starting at flat index idx0 (a multiple of 4: the
// tensor-core kernels only see row pitches and column offsets that are multiples of 8).
__device__ __forceinline__ void add_noise32(const NoiseKey& nk, size_t idx0, float v[32]) {
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    float z[4];
    noise_group(nk, (idx0 >> 2) + g, z);
    v[4 * g] += z[0]; v[4 * g + 1] += z[1]; v[4 * g + 2] += z[2]; v[4 * g + 3] += z[3];
  }
}

// Finish 32 adjacent output columns of row m starting at column n: bias, noise (NOISE), convert, store.
template <bool NOISE>
__device__ __forceinline__ void store_chunk32(const TcArgs& args, float v[32], int m, int n) {
  if (m >= args.M || n >= args.N) return;
  const size_t idx0 = static_cast<size_t>(m) * args.ld_out + n;
  if (args.bias != nullptr) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (n + j < args.N) v[j] += load_as(args.bias, args.bias_dt, n + j);
  }
  if (NOISE && args.nk.std != 0.f) add_noise32(args.nk, idx0, v);
  const bool vec_ok = (args.ld_out * static_cast<long long>(dtype_size(args.out_dt))) % 16 == 0;
  if (n + 32 <= args.N && vec_ok) {
    if (args.out_dt == FDP_F32) {
      float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(args.out) + idx0);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
      uint4* o = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(args.out) + idx0);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float lo = v[8 * j + 2 * e], hi = v[8 * j + 2 * e + 1];
          if (args.out_dt == FDP_BF16) {
            __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
            w[e] = *reinterpret_cast<uint32_t*>(&h);
          } else {
            __half2 h = __floats2half2_rn(lo, hi);
            w[e] = *reinterpret_cast<uint32_t*>(&h);
          }
        }
        o[j] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (n + j < args.N) store_as(args.out, args.out_dt, idx0 + j, v[j]);
  }
}

// accr[4g .. 4g+3] += z * f with g known only at run time: a switch keeps every index static, so
// the 128 accumulators stay in registers.
__device__ __forceinline__ void add_group(float (&accr)[128], int g, const float z[4], float f) {
#define FDP_ADD_GROUP(G) case G: accr[4 * G] = fmaf(z[0], f, accr[4 * G]); accr[4 * G + 1] = fmaf(z[1], f, accr[4 * G + 1]); \
    accr[4 * G + 2] = fmaf(z[2], f, accr[4 * G + 2]); accr[4 * G + 3] = fmaf(z[3], f, accr[4 * G + 3]); break;
  switch (g) {
    FDP_ADD_GROUP(0) FDP_ADD_GROUP(1) FDP_ADD_GROUP(2) FDP_ADD_GROUP(3) FDP_ADD_GROUP(4) FDP_ADD_GROUP(5)
    FDP_ADD_GROUP(6) FDP_ADD_GROUP(7) FDP_ADD_GROUP(8) FDP_ADD_GROUP(9) FDP_ADD_GROUP(10) FDP_ADD_GROUP(11)
    FDP_ADD_GROUP(12) FDP_ADD_GROUP(13) FDP_ADD_GROUP(14) FDP_ADD_GROUP(15) FDP_ADD_GROUP(16) FDP_ADD_GROUP(17)
    FDP_ADD_GROUP(18) FDP_ADD_GROUP(19) FDP_ADD_GROUP(20) FDP_ADD_GROUP(21) FDP_ADD_GROUP(22) FDP_ADD_GROUP(23)
    FDP_ADD_GROUP(24) FDP_ADD_GROUP(25) FDP_ADD_GROUP(26) FDP_ADD_GROUP(27) FDP_ADD_GROUP(28) FDP_ADD_GROUP(29)
    FDP_ADD_GROUP(30) FDP_ADD_GROUP(31)
    default: break;
  }
#undef FDP_ADD_GROUP
}

// ---- the kernel ---------------------------------------------------------------------------------------
// CTAS = 2: a cluster of two CTAs works on one 256x256 tile.  Each CTA loads its 128 rows of A and
// its 128 columns of B (32 KiB per stage instead of 48, six stages), the even CTA issues
// tcgen05.mma.cta_group::2 (M = 256) for both, each CTA drains its own 128 accumulator rows.
template <bool A_MN, bool B_MN, int EPI, int CTAS>
__global__ void __launch_bounds__(threads_for(EPI), 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
               const __grid_constant__ TcArgs args) {
  constexpr int NST = (CTAS == 2) ? 6 : STAGES;          // ring depth
  constexpr int B_BYTES = B_STAGE_BYTES / CTAS;          // this CTA's share of the B stage
  constexpr int STG = A_STAGE_BYTES + B_BYTES;
  constexpr int BN_CTA = BN / CTAS;                      // B columns (rows if K-major) loaded by this CTA
  constexpr int EPI_WARPS = epi_warps_for(EPI);
  static_assert(NST * STG <= STAGES * STAGE_BYTES, "ring size");
  static_assert(CTAS == 1 || EPI == EPI_STORE || EPI == EPI_STORE_SCALED, "pairs: store epilogues only");
  const uint32_t cta_rank = (CTAS == 2) ? cluster_ctarank() : 0u;
  const bool is_leader = cta_rank == 0;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw_addr);
  const uint32_t bar_base = base + NST * STG;
  uint8_t* bar_gen = gen_base + NST * STG;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (NST + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * NST + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * NST + 2 + a); };
  const uint32_t drain_bar = bar_base + 8u * (2 * NST + 4);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * (2 * NST + 5));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_gen + 8 * (2 * NST + 5) + 4);
  float* sfac = reinterpret_cast<float*>(bar_gen + BAR_BYTES);   // EPI_STORE_SCALED: clip factors [segs]
  const WaitCtx wctx{abort_flag, args.status, args.sticky, WAIT_LIMIT_CYCLES};

  constexpr int NUM_ACC = (EPI == EPI_GRAM) ? 1 : 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_tiles = args.batch * args.tiles_per_batch;
  const int kst_total = args.k_stages + (EPI == EPI_GRAM ? args.k_stages2 : 0);
  const int total_units = args.units_full + (total_tiles - args.units_full) * args.split;

  if (threadIdx.x == 0) {
    // (a wait can only run out a second from now, so no report of this call can precede the clearing)
    if (args.zero_status && blockIdx.x == 0 && args.status != nullptr) *args.status = 0;
    for (int s = 0; s < NST; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), EPI_WARPS * CTAS); }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (CTAS == 2) {
    // the peer's barriers must be initialised before anything is signalled across the pair
    __syncthreads();
    cluster_sync_all();
  }
  if (warp == 1) {
    if (CTAS == 2) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                   ::"r"(smem_u32(const_cast<uint32_t*>(tmem_slot))), "r"(TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                   ::"r"(smem_u32(const_cast<uint32_t*>(tmem_slot))), "r"(TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // Barriers, TMEM and the shared-memory carve-up are ready.  Let the kernel that follows in the
  // stream be scheduled as SMs free up (it waits at this same point), and, if this launch is itself
  // a programmatic dependent, wait here for the kernel before it: nothing above touched global
  // memory that an earlier kernel writes.
  pdl_trigger();
  pdl_wait();
  // work is dealt to CTAs (or CTA pairs) round-robin
  const int wid = blockIdx.x / CTAS, wstep = gridDim.x / CTAS;
  const uint32_t tmem_base = *tmem_slot;

  // tile -> (batch, m0, n0, half).  EPI_GRAM: m0 = first row of the t-block, n0 / n1 = first rows of
  // the two s-blocks (n1 < 0 and half = 1 for a single-block unit)
  int gram_n1 = -1;
  auto decode = [&](int tile, int& b, int& m0, int& n0, int& half) {
    half = 0;
    b = tile / args.tiles_per_batch;
    int q = tile - b * args.tiles_per_batch;
    if (EPI == EPI_GRAM) {
      int i, j1, j2;
      gram_decode(args.gram_nb, q, i, j1, j2);
      m0 = i * BM; n0 = j1 * BM;
      gram_n1 = j2 >= 0 ? j2 * BM : -1;
      half = j2 < 0;
      return;
    }
    int mi, ni;
    if (args.n_fastest) {
      ni = q % args.tiles_n; mi = q / args.tiles_n;
    } else if (args.m_group > 0) {
      const int per_group = args.m_group * args.tiles_n;
      const int g = q / per_group, r = q - g * per_group;
      const int gm = min(args.m_group, args.tiles_m - g * args.m_group);
      mi = g * args.m_group + r % gm; ni = r / gm;
    } else {
      mi = q % args.tiles_m; ni = q / args.tiles_m;
    }
    m0 = mi * (BM * CTAS) + cta_rank * BM;
    n0 = ni * BN;
  };

  // work unit -> tile, K-stage range, slot in split_ws (-1: whole tile, normal epilogue)
  auto decode_unit = [&](int u, int& tile, int& ks0, int& ks1, int& slot) {
    if (u < args.units_full) { tile = u; ks0 = 0; ks1 = kst_total; slot = -1; return; }
    const int v = u - args.units_full;
    const int part = v % args.split;
    tile = args.units_full + v / args.split;
    ks0 = static_cast<int>(static_cast<long long>(kst_total) * part / args.split);
    ks1 = static_cast<int>(static_cast<long long>(kst_total) * (part + 1) / args.split);
    slot = v;
  };
  // EPI_STORE_SCALED: end of the sample segment that contains stage ks, cut at the unit's end
  // (sub_stages divides seg_stages: a hand-off never spans two samples.  With fp32 inputs it is a few
  // stages only: the tensor cores add into the TMEM accumulator by truncation, about one unit in the
  // last place per K = 16 step and all of one sign, so a long chain drifts; short chains summed in
  // registers with round-to-nearest do not.)
  auto segment_end = [&](int ks, int ks1) {
    const int e = (ks / args.sub_stages + 1) * args.sub_stages;
    return e < ks1 ? e : ks1;
  };

  // K stage `kl` of an operand pair's K order -> stage within the K range, and which term it belongs to
  // (0: hi*hi, 1: hi*lo, 2: lo*hi); a no-op for 16-bit inputs (terms == 1)
  auto term_of = [&](int& kl, bool second) {
    if (args.terms <= 1) return 0;
    const int ts = second ? args.term_stages2 : args.term_stages;
    const int run = args.terms * ts;
    const int blk = kl / run, w = kl - blk * run;
    const int term = w / ts;
    kl = blk * ts + (w - term * ts);
    return term;
  };

  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int u = wid; u < total_units && ok; u += wstep) {
        int tile, ks0, ks1, slot, b, m0, n0, half;
        decode_unit(u, tile, ks0, ks1, slot);
        decode(tile, b, m0, n0, half);
        const int row0 = b * args.batch_rows;
        for (int ks = ks0; ks < ks1; ++ks) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, wctx, 1)) { ok = false; break; }
          const bool second = (EPI == EPI_GRAM) && ks >= args.k_stages;
          const CUtensorMap* ma = second ? &tmA2 : &tmA;
          const CUtensorMap* mb = second ? &tmB2 : &tmB;
          int kl = second ? ks - args.k_stages : ks;
          const int term = term_of(kl, second);
          const int k0 = kl * BK;
          // column offsets of the planes this term reads (A low halves in term 2, B low halves in term 1)
          const int ca = term == 2 ? (second ? args.plane_a2 : args.plane_a) : 0;
          const int cb = term == 1 ? (second ? args.plane_b2 : args.plane_b) : 0;
          const uint32_t sa = base + stage * STG, sb = sa + A_STAGE_BYTES;
          if (EPI == EPI_GRAM) {
            // A: the t-block; B: two independent 128-row s-blocks, one per half of the stage
            // (a unit that contains the diagonal block (i, i) has its t-block in the B stage already:
            // the MMA warp points the A descriptor there and no A copy is made)
            constexpr uint32_t HALF_B = B_STAGE_BYTES / 2;
            const bool a_in_b = term == 0 && ((n0 == m0) || (gram_n1 == m0));
            mbar_expect_tx(full_bar(stage), (a_in_b ? 0 : A_STAGE_BYTES) + (gram_n1 >= 0 ? 2 : 1) * HALF_B);
            if (!a_in_b) tma_load_2d(sa, ma, k0 + ca, row0 + m0, full_bar(stage));
            tma_load_2d(sb, mb, k0 + cb, row0 + n0, full_bar(stage));
            if (gram_n1 >= 0) tma_load_2d(sb + HALF_B, mb, k0 + cb, row0 + gram_n1, full_bar(stage));
          } else if (CTAS == 1) {
            mbar_expect_tx(full_bar(stage), STG);
            if (A_MN) {
#pragma unroll
              for (int i = 0; i < BM / 64; ++i) tma_load_2d(sa + i * (BK * 128), ma, m0 + 64 * i + ca, row0 + k0, full_bar(stage));
            } else {
              tma_load_2d(sa, ma, k0 + ca, row0 + m0, full_bar(stage));
            }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * (BK * 128), mb, n0 + 64 * j + cb, row0 + k0, full_bar(stage));
            } else {
              tma_load_2d(sb, mb, k0 + cb, row0 + n0, full_bar(stage));
            }
          } else {
            // both CTAs' copies complete on the leader's barrier, which expects the bytes of both
            const uint32_t lbar = mapa_u32(full_bar(stage), 0);
            if (is_leader) mbar_expect_tx(full_bar(stage), 2 * STG);
            const int nb0 = n0 + static_cast<int>(cta_rank) * BN_CTA;
            if (A_MN) {
#pragma unroll
              for (int i = 0; i < BM / 64; ++i) tma_load_2d_pair(sa + i * (BK * 128), ma, m0 + 64 * i + ca, row0 + k0, lbar);
            } else {
              tma_load_2d_pair(sa, ma, k0 + ca, row0 + m0, lbar);
            }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN_CTA / 64; ++j) tma_load_2d_pair(sb + j * (BK * 128), mb, nb0 + 64 * j + cb, row0 + k0, lbar);
            } else {
              tma_load_2d_pair(sb, mb, k0 + cb, row0 + nb0, lbar);
            }
          }
          if (++stage == NST) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // wait (bounded) for the copies already in flight before the CTA may leave
        for (int s = 0; s < NST; ++s) {
          const long long t0 = clock64();
          const uint32_t ph = (s < stage) ? phase : (phase ^ 1u);
          while (!mbar_try(full_bar(s), ph) && clock64() - t0 < WAIT_LIMIT_CYCLES / 8) {}
        }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer (the leader CTA of a pair issues for both) =================
    if (lane == 0 && is_leader) {
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int u = wid; u < total_units && ok; u += wstep) {
        int tile, ks0, ks1, slot, tb, tm0, tn0, half;
        decode_unit(u, tile, ks0, ks1, slot);
        decode(tile, tb, tm0, tn0, half);
        // a single-block unit multiplies by the first 128 rows of the B stage only (N = 128)
        const uint32_t idesc = half ? args.idesc_half : args.idesc;
        int ks = ks0;
        // one accumulator per segment: the whole unit, or one sample's share of it for EPI_STORE_SCALED
        while (ks < ks1 && ok) {
          const int seg_begin = ks;
          const int seg_end = (EPI == EPI_STORE_SCALED) ? segment_end(ks, ks1) : ks1;
          const int acc = it % NUM_ACC;
          const uint32_t acc_phase = (it / NUM_ACC) & 1u;
          if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, wctx, 2)) { ok = false; break; }
          tc_fence_after();
          for (; ks < seg_end; ++ks) {
            if (!mbar_wait(full_bar(stage), phase, wctx, 3)) { ok = false; break; }
            tc_fence_after();
            const bool second = (EPI == EPI_GRAM) && ks >= args.k_stages;
            const uint32_t d = tmem_base + (EPI == EPI_GRAM ? (second ? BN : 0) : acc * BN);
            const bool first_stage = second ? (ks == args.k_stages) : (ks == seg_begin);
            uint32_t sa = base + stage * STG;
            const uint32_t sb = sa + A_STAGE_BYTES;
            if (EPI == EPI_GRAM) {   // diagonal block in this unit: A is the matching half of the B stage
              int kl = second ? ks - args.k_stages : ks;
              if (term_of(kl, second) == 0) {
                if (tn0 == tm0) sa = sb;
                else if (gram_n1 == tm0) sa = sb + B_STAGE_BYTES / 2;
              }
            }
#pragma unroll
            for (int k16 = 0; k16 < BK / UMMA_K; ++k16) {
              if (CTAS == 1)
                tc_mma(d, operand_desc<A_MN>(sa, k16), operand_desc<B_MN>(sb, k16), idesc,
                       (first_stage && k16 == 0) ? 0u : 1u);
              else
                tc_mma_pair(d, operand_desc<A_MN>(sa, k16), operand_desc<B_MN>(sb, k16), idesc,
                            (first_stage && k16 == 0) ? 0u : 1u);
            }
            // frees the stage (in both CTAs of a pair) once these MMAs have read it
            if (CTAS == 1) {
              tc_commit(empty_bar(stage));
            } else {
              tc_commit_pair(empty_bar(stage));
              tc_commit_pair(mapa_u32(empty_bar(stage), 1));
            }
            if (++stage == NST) { stage = 0; phase ^= 1u; }
          }
          if (ok) {
            if (CTAS == 1) {
              tc_commit(tfull_bar(acc));
            } else {
              tc_commit_pair(tfull_bar(acc));
              tc_commit_pair(mapa_u32(tfull_bar(acc), 1));
            }
            ++it;
          }
        }
      }
      if (!ok) {
        // let MMAs already issued finish before TMEM is released
        if (CTAS == 1) tc_commit(drain_bar); else tc_commit_pair(drain_bar);
        const long long t0 = clock64();
        while (!mbar_try(drain_bar, 0) && clock64() - t0 < WAIT_LIMIT_CYCLES / 8) {}
      }
    }
  } else {
    // ================= epilogue: warps 2.., TMEM lane quarter = warp % 4 =================
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int ew = warp - 2;
    int it = 0;
    bool ok = true;
    if (EPI == EPI_STORE_SCALED && args.norm_partials != nullptr) {
      // clip factors of all samples from the norm pass's partial sums (fixed order: a lane adds every
      // 32nd partial, then the shuffle tree), while the producer and MMA warps start the main loop
      for (int b = ew; b < args.segs; b += EPI_WARPS) {
        const float* pp = args.norm_partials + static_cast<size_t>(b) * args.norm_nparts;
        float sq = 0.f;
        for (int i = lane; i < args.norm_nparts; i += 32) sq += pp[i];
        sq = warp_sum(sq);
        if (lane == 0) {
          const float n = sqrtf(fmaxf(sq, 0.f));
          const float f = clip_factor(n, args.C, args.clamp);
          sfac[b] = f;
          if (blockIdx.x == 0) {
            if (args.norms_out != nullptr) args.norms_out[b] = n;
            if (args.factors_out != nullptr) args.factors_out[b] = f;
          }
        }
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");   // the eight epilogue warps
    }
    for (int u = wid; u < total_units && ok; u += wstep) {
      int tile, ks0, ks1, slot, b, m0, n0, half;
      decode_unit(u, tile, ks0, ks1, slot);
      decode(tile, b, m0, n0, half);
      const int m = m0 + row;
      if (EPI == EPI_STORE_SCALED) {
        // eight warps: two per lane quarter, each owning 128 of the tile's 256 columns in registers
        const int chalf = ew >> 2;
        float accr[128];
#pragma unroll
        for (int i = 0; i < 128; ++i) accr[i] = 0.f;
        // A whole tile's Gaussian noise goes into the accumulators a few element groups per sample
        // segment, in the time these warps would otherwise wait for the next segment's MMAs; K-split
        // parts stay noise-free (the fix-up kernel adds the noise once per tile).
        const bool pre_noise = slot < 0 && args.nk.std != 0.f && m < args.M;
        const uint64_t g0 = (static_cast<uint64_t>(m) * args.ld_out + n0 + chalf * 128) >> 2;
        const int nseg = (ks1 - 1) / args.sub_stages - ks0 / args.sub_stages + 1;
        int ng = 0, seg = 0;
        for (int ks = ks0; ks < ks1 && ok; ks = segment_end(ks, ks1), ++it) {
          const int acc = it % NUM_ACC;
          const uint32_t acc_phase = (it / NUM_ACC) & 1u;
          if (!mbar_wait_warp(tfull_bar(acc), acc_phase, wctx, 4)) { ok = false; break; }
          tc_fence_after();
          const int sample = ks / args.seg_stages;
          // the divisor goes into the factor, so the noise is added as it is drawn
          const float cbs = args.norm_mode == 1 ? 1.0f : args.norm_mode == 2 ? args.scale
                          : (args.norm_partials != nullptr ? sfac[sample] : __ldg(args.factors + sample)) * args.scale;
          const uint32_t tb = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN + chalf * 128;
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            uint32_t r[32];
            tc_ld32(tb + c4 * 32, r);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) accr[c4 * 32 + j] = fmaf(cbs, __uint_as_float(r[j]), accr[c4 * 32 + j]);
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (CTAS == 1 || is_leader) mbar_arrive(tempty_bar(acc));
            else mbar_arrive_cluster(mapa_u32(tempty_bar(acc), 0));
          }
          ++seg;
          if (pre_noise) {
            const int target = (32 * seg) / nseg;
            for (; ng < target; ++ng) {
              float z[4];
              noise_group(args.nk, g0 + ng, z);
              add_group(accr, ng, z, 1.0f);
            }
          }
        }
        if (!ok) break;
        if (args.norm_mode == 1) {
          // the unit is one sample's product tile: its squares, without the rows and columns past the
          // matrix (with split operands a tile that overhangs reads the other half's columns, not zeros)
          float part = 0.f;
          const int nb = n0 + chalf * 128;
          if (m < args.M) {
#pragma unroll
            for (int i = 0; i < 128; ++i) part = fmaf((nb + i < args.N) ? accr[i] : 0.f, accr[i], part);
          }
          part = warp_sum(part);
          if (lane == 0) args.partials[(static_cast<size_t>(tile) * CTAS + cta_rank) * EPI_WARPS + ew] = part;
          continue;
        }
        if (slot < 0) {
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = accr[c4 * 32 + j];
            store_chunk32<false>(args, v, m, n0 + chalf * 128 + c4 * 32);
          }
        } else {
          // park this part (already divided by the batch) for the fix-up kernel
          float4* dst = reinterpret_cast<float4*>(args.split_ws + ((static_cast<size_t>(slot) * CTAS + cta_rank) * BM + row) * BN + chalf * 128);
#pragma unroll
          for (int j = 0; j < 32; ++j)
            dst[j] = make_float4(accr[4 * j], accr[4 * j + 1], accr[4 * j + 2], accr[4 * j + 3]);
        }
        continue;
      }
      const int acc = it % NUM_ACC;
      const uint32_t acc_phase = (it / NUM_ACC) & 1u;
      if (!mbar_wait_warp(tfull_bar(acc), acc_phase, wctx, 4)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tbase = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + (EPI == EPI_GRAM ? 0 : acc * BN);
      float part = 0.f;
      constexpr int C_SPAN = BN * 4 / EPI_WARPS;     // store epilogue: this warp's share of the tile's columns
      const int c_begin = (ew >> 2) * C_SPAN;
      if (EPI == EPI_STORE && slot >= 0) {
        // K-split unit: park the raw accumulator for the fix-up kernel
        float4* dst = reinterpret_cast<float4*>(args.split_ws + ((static_cast<size_t>(slot) * CTAS + cta_rank) * BM + row) * BN);
#pragma unroll 1
        for (int c = c_begin; c < c_begin + C_SPAN; c += 32) {
          uint32_t r[32];
          tc_ld32(tbase + c, r);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            dst[c / 4 + j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                         __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
        }
      } else if (EPI == EPI_STORE) {
#pragma unroll 1
        for (int c = c_begin; c < c_begin + C_SPAN; c += 32) {
          uint32_t r[32];
          tc_ld32(tbase + c, r);
          tc_wait_ld();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * args.scale;
          store_chunk32<true>(args, v, m, n0 + c);
        }
      } else if (EPI == EPI_SUMSQ) {
        // rows / columns outside the matrix were zero-filled by TMA, so they add nothing
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tc_ld32(tbase + c, r);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) { const float f = __uint_as_float(r[j]); part = fmaf(f, f, part); }
        }
      } else {
        // columns 0..127 belong to s-block n0, 128..255 to s-block gram_n1; a diagonal block counts
        // once, any other block twice (it stands for its mirror image too); rows and columns past the
        // end of the sample (they belong to the next one) count nothing
        const int t = m0 + row;
        const int ncols = half ? BN / 2 : BN;
#pragma unroll 1
        for (int c = 0; c < ncols; c += 32) {
          uint32_t p[32], q[32];
          tc_ld32(tbase + c, p);
          tc_ld32(tbase + BN + c, q);
          tc_wait_ld();
          const int sb0 = (c < BN / 2) ? n0 : gram_n1;          // first row of this chunk's s-block
          const int s0 = sb0 + (c & (BN / 2 - 1));
          const float wblk = (sb0 == m0) ? 1.f : 2.f;
          if (t < args.T) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float w = (s0 + j < args.T) ? wblk : 0.f;
              part = fmaf(w * __uint_as_float(p[j]), __uint_as_float(q[j]), part);
            }
          }
        }
      }
      // accumulator drained: hand it back to the MMA warp (of the leader CTA)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (CTAS == 1 || is_leader) mbar_arrive(tempty_bar(acc));
        else mbar_arrive_cluster(mapa_u32(tempty_bar(acc), 0));
      }
      ++it;
      if (EPI == EPI_SUMSQ || EPI == EPI_GRAM) {
        // one partial per (unit, epilogue warp); units are numbered sample by sample
        part = warp_sum(part);
        if (lane == 0) args.partials[static_cast<size_t>(tile) * 4 + quarter] = part;
      }
    }
  }

  // ================= teardown =================
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (CTAS == 2) cluster_sync_all();  // neither CTA leaves (or frees TMEM) while its peer may still signal it
  if (warp == 1) {
    tc_fence_after();
    if (CTAS == 2)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---- split-K fix-up: out = scale * (part_0 + part_1 + ...) + noise for the K-split tiles --------------
__global__ void __launch_bounds__(256) splitk_fixup_kernel(const float* __restrict__ ws, int first_tile, int split,
                                                           int tile_rows, int M, int N, int tiles_m, int tiles_n, int n_fastest,
                                                           int m_group,
                                                           void* __restrict__ out, int out_dt, long long ld_out,
                                                           float scale, NoiseKey nk) {
  pdl_wait();
  const int t = blockIdx.y;  // index among the split tiles
  const int q = first_tile + t;
  int mi, ni;  // the tile order of tc_gemm_kernel's decode
  if (n_fastest) {
    ni = q % tiles_n; mi = q / tiles_n;
  } else if (m_group > 0) {
    const int per_group = m_group * tiles_n;
    const int g = q / per_group, r = q - g * per_group;
    const int gm = min(m_group, tiles_m - g * m_group);
    mi = g * m_group + r % gm; ni = r / gm;
  } else {
    mi = q % tiles_m; ni = q / tiles_m;
  }
  const int m0 = mi * tile_rows, n0 = ni * BN;
  const int e = (blockIdx.x * 256 + threadIdx.x) * 4;  // element of the tile, 4 adjacent columns
  const int row = e / BN, col = e % BN;
  const int m = m0 + row, n = n0 + col;
  if (m >= M || n >= N) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int p = 0; p < split; ++p) {
    const float4 v = *reinterpret_cast<const float4*>(ws + (static_cast<size_t>(t * split + p) * tile_rows + row) * BN + col);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  float v[4] = {acc.x * scale, acc.y * scale, acc.z * scale, acc.w * scale};
  const size_t idx0 = static_cast<size_t>(m) * ld_out + n;
  if (nk.std != 0.f) {   // idx0 is a multiple of 4: the row pitch and n are
    float z[4];
    noise_group(nk, idx0 >> 2, z);
    v[0] += z[0]; v[1] += z[1]; v[2] += z[2]; v[3] += z[3];
  }
  for (int j = 0; j < 4; ++j)
    if (n + j < N) store_as(out, out_dt, idx0 + j, v[j]);
}

// ---- c_b pre-scale: Gs[r,:] = c[r / T] * G[r,:] (HBM-bound, 16-byte vectors) ------------------------
template <typename Tin>
__global__ void __launch_bounds__(256) prescale_kernel(const Tin* __restrict__ G, const float* __restrict__ factors,
                                                       Tin* __restrict__ Gs, size_t nvec, int vec_per_sample) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const float c = factors[i / vec_per_sample];
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(G) + i);
    const Tin* e = reinterpret_cast<const Tin*>(&raw);
    uint4 outv;
    Tin* o = reinterpret_cast<Tin*>(&outv);
#pragma unroll
    for (int v = 0; v < 8; ++v) o[v] = from_f32<Tin>(to_f32<Tin>(e[v]) * c);
    reinterpret_cast<uint4*>(Gs)[i] = outv;
  }
}

// ---- fp32 -> (hi, lo) bf16 halves: dst[r, c] = bf16(x), dst[r, n + c] = bf16(x - hi) ---------------------
__global__ void __launch_bounds__(256) split3_kernel(const float4* __restrict__ src, uint2* __restrict__ dst,
                                                     size_t nvec, int vec_per_row) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const float4 v = __ldg(src + i);
    const float f[4] = {v.x, v.y, v.z, v.w};
    uint16_t hi[4], lo[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __nv_bfloat16 h = __float2bfloat16_rn(f[e]);
      const __nv_bfloat16 l = __float2bfloat16_rn(f[e] - __bfloat162float(h));
      hi[e] = *reinterpret_cast<const uint16_t*>(&h);
      lo[e] = *reinterpret_cast<const uint16_t*>(&l);
    }
    const size_t row = i / vec_per_row, cv = i - row * vec_per_row;
    uint2* o = dst + row * (2 * static_cast<size_t>(vec_per_row)) + cv;
    o[0] = make_uint2(hi[0] | (static_cast<uint32_t>(hi[1]) << 16), hi[2] | (static_cast<uint32_t>(hi[3]) << 16));
    o[vec_per_row] = make_uint2(lo[0] | (static_cast<uint32_t>(lo[1]) << 16), lo[2] | (static_cast<uint32_t>(lo[3]) << 16));
  }
}

// ---- host side ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static std::mutex mu;
  static EncodeTiledFn fn = nullptr;
  std::lock_guard<std::mutex> lk(mu);
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      cudaGetLastError();
  }
  return fn;
}

// 2-D map over a row-major [rows, cols] matrix of 16-bit elements, 128-byte swizzle, zero fill
bool make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_cols,
              uint32_t box_rows, int dt) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(m, dt == FDP_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                        const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

uint32_t make_idesc(int dt, bool a_mn, bool b_mn, int ctas = 1, int n = BN) {
  uint32_t d = 0;
  d |= 1u << 4;                                   // accumulator format: F32
  d |= (dt == FDP_BF16 ? 1u : 0u) << 7;           // A format
  d |= (dt == FDP_BF16 ? 1u : 0u) << 10;          // B format
  d |= (a_mn ? 1u : 0u) << 15;                    // A major: 1 = MN-major
  d |= (b_mn ? 1u : 0u) << 16;                    // B major
  d |= static_cast<uint32_t>(n >> 3) << 17;       // N
  d |= static_cast<uint32_t>((BM * ctas) >> 4) << 24;  // M (256 for a CTA pair)
  return d;
}

// SMs of the current device (cached per device).
int sm_count() {
  static std::mutex mu;
  static int cache[64];
  static bool have[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return 148; }
  std::lock_guard<std::mutex> lk(mu);
  if (!have[dev]) {
    int n = 148;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) { cudaGetLastError(); n = 148; }
    cache[dev] = n; have[dev] = true;
  }
  return cache[dev];
}
// SMs the next persistent GEMM grid may occupy: all of them minus the current reservation
// (fdp_set_sm_reserve; FDP_TC_RESERVE_SMS is its initial value).  A persistent CTA holds a whole SM's
// shared memory, so a collective kernel launched beside such a grid cannot start until SMs are free;
// a caller that overlaps a GEMM with a collective reserves a few SMs for the duration of that call.
std::atomic<int> g_sm_reserve{[] { const char* e = getenv("FDP_TC_RESERVE_SMS"); return e ? atoi(e) : 0; }()};
int launch_sms() {
  int n = sm_count();
  const int reserve = g_sm_reserve.load(std::memory_order_relaxed);
  if (n > MAX_SMS) n = MAX_SMS;   // the parking area is sized for MAX_SMS workers
  if (reserve > 0 && n - reserve >= 16) n -= reserve;
  return n & ~1;  // CTA pairs
}

template <bool A_MN, bool B_MN, int EPI, int CTAS = 1>
int launch(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& a2, const CUtensorMap& b2,
           const TcArgs& args, cudaStream_t s) {
  static std::mutex mu;
  static bool done[64];
  constexpr int SMEM = smem_for(EPI);
  if (!smem_opt_in(done, mu, tc_gemm_kernel<A_MN, B_MN, EPI, CTAS>, SMEM)) return FDP_ERR_LAUNCH;
  TcArgs la = args;
  la.sticky = sticky_status_slot();
  const int total = la.batch * la.tiles_per_batch;
  if (la.split <= 1) { la.split = 1; la.units_full = total; }
  int units = la.units_full + (total - la.units_full) * la.split;
  const int workers = launch_sms() / CTAS;   // CTAs, or CTA pairs
  const int grid = CTAS * (units < workers ? units : workers);
  const bool dependent = la.dependent != 0 && pdl_enabled();
  if (CTAS == 1 && !dependent) {
    tc_gemm_kernel<A_MN, B_MN, EPI, CTAS><<<grid, threads_for(EPI), SMEM, s>>>(a, b, a2, b2, la);
  } else {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(threads_for(EPI));
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (CTAS == 2) {
      attr[na].id = cudaLaunchAttributeClusterDimension;
      attr[na].val.clusterDim.x = 2; attr[na].val.clusterDim.y = 1; attr[na].val.clusterDim.z = 1;
      ++na;
    }
    if (dependent) {
      attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[na].val.programmaticStreamSerializationAllowed = 1;
      ++na;
    }
    cfg.attrs = attr; cfg.numAttrs = na;
    if (cudaLaunchKernelEx(&cfg, tc_gemm_kernel<A_MN, B_MN, EPI, CTAS>, a, b, a2, b2, la) != cudaSuccess) {
      cudaGetLastError();
      return FDP_ERR_LAUNCH;
    }
  }
  note_launch();
  return cudaPeekAtLastError() == cudaSuccess ? FDP_OK : (cudaGetLastError(), FDP_ERR_LAUNCH);
}

// CTA pairs (cta_group::2) for the store-epilogue GEMMs; FDP_TC_CTAS=1 / 2 forces single CTAs / pairs
int forced_ctas() {
  static const int v = [] { const char* e = getenv("FDP_TC_CTAS"); return (e && (e[0] == '1' || e[0] == '2')) ? e[0] - '0' : 0; }();
  return v;
}
int ctas_per_tile() { return forced_ctas() == 1 ? 1 : 2; }
// (Tried for the clipped-sum GEMM of small layers: single-CTA 128 x 256 tiles run whole, without K split,
// parked accumulators or fix-up, whenever the pair tiles do not fill one wave of CTA pairs.  At the four
// GPT-2-medium layer shapes that was 1-3 % slower than pairs with the K split, so pairs stay.)

// K-split of the tail wave: `rem` tiles left after the full waves (all of them when there are fewer
// tiles than workers) are cut into s parts of equal K-stage count, so that the last round keeps more
// SMs busy; cost in tile-times = ceil(rem*s/workers)/s plus the cost of parking and re-reading the
// accumulators.  At most 2 * workers parked parts (workers <= MAX_SMS / CTAS).
// That cost, in tile-times: 0.05 for the fix-up launch plus 0.15 per parked part and worker (the
// parts are written and read again).  With 48 pair tiles of 128 K stages for 74 pairs (a GPT-2
// layer, B=8, T=1024) three parts of 43 stages in two rounds measured no faster than the tiles
// unsplit (100.8 against 98.6 us per call: parking, the second round's hand-over and the fix-up
// launch eat the 42 stages saved), while 16 tiles in four parts (52 against 82 us) and the tails of
// the larger layers do pay.
int plan_tail_split(int total_tiles, int k_stages, int workers) {
  const int rem = total_tiles <= workers ? total_tiles : total_tiles % workers;
  if (rem == 0 || k_stages < 32) return 1;
  // FDP_TC_SPLIT=n forces the number of parts (measurements), within the same limits
  static const int forced = [] { const char* e = getenv("FDP_TC_SPLIT"); return e ? atoi(e) : 0; }();
  if (forced >= 1) return (rem * forced > 2 * workers || k_stages / forced < 8) ? 1 : forced;
  int best_s = 1; double best = 1.0;
  for (int sp = 2; sp <= 16; ++sp) {
    if (rem * sp > 2 * workers || k_stages / sp < 8) break;
    const double cost = static_cast<double>((rem * sp + workers - 1) / workers) / sp +
                        0.15 * (static_cast<double>(rem) * sp / workers) + 0.05;
    if (cost < best - 0.03) { best = cost; best_s = sp; }
  }
  return best_s;
}
// parked accumulators: up to 2 * MAX_SMS parts of 128 x 256 fp32 (a CTA pair parks two per part)
size_t split_ws_bytes() { return static_cast<size_t>(2) * MAX_SMS * BM * BN * sizeof(float); }
size_t align256(size_t n) { return (n + 255) & ~static_cast<size_t>(255); }

int gram_tiles(int T) { return gram_units(ceil_div(T, BM)); }   // work units (128 x 256 tiles) per sample

// A warp waits on a barrier nobody arrives on, so the wait runs out after `limit` cycles and takes the
// reporting path of every bounded wait of the library: abort flag, status word, host-visible slot.
__global__ void __launch_bounds__(32) wait_selftest_kernel(int* status, int* sticky, long long limit) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); abort_flag = 0; mbar_fence_init(); }
  __syncwarp();
  const WaitCtx w{&abort_flag, status, sticky, limit};
  mbar_wait_warp(smem_u32(&bar), 0, w, 9);
}

}  // namespace

int sm_reserve_exchange(int n) { return g_sm_reserve.exchange(n < 0 ? 0 : n); }

int tc_wait_selftest(int* status, long long limit_cycles, cudaStream_t s) {
  if (limit_cycles < 1) limit_cycles = 1;
  if (limit_cycles > WAIT_LIMIT_CYCLES) limit_cycles = WAIT_LIMIT_CYCLES;
  wait_selftest_kernel<<<1, 32, 0, s>>>(status, sticky_status_slot(), limit_cycles);
  note_launch();
  return cudaPeekAtLastError() == cudaSuccess ? FDP_OK : (cudaGetLastError(), FDP_ERR_LAUNCH);
}

// K stages per accumulator hand-off for fp32 inputs (three bf16 products): the largest divisor of a
// sample's stage count that is at most FDP_TC_CHAIN_STAGES (default 8: 32 steps of K = 16 per chain).
// B=8, T=1024, 4096x4096, against float64: norms 1.1e-7 / 2.5e-7 / 4.4e-7 / 5e-6 and 2.15 / 1.48 /
// 1.42 / 1.37 ms per call with 2 / 4 / 8 / all stages per chain (1e-5 at T=2048 with one chain).
static int chain_stages(int seg_stages) {
  static const int cap = [] {
    const char* e = getenv("FDP_TC_CHAIN_STAGES");
    const int v = e ? atoi(e) : 8;
    return v < 1 ? 1 : v;
  }();
  int c = cap < seg_stages ? cap : seg_stages;
  while (seg_stages % c != 0) --c;
  return c;
}

// The tensor-core path needs 16-bit inputs, row pitches that are multiples of 16 bytes, and
// matrices large enough that the 128x256 tile is not mostly padding.
TcPlan tc_plan(int B, int T, int n_in, int n_out, int dt, int norm_algo) {
  TcPlan p; p.ok = false; p.algo = FDP_NORM_DIRECT; p.ws_bytes = 0; p.nparts = 0; p.scaled_epilogue = false;
  p.short_seq = false; p.split_bytes = 0;
  p.split3 = false; p.split3_g_bytes = p.split3_x_bytes = 0;
  const bool fp32_tensor = (norm_algo & FDP_FP32_TENSOR) != 0;
  norm_algo &= FDP_NORM_MASK;
  if (dt == FDP_F32) {
    // fp32 on the tensor cores as three bf16 products (hi*hi + hi*lo + lo*hi, fp32 accumulation), when
    // the caller asks for it (FDP_FP32_TENSOR).  The tensor cores add into their fp32 accumulators by
    // truncation, a one-sided error of about 2^-24 per K=16 step, so no accumulator runs for more than
    // a few K stages: it is handed to the epilogue warps, which add it to registers with
    // round-to-nearest (chain_stages).  Needs whole 64-column K stages per half, samples made of whole
    // 64-row stages, and the per-sample epilogue (a pre-scaled copy would round c_b * G to bf16 again).
    if (!fp32_tensor || n_in % BK != 0 || n_out % BK != 0 || n_in < 128 || n_out < 128 || T % BK != 0 || T < 2 * BK) return p;
    p.split3 = true;
    p.split3_g_bytes = align256(static_cast<size_t>(B) * T * n_out * 4);
    p.split3_x_bytes = align256(static_cast<size_t>(B) * T * n_in * 4);
  } else if (dt != FDP_BF16 && dt != FDP_F16) {
    return p;
  }
  if (n_in % 8 != 0 || n_out % 8 != 0 || n_in < 128 || n_out < 128) return p;
  if (T < SHORT_SEQ) {
    // short sequences: the norms come from the small Gram kernel (one partial per sample); the
    // clipped sum is still one GEMM with K = B*T over the pre-scaled copy of G, if K is worth a tile
    if (norm_algo == FDP_NORM_DIRECT || static_cast<long long>(B) * T < 4 * BK) return p;
    p.ok = true; p.algo = FDP_NORM_GRAM; p.short_seq = true; p.nparts = 1;
    p.split_bytes = split_ws_bytes();
    p.ws_bytes = p.split_bytes + align256(static_cast<size_t>(B) * T * n_out * 2);
    return p;
  }
  // direct: a K stage must not run into the next sample's rows
  const bool direct_ok = (T % BK == 0);
  // Cost of the two norm algorithms in K stages on the critical path: both kernels deal equal work
  // units (128x256 tiles) round-robin to one CTA per SM, so a pass takes
  // ceil(units / SMs) * (stages per unit + a fixed cost per unit of about four stages).  The SM
  // count is a constant here: the workspace query and the launch must pick the same algorithm.
  constexpr long long PLAN_SMS = 148, UNIT_FIXED_STAGES = 4;
  const long long units_d = static_cast<long long>(B) * ceil_div(n_out, BM) * ceil_div(n_in, BN);
  const long long units_g = static_cast<long long>(B) * gram_tiles(T);
  const int terms = p.split3 ? 3 : 1;
  const double direct = static_cast<double>((units_d + PLAN_SMS - 1) / PLAN_SMS) * (terms * ceil_div(T, BK) + UNIT_FIXED_STAGES);
  const double gram = static_cast<double>((units_g + PLAN_SMS - 1) / PLAN_SMS) *
                      (terms * (ceil_div(n_in, BK) + ceil_div(n_out, BK)) + UNIT_FIXED_STAGES);
  int algo = norm_algo;
  if (algo == FDP_NORM_AUTO) algo = (direct_ok && direct <= gram) ? FDP_NORM_DIRECT : FDP_NORM_GRAM;
  if (algo == FDP_NORM_DIRECT && !direct_ok) algo = FDP_NORM_GRAM;
  // split operands: always the product form, accumulated in short chains (tc_norms); the Gram form
  // needs both T x T tiles complete in TMEM before its epilogue can multiply them, i.e. one chain of
  // 3 * (in + out) / 16 truncating additions
  if (p.split3) algo = FDP_NORM_DIRECT;
  p.ok = true;
  p.algo = algo;
  // clip factors applied in the GEMM epilogue (no scaled copy of G) when every 64-row K stage lies
  // inside one sample and a sample's main loop is long enough to hide the per-sample drain;
  // FDP_WGRAD_PRESCALE=1 forces the pre-scale pass (for A/B measurements)
  static const bool force_prescale = [] { const char* e = getenv("FDP_WGRAD_PRESCALE"); return e && e[0] == '1'; }();
  p.scaled_epilogue = p.split3 || (!force_prescale && (T % BK == 0) && T >= 256);
  // one partial per work unit and epilogue warp
  p.nparts = 4 * ((algo == FDP_NORM_DIRECT) ? ceil_div(n_out, BM) * ceil_div(n_in, BN) : gram_tiles(T));
  if (p.split3) {   // the chained norm pass: tiles of the clipped-sum GEMM, eight epilogue warps per CTA
    const int ctas = ctas_per_tile();
    p.nparts = ceil_div(n_out, BM * ctas) * ceil_div(n_in, BN) * ctas * epi_warps_for(EPI_STORE_SCALED);
  }
  // the parked accumulators of the split-K tail, then (pre-scale path only) the c_b-scaled copy of G
  p.split_bytes = split_ws_bytes();
  p.ws_bytes = p.split_bytes + (p.scaled_epilogue ? 0 : align256(static_cast<size_t>(B) * T * n_out * 2)) +
               p.split3_g_bytes + p.split3_x_bytes;
  return p;
}

int tc_split3(const void* src, void* dst, size_t rows, int n, cudaStream_t s) {
  const size_t nvec = rows * n / 4;
  size_t blocks = (nvec + 255) / 256;
  const size_t cap = static_cast<size_t>(sm_count()) * 16;
  split3_kernel<<<static_cast<unsigned>(blocks < cap ? blocks : cap), 256, 0, s>>>(
      static_cast<const float4*>(src), static_cast<uint2*>(dst), nvec, n / 4);
  note_launch();
  return cudaPeekAtLastError() == cudaSuccess ? FDP_OK : (cudaGetLastError(), FDP_ERR_LAUNCH);
}

int tc_norms(const void* G, const void* X, float* partials, int* dev_status, int B, int T, int n_in,
             int n_out, int dt, const TcPlan& pl, cudaStream_t s) {
  const uint64_t rows = static_cast<uint64_t>(B) * T;
  const int terms = pl.split3 ? 3 : 1;
  const int wo = pl.split3 ? 2 * n_out : n_out, wi = pl.split3 ? 2 * n_in : n_in;   // matrix widths
  CUtensorMap a, b, a2, b2;
  TcArgs args{};
  args.batch = B; args.batch_rows = T; args.partials = partials; args.status = dev_status; args.T = T;
  args.zero_status = 1;      // the norm pass is the first launch of a weight-gradient call
  args.terms = terms;
  if (pl.split3) {
    // fp32 inputs: the per-sample products G_b^T X_b themselves, on the tiles and CTA pairs of the
    // clipped-sum GEMM, handed to the epilogue every few K stages and summed there in registers; a
    // unit is (sample, tile) and ends with the sum of its squares instead of a store
    if (!make_map(&a, G, rows, wo, 64, BK, dt) || !make_map(&b, X, rows, wi, 64, BK, dt)) return FDP_ERR_LAUNCH;
    const int ctas = ctas_per_tile();
    args.M = n_out; args.N = n_in; args.ld_out = n_in;
    args.tiles_m = ceil_div(n_out, BM * ctas); args.tiles_n = ceil_div(n_in, BN);
    args.tiles_per_batch = args.tiles_m * args.tiles_n;
    args.term_stages = T / BK;
    args.k_stages = terms * (T / BK);
    args.plane_a = n_out; args.plane_b = n_in;
    args.idesc = make_idesc(dt, true, true, ctas);
    args.segs = 1; args.seg_stages = args.k_stages; args.sub_stages = chain_stages(args.seg_stages);
    args.norm_mode = 1; args.scale = 1.0f; args.nk = NoiseKey{};
    return ctas == 2 ? launch<true, true, EPI_STORE_SCALED, 2>(a, b, a, b, args, s)
                     : launch<true, true, EPI_STORE_SCALED, 1>(a, b, a, b, args, s);
  }
  if (pl.algo == FDP_NORM_DIRECT) {
    if (!make_map(&a, G, rows, wo, 64, BK, dt) || !make_map(&b, X, rows, wi, 64, BK, dt)) return FDP_ERR_LAUNCH;
    args.M = n_out; args.N = n_in;
    args.tiles_m = ceil_div(n_out, BM); args.tiles_n = ceil_div(n_in, BN);
    args.tiles_per_batch = args.tiles_m * args.tiles_n;
    args.term_stages = T / BK;
    args.k_stages = terms * (T / BK);
    args.plane_a = n_out; args.plane_b = n_in;
    args.idesc = make_idesc(dt, true, true);
    return launch<true, true, EPI_SUMSQ>(a, b, a, b, args, s);
  }
  // A and B boxes are both 128 rows: a B stage is filled by two independent copies
  if (!make_map(&a, G, rows, wo, BK, BM, dt) || !make_map(&b, G, rows, wo, BK, BN / 2, dt) ||
      !make_map(&a2, X, rows, wi, BK, BM, dt) || !make_map(&b2, X, rows, wi, BK, BN / 2, dt))
    return FDP_ERR_LAUNCH;
  args.M = T; args.N = T;
  args.gram_nb = ceil_div(T, BM);
  args.tiles_m = args.gram_nb; args.tiles_n = args.gram_nb;
  args.tiles_per_batch = gram_tiles(T);
  args.idesc_half = make_idesc(dt, false, false, 1, BN / 2);
  args.term_stages = ceil_div(n_out, BK); args.term_stages2 = ceil_div(n_in, BK);
  args.k_stages = terms * args.term_stages; args.k_stages2 = terms * args.term_stages2;
  args.plane_a = args.plane_b = n_out; args.plane_a2 = args.plane_b2 = n_in;
  args.idesc = make_idesc(dt, false, false);
  return launch<false, false, EPI_GRAM>(a, b, a2, b2, args, s);
}

int tc_prescale(const void* G, const float* factors, void* Gs, int B, int T, int n_out, int dt, cudaStream_t s) {
  const size_t nvec = static_cast<size_t>(B) * T * n_out / 8;
  const int vps = T * (n_out / 8);
  const int grid = sm_count() * 8;
  if (dt == FDP_BF16)
    prescale_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)G, factors, (__nv_bfloat16*)Gs, nvec, vps);
  else
    prescale_kernel<__half><<<grid, 256, 0, s>>>((const __half*)G, factors, (__half*)Gs, nvec, vps);
  note_launch();
  return FDP_OK;
}

bool tc_fused_factors_ok(int B) { return B <= MAX_SMEM_FACTORS; }

int tc_clipped_wgrad(const void* Gs, const void* X, const TcFactorSource* fs, float* split_ws,
                     void* dW, int* dev_status, int B, int T, int n_in, int n_out, int dt, int out_dt,
                     int layout, float inv_div, NoiseKey nk, cudaStream_t s, int terms) {
  const uint64_t rows = static_cast<uint64_t>(B) * T;
  const bool scaled = fs != nullptr;  // Gs is then the unscaled G
  if (terms != 1 && !(terms == 3 && scaled)) return FDP_ERR_ARG;
  CUtensorMap mg, mx;
  if (!make_map(&mg, Gs, rows, terms == 3 ? 2 * n_out : n_out, 64, BK, dt) ||
      !make_map(&mx, X, rows, terms == 3 ? 2 * n_in : n_in, 64, BK, dt)) return FDP_ERR_LAUNCH;
  TcArgs args{};
  args.batch = 1; args.batch_rows = 0; args.status = dev_status;
  args.dependent = 1;             // always follows a kernel of the same call (norm pass, clip factors or pre-scale)
  args.terms = terms;
  args.term_stages = T / BK;      // used when terms == 3: every sample's rows are visited three times
  args.k_stages = terms * static_cast<int>((rows + BK - 1) / BK);
  args.out = dW; args.out_dt = out_dt; args.scale = inv_div; args.nk = nk;
  // [out,in]: A = G (M = n_out), B = X (N = n_in); [in,out]: operands swap roles, no transpose pass
  const bool oi = (layout == FDP_OUT_IN);
  args.M = oi ? n_out : n_in; args.N = oi ? n_in : n_out; args.ld_out = args.N;
  const int ctas = ctas_per_tile();
  args.idesc = make_idesc(dt, true, true, ctas);
  if (scaled) {
    args.segs = B; args.seg_stages = terms * (T / BK);
    args.sub_stages = terms == 3 ? chain_stages(args.seg_stages) : args.seg_stages;
    args.factors = fs->factors;
    if (fs->factors == nullptr) {
      if (!tc_fused_factors_ok(B) || fs->norm_partials == nullptr) return FDP_ERR_ARG;
      args.norm_partials = fs->norm_partials; args.norm_nparts = fs->nparts;
      args.C = fs->C; args.clamp = fs->clamp;
      args.norms_out = fs->norms_out; args.factors_out = fs->factors_out;
    }
  }
  args.plane_a = args.M; args.plane_b = args.N;
  args.tiles_m = ceil_div(args.M, BM * ctas); args.tiles_n = ceil_div(args.N, BN);
  args.tiles_per_batch = args.tiles_m * args.tiles_n;
  static const int m_group = [] { const char* e = getenv("FDP_TC_MGROUP"); return e ? atoi(e) : 8; }();
  args.m_group = m_group;
  // tail wave: split K so the SMs left idle by the tile count get work; the parts are parked in the
  // workspace and summed in fixed order by the fix-up kernel (deterministic, no waits)
  const int total = args.tiles_per_batch, workers = launch_sms() / ctas;
  const int split = plan_tail_split(total, args.k_stages, workers);
  int n_split_tiles = 0;
  if (split > 1) {
    n_split_tiles = total <= workers ? total : total % workers;
    args.split = split;
    args.units_full = total - n_split_tiles;
    args.split_ws = split_ws;
  }
  int st;
#define FDP_WGRAD_LAUNCH(EPI_, CT_) (oi ? launch<true, true, EPI_, CT_>(mg, mx, mg, mx, args, s) \
                                        : launch<true, true, EPI_, CT_>(mx, mg, mx, mg, args, s))
  if (scaled) st = ctas == 2 ? FDP_WGRAD_LAUNCH(EPI_STORE_SCALED, 2) : FDP_WGRAD_LAUNCH(EPI_STORE_SCALED, 1);
  else st = ctas == 2 ? FDP_WGRAD_LAUNCH(EPI_STORE, 2) : FDP_WGRAD_LAUNCH(EPI_STORE, 1);
#undef FDP_WGRAD_LAUNCH
  if (st != FDP_OK || split <= 1) return st;
  // the scaled epilogue parks its parts already divided by the batch
  dim3 grid(BM * ctas * BN / (256 * 4), n_split_tiles);
  launch_dependent(splitk_fixup_kernel, grid, dim3(256), 0, s, args.split_ws, args.units_full, split, BM * ctas, args.M,
                   args.N, args.tiles_m, args.tiles_n, args.n_fastest, args.m_group, dW, out_dt, args.ld_out,
                   scaled ? 1.0f : inv_div, nk);
  note_launch();
  return FDP_OK;
}

bool tc_dgrad_ok(int rows, int n_in, int n_out, int dt) {
  return (dt == FDP_BF16 || dt == FDP_F16) && n_in % 8 == 0 && n_out % 8 == 0 && n_in >= 128 && n_out >= 64 && rows >= 128;
}

int tc_dgrad(const void* G, const void* W, void* dX, int* dev_status, int rows, int n_in, int n_out,
             int dt, int out_dt, int w_layout, cudaStream_t s) {
  CUtensorMap mg, mw;
  const int ctas = ctas_per_tile();
  if (!make_map(&mg, G, rows, n_out, BK, BM, dt)) return FDP_ERR_LAUNCH;
  TcArgs args{};
  args.batch = 1; args.batch_rows = 0; args.status = dev_status; args.zero_status = 1;
  args.M = rows; args.N = n_in; args.ld_out = n_in;
  args.tiles_m = ceil_div(rows, BM * ctas); args.tiles_n = ceil_div(n_in, BN);
  args.tiles_per_batch = args.tiles_m * args.tiles_n;
  args.k_stages = ceil_div(n_out, BK);
  // G is streamed once: CTAs that run together cover a band of rows times all of n_in, so the
  // band of G and the whole of W stay in L2 (walking along M first would re-read G per n-tile)
  args.n_fastest = 1;
  args.out = dX; args.out_dt = out_dt; args.scale = 1.0f; args.nk = NoiseKey{};
  if (w_layout == FDP_OUT_IN) {  // W [n_out, n_in]: rows are K, N contiguous
    if (!make_map(&mw, W, n_out, n_in, 64, BK, dt)) return FDP_ERR_LAUNCH;
    args.idesc = make_idesc(dt, false, true, ctas);
    return ctas == 2 ? launch<false, true, EPI_STORE, 2>(mg, mw, mg, mw, args, s)
                     : launch<false, true, EPI_STORE, 1>(mg, mw, mg, mw, args, s);
  }
  // W [n_in, n_out]: K contiguous; a CTA of a pair loads half of the 256 B rows
  if (!make_map(&mw, W, n_in, n_out, BK, BN / ctas, dt)) return FDP_ERR_LAUNCH;
  args.idesc = make_idesc(dt, false, false, ctas);
  return ctas == 2 ? launch<false, false, EPI_STORE, 2>(mg, mw, mg, mw, args, s)
                   : launch<false, false, EPI_STORE, 1>(mg, mw, mg, mw, args, s);
}

// forward: A = X [rows, n_in] K-major; B = W, K-major for [n_out, n_in] (Linear), MN-major for
// [n_in, n_out] (Conv1D); bias added in the epilogue
int tc_fwd(const void* X, const void* W, const void* bias, void* Y, int* dev_status, int rows, int n_in,
           int n_out, int dt, int out_dt, int w_layout, cudaStream_t s) {
  CUtensorMap mx, mw;
  const int ctas = ctas_per_tile();
  if (!make_map(&mx, X, rows, n_in, BK, BM, dt)) return FDP_ERR_LAUNCH;
  TcArgs args{};
  args.batch = 1; args.batch_rows = 0; args.status = dev_status; args.zero_status = 1;
  args.M = rows; args.N = n_out; args.ld_out = n_out;
  args.tiles_m = ceil_div(rows, BM * ctas); args.tiles_n = ceil_div(n_out, BN);
  args.tiles_per_batch = args.tiles_m * args.tiles_n;
  args.k_stages = ceil_div(n_in, BK);
  args.n_fastest = 1;  // X is streamed once, W stays in L2
  args.out = Y; args.out_dt = out_dt; args.scale = 1.0f; args.nk = NoiseKey{};
  args.bias = bias; args.bias_dt = dt;
  if (w_layout == FDP_OUT_IN) {  // W [n_out, n_in]: K contiguous
    if (!make_map(&mw, W, n_out, n_in, BK, BN / ctas, dt)) return FDP_ERR_LAUNCH;
    args.idesc = make_idesc(dt, false, false, ctas);
    return ctas == 2 ? launch<false, false, EPI_STORE, 2>(mx, mw, mx, mw, args, s)
                     : launch<false, false, EPI_STORE, 1>(mx, mw, mx, mw, args, s);
  }
  if (!make_map(&mw, W, n_in, n_out, 64, BK, dt)) return FDP_ERR_LAUNCH;  // W [n_in, n_out]: N contiguous
  args.idesc = make_idesc(dt, false, true, ctas);
  return ctas == 2 ? launch<false, true, EPI_STORE, 2>(mx, mw, mx, mw, args, s)
                   : launch<false, true, EPI_STORE, 1>(mx, mw, mx, mw, args, s);
}

// ---- fp32 products on the tensor cores: Y[rows, N] = A[rows, K] * W (+ bias) --------------------------
// A3 is [rows, 2K] and W3 [K, 2N] (w_kn) or [N, 2K] (else): bf16 high halves then low halves (tc_split3).
// Three bf16 products per K range into accumulators that the epilogue warps take over every few K
// stages and sum in registers (chain_stages), then the ordinary store epilogue.
bool tc_gemm3_ok(int rows, int K, int N) {
  return rows >= 128 && K >= 128 && N >= 128 && K % BK == 0 && N % 8 == 0;
}
size_t tc_gemm3_ws_bytes(int rows, int K, int N) {
  return align256(static_cast<size_t>(rows) * K * 4) + align256(static_cast<size_t>(K) * N * 4);
}
int tc_gemm3(const void* A3, const void* W3, const void* bias, void* Y, int* dev_status, int rows, int K, int N,
             int out_dt, bool w_kn, cudaStream_t s) {
  CUtensorMap ma, mw;
  const int ctas = ctas_per_tile();
  if (!make_map(&ma, A3, rows, 2 * K, BK, BM, FDP_BF16)) return FDP_ERR_LAUNCH;
  TcArgs args{};
  args.batch = 1; args.batch_rows = 0; args.status = dev_status;
  args.dependent = 1;            // follows the split kernels of the same call
  args.M = rows; args.N = N; args.ld_out = N;
  args.tiles_m = ceil_div(rows, BM * ctas); args.tiles_n = ceil_div(N, BN);
  args.tiles_per_batch = args.tiles_m * args.tiles_n;
  args.terms = 3;
  args.term_stages = K / BK;
  args.k_stages = 3 * (K / BK);
  args.plane_a = K; args.plane_b = w_kn ? N : K;
  args.n_fastest = 1;
  args.out = Y; args.out_dt = out_dt; args.scale = 1.0f; args.nk = NoiseKey{};
  args.bias = bias; args.bias_dt = FDP_F32;
  args.segs = 1; args.seg_stages = args.k_stages; args.sub_stages = chain_stages(args.seg_stages);
  args.norm_mode = 2;
  if (w_kn) {   // rows of W3 are K, N contiguous
    if (!make_map(&mw, W3, K, 2 * N, 64, BK, FDP_BF16)) return FDP_ERR_LAUNCH;
    args.idesc = make_idesc(FDP_BF16, false, true, ctas);
    return ctas == 2 ? launch<false, true, EPI_STORE_SCALED, 2>(ma, mw, ma, mw, args, s)
                     : launch<false, true, EPI_STORE_SCALED, 1>(ma, mw, ma, mw, args, s);
  }
  if (!make_map(&mw, W3, N, 2 * K, BK, BN / ctas, FDP_BF16)) return FDP_ERR_LAUNCH;   // K contiguous
  args.idesc = make_idesc(FDP_BF16, false, false, ctas);
  return ctas == 2 ? launch<false, false, EPI_STORE_SCALED, 2>(ma, mw, ma, mw, args, s)
                   : launch<false, false, EPI_STORE_SCALED, 1>(ma, mw, ma, mw, args, s);
}

}  // namespace fdp
