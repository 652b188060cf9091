// LayerNorm forward, backward (dx + per-sample dgamma/dbeta partials) and the per-sample
// clip / mean / noise finalisation.  All HBM-bound: 16-byte loads, each thread owns fixed columns
// so the per-sample column sums accumulate in registers, no atomics, fixed reduction order.
#include "fdp_async.cuh"
#include "fdp_kernels.h"

namespace fdp {

// named barrier `id` over `nthreads` threads that also ANDs a predicate across them
__device__ __forceinline__ bool bar_red_and(int id, int nthreads, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 q, %3, 0;\n\t"
      "bar.red.and.pred p, %1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r) : "r"(id), "r"(nthreads), "r"(static_cast<uint32_t>(pred)) : "memory");
  return r != 0;
}

// VEC adjacent affine parameters starting at column c (a multiple of VEC) as fp32: one or two
// 16-byte loads when the parameter array is 16-byte aligned, scalar loads otherwise
template <int VEC>
__device__ __forceinline__ void load_params(const void* p, int pdt, int c, bool vec_ok, float out[VEC]) {
  if (vec_ok && VEC >= 4) {
    if (pdt == FDP_F32) {
#pragma unroll
      for (int k = 0; k < VEC / 4; ++k) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(p) + c / 4 + k);
        out[4 * k] = v.x; out[4 * k + 1] = v.y; out[4 * k + 2] = v.z; out[4 * k + 3] = v.w;
      }
    } else {
      const uint2* q = reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(p) + c);
#pragma unroll
      for (int k = 0; k < VEC / 4; ++k) {
        const uint2 raw = __ldg(q + k);
        const uint32_t w[2] = {raw.x, raw.y};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          if (pdt == FDP_BF16) {
            const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[e]);
            out[4 * k + 2 * e] = __bfloat162float(h.x); out[4 * k + 2 * e + 1] = __bfloat162float(h.y);
          } else {
            const __half2 h = *reinterpret_cast<const __half2*>(&w[e]);
            out[4 * k + 2 * e] = __half2float(h.x); out[4 * k + 2 * e + 1] = __half2float(h.y);
          }
        }
      }
    }
  } else {
#pragma unroll
    for (int v = 0; v < VEC; ++v) out[v] = load_as(p, pdt, c + v);
  }
}

// ---------------------------------------------------------------------------------------------
// forward: one warp per row; mean, biased variance (two-pass), rstd, y = xhat*gamma + beta
// (flashdp/core/layernorm_clip.py:11-60)
// ---------------------------------------------------------------------------------------------
template <typename Tin, int VEC>
__global__ void __launch_bounds__(128) ln_fwd_kernel(const Tin* __restrict__ x,
                                                     const void* __restrict__ gamma,
                                                     const void* __restrict__ beta,
                                                     Tin* __restrict__ y, float* __restrict__ mean,
                                                     float* __restrict__ rstd, int rows, int d,
                                                     float eps, int pdt) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const Tin* xr = x + static_cast<size_t>(row) * d;
  Tin* yr = y + static_cast<size_t>(row) * d;
  float s = 0.f;
  if (VEC > 1) {
    for (int c = lane * VEC; c < d; c += 32 * VEC) {
      const uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
      const Tin* e = reinterpret_cast<const Tin*>(&raw);
#pragma unroll
      for (int v = 0; v < VEC; ++v) s += to_f32<Tin>(e[v]);
    }
  } else {
    for (int c = lane; c < d; c += 32) s += to_f32<Tin>(xr[c]);
  }
  const float mu = warp_sum(s) / d;
  float q = 0.f;
  if (VEC > 1) {
    for (int c = lane * VEC; c < d; c += 32 * VEC) {
      const uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
      const Tin* e = reinterpret_cast<const Tin*>(&raw);
#pragma unroll
      for (int v = 0; v < VEC; ++v) { const float t = to_f32<Tin>(e[v]) - mu; q = fmaf(t, t, q); }
    }
  } else {
    for (int c = lane; c < d; c += 32) { const float t = to_f32<Tin>(xr[c]) - mu; q = fmaf(t, t, q); }
  }
  const float rs = 1.0f / sqrtf(warp_sum(q) / d + eps);
  if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
  if (VEC > 1) {
    for (int c = lane * VEC; c < d; c += 32 * VEC) {
      const uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
      const Tin* e = reinterpret_cast<const Tin*>(&raw);
      uint4 outv;
      Tin* o = reinterpret_cast<Tin*>(&outv);
#pragma unroll
      for (int v = 0; v < VEC; ++v)
        o[v] = from_f32<Tin>((to_f32<Tin>(e[v]) - mu) * rs * load_as(gamma, pdt, c + v) + load_as(beta, pdt, c + v));
      *reinterpret_cast<uint4*>(yr + c) = outv;
    }
  } else {
    for (int c = lane; c < d; c += 32)
      yr[c] = from_f32<Tin>((to_f32<Tin>(xr[c]) - mu) * rs * load_as(gamma, pdt, c) + load_as(beta, pdt, c));
  }
}

// Staged forward: a producer warp streams groups of 8 rows into a shared-memory ring with bulk
// async copies (several groups in flight per SM, so HBM latency is covered whatever the occupancy);
// eight consumer warps take one row each, reduce mean and variance out of shared memory and write y.
constexpr int LN_MAX_STAGES = 8;
constexpr int LN_MAX_ROWS_PER_BLOCK = 256;
constexpr size_t LN_SMEM_BUDGET = 192 * 1024;
// NV > 0: a lane keeps its NV vectors of the row, gamma and beta in registers (d <= 32*VEC*NV), so the
// row is read from shared memory once; NV = 0: generic three-pass loop for longer rows.
template <typename Tin, int NV>
__global__ void __launch_bounds__(288) ln_fwd_staged_kernel(const Tin* __restrict__ x,
                                                            const void* __restrict__ gamma,
                                                            const void* __restrict__ beta,
                                                            Tin* __restrict__ y, float* __restrict__ mean,
                                                            float* __restrict__ rstd, int rows, int d,
                                                            float eps, int pdt, int n_stages,
                                                            int pvec_ok, int* sticky) {
  constexpr int VEC = 16 / sizeof(Tin);
  extern __shared__ __align__(128) unsigned char ln_smem[];
  __shared__ __align__(8) unsigned long long bars[2 * LN_MAX_STAGES];
  __shared__ int abort_flag_s;
  const WaitCtx wctx{&abort_flag_s, nullptr, sticky, WAIT_LIMIT_CYCLES};
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t row_bytes = static_cast<uint32_t>(d) * sizeof(Tin);
  const uint32_t stage_bytes = 8 * row_bytes;
  // groups of 8 rows are dealt round-robin to a grid of two blocks per SM, so every block gets
  // within one group of the same amount of work
  const int g0 = blockIdx.x, g1 = (rows + 7) / 8, gstep = gridDim.x;
  if (threadIdx.x == 0) {
    for (int s = 0; s < n_stages; ++s) { mbar_init(smem_u32(&bars[s]), 1); mbar_init(smem_u32(&bars[LN_MAX_STAGES + s]), 8); }
    abort_flag_s = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (warp == 8) {
    if (lane == 0) {
      int s = 0; uint32_t ph = 0;
      for (int g = g0; g < g1; g += gstep) {
        if (!mbar_wait(smem_u32(&bars[LN_MAX_STAGES + s]), ph ^ 1u, wctx, 5)) break;
        const int nrows = min(8, rows - g * 8);
        mbar_expect_tx(smem_u32(&bars[s]), nrows * row_bytes);
        bulk_load(smem_u32(ln_smem + s * stage_bytes), x + static_cast<size_t>(g) * 8 * d, nrows * row_bytes, smem_u32(&bars[s]));
        if (++s == n_stages) { s = 0; ph ^= 1u; }
      }
    }
    return;
  }
  constexpr int NR = NV > 0 ? NV * VEC : 1;
  float gv[NR], bv[NR];
  if (NV > 0) {
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = (j * 32 + lane) * VEC;
      if (c < d) {
        load_params<VEC>(gamma, pdt, c, pvec_ok != 0, gv + j * VEC);
        load_params<VEC>(beta, pdt, c, pvec_ok != 0, bv + j * VEC);
      }
    }
  }
  int s = 0; uint32_t ph = 0;
  for (int g = g0; g < g1; g += gstep) {
    if (!mbar_wait_warp(smem_u32(&bars[s]), ph, wctx, 6)) break;
    const int row = g * 8 + warp;
    if (NV > 0) {
      // ---- the row lives in registers ----
      const Tin* xr = reinterpret_cast<const Tin*>(ln_smem + s * stage_bytes + warp * row_bytes);
      float xv[NR];
      float sum = 0.f;
      if (row < rows) {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          const int c = (j * 32 + lane) * VEC;
          if (c < d) {
            const uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
            const Tin* e = reinterpret_cast<const Tin*>(&raw);
#pragma unroll
            for (int v = 0; v < VEC; ++v) { xv[j * VEC + v] = to_f32<Tin>(e[v]); sum += xv[j * VEC + v]; }
          }
        }
      }
      // the stage is in registers: give it back before the arithmetic
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars[LN_MAX_STAGES + s]));
      if (++s == n_stages) { s = 0; ph ^= 1u; }
      if (row >= rows) continue;
      const float mu = warp_sum(sum) / d;
      float q = 0.f;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        if ((j * 32 + lane) * VEC < d) {
#pragma unroll
          for (int v = 0; v < VEC; ++v) { const float t = xv[j * VEC + v] - mu; q = fmaf(t, t, q); }
        }
      }
      const float rs = 1.0f / sqrtf(warp_sum(q) / d + eps);
      if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
      Tin* yr = y + static_cast<size_t>(row) * d;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int c = (j * 32 + lane) * VEC;
        if (c < d) {
          uint4 outv;
          Tin* o = reinterpret_cast<Tin*>(&outv);
#pragma unroll
          for (int v = 0; v < VEC; ++v)
            o[v] = from_f32<Tin>(fmaf((xv[j * VEC + v] - mu) * rs, gv[j * VEC + v], bv[j * VEC + v]));
          *reinterpret_cast<uint4*>(yr + c) = outv;
        }
      }
      continue;
    }
    if (row < rows) {
      const Tin* xr = reinterpret_cast<const Tin*>(ln_smem + s * stage_bytes + warp * row_bytes);
      float sum = 0.f;
      for (int c = lane * VEC; c < d; c += 32 * VEC) {
        const uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
        const Tin* e = reinterpret_cast<const Tin*>(&raw);
#pragma unroll
        for (int v = 0; v < VEC; ++v) sum += to_f32<Tin>(e[v]);
      }
      const float mu = warp_sum(sum) / d;
      float q = 0.f;
      for (int c = lane * VEC; c < d; c += 32 * VEC) {
        const uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
        const Tin* e = reinterpret_cast<const Tin*>(&raw);
#pragma unroll
        for (int v = 0; v < VEC; ++v) { const float t = to_f32<Tin>(e[v]) - mu; q = fmaf(t, t, q); }
      }
      const float rs = 1.0f / sqrtf(warp_sum(q) / d + eps);
      if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
      Tin* yr = y + static_cast<size_t>(row) * d;
      for (int c = lane * VEC; c < d; c += 32 * VEC) {
        const uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
        const Tin* e = reinterpret_cast<const Tin*>(&raw);
        float gq[VEC], bq[VEC];
        load_params<VEC>(gamma, pdt, c, pvec_ok != 0, gq);
        load_params<VEC>(beta, pdt, c, pvec_ok != 0, bq);
        uint4 outv;
        Tin* o = reinterpret_cast<Tin*>(&outv);
#pragma unroll
        for (int v = 0; v < VEC; ++v) o[v] = from_f32<Tin>(fmaf((to_f32<Tin>(e[v]) - mu) * rs, gq[v], bq[v]));
        *reinterpret_cast<uint4*>(yr + c) = outv;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&bars[LN_MAX_STAGES + s]));
    if (++s == n_stages) { s = 0; ph ^= 1u; }
  }
}

// Direct forward for rows that fit a warp's registers (d <= 32 columns per lane): one warp per row,
// grid-stride, the row held as the raw 16-byte vectors it was loaded as (values are re-converted in
// each of the three passes, which keeps the kernel near 48 registers and ~40 warps resident per SM --
// the kernel is bound by instruction issue, so resident warps matter more than anything else);
// gamma and beta sit in shared memory as fp32.
template <typename Tin, int NV>
__global__ void __launch_bounds__(256, 4) ln_fwd_rows_kernel(const Tin* __restrict__ x,
                                                             const void* __restrict__ gamma,
                                                             const void* __restrict__ beta,
                                                             Tin* __restrict__ y, float* __restrict__ mean,
                                                             float* __restrict__ rstd, int rows, int d,
                                                             float eps, int pdt) {
  constexpr int VEC = 16 / sizeof(Tin);
  // gamma[d] then beta[d] as fp32, stored so that a warp's 16-byte reads are adjacent: the four
  // values k*4..k*4+3 of vector q (columns q*VEC ..) sit at float4 slot k*(d/VEC) + q.  With the
  // plain column order a lane's two float4 reads would be 32 bytes apart and every read a two-way
  // bank conflict.
  extern __shared__ __align__(16) float ln_params[];
  const int nvec = d / VEC;
  for (int c = threadIdx.x; c < d; c += 256) {
    const int q = c / VEC, i = c % VEC;
    const int idx = ((i >> 2) * nvec + q) * 4 + (i & 3);
    ln_params[idx] = load_as(gamma, pdt, c);
    ln_params[d + idx] = load_as(beta, pdt, c);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int nwarps = gridDim.x * 8;
  const float inv_d = 1.0f / d;
  for (int row = blockIdx.x * 8 + (threadIdx.x >> 5); row < rows; row += nwarps) {
    const Tin* xr = x + static_cast<size_t>(row) * d;
    uint4 raw[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = (j * 32 + lane) * VEC;
      raw[j] = (c < d) ? __ldg(reinterpret_cast<const uint4*>(xr + c)) : make_uint4(0, 0, 0, 0);
    }
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      float f[VEC];
      unpack16<Tin>(raw[j], f);
#pragma unroll
      for (int v = 0; v < VEC; ++v) sum += f[v];     // padding vectors are zero
    }
    const float mu = warp_sum(sum) * inv_d;
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      if ((j * 32 + lane) * VEC < d) {
        float f[VEC];
        unpack16<Tin>(raw[j], f);
#pragma unroll
        for (int v = 0; v < VEC; ++v) { const float t = f[v] - mu; q = fmaf(t, t, q); }
      }
    }
    const float rs = 1.0f / sqrtf(warp_sum(q) * inv_d + eps);
    if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
    Tin* yr = y + static_cast<size_t>(row) * d;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int vq = j * 32 + lane;
      if (vq * VEC < d) {
        float f[VEC], o[VEC];
        unpack16<Tin>(raw[j], f);
#pragma unroll
        for (int v4 = 0; v4 < VEC / 4; ++v4) {
          const float4 g = *reinterpret_cast<const float4*>(ln_params + (v4 * nvec + vq) * 4);
          const float4 b = *reinterpret_cast<const float4*>(ln_params + d + (v4 * nvec + vq) * 4);
          o[4 * v4 + 0] = fmaf((f[4 * v4 + 0] - mu) * rs, g.x, b.x);
          o[4 * v4 + 1] = fmaf((f[4 * v4 + 1] - mu) * rs, g.y, b.y);
          o[4 * v4 + 2] = fmaf((f[4 * v4 + 2] - mu) * rs, g.z, b.z);
          o[4 * v4 + 3] = fmaf((f[4 * v4 + 3] - mu) * rs, g.w, b.w);
        }
        *reinterpret_cast<uint4*>(yr + vq * VEC) = pack16<Tin>(o);
      }
    }
  }
}

template <typename Tin>
static void ln_fwd_t(const void* x, const void* gamma, const void* beta, void* y, float* mean,
                     float* rstd, int rows, int d, float eps, int pdt, bool vec, cudaStream_t s) {
  constexpr int V = 16 / sizeof(Tin);
  if (vec && d <= 1024 && d % 4 == 0) {
    // rows of up to 32 columns per lane: registers only, as many resident warps as possible
    constexpr int NVR = 32 / V;
    int grid = ceil_div(rows, 8);
    if (grid > 148 * 8) grid = 148 * 8;
    ln_fwd_rows_kernel<Tin, NVR><<<grid, 256, static_cast<size_t>(2) * d * sizeof(float), s>>>(
        (const Tin*)x, gamma, beta, (Tin*)y, mean, rstd, rows, d, eps, pdt);
    note_launch();
    return;
  }
  const size_t stage_bytes = static_cast<size_t>(8) * d * sizeof(Tin);
  if (vec && stage_bytes * 2 <= LN_SMEM_BUDGET) {
    const int groups = ceil_div(rows, 8);
    // two resident blocks per SM, each with a ring of up to 96 KiB
    int n_stages = static_cast<int>((96 * 1024) / stage_bytes);
    if (n_stages > LN_MAX_STAGES) n_stages = LN_MAX_STAGES;
    if (n_stages < 2) n_stages = 2;
    const int grid = groups < 2 * 148 ? groups : 2 * 148;
    constexpr int NVR = 32 / V;           // register-resident rows: up to 32 columns per lane
    const bool in_regs = d <= 32 * V * NVR;
    static bool done[64], done_r[64];
    static std::mutex mu;
    const int pv = aligned16(gamma) && aligned16(beta) ? 1 : 0;
    if (in_regs && smem_opt_in(done_r, mu, ln_fwd_staged_kernel<Tin, NVR>, LN_SMEM_BUDGET)) {
      ln_fwd_staged_kernel<Tin, NVR><<<grid, 288, n_stages * stage_bytes, s>>>(
          (const Tin*)x, gamma, beta, (Tin*)y, mean, rstd, rows, d, eps, pdt, n_stages, pv, sticky_status_slot());
      note_launch();
      return;
    }
    if (smem_opt_in(done, mu, ln_fwd_staged_kernel<Tin, 0>, LN_SMEM_BUDGET)) {
      ln_fwd_staged_kernel<Tin, 0><<<grid, 288, n_stages * stage_bytes, s>>>(
          (const Tin*)x, gamma, beta, (Tin*)y, mean, rstd, rows, d, eps, pdt, n_stages, pv, sticky_status_slot());
      note_launch();
      return;
    }
  }
  dim3 grid(ceil_div(rows, 4));
  if (vec)
    ln_fwd_kernel<Tin, V><<<grid, 128, 0, s>>>((const Tin*)x, gamma, beta, (Tin*)y, mean, rstd, rows, d, eps, pdt);
  else
    ln_fwd_kernel<Tin, 1><<<grid, 128, 0, s>>>((const Tin*)x, gamma, beta, (Tin*)y, mean, rstd, rows, d, eps, pdt);
  note_launch();
}

void ln_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
            int rows, int d, float eps, int dt, int pdt, cudaStream_t s) {
  const int V = 16 / static_cast<int>(dtype_size(dt));
  const bool vec = (d % V == 0) && aligned16(x) && aligned16(y);
  if (dt == FDP_F32) ln_fwd_t<float>(x, gamma, beta, y, mean, rstd, rows, d, eps, pdt, vec, s);
  else if (dt == FDP_BF16) ln_fwd_t<__nv_bfloat16>(x, gamma, beta, y, mean, rstd, rows, d, eps, pdt, vec, s);
  else ln_fwd_t<__half>(x, gamma, beta, y, mean, rstd, rows, d, eps, pdt, vec, s);
}

// ---------------------------------------------------------------------------------------------
// backward.  A block of CW consumer threads (256 or 512) is RG = CW/TPR row groups of TPR threads; a row group walks
// rows of one chunk of one sample, each thread owning NV vectors of VEC columns (vector j at
// column (j*TPR + t)*VEC).  Per row: xhat, wdy = gamma*dy, the two row means, dx
// (flashdp/core/layernorm_clip.py:95-103); per thread: running sums of dy*xhat and dy over the
// rows it saw.  At the end the row groups are summed in fixed order and one partial
// [sample, chunk, d] is written per tensor.
// ---------------------------------------------------------------------------------------------
// STAGED: a ninth warp streams the rows of x and dy into a shared-memory ring with bulk async
// copies (one stage = the RG rows the row groups work on at once), so several stages are in flight
// per SM whatever the register-limited occupancy; the row groups read their row from the ring.
#ifndef FDP_LN_BWD_PRODUCER_WARP
#define FDP_LN_BWD_PRODUCER_WARP 0
#endif
// Who feeds the ring.  0: thread 0 of the block, between its own rows -- the block is then exactly
// CW threads; with CW = 512 that is four warps per scheduler and 128 registers per thread.  1: an
// extra warp -- a fifth warp on one scheduler, which caps every thread at 96 registers.
constexpr bool LN_BWD_PW = FDP_LN_BWD_PRODUCER_WARP != 0;
#ifndef FDP_LN_BWD_STAGES
#define FDP_LN_BWD_STAGES 3
#endif
#ifndef FDP_LN_BWD_RING_KB
#define FDP_LN_BWD_RING_KB 96
#endif
// EXACT: d == TPR * NV * VEC, every thread's columns exist (no column checks, no zero fill).
template <typename Tin, int VEC, int NV, int TPR, bool STAGED, int CW, bool EXACT = false>
__global__ void __launch_bounds__((STAGED && LN_BWD_PW) ? CW + 32 : CW) ln_bwd_kernel(
    const Tin* __restrict__ dy, const Tin* __restrict__ x, const void* __restrict__ gamma,
    const float* __restrict__ mean, const float* __restrict__ rstd, Tin* __restrict__ dx,
    float* __restrict__ dg_part, float* __restrict__ db_part, int T, int d, int pdt,
    int rows_per_block, int chunks, int n_stages, int* sticky) {
  constexpr int RG = CW / TPR;
  constexpr int NWG = TPR / 32;  // warps per row group
  // dynamic shared memory: the ring (STAGED), reused at the end as [2][RG][TPR*NV*VEC] floats for the
  // cross-group sum
  extern __shared__ __align__(128) unsigned char ln_smem[];
  float* sm = reinterpret_cast<float*>(ln_smem);
  __shared__ float2 xch[2][RG][NWG > 1 ? NWG : 1];   // row sums of the group's warps, alternating by iteration
  __shared__ __align__(8) unsigned long long bars[2 * LN_MAX_STAGES];
  __shared__ int abort_flag_s;
  __shared__ float s_mean[LN_MAX_ROWS_PER_BLOCK], s_rstd[LN_MAX_ROWS_PER_BLOCK];  // this chunk's row statistics
  const WaitCtx wctx{&abort_flag_s, nullptr, sticky, WAIT_LIMIT_CYCLES};
  const int rg = (threadIdx.x % CW) / TPR, t = threadIdx.x % TPR;
  const int lane = threadIdx.x & 31, wig = (threadIdx.x % TPR) >> 5;
  // one-dimensional grid (the batch may exceed 65535): block = b * chunks + chunk
  const int b = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
  const int r0 = chunk * rows_per_block, r1 = min(T, r0 + rows_per_block);
  const int n_iter = (r1 - r0 + RG - 1) / RG;
  const uint32_t row_bytes = static_cast<uint32_t>(d) * sizeof(Tin);
  const uint32_t stage_bytes = 2 * RG * row_bytes;

  // the RG rows of iteration `it` (x, then dy) into stage `st`; one thread
  auto issue_stage = [&](int it, int st) {
    const int rb = r0 + it * RG;
    const int nrows = min(RG, r1 - rb);
    const size_t goff = (static_cast<size_t>(b) * T + rb) * d;
    mbar_expect_tx(smem_u32(&bars[st]), 2 * nrows * row_bytes);
    bulk_load(smem_u32(ln_smem + st * stage_bytes), x + goff, nrows * row_bytes, smem_u32(&bars[st]));
    bulk_load(smem_u32(ln_smem + st * stage_bytes + RG * row_bytes), dy + goff, nrows * row_bytes, smem_u32(&bars[st]));
  };
  if (STAGED && threadIdx.x == 0) {
    for (int s = 0; s < n_stages; ++s) { mbar_init(smem_u32(&bars[s]), 1); mbar_init(smem_u32(&bars[LN_MAX_STAGES + s]), CW / 32); }
    abort_flag_s = 0;
    mbar_fence_init();
    // the first stages are on their way before anything else of the block touches global memory:
    // their latency overlaps the fetch of the row statistics and of gamma below
    if (!LN_BWD_PW)
      for (int it = 0; it < n_stages && it < n_iter; ++it) issue_stage(it, it);
  }
  // one parallel fetch of the chunk's mean / rstd, so no row waits on a global load of its own
  if (threadIdx.x < r1 - r0) {
    s_mean[threadIdx.x] = mean[static_cast<size_t>(b) * T + r0 + threadIdx.x];
    s_rstd[threadIdx.x] = rstd[static_cast<size_t>(b) * T + r0 + threadIdx.x];
  }
  __syncthreads();

  float gam[NV * VEC], accg[NV * VEC], accb[NV * VEC];
#pragma unroll
  for (int j = 0; j < NV; ++j)
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      const int c = (j * TPR + t) * VEC + v;
      gam[j * VEC + v] = (EXACT || c < d) ? load_as(gamma, pdt, c) : 0.f;
      accg[j * VEC + v] = 0.f; accb[j * VEC + v] = 0.f;
    }
  const float inv_d = 1.0f / d;

  if (STAGED && LN_BWD_PW && threadIdx.x >= CW) {
    // ---- producer warp ----
    if (threadIdx.x == CW) {
      int s = 0; uint32_t ph = 0;
      for (int it = 0; it < n_iter; ++it) {
        if (!mbar_wait(smem_u32(&bars[LN_MAX_STAGES + s]), ph ^ 1u, wctx, 7)) break;
        issue_stage(it, s);
        if (++s == n_stages) { s = 0; ph ^= 1u; }
      }
    }
  } else {
    // ---- row groups ----
    int s = 0; uint32_t ph = 0;
    int prev_s = 0; uint32_t prev_ph = 0;
    for (int it = 0; it < n_iter; ++it) {
      const int r = r0 + it * RG + rg;
      const bool valid = r < r1;
      const size_t row = static_cast<size_t>(b) * T + r;
      const Tin* xr = x + row * d;
      const Tin* dyr = dy + row * d;
      bool ok = true;   // whether this warp saw the stage arrive; agreed on by the row group below
      if (STAGED) {
        ok = mbar_wait_warp(smem_u32(&bars[s]), ph, wctx, 8);
        if (NWG == 1 && !ok) break;
        xr = reinterpret_cast<const Tin*>(ln_smem + s * stage_bytes + rg * row_bytes);
        dyr = reinterpret_cast<const Tin*>(ln_smem + s * stage_bytes + (RG + rg) * row_bytes);
      }
      float xh[NV * VEC], wd[NV * VEC];
      float s1 = 0.f, s2 = 0.f;
      float mu = 0.f, rs = 0.f;
      if (valid) {
        mu = s_mean[r - r0]; rs = s_rstd[r - r0];
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          const int c = (j * TPR + t) * VEC;
          if constexpr (VEC > 1) {
            if (EXACT || c < d) {
              float ex[VEC], ed[VEC];
              unpack16<Tin>(*reinterpret_cast<const uint4*>(xr + c), ex);
              unpack16<Tin>(*reinterpret_cast<const uint4*>(dyr + c), ed);
#pragma unroll
              for (int v = 0; v < VEC; ++v) {
                const int i = j * VEC + v;
                const float xv = (ex[v] - mu) * rs, dv = ed[v];
                xh[i] = xv; wd[i] = dv * gam[i];
                accg[i] = fmaf(dv, xv, accg[i]); accb[i] += dv;
                s1 = fmaf(xv, wd[i], s1); s2 += wd[i];
              }
            } else {
#pragma unroll
              for (int v = 0; v < VEC; ++v) { xh[j * VEC + v] = 0.f; wd[j * VEC + v] = 0.f; }
            }
          } else {
            const int i = j;
            if (c < d) {
              const float xv = (to_f32<Tin>(xr[c]) - mu) * rs, dv = to_f32<Tin>(dyr[c]);
              xh[i] = xv; wd[i] = dv * gam[i];
              accg[i] = fmaf(dv, xv, accg[i]); accb[i] += dv;
              s1 = fmaf(xv, wd[i], s1); s2 += wd[i];
            } else { xh[i] = 0.f; wd[i] = 0.f; }
          }
        }
      }
      if (STAGED) {
        // the row is in registers: hand the stage back to the producer
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars[LN_MAX_STAGES + s]));
        if (!LN_BWD_PW && threadIdx.x == 0 && it >= 1 && it - 1 + n_stages < n_iter) {
          // refill the stage of the PREVIOUS iteration: by now every warp has normally taken its row
          // of that stage into registers, so this wait rarely spins, and no row group is tied to the
          // slowest one of the current iteration.  If the wait runs out nothing is issued and the
          // consumers' own bounded waits end the block.
          if (mbar_wait(smem_u32(&bars[LN_MAX_STAGES + prev_s]), prev_ph, wctx, 7)) issue_stage(it - 1 + n_stages, prev_s);
        }
        prev_s = s; prev_ph = ph;
        if (++s == n_stages) { s = 0; ph ^= 1u; }
      }
      if (!valid) { if (!ok) break; continue; }     // `valid` is the same for the whole row group
      s1 = warp_sum(s1); s2 = warp_sum(s2);
      if (NWG > 1) {
        // One barrier per row: the slot alternates, and a thread writes slot (it+1)&1 only after
        // this iteration's barrier, which every thread of the group reaches after its reads of that
        // slot in iteration it-1.
        if (lane == 0) xch[it & 1][rg][wig] = make_float2(s1, s2);
        // the barrier also carries the row group's verdict on the wait: either all of its warps go
        // on or all of them leave, so none is left waiting at a barrier the others never reach
        if (!bar_red_and(1 + rg, TPR, ok)) break;
        s1 = 0.f; s2 = 0.f;
#pragma unroll
        for (int w = 0; w < NWG; ++w) { s1 += xch[it & 1][rg][w].x; s2 += xch[it & 1][rg][w].y; }
      }
      if (dx != nullptr) {
        const float a1 = -(s1 * inv_d) * rs, a2 = -(s2 * inv_d) * rs;
        Tin* dxr = dx + row * d;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          const int c = (j * TPR + t) * VEC;
          if (!EXACT && c >= d) continue;
          if constexpr (VEC > 1) {
            float o[VEC];
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
              const int i = j * VEC + v;
              o[v] = fmaf(xh[i], a1, fmaf(wd[i], rs, a2));   // (wd - (xhat*c1 + c2)) * rs
            }
            *reinterpret_cast<uint4*>(dxr + c) = pack16<Tin>(o);
          } else {
            dxr[c] = from_f32<Tin>(fmaf(xh[j], a1, fmaf(wd[j], rs, a2)));
          }
        }
      }
    }
  }

  // the reduction kernel may be scheduled while this block finishes (triggering at the top of the kernel
  // instead, so that its blocks sit waiting beside the row loop, cost 1.3 us per call)
  pdl_trigger();
  // cross-row-group sum, fixed order, both tensors in one pass: [2][RG][CPG] floats in the buffer
  // the ring occupied (every consumer is past its last stage once it is past the barrier below)
  constexpr int CPG = TPR * NV * VEC;  // columns covered by a row group
  __syncthreads();
  if (threadIdx.x < CW) {
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      float* dstp = sm + which * RG * CPG + rg * CPG;
      const float* acc = which == 0 ? accg : accb;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        if constexpr (VEC % 4 == 0) {
#pragma unroll
          for (int v = 0; v < VEC; v += 4) {
            const float* a = acc + j * VEC + v;
            *reinterpret_cast<float4*>(&dstp[(j * TPR + t) * VEC + v]) = make_float4(a[0], a[1], a[2], a[3]);
          }
        } else {
#pragma unroll
          for (int v = 0; v < VEC; ++v) dstp[(j * TPR + t) * VEC + v] = acc[j * VEC + v];
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x < CW) {
    const size_t off = (static_cast<size_t>(b) * chunks + chunk) * d;
    for (int c2 = threadIdx.x; c2 < 2 * d; c2 += CW) {
      const int which = c2 >= d ? 1 : 0;
      const int c = c2 - which * d;
      const float* src = sm + which * RG * CPG + c;
      float tot = 0.f;
#pragma unroll
      for (int g = 0; g < RG; ++g) tot += src[g * CPG];
      (which == 0 ? dg_part : db_part)[off + c] = tot;
    }
  }
}

LnPlan ln_plan(int B, int T, int d, int dt) {
  LnPlan pl;
  const int V = 16 / static_cast<int>(dtype_size(dt));
  pl.vec = (d % V == 0);
  const int vec = pl.vec ? V : 1;
  // Vector path up to d = 4096: 16 columns per thread and 512 consumer threads (16 warps hide the
  // latency of the row arithmetic; about 115 registers each).  Otherwise 32 columns, 256 threads
  // (one warp per row at d = 1024, no exchange between warps, but only 8 warps per SM: 37.2 against
  // 36.2 us per call at B=16, T=1024, d=1024, bf16).
  int nv_max = pl.vec ? (32 / V) : 32;
  pl.cw = 256;
  if (pl.vec && d <= 4096) { nv_max = 16 / V; pl.cw = 512; }
  pl.cpt = nv_max * vec;
  pl.tpr = 32;
  while (pl.tpr < 256 && pl.tpr * pl.cpt < d) pl.tpr *= 2;
  // Partials are [B, chunks, d]; one chunk = rows_per_block rows of one sample = one block.  The
  // backward kernel holds one block per SM, so B * chunks blocks run in whole waves of LN_SMS: pick
  // the chunk length that minimises waves * (rows + fixed cost per block); ties go to the longer
  // chunk (fewer partials).  The count must not depend on the device in use -- the workspace
  // query has to agree with the launch -- hence the constant.
  constexpr int LN_SMS = 148, BLOCK_FIXED_ROWS = 6;
  const int rg = pl.cw / pl.tpr;   // rows a block works on at a time
  int best_r = 64, best_cost = 1 << 30;
  for (int r = 32; r <= LN_MAX_ROWS_PER_BLOCK; r += 8) {
    if (r % rg != 0) continue;
    const long long blocks = static_cast<long long>(B) * ceil_div(T, r);
    const long long waves = (blocks + LN_SMS - 1) / LN_SMS;
    const long long cost = waves * (r + BLOCK_FIXED_ROWS);
    if (cost <= best_cost) { best_cost = static_cast<int>(cost < (1 << 30) ? cost : (1 << 30) - 1); best_r = r; }
  }
  pl.rows_per_block = best_r;
  pl.chunks = ceil_div(T, pl.rows_per_block);
  return pl;
}

template <typename Tin, int VEC, int NV, int TPRV, bool STAGED, int CW, bool EXACT = false>
static bool ln_bwd_launch_one(const void* dy, const void* x, const void* gamma, const float* mean,
                              const float* rstd, void* dx, float* dg_part, float* db_part, int B, int T,
                              int d, int pdt, const LnPlan& pl, int n_stages, cudaStream_t s) {
  const unsigned grid = static_cast<unsigned>(static_cast<size_t>(B) * pl.chunks);
  constexpr int RG = CW / TPRV;
  const size_t reduce_bytes = static_cast<size_t>(2) * CW * NV * VEC * sizeof(float);   // both tensors at once
  const size_t stage_bytes = static_cast<size_t>(2) * RG * d * sizeof(Tin);
  size_t smem = reduce_bytes;
  if (STAGED && n_stages * stage_bytes > smem) smem = n_stages * stage_bytes;
  static bool done[64];
  static std::mutex mu;
  if (smem > 48 * 1024 && !smem_opt_in(done, mu, ln_bwd_kernel<Tin, VEC, NV, TPRV, STAGED, CW, EXACT>, LN_SMEM_BUDGET)) return false;
  ln_bwd_kernel<Tin, VEC, NV, TPRV, STAGED, CW, EXACT><<<grid, (STAGED && LN_BWD_PW) ? CW + 32 : CW, smem, s>>>(
      (const Tin*)dy, (const Tin*)x, gamma, mean, rstd, (Tin*)dx, dg_part, db_part, T, d, pdt,
      pl.rows_per_block, pl.chunks, n_stages, sticky_status_slot());
  note_launch();
  return true;
}

template <typename Tin, int VEC, int NV, int CW>
static void ln_bwd_launch(const void* dy, const void* x, const void* gamma, const float* mean,
                          const float* rstd, void* dx, float* dg_part, float* db_part, int B, int T,
                          int d, int pdt, const LnPlan& pl, cudaStream_t s) {
  // ring of up to FDP_LN_BWD_STAGES stages within FDP_LN_BWD_RING_KB (five stages in 160 KiB measured
  // no faster than three in 96 KiB: 36.1 against 35.3 us per call at B=16, T=1024, d=1024, bf16);
  // needs 16-byte rows, i.e. the vector path
  const size_t stage_bytes = static_cast<size_t>(2) * (CW / pl.tpr) * d * sizeof(Tin);
  int n_stages = static_cast<int>((static_cast<size_t>(FDP_LN_BWD_RING_KB) * 1024) / stage_bytes);
  if (n_stages > FDP_LN_BWD_STAGES) n_stages = FDP_LN_BWD_STAGES;
  const int n_iter = ceil_div(pl.rows_per_block, CW / pl.tpr);
  if (n_stages > n_iter) n_stages = n_iter;
  const bool staged = VEC > 1 && n_stages >= 2;
#define FDP_LN_CASE(TPRV)                                                                                      \
  if (staged && d == TPRV * NV * VEC &&                                                                        \
      ln_bwd_launch_one<Tin, VEC, NV, TPRV, (VEC > 1), CW, (VEC > 1)>(dy, x, gamma, mean, rstd, dx, dg_part, db_part, \
                                                                      B, T, d, pdt, pl, n_stages, s))          \
    return;                                                                                                    \
  if (staged && ln_bwd_launch_one<Tin, VEC, NV, TPRV, (VEC > 1), CW>(dy, x, gamma, mean, rstd, dx, dg_part, db_part, \
                                                                     B, T, d, pdt, pl, n_stages, s))                 \
    return;                                                                                                    \
  ln_bwd_launch_one<Tin, VEC, NV, TPRV, false, CW>(dy, x, gamma, mean, rstd, dx, dg_part, db_part, B, T, d, pdt, pl, 0, s)
  switch (pl.tpr) {
    case 32: FDP_LN_CASE(32); break;
    case 64: FDP_LN_CASE(64); break;
    case 128: FDP_LN_CASE(128); break;
    default: FDP_LN_CASE(256); break;
  }
#undef FDP_LN_CASE
}

void ln_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
            void* dx, float* dg_part, float* db_part, int B, int T, int d, int dt, int pdt,
            const LnPlan& pl, cudaStream_t s) {
  const bool vec = pl.vec && aligned16(dy) && aligned16(x) && (dx == nullptr || aligned16(dx));
#define FDP_LN_ARGS dy, x, gamma, mean, rstd, dx, dg_part, db_part, B, T, d, pdt, pl, s
  if (dt == FDP_F32) {
    if (vec && pl.cw == 512) ln_bwd_launch<float, 4, 4, 512>(FDP_LN_ARGS);
    else if (vec) ln_bwd_launch<float, 4, 8, 256>(FDP_LN_ARGS);
    else ln_bwd_launch<float, 1, 32, 256>(FDP_LN_ARGS);
  } else if (dt == FDP_BF16) {
    if (vec && pl.cw == 512) ln_bwd_launch<__nv_bfloat16, 8, 2, 512>(FDP_LN_ARGS);
    else if (vec) ln_bwd_launch<__nv_bfloat16, 8, 4, 256>(FDP_LN_ARGS);
    else ln_bwd_launch<__nv_bfloat16, 1, 32, 256>(FDP_LN_ARGS);
  } else {
    if (vec && pl.cw == 512) ln_bwd_launch<__half, 8, 2, 512>(FDP_LN_ARGS);
    else if (vec) ln_bwd_launch<__half, 8, 4, 256>(FDP_LN_ARGS);
    else ln_bwd_launch<__half, 1, 32, 256>(FDP_LN_ARGS);
  }
#undef FDP_LN_ARGS
}

// ---------------------------------------------------------------------------------------------
// per-sample finalisation.  `part` holds [2 tensors][B][chunks][d]; the reduced per-sample
// gradient lands in chunk slot 0.  sumsq[tensor*B + b] = ||per-sample grad||^2 over d.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ln_psgrad_reduce_kernel(float* __restrict__ part,
                                                               float* __restrict__ sumsq, int chunks,
                                                               int d) {
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  // one-dimensional grid: block = (tensor*B + b) * column blocks + block of 256 columns
  const int nblk = (d + 255) / 256;
  const int sample = blockIdx.x / nblk, cblk = blockIdx.x % nblk;
  float* p = part + static_cast<size_t>(sample) * chunks * d;
  const int c = cblk * 256 + threadIdx.x;
  float sq = 0.f;
  if (c < d) {
    float t = 0.f;
    for (int k = 0; k < chunks; ++k) t += p[static_cast<size_t>(k) * d + c];
    p[c] = t;
    sq = t * t;
  }
  sq = block_sum(sq, red);
  if (threadIdx.x == 0) sumsq[blockIdx.x] = sq;
}

int ln_sumsq_parts(int d) { return ceil_div(d, 256); }

void ln_psgrad_reduce(float* part, float* sumsq, int B, int chunks, int d, cudaStream_t s) {
  const unsigned grid = static_cast<unsigned>(static_cast<size_t>(2) * B * ln_sumsq_parts(d));
  launch_dependent(ln_psgrad_reduce_kernel, dim3(grid), dim3(256), 0, s, part, sumsq, chunks, d);
  note_launch();
}

__global__ void __launch_bounds__(256) ln_psgrad_finalize_kernel(const float* __restrict__ part,
                                                                 const float* __restrict__ factors,
                                                                 void* __restrict__ out0, void* __restrict__ out1,
                                                                 int B, int chunks, int d, int out_dt,
                                                                 float inv_div, NoiseKey nk0, NoiseKey nk1) {
  pdl_wait();
  const int c = blockIdx.x * 256 + threadIdx.x;
  const int tensor = blockIdx.y;
  void* out = tensor == 0 ? out0 : out1;
  if (c >= d || out == nullptr) return;
  const float* p = part + static_cast<size_t>(tensor) * B * chunks * d;
  const float* f = factors + tensor * B;
  float acc = 0.f;
  for (int b = 0; b < B; ++b) acc = fmaf(f[b], p[static_cast<size_t>(b) * chunks * d + c], acc);
  float v = acc * inv_div;
  const NoiseKey& nk = tensor == 0 ? nk0 : nk1;
  if (nk.std != 0.f) v += noise_at(nk, c);
  store_as(out, out_dt, c, v);
}

void ln_psgrad_finalize(const float* part, const float* factors, void* out0, void* out1, int B, int chunks,
                        int d, int out_dt, float inv_div, NoiseKey nk0, NoiseKey nk1, cudaStream_t s) {
  dim3 grid(ceil_div(d, 256), 2);
  launch_dependent(ln_psgrad_finalize_kernel, grid, dim3(256), 0, s, part, factors, out0, out1, B, chunks, d, out_dt, inv_div, nk0, nk1);
  note_launch();
}

__global__ void __launch_bounds__(256) ln_clip_finalize_kernel(
    const float* __restrict__ part, const float* __restrict__ sumsq, int nparts, float C, float clamp,
    float* __restrict__ norms0, float* __restrict__ norms1, void* __restrict__ out0, void* __restrict__ out1,
    int B, int chunks, int d, int out_dt, float inv_div, NoiseKey nk0, NoiseKey nk1) {
  extern __shared__ float s_fac[];  // [B] factors of this block's tensor
  const int tensor = blockIdx.y;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  pdl_wait();
  for (int b = w; b < B; b += 8) {
    float sq = 0.f;
    for (int i = lane; i < nparts; i += 32) sq += sumsq[static_cast<size_t>(tensor * B + b) * nparts + i];
    sq = warp_sum(sq);
    if (lane == 0) {
      const float n = sqrtf(fmaxf(sq, 0.f));
      s_fac[b] = clip_factor(n, C, clamp);
      float* no = tensor == 0 ? norms0 : norms1;
      if (blockIdx.x == 0 && no != nullptr) no[b] = n;
    }
  }
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  void* out = tensor == 0 ? out0 : out1;
  if (c >= d || out == nullptr) return;
  const float* p = part + static_cast<size_t>(tensor) * B * chunks * d;
  float acc = 0.f;
  for (int b = 0; b < B; ++b) acc = fmaf(s_fac[b], p[static_cast<size_t>(b) * chunks * d + c], acc);
  float v = acc * inv_div;
  const NoiseKey& nk = tensor == 0 ? nk0 : nk1;
  if (nk.std != 0.f) v += noise_at(nk, c);
  store_as(out, out_dt, c, v);
}

void ln_clip_finalize(const float* part, const float* sumsq, int nparts, float C, float clamp, float* factors_ws,
                      float* norms0, float* norms1, void* out0, void* out1, int B, int chunks, int d, int out_dt,
                      float inv_div, NoiseKey nk0, NoiseKey nk1, cudaStream_t s) {
  if (static_cast<size_t>(B) * sizeof(float) <= 32 * 1024) {
    dim3 grid(ceil_div(d, 256), 2);
    launch_dependent(ln_clip_finalize_kernel, grid, dim3(256), B * sizeof(float), s, part, sumsq, nparts, C, clamp,
                     norms0, norms1, out0, out1, B, chunks, d, out_dt, inv_div, nk0, nk1);
    note_launch();
    return;
  }
  clip_factors_pair(sumsq, nparts, B, C, clamp, factors_ws, norms0, norms1, s);
  ln_psgrad_finalize(part, factors_ws, out0, out1, B, chunks, d, out_dt, inv_div, nk0, nk1, s);
}

// ---------------------------------------------------------------------------------------------
// Compatibility: the "clipped" dgamma / dbeta of the reference's fused LayerNorm backward
// (flashdp/core/layernorm_clip.py:109-131, summed by :134-160).  Row r adds its dy*xhat and dy to
// buffer r % G; every addition after a buffer's first one first saturates the buffer element by
// element, buf <- partial + buf * min(clamp, C / (|buf| + 1e-10)).  In the reference the rows of a
// buffer arrive in whatever order the row programs win a spin lock; here they are taken in
// increasing row order, which makes the result a function of the inputs.  One thread owns one
// (buffer, column) pair and walks that buffer's rows; no locks, no atomics.  No division by the
// batch and no noise (the reference's fused path has neither, flashdp/layers/layernorm.py:179-203).
// ---------------------------------------------------------------------------------------------
template <typename Tin>
__global__ void __launch_bounds__(128) ln_saturate_kernel(const Tin* __restrict__ dy, const Tin* __restrict__ x,
                                                          const float* __restrict__ mean, const float* __restrict__ rstd,
                                                          float* __restrict__ dw_buf, float* __restrict__ db_buf,
                                                          int rows, int d, int groups, int pdt, float C, float clamp) {
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int g = blockIdx.y;
  if (c >= d) return;
  float bw = 0.f, bb = 0.f;
  bool first = true;
  for (int r = g; r < rows; r += groups) {
    const size_t i = static_cast<size_t>(r) * d + c;
    const float dv = to_f32<Tin>(dy[i]);
    const float xh = (to_f32<Tin>(x[i]) - mean[r]) * rstd[r];
    // the partial sums are rounded to the parameter dtype before they are accumulated (:106-107)
    float pw = dv * xh, pb = dv;
    if (pdt == FDP_BF16) { pw = __bfloat162float(__float2bfloat16_rn(pw)); pb = __bfloat162float(__float2bfloat16_rn(pb)); }
    else if (pdt == FDP_F16) { pw = __half2float(__float2half_rn(pw)); pb = __half2float(__float2half_rn(pb)); }
    if (first) { bw = pw; bb = pb; first = false; }
    else {
      bw = pw + bw * clip_factor(fabsf(bw), C, clamp);
      bb = pb + bb * clip_factor(fabsf(bb), C, clamp);
    }
  }
  dw_buf[static_cast<size_t>(g) * d + c] = bw;
  db_buf[static_cast<size_t>(g) * d + c] = bb;
}

__global__ void __launch_bounds__(128) ln_saturate_sum_kernel(const float* __restrict__ dw_buf, const float* __restrict__ db_buf,
                                                              void* __restrict__ dgamma, void* __restrict__ dbeta, int d,
                                                              int groups, int out_dt) {
  const int c = blockIdx.x * 128 + threadIdx.x;
  if (c >= d) return;
  float sw = 0.f, sb = 0.f;
  for (int g = 0; g < groups; ++g) { sw += dw_buf[static_cast<size_t>(g) * d + c]; sb += db_buf[static_cast<size_t>(g) * d + c]; }
  store_as(dgamma, out_dt, c, sw);
  if (dbeta != nullptr) store_as(dbeta, out_dt, c, sb);
}

int ln_saturate_groups(int rows, int d) {
  // flashdp/core/layernorm_clip.py:261-264, and min(GROUP_SIZE_M, M) of :309
  int g = 64;
  if (d <= 8192) g = 96;
  if (d <= 4096) g = 128;
  if (d <= 1024) g = 256;
  return g < rows ? g : rows;
}

void ln_saturate(const void* dy, const void* x, const float* mean, const float* rstd, float* dw_buf, float* db_buf,
                 void* dgamma, void* dbeta, int rows, int d, int dt, int pdt, float C, float clamp, cudaStream_t s) {
  const int groups = ln_saturate_groups(rows, d);
  dim3 grid(ceil_div(d, 128), groups);
  if (dt == FDP_F32)
    ln_saturate_kernel<float><<<grid, 128, 0, s>>>((const float*)dy, (const float*)x, mean, rstd, dw_buf, db_buf, rows, d, groups, pdt, C, clamp);
  else if (dt == FDP_BF16)
    ln_saturate_kernel<__nv_bfloat16><<<grid, 128, 0, s>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, mean, rstd, dw_buf, db_buf, rows, d, groups, pdt, C, clamp);
  else
    ln_saturate_kernel<__half><<<grid, 128, 0, s>>>((const __half*)dy, (const __half*)x, mean, rstd, dw_buf, db_buf, rows, d, groups, pdt, C, clamp);
  note_launch();
  ln_saturate_sum_kernel<<<ceil_div(d, 128), 128, 0, s>>>(dw_buf, db_buf, dgamma, dbeta, d, groups, pdt);
  note_launch();
}

}  // namespace fdp
