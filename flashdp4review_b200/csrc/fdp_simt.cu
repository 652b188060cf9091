// Generic-shape kernels: per-sample norm, clip factors, clipped-sum weight gradient, input
// gradient and the bias-gradient reduction.  Any dtype, any size, true fp32 FMA accumulation
// (the 1e-5 fp32 tolerance rules out TF32).  The aligned bf16/fp16 shapes take the tcgen05
// kernels instead; these cover fp32 and ragged shapes.
#include "fdp_kernels.h"

namespace fdp {

constexpr int TM = 64, TN = 64, TK = 16;  // block tile; 256 threads, 4x4 outputs per thread

// acc[i][j] += sum_k A(k, m0+4*ty+i) * B(k, n0+4*tx+j), operands addressed through strides so the
// same body serves the weight gradient (contraction over rows) and the input gradient.
// SCALED multiplies A(k, .) by factors[k / T] (the per-sample clip factor of row k).
template <typename Tin, bool SCALED>
__device__ __forceinline__ void simt_tile(const Tin* __restrict__ A, long sAk, long sAm,
                                          const Tin* __restrict__ Bm, long sBk, long sBn, int K,
                                          int M, int N, int m0, int n0,
                                          const float* __restrict__ factors, int T,
                                          float acc[4][4]) {
  __shared__ __align__(16) float As[TK][TM];
  __shared__ __align__(16) float Bs[TK][TN];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256;
      int kk, mm;
      if (sAm == 1) { kk = idx >> 6; mm = idx & 63; } else { mm = idx >> 4; kk = idx & 15; }
      const int k = k0 + kk, m = m0 + mm;
      float v = 0.f;
      if (k < K && m < M) {
        v = to_f32<Tin>(A[k * sAk + m * sAm]);
        if (SCALED) v *= factors[k / T];
      }
      As[kk][mm] = v;
      int nn;
      if (sBn == 1) { kk = idx >> 6; nn = idx & 63; } else { nn = idx >> 4; kk = idx & 15; }
      const int kb = k0 + kk, n = n0 + nn;
      Bs[kk][nn] = (kb < K && n < N) ? to_f32<Tin>(Bm[kb * sBk + n * sBn]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      const float4 a = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
}

// ---- fp32 fast path: 128 x 128 block tiles, 8 x 8 outputs per thread, double-buffered stages --------
// For fp32 operands whose contraction runs over rows (the weight gradient and its per-sample norm):
// A(k, m) = A[k * lda + m], B(k, n) = Bm[k * ldb + n], both row pitches multiples of four elements and
// both bases 16-byte aligned, so a stage (16 rows x 128 columns of each operand) is fetched with
// 16-byte loads; the next stage is prefetched into registers while the current one is multiplied.
// A thread owns rows {4ty..4ty+3, 64+4ty..} and columns {4tx..4tx+3, 64+4tx..} of the tile: its
// shared-memory reads are broadcasts (A) or conflict-free 16-byte reads (B), four per 64 FMAs.
constexpr int FM = 128, FN = 128, FK = 16;

template <bool SCALED>
__device__ __forceinline__ void fast_tile(const float* __restrict__ A, int lda, const float* __restrict__ Bm, int ldb,
                                          int K, int M, int N, int m0, int n0,
                                          const float* __restrict__ factors, int T, float acc[8][8]) {
  __shared__ __align__(16) float As[2][FK][FM];
  __shared__ __align__(16) float Bs[2][FK][FN];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int lk = tid >> 5, lc = (tid & 31) * 4;       // this thread's rows lk, lk + 8 and columns lc..lc+3 of a stage
  float4 ra[2], rb[2];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int k = k0 + lk + 8 * i;
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
      if (k < K) {
        if (m0 + lc < M) a = __ldg(reinterpret_cast<const float4*>(A + static_cast<size_t>(k) * lda + m0 + lc));
        if (n0 + lc < N) b = __ldg(reinterpret_cast<const float4*>(Bm + static_cast<size_t>(k) * ldb + n0 + lc));
        if (SCALED) { const float f = factors[k / T]; a.x *= f; a.y *= f; a.z *= f; a.w *= f; }
      }
      ra[i] = a; rb[i] = b;
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      *reinterpret_cast<float4*>(&As[buf][lk + 8 * i][lc]) = ra[i];
      *reinterpret_cast<float4*>(&Bs[buf][lk + 8 * i][lc]) = rb[i];
    }
  };
  fetch(0);
  stash(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < K; k0 += FK) {
    const bool more = k0 + FK < K;
    if (more) fetch(k0 + FK);
#pragma unroll
    for (int kk = 0; kk < FK; ++kk) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][kk][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][kk][64 + tx * 4]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (more) stash(buf ^ 1);     // the other buffer was last read before the previous barrier
    __syncthreads();
    buf ^= 1;
  }
}

// fp32 operands that the fast path can take
inline bool fast_ok(const void* G, const void* X, int n_in, int n_out, int dt) {
  return dt == FDP_F32 && n_in % 4 == 0 && n_out % 4 == 0 && aligned16(G) && aligned16(X);
}

__global__ void __launch_bounds__(256) fast_norm_direct_kernel(const float* __restrict__ G, const float* __restrict__ X,
                                                               float* __restrict__ partials, int T, int n_in,
                                                               int n_out, int tiles_n, int tiles_m) {
  __shared__ float red[32];
  const int bx = blockIdx.x % tiles_n, by = (blockIdx.x / tiles_n) % tiles_m;
  const int b = blockIdx.x / (tiles_n * tiles_m);
  float acc[8][8] = {};
  fast_tile<false>(G + static_cast<size_t>(b) * T * n_out, n_out, X + static_cast<size_t>(b) * T * n_in, n_in, T,
                   n_out, n_in, by * FM, bx * FN, nullptr, 1, acc);
  float s = 0.f;     // rows and columns outside the matrix were fetched as zeros
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) s = fmaf(acc[i][j], acc[i][j], s);
  s = block_sum(s, red);
  if (threadIdx.x == 0) partials[blockIdx.x] = s;
}

__global__ void __launch_bounds__(256) fast_clipped_wgrad_kernel(const float* __restrict__ G, const float* __restrict__ X,
                                                                 const float* __restrict__ factors, void* __restrict__ dW,
                                                                 int B, int T, int n_in, int n_out, int out_dt,
                                                                 int layout, float inv_div, NoiseKey nk) {
  float acc[8][8] = {};
  const int m0 = blockIdx.y * FM, n0 = blockIdx.x * FN;
  fast_tile<true>(G, n_out, X, n_in, B * T, n_out, n_in, m0, n0, factors, T, acc);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
  for (int ih = 0; ih < 2; ++ih)
#pragma unroll
    for (int jh = 0; jh < 2; ++jh) {
      const int mb = m0 + 64 * ih + ty * 4, nb = n0 + 64 * jh + tx * 4;   // a 4 x 4 patch; M, N multiples of 4
      if (mb >= n_out || nb >= n_in) continue;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        // four elements adjacent in the output: along n for [out,in], along m for [in,out]
        const bool oi = layout == FDP_OUT_IN;
        const size_t idx0 = oi ? static_cast<size_t>(mb + q) * n_in + nb : static_cast<size_t>(nb + q) * n_out + mb;
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = (oi ? acc[4 * ih + q][4 * jh + e] : acc[4 * ih + e][4 * jh + q]) * inv_div;
        if (nk.std != 0.f) {      // idx0 is a multiple of 4
          float z[4];
          noise_group(nk, idx0 >> 2, z);
          v[0] += z[0]; v[1] += z[1]; v[2] += z[2]; v[3] += z[3];
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) store_as(dW, out_dt, idx0 + e, v[e]);
      }
    }
}

// ---- fp32 fast path, Gram form of the per-sample norm ----------------------------------------------
// ||G_b^T X_b||_F^2 = sum_{t,s} (G_b G_b^T)[t,s] (X_b X_b^T)[t,s] on 128 x 128 blocks of the T x T
// plane, blocks j >= i only (off-diagonal ones count twice): 128^2 (in + out) FMAs per block instead of
// T in out per sample for the direct form.  Here both operands of a product are row blocks of the same
// matrix and the contraction runs along the rows' contiguous columns, so a stage is fetched with
// 16-byte loads along K and written to shared memory transposed (K-major rows of 128 + 4 floats).
constexpr int GK_PITCH = FM + 4;

// acc[i][j] += sum_k M[row_a + r_i][k] * M[row_b + r_j][k]; rows at or beyond `row_end` read as zero
__device__ __forceinline__ void gram_fast_tile(const float* __restrict__ Mx, int ld, int K, int row_a, int row_b,
                                               int row_end, float (*As)[GK_PITCH], float (*Bs)[GK_PITCH],
                                               float acc[8][8]) {
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  float4 ra[2], rb[2];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = tid + 256 * i, r = idx >> 2, k = k0 + 4 * (idx & 3);
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
      if (k < K) {
        if (row_a + r < row_end) a = __ldg(reinterpret_cast<const float4*>(Mx + static_cast<size_t>(row_a + r) * ld + k));
        if (row_b + r < row_end) b = __ldg(reinterpret_cast<const float4*>(Mx + static_cast<size_t>(row_b + r) * ld + k));
      }
      ra[i] = a; rb[i] = b;
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = tid + 256 * i, r = idx >> 2, kk = 4 * (idx & 3);
      float (*A)[GK_PITCH] = As + buf * FK;
      float (*Bq)[GK_PITCH] = Bs + buf * FK;
      A[kk][r] = ra[i].x; A[kk + 1][r] = ra[i].y; A[kk + 2][r] = ra[i].z; A[kk + 3][r] = ra[i].w;
      Bq[kk][r] = rb[i].x; Bq[kk + 1][r] = rb[i].y; Bq[kk + 2][r] = rb[i].z; Bq[kk + 3][r] = rb[i].w;
    }
  };
  __syncthreads();              // the buffers may still be read by the previous call
  fetch(0);
  stash(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < K; k0 += FK) {
    const bool more = k0 + FK < K;
    if (more) fetch(k0 + FK);
#pragma unroll
    for (int kk = 0; kk < FK; ++kk) {
      const float* ar = As[buf * FK + kk];
      const float* br = Bs[buf * FK + kk];
      const float4 a0 = *reinterpret_cast<const float4*>(ar + ty * 4), a1 = *reinterpret_cast<const float4*>(ar + 64 + ty * 4);
      const float4 b0 = *reinterpret_cast<const float4*>(br + tx * 4), b1 = *reinterpret_cast<const float4*>(br + 64 + tx * 4);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (more) stash(buf ^ 1);
    __syncthreads();
    buf ^= 1;
  }
}

__global__ void __launch_bounds__(256) fast_norm_gram_kernel(const float* __restrict__ G, const float* __restrict__ X,
                                                             float* __restrict__ partials, int T, int n_in, int n_out,
                                                             int nb, int nblk) {
  __shared__ __align__(16) float As[2 * FK][GK_PITCH];
  __shared__ __align__(16) float Bs[2 * FK][GK_PITCH];
  __shared__ float red[32];
  const int b = blockIdx.x / nblk;
  int q = blockIdx.x - b * nblk, i = 0;
  while (q >= nb - i) { q -= nb - i; ++i; }      // block (i, j = i + q) of the upper triangle
  const int j = i + q;
  const int row0 = b * T;
  float p[8][8] = {}, x[8][8] = {};
  gram_fast_tile(G, n_out, n_out, row0 + i * FM, row0 + j * FM, row0 + T, As, Bs, p);
  gram_fast_tile(X, n_in, n_in, row0 + i * FM, row0 + j * FM, row0 + T, As, Bs, x);
  float s = 0.f;       // rows past the sample's end were fetched as zeros
#pragma unroll
  for (int a = 0; a < 8; ++a)
#pragma unroll
    for (int c = 0; c < 8; ++c) s = fmaf(p[a][c], x[a][c], s);
  s = block_sum(s, red);
  if (threadIdx.x == 0) partials[blockIdx.x] = (i == j) ? s : 2.f * s;
}

// ---- per-sample norm, direct: one block = one 64x64 tile of G_b^T X_b, squared and summed -------
template <typename Tin>
__global__ void __launch_bounds__(256) simt_norm_direct_kernel(const Tin* __restrict__ G,
                                                               const Tin* __restrict__ X,
                                                               float* __restrict__ partials, int T,
                                                               int n_in, int n_out, int tiles_n, int tiles_m) {
  __shared__ float red[32];
  // one-dimensional grid (the batch may exceed the 65535 limit of the other grid dimensions):
  // block = (b * tiles_m + tile row) * tiles_n + tile column
  const int bx = blockIdx.x % tiles_n, by = (blockIdx.x / tiles_n) % tiles_m;
  const int b = blockIdx.x / (tiles_n * tiles_m);
  const Tin* Gb = G + static_cast<size_t>(b) * T * n_out;
  const Tin* Xb = X + static_cast<size_t>(b) * T * n_in;
  float acc[4][4] = {};
  simt_tile<Tin, false>(Gb, n_out, 1, Xb, n_in, 1, T, n_out, n_in, by * TM, bx * TN, nullptr, 1, acc);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) s = fmaf(acc[i][j], acc[i][j], s);
  s = block_sum(s, red);
  if (threadIdx.x == 0)
    partials[blockIdx.x] = s;
}

int simt_norm_tiles(int n_in, int n_out) { return ceil_div(n_in, TN) * ceil_div(n_out, TM); }

int simt_norm_direct(const void* G, const void* X, float* partials, int B, int T, int n_in,
                     int n_out, int dt, int norm_algo, cudaStream_t s) {
  if (fast_ok(G, X, n_in, n_out, dt)) {
    // Gram form when it is the cheaper one (long sequences) and its partials fit the workspace, which
    // is sized for the 64 x 64 tiles of the direct form
    const int nb = ceil_div(T, FM), nblk = nb * (nb + 1) / 2;
    const double gram_cost = static_cast<double>(nblk) * FM * FM * (static_cast<double>(n_in) + n_out);
    const double direct_cost = static_cast<double>(T) * n_in * n_out;
    const bool want_gram = norm_algo == FDP_NORM_GRAM || (norm_algo == FDP_NORM_AUTO && gram_cost < 0.8 * direct_cost);
    if (want_gram && nblk <= simt_norm_tiles(n_in, n_out)) {
      fast_norm_gram_kernel<<<static_cast<unsigned>(static_cast<size_t>(B) * nblk), 256, 0, s>>>(
          (const float*)G, (const float*)X, partials, T, n_in, n_out, nb, nblk);
      note_launch();
      return nblk;
    }
    const int tn = ceil_div(n_in, FN), tm = ceil_div(n_out, FM);
    fast_norm_direct_kernel<<<static_cast<unsigned>(static_cast<size_t>(B) * tn * tm), 256, 0, s>>>(
        (const float*)G, (const float*)X, partials, T, n_in, n_out, tn, tm);
    note_launch();
    return tn * tm;
  }
  const int tn = ceil_div(n_in, TN), tm = ceil_div(n_out, TM);
  const unsigned grid = static_cast<unsigned>(static_cast<size_t>(B) * tn * tm);
  if (dt == FDP_F32)
    simt_norm_direct_kernel<float><<<grid, 256, 0, s>>>((const float*)G, (const float*)X, partials, T, n_in, n_out, tn, tm);
  else if (dt == FDP_BF16)
    simt_norm_direct_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)G, (const __nv_bfloat16*)X, partials, T, n_in, n_out, tn, tm);
  else
    simt_norm_direct_kernel<__half><<<grid, 256, 0, s>>>((const __half*)G, (const __half*)X, partials, T, n_in, n_out, tn, tm);
  note_launch();
  return tn * tm;
}

// ---- per-sample norm for short sequences (T < 64), through the T x T Gram matrices ---------------
//   ||G_b^T X_b||_F^2 = sum_{t,s} (G_b G_b^T)[t,s] * (X_b X_b^T)[t,s]
// costs T^2 (in + out) multiply-adds per sample instead of T * in * out; for T = 1 (2-D layer
// inputs) it is the rank-one identity ||g||^2 ||x||^2 and one read of G and X.  One block per
// sample.  The (t,s) plane is cut into 4x4 blocks, one per thread group; a group's `cs` lanes
// split the 64 columns of a staged chunk and combine by shuffles, so short sequences still use
// whole warps.  Rows t >= T of the staged chunk are zero and add nothing.
constexpr int GS_COLS = 64, GS_PITCH = 68;   // chunk columns; floats per staged column (T padded, 16-byte rows)

template <typename Tin>
__device__ __forceinline__ void gram_small_accumulate(const Tin* __restrict__ Mb, int T, int n, int tb,
                                                      int cs, float (*tile)[GS_PITCH], float acc[4][4]) {
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int blk = tid / cs, part = tid % cs;
  const int bt = blk / tb, bs = blk % tb;
  const bool active = blk < tb * tb;
  const int tp = tb * 4;
  for (int c0 = 0; c0 < n; c0 += GS_COLS) {
    __syncthreads();
    for (int i = tid; i < tp * GS_COLS; i += nthreads) {
      const int t = i / GS_COLS, c = i % GS_COLS;
      tile[c][t] = (t < T && c0 + c < n) ? to_f32<Tin>(Mb[static_cast<size_t>(t) * n + c0 + c]) : 0.f;
    }
    __syncthreads();
    if (active) {
      for (int c = part; c < GS_COLS; c += cs) {
        const float4 a = *reinterpret_cast<const float4*>(&tile[c][bt * 4]);
        const float4 b = *reinterpret_cast<const float4*>(&tile[c][bs * 4]);
        const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
      }
    }
  }
  // the lanes of a group are adjacent and cs is a power of two <= 32: butterfly inside the group
  for (int o = cs >> 1; o > 0; o >>= 1) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] += __shfl_xor_sync(0xffffffffu, acc[i][j], o);
  }
}

template <typename Tin>
__global__ void __launch_bounds__(256) gram_small_norm_kernel(const Tin* __restrict__ G,
                                                              const Tin* __restrict__ X,
                                                              float* __restrict__ sumsq, int T, int n_in,
                                                              int n_out, int tb, int cs) {
  __shared__ __align__(16) float tile[GS_COLS][GS_PITCH];
  __shared__ float red[32];
  const int b = blockIdx.x;
  float gg[4][4] = {}, xx[4][4] = {};
  gram_small_accumulate<Tin>(G + static_cast<size_t>(b) * T * n_out, T, n_out, tb, cs, tile, gg);
  gram_small_accumulate<Tin>(X + static_cast<size_t>(b) * T * n_in, T, n_in, tb, cs, tile, xx);
  float v = 0.f;
  if (threadIdx.x % cs == 0 && threadIdx.x / cs < tb * tb) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) v = fmaf(gg[i][j], xx[i][j], v);
  }
  v = block_sum(v, red);
  if (threadIdx.x == 0) sumsq[b] = v;
}

void simt_norm_gram_small(const void* G, const void* X, float* sumsq, int B, int T, int n_in, int n_out,
                          int dt, cudaStream_t s) {
  const int tb = ceil_div(T, 4);                 // T < 64: at most 16 x 16 thread groups
  int cs = 32;
  while (cs > 1 && tb * tb * cs > 256) cs >>= 1;
  const int threads = ceil_div(tb * tb * cs, 32) * 32;
  if (dt == FDP_F32)
    gram_small_norm_kernel<float><<<B, threads, 0, s>>>((const float*)G, (const float*)X, sumsq, T, n_in, n_out, tb, cs);
  else if (dt == FDP_BF16)
    gram_small_norm_kernel<__nv_bfloat16><<<B, threads, 0, s>>>((const __nv_bfloat16*)G, (const __nv_bfloat16*)X, sumsq, T, n_in, n_out, tb, cs);
  else
    gram_small_norm_kernel<__half><<<B, threads, 0, s>>>((const __half*)G, (const __half*)X, sumsq, T, n_in, n_out, tb, cs);
  note_launch();
}

// ---- clip factors --------------------------------------------------------------------------------
// split > 0: entries [split, ..) report their norm to norms_out2[b - split] (two tensors, one launch)
__global__ void __launch_bounds__(256) clip_factors_kernel(const float* __restrict__ partials,
                                                           int nparts, float C, float clamp,
                                                           float* norms, float* factors,
                                                           float* norms_out, float* factors_out,
                                                           int split, float* norms_out2) {
  __shared__ float red[32];
  const int b = blockIdx.x;
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += partials[static_cast<size_t>(b) * nparts + i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) {
    const float n = sqrtf(fmaxf(s, 0.f));
    const float f = clip_factor(n, C, clamp);
    if (norms) norms[b] = n;
    factors[b] = f;
    if (split > 0 && b >= split) {
      if (norms_out2) norms_out2[b - split] = n;
    } else {
      if (norms_out) norms_out[b] = n;
      if (factors_out) factors_out[b] = f;
    }
  }
}

void clip_factors(const float* partials, int nparts, int B, float C, float clamp, float* norms,
                  float* factors, float* norms_out, float* factors_out, cudaStream_t s) {
  clip_factors_kernel<<<B, 256, 0, s>>>(partials, nparts, C, clamp, norms, factors, norms_out, factors_out, 0, nullptr);
  note_launch();
}

void clip_factors_pair(const float* partials, int nparts, int B, float C, float clamp, float* factors,
                       float* norms_out_first, float* norms_out_second, cudaStream_t s) {
  clip_factors_kernel<<<2 * B, 256, 0, s>>>(partials, nparts, C, clamp, nullptr, factors, norms_out_first, nullptr, B,
                                            norms_out_second);
  note_launch();
}

// ---- clipped-sum weight gradient: one GEMM over K = B*T with c_b folded into the G operand ------
template <typename Tin>
__global__ void __launch_bounds__(256) simt_clipped_wgrad_kernel(
    const Tin* __restrict__ G, const Tin* __restrict__ X, const float* __restrict__ factors,
    void* __restrict__ dW, int B, int T, int n_in, int n_out, int out_dt, int layout, float inv_div,
    NoiseKey nk) {
  float acc[4][4] = {};
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  simt_tile<Tin, true>(G, n_out, 1, X, n_in, 1, B * T, n_out, n_in, m0, n0, factors, T, acc);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= n_out) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= n_in) continue;
      const size_t idx = (layout == FDP_OUT_IN) ? static_cast<size_t>(m) * n_in + n
                                                : static_cast<size_t>(n) * n_out + m;
      float v = acc[i][j] * inv_div;
      if (nk.std != 0.f) v += noise_at(nk, idx);
      store_as(dW, out_dt, idx, v);
    }
  }
}

void simt_clipped_wgrad(const void* G, const void* X, const float* factors, void* dW, int B, int T,
                        int n_in, int n_out, int dt, int out_dt, int layout, float inv_div,
                        NoiseKey nk, cudaStream_t s) {
  if (fast_ok(G, X, n_in, n_out, dt) && (out_dt != FDP_F32 || aligned16(dW))) {
    dim3 fgrid(ceil_div(n_in, FN), ceil_div(n_out, FM));
    fast_clipped_wgrad_kernel<<<fgrid, 256, 0, s>>>((const float*)G, (const float*)X, factors, dW, B, T, n_in, n_out,
                                                    out_dt, layout, inv_div, nk);
    note_launch();
    return;
  }
  dim3 grid(ceil_div(n_in, TN), ceil_div(n_out, TM));
  if (dt == FDP_F32)
    simt_clipped_wgrad_kernel<float><<<grid, 256, 0, s>>>((const float*)G, (const float*)X, factors, dW, B, T, n_in, n_out, out_dt, layout, inv_div, nk);
  else if (dt == FDP_BF16)
    simt_clipped_wgrad_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)G, (const __nv_bfloat16*)X, factors, dW, B, T, n_in, n_out, out_dt, layout, inv_div, nk);
  else
    simt_clipped_wgrad_kernel<__half><<<grid, 256, 0, s>>>((const __half*)G, (const __half*)X, factors, dW, B, T, n_in, n_out, out_dt, layout, inv_div, nk);
  note_launch();
}

// ---- input gradient: dX[r,i] = sum_o G[r,o] W(o,i) ------------------------------------------------
template <typename Tin>
__global__ void __launch_bounds__(256) simt_dgrad_kernel(const Tin* __restrict__ G,
                                                         const Tin* __restrict__ W,
                                                         void* __restrict__ dX, int out_dt, int rows,
                                                         int n_in, int n_out, int w_layout) {
  float acc[4][4] = {};
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  // A(k=o, m=r) = G[r*n_out + o];  B(k=o, n=i) = W[o*n_in + i] (OUT_IN) or W[i*n_out + o] (IN_OUT)
  const long sBk = (w_layout == FDP_OUT_IN) ? n_in : 1, sBn = (w_layout == FDP_OUT_IN) ? 1 : n_out;
  simt_tile<Tin, false>(G, 1, n_out, W, sBk, sBn, n_out, rows, n_in, m0, n0, nullptr, 1, acc);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < n_in) store_as(dX, out_dt, static_cast<size_t>(m) * n_in + n, acc[i][j]);
    }
  }
}

void simt_dgrad(const void* G, const void* W, void* dX, int rows, int n_in, int n_out, int dt,
                int out_dt, int w_layout, cudaStream_t s) {
  dim3 grid(ceil_div(n_in, TN), ceil_div(rows, TM));
  if (dt == FDP_F32)
    simt_dgrad_kernel<float><<<grid, 256, 0, s>>>((const float*)G, (const float*)W, dX, out_dt, rows, n_in, n_out, w_layout);
  else if (dt == FDP_BF16)
    simt_dgrad_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)G, (const __nv_bfloat16*)W, dX, out_dt, rows, n_in, n_out, w_layout);
  else
    simt_dgrad_kernel<__half><<<grid, 256, 0, s>>>((const __half*)G, (const __half*)W, dX, out_dt, rows, n_in, n_out, w_layout);
  note_launch();
}

// ---- forward: Y[r,o] = sum_i X[r,i] W(i,o) + bias[o] ---------------------------------------------
template <typename Tin>
__global__ void __launch_bounds__(256) simt_fwd_kernel(const Tin* __restrict__ X, const Tin* __restrict__ W,
                                                       const Tin* __restrict__ bias, void* __restrict__ Y,
                                                       int out_dt, int rows, int n_in, int n_out, int w_layout) {
  float acc[4][4] = {};
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  // A(k=i, m=r) = X[r*n_in + i];  B(k=i, n=o) = W[o*n_in + i] (OUT_IN) or W[i*n_out + o] (IN_OUT)
  const long sBk = (w_layout == FDP_OUT_IN) ? 1 : n_out, sBn = (w_layout == FDP_OUT_IN) ? n_in : 1;
  simt_tile<Tin, false>(X, 1, n_in, W, sBk, sBn, n_in, rows, n_out, m0, n0, nullptr, 1, acc);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < n_out)
        store_as(Y, out_dt, static_cast<size_t>(m) * n_out + n, acc[i][j] + (bias ? to_f32<Tin>(bias[n]) : 0.f));
    }
  }
}

void simt_fwd(const void* X, const void* W, const void* bias, void* Y, int rows, int n_in, int n_out, int dt,
              int out_dt, int w_layout, cudaStream_t s) {
  dim3 grid(ceil_div(n_out, TN), ceil_div(rows, TM));
  if (dt == FDP_F32)
    simt_fwd_kernel<float><<<grid, 256, 0, s>>>((const float*)X, (const float*)W, (const float*)bias, Y, out_dt, rows, n_in, n_out, w_layout);
  else if (dt == FDP_BF16)
    simt_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)X, (const __nv_bfloat16*)W, (const __nv_bfloat16*)bias, Y, out_dt, rows, n_in, n_out, w_layout);
  else
    simt_fwd_kernel<__half><<<grid, 256, 0, s>>>((const __half*)X, (const __half*)W, (const __half*)bias, Y, out_dt, rows, n_in, n_out, w_layout);
  note_launch();
}

// ---- bias gradient statistics: one read of G -> per-sample sum of squares + column sums ---------
// Block = 32 column-threads x 8 row-threads.  A column-thread owns VEC adjacent columns (one
// 16-byte load per row); the 8 row-threads stride over the rows of the chunk.  Partials are
// combined in a fixed order, so results are bit-reproducible.
#ifndef FDP_GSTATS_UNROLL
#define FDP_GSTATS_UNROLL 8
#endif
template <typename Tin, int VEC>
__global__ void __launch_bounds__(256, 4) gstats_kernel(const Tin* __restrict__ G,
                                                     float* __restrict__ colsum_part,
                                                     float* __restrict__ sq_part, int T, int n_out,
                                                     int rows_per_chunk, int vec_ok, int col_chunks, int row_chunks) {
  __shared__ float cs[8][32 * VEC];
  __shared__ float red[32];
  const int x = threadIdx.x & 31, y = threadIdx.x >> 5;
  // one-dimensional grid (the batch may exceed 65535): block = (b * row_chunks + rc) * col_chunks + cc
  const int cc = blockIdx.x % col_chunks, rc = (blockIdx.x / col_chunks) % row_chunks;
  const int b = blockIdx.x / (col_chunks * row_chunks);
  const int c0 = (cc * 32 + x) * VEC;
  const int r0 = rc * rows_per_chunk, r1 = min(T, r0 + rows_per_chunk);
  const Tin* Gb = G + static_cast<size_t>(b) * T * n_out;
  float acc[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
  float sq = 0.f;
  if (vec_ok) {
    if (c0 < n_out) {
      // U independent 16-byte loads in flight per thread before any of them is consumed: the kernel
      // waits on memory latency, and four resident blocks of 256 threads with eight loads each keep
      // about 128 KB in flight per SM
      constexpr int U = FDP_GSTATS_UNROLL;
      int r = r0 + y;
      for (; r + 8 * (U - 1) < r1; r += 8 * U) {
        uint4 raw[U];
#pragma unroll
        for (int k = 0; k < U; ++k)
          raw[k] = __ldg(reinterpret_cast<const uint4*>(Gb + static_cast<size_t>(r + 8 * k) * n_out + c0));
#pragma unroll
        for (int k = 0; k < U; ++k) {
          float f[VEC];
          unpack16<Tin>(raw[k], f);
#pragma unroll
          for (int v = 0; v < VEC; ++v) { acc[v] += f[v]; sq = fmaf(f[v], f[v], sq); }
        }
      }
      for (; r < r1; r += 8) {
        float f[VEC];
        unpack16<Tin>(__ldg(reinterpret_cast<const uint4*>(Gb + static_cast<size_t>(r) * n_out + c0)), f);
#pragma unroll
        for (int v = 0; v < VEC; ++v) { acc[v] += f[v]; sq = fmaf(f[v], f[v], sq); }
      }
    }
  } else {
    for (int r = r0 + y; r < r1; r += 8) {
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        if (c0 + v < n_out) {
          const float f = to_f32<Tin>(Gb[static_cast<size_t>(r) * n_out + c0 + v]);
          acc[v] += f; sq = fmaf(f, f, sq);
        }
      }
    }
  }
  pdl_trigger();   // the finalisation kernel may be scheduled while this block reduces and stores
#pragma unroll
  for (int v = 0; v < VEC; ++v) cs[y][x * VEC + v] = acc[v];
  sq = block_sum(sq, red);  // contains the __syncthreads that publishes cs
  if (threadIdx.x == 0)
    sq_part[blockIdx.x] = sq;
  for (int c = threadIdx.x; c < 32 * VEC; c += 256) {
    const int col = cc * 32 * VEC + c;
    if (col < n_out) {
      float t = 0.f;
#pragma unroll
      for (int yy = 0; yy < 8; ++yy) t += cs[yy][c];
      colsum_part[(static_cast<size_t>(b) * row_chunks + rc) * n_out + col] = t;
    }
  }
}

#ifndef FDP_GSTATS_BALANCE
#define FDP_GSTATS_BALANCE 1
#endif
GstatsPlan gstats_plan(int B, int T, int n_out, int dt) {
  GstatsPlan pl;
  pl.vec = (dt == FDP_F32) ? 4 : 8;
  pl.cols_per_block = 32 * pl.vec;
  pl.col_chunks = ceil_div(n_out, pl.cols_per_block);
  // 256 rows per block (32 per thread) when that still leaves four blocks for each of the 148 SMs:
  // half the partials and a shorter finalisation (27.6 us against 30.8 us per call at B=16, T=1024,
  // 3072 columns); otherwise 128 rows, which keeps the grid large at small batch sizes
  pl.rows_per_chunk = 256;
  if (static_cast<long long>(B) * pl.col_chunks * ceil_div(T, 256) < 4 * 148) pl.rows_per_chunk = 128;
  pl.row_chunks = ceil_div(T, pl.rows_per_chunk);
  // Blocks are handed to the 148 SMs as they free up, so the kernel ends when the SM with the most
  // blocks ends: pick the number of row chunks (at most 4x finer than the rule above, each at least
  // 64 rows) that minimises ceil(blocks / 148) * (rows per chunk + a fixed cost per block); ties go to
  // fewer chunks (fewer partials).  B=16, T=1024, 3072 columns: 3 chunks of 342 rows (576 blocks,
  // 4 on the fullest SM against 3.9 on average) instead of 4 of 256 (768 blocks, 6 against 5.2).
  // The constant keeps the workspace query and the launch in agreement on every device.
  if (FDP_GSTATS_BALANCE) {
    constexpr int GS_SMS = 148, BLOCK_FIXED_ROWS = 8;
    const long long strips = static_cast<long long>(B) * pl.col_chunks;
    const int base = pl.row_chunks;
    long long best = -1;
    for (int rc = 1; rc <= 4 * base && ceil_div(T, rc) >= 64; ++rc) {
      const long long blocks = strips * rc;
      const long long cost = ((blocks + GS_SMS - 1) / GS_SMS) * (ceil_div(T, rc) + BLOCK_FIXED_ROWS);
      if (best < 0 || cost < best) { best = cost; pl.row_chunks = rc; }
    }
    pl.rows_per_chunk = ceil_div(T, pl.row_chunks);
    pl.row_chunks = ceil_div(T, pl.rows_per_chunk);
  }
  return pl;
}

void gstats(const void* G, float* colsum_part, float* sq_part, int B, int T, int n_out, int dt,
            const GstatsPlan& pl, cudaStream_t s) {
  const unsigned grid = static_cast<unsigned>(static_cast<size_t>(B) * pl.row_chunks * pl.col_chunks);
  const int vec_ok = (n_out % pl.vec == 0) && aligned16(G);
  if (dt == FDP_F32)
    gstats_kernel<float, 4><<<grid, 256, 0, s>>>((const float*)G, colsum_part, sq_part, T, n_out, pl.rows_per_chunk, vec_ok, pl.col_chunks, pl.row_chunks);
  else if (dt == FDP_BF16)
    gstats_kernel<__nv_bfloat16, 8><<<grid, 256, 0, s>>>((const __nv_bfloat16*)G, colsum_part, sq_part, T, n_out, pl.rows_per_chunk, vec_ok, pl.col_chunks, pl.row_chunks);
  else
    gstats_kernel<__half, 8><<<grid, 256, 0, s>>>((const __half*)G, colsum_part, sq_part, T, n_out, pl.rows_per_chunk, vec_ok, pl.col_chunks, pl.row_chunks);
  note_launch();
}

// db[o] = inv_div * sum_b c_b * sum_rc colsum_part[b,rc,o] + noise.
// Block = 32 columns x 8 slices: slice s adds the (b,rc) pairs s, s+8, ... in order, then the eight
// slice sums are added in order -- many loads in flight, still a fixed summation order.
__global__ void __launch_bounds__(256) bias_finalize_kernel(const float* __restrict__ colsum_part,
                                                            const float* __restrict__ factors,
                                                            void* __restrict__ db, int B, int n_out,
                                                            int row_chunks, int out_dt,
                                                            float inv_div, NoiseKey nk) {
  __shared__ float part[8][32];
  const int col = threadIdx.x & 31, sl = threadIdx.x >> 5;
  const int o = blockIdx.x * 32 + col;
  const int pairs = B * row_chunks;
  float acc = 0.f;
  if (o < n_out) {
    for (int p = sl; p < pairs; p += 8)
      acc = fmaf(factors[p / row_chunks], colsum_part[static_cast<size_t>(p) * n_out + o], acc);
  }
  part[sl][col] = acc;
  __syncthreads();
  if (sl == 0 && o < n_out) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += part[k][col];
    float v = t * inv_div;
    if (nk.std != 0.f) v += noise_at(nk, o);
    store_as(db, out_dt, o, v);
  }
}

void bias_finalize(const float* colsum_part, const float* factors, void* db, int B, int n_out,
                   int row_chunks, int out_dt, float inv_div, NoiseKey nk, cudaStream_t s) {
  bias_finalize_kernel<<<ceil_div(n_out, 32), 256, 0, s>>>(colsum_part, factors, db, B, n_out, row_chunks, out_dt, inv_div, nk);
  note_launch();
}

// The same with the clip factors computed in the kernel (one launch less): every block derives the
// B factors from the sum-of-squares partials in the same fixed order (warp w takes samples w, w+8, ...),
// block 0 also reports norms and factors.
__global__ void __launch_bounds__(256) bias_finalize_fused_kernel(
    const float* __restrict__ colsum_part, const float* __restrict__ sq_part, int nparts, float C, float clamp,
    float* __restrict__ norms_out, float* __restrict__ factors_out, void* __restrict__ db, int B, int n_out,
    int row_chunks, int out_dt, float inv_div, NoiseKey nk) {
  extern __shared__ float s_fac[];  // [B]
  __shared__ float part[8][32];
  const int col = threadIdx.x & 31, sl = threadIdx.x >> 5;
  pdl_wait();
  for (int b = sl; b < B; b += 8) {
    float sq = 0.f;
    for (int i = col; i < nparts; i += 32) sq += sq_part[static_cast<size_t>(b) * nparts + i];
    sq = warp_sum(sq);
    if (col == 0) {
      const float n = sqrtf(fmaxf(sq, 0.f));
      const float f = clip_factor(n, C, clamp);
      s_fac[b] = f;
      if (blockIdx.x == 0) {
        if (norms_out) norms_out[b] = n;
        if (factors_out) factors_out[b] = f;
      }
    }
  }
  __syncthreads();
  const int o = blockIdx.x * 32 + col;
  const int pairs = B * row_chunks;
  float acc = 0.f;
  if (o < n_out) {
    for (int p = sl; p < pairs; p += 8)
      acc = fmaf(s_fac[p / row_chunks], colsum_part[static_cast<size_t>(p) * n_out + o], acc);
  }
  part[sl][col] = acc;
  __syncthreads();
  if (sl == 0 && o < n_out) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += part[k][col];
    float v = t * inv_div;
    if (nk.std != 0.f) v += noise_at(nk, o);
    store_as(db, out_dt, o, v);
  }
}

void bias_clip_finalize(const float* colsum_part, const float* sq_part, int nparts, float C, float clamp,
                        float* factors_ws, float* norms_out, float* factors_out, void* db, int B, int n_out,
                        int row_chunks, int out_dt, float inv_div, NoiseKey nk, cudaStream_t s) {
  if (static_cast<size_t>(B) * sizeof(float) <= 32 * 1024) {
    launch_dependent(bias_finalize_fused_kernel, dim3(ceil_div(n_out, 32)), dim3(256), B * sizeof(float), s,
                     colsum_part, sq_part, nparts, C, clamp, norms_out, factors_out, db, B, n_out, row_chunks, out_dt,
                     inv_div, nk);
    note_launch();
    return;
  }
  clip_factors(sq_part, nparts, B, C, clamp, nullptr, factors_ws, norms_out, factors_out, s);
  bias_finalize(colsum_part, factors_ws, db, B, n_out, row_chunks, out_dt, inv_div, nk, s);
}

}  // namespace fdp
