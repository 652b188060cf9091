// Host-side launchers shared between the translation units of the library (internal).
#pragma once
#include "fdp_common.cuh"

namespace fdp {

// every kernel launch of the library is counted (fdp_launch_count)
void note_launch(int n = 1);
// The current device's slot of the host-visible (mapped, pinned) status array, as a pointer kernels
// may write through; null when the array could not be set up.  A bounded wait that runs out stores
// its code there, and every later entry-point call on that device returns FDP_ERR_TIMEOUT until
// fdp_clear_async_status.
int* sticky_status_slot();
// SMs persistent GEMM grids leave free (fdp_set_sm_reserve)
int sm_reserve_exchange(int n);

// Programmatic dependent launch for the second and later kernels of one entry point.  A kernel
// launched with launch_dependent() may be scheduled as soon as every block of the kernel before it
// in the stream has called pdl_trigger() (or exited), so its launch latency and prologue overlap
// that kernel's tail; it must call pdl_wait() before it touches anything the earlier kernel wrote
// (the wait returns when the earlier grid has completed and its writes are visible).  The first
// kernel of an entry point is always launched the ordinary way, so nothing of the library ever
// overtakes the caller's own work in the stream.  FDP_PDL=0 in the environment turns it off.
bool pdl_enabled();
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
template <typename... KArgs, typename... Args>
inline void launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                             Args&&... args) {
  if (!pdl_enabled()) {
    kernel<<<grid, block, smem, s>>>(static_cast<KArgs>(args)...);
    return;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// ---- generic-shape kernels (any dtype, any size; fp32 FMA accumulation) -----------------------
int simt_norm_tiles(int n_in, int n_out);
// partials[b*nparts + part] add up to ||G_b^T X_b||_F^2; returns nparts, which is at most simt_norm_tiles
// (64 x 64 tiles of the product; aligned fp32 operands take 128 x 128 tiles, or, when cheaper or asked for
// by norm_algo, 128 x 128 blocks of the T x T Gram form)
int simt_norm_direct(const void* G, const void* X, float* partials, int B, int T, int n_in,
                     int n_out, int dt, int norm_algo, cudaStream_t s);
// short sequences (T < SHORT_SEQ): sumsq[b] = ||G_b^T X_b||_F^2 through the T x T Gram matrices
constexpr int SHORT_SEQ = 64;
void simt_norm_gram_small(const void* G, const void* X, float* sumsq, int B, int T, int n_in, int n_out,
                          int dt, cudaStream_t s);
// sumsq_b = fixed-order sum of partials[b, 0..nparts); norm = sqrt; factor = clip_factor(norm)
void clip_factors(const float* partials, int nparts, int B, float C, float clamp, float* norms,
                  float* factors, float* norms_out, float* factors_out, cudaStream_t s);
// the same for 2B entries (two tensors of B samples): factors[2B]; norms go to two outputs
void clip_factors_pair(const float* partials, int nparts, int B, float C, float clamp, float* factors,
                       float* norms_out_first, float* norms_out_second, cudaStream_t s);
// dW = inv_div * sum_{b,t} c_b G[b,t,:]^T X[b,t,:] + noise, stored as out_dt in `layout`
void simt_clipped_wgrad(const void* G, const void* X, const float* factors, void* dW, int B, int T,
                        int n_in, int n_out, int dt, int out_dt, int layout, float inv_div,
                        NoiseKey nk, cudaStream_t s);
// dX[rows,n_in] = G[rows,n_out] * W (W [n_out,n_in] if w_layout==FDP_OUT_IN else [n_in,n_out]^T)
void simt_dgrad(const void* G, const void* W, void* dX, int rows, int n_in, int n_out, int dt,
                int out_dt, int w_layout, cudaStream_t s);

// Y[rows,n_out] = X[rows,n_in] * W^T (+ bias); W [n_out,n_in] if w_layout==FDP_OUT_IN else [n_in,n_out]
void simt_fwd(const void* X, const void* W, const void* bias, void* Y, int rows, int n_in, int n_out, int dt,
              int out_dt, int w_layout, cudaStream_t s);

// ---- bias gradient (HBM-bound; G read once) ----------------------------------------------------
struct GstatsPlan { int vec, cols_per_block, col_chunks, rows_per_chunk, row_chunks; };
GstatsPlan gstats_plan(int B, int T, int n_out, int dt);
void gstats(const void* G, float* colsum_part, float* sq_part, int B, int T, int n_out, int dt,
            const GstatsPlan& pl, cudaStream_t s);
void bias_finalize(const float* colsum_part, const float* factors, void* db, int B, int n_out,
                   int row_chunks, int out_dt, float inv_div, NoiseKey nk, cudaStream_t s);
// clip factors from sq_part[B, nparts] and the finalisation in one launch (two for very large B)
void bias_clip_finalize(const float* colsum_part, const float* sq_part, int nparts, float C, float clamp,
                        float* factors_ws, float* norms_out, float* factors_out, void* db, int B, int n_out,
                        int row_chunks, int out_dt, float inv_div, NoiseKey nk, cudaStream_t s);

// ---- LayerNorm -----------------------------------------------------------------------------------
struct LnPlan { int tpr, cpt, cw, rows_per_block, chunks; bool vec; };
LnPlan ln_plan(int B, int T, int d, int dt);
void ln_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
            int rows, int d, float eps, int dt, int pdt, cudaStream_t s);
void ln_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
            void* dx, float* dg_part, float* db_part, int B, int T, int d, int dt, int pdt,
            const LnPlan& pl, cudaStream_t s);
// reduce partials over chunks -> per-sample grads [2,B,d] (in place in chunk slot 0) and partial sums
// of squares sumsq[(tensor*B + b) * ln_sumsq_parts(d) + column block]
int ln_sumsq_parts(int d);
void ln_psgrad_reduce(float* part, float* sumsq, int B, int chunks, int d, cudaStream_t s);
// both tensors in one launch: out0/nk0 for dgamma, out1/nk1 for dbeta (out1 may be null)
void ln_psgrad_finalize(const float* part, const float* factors, void* out0, void* out1, int B, int chunks,
                        int d, int out_dt, float inv_div, NoiseKey nk0, NoiseKey nk1, cudaStream_t s);
// clip factors from sumsq[2B, nparts] and the finalisation of both tensors in one launch
void ln_clip_finalize(const float* part, const float* sumsq, int nparts, float C, float clamp, float* factors_ws,
                      float* norms0, float* norms1, void* out0, void* out1, int B, int chunks, int d, int out_dt,
                      float inv_div, NoiseKey nk0, NoiseKey nk1, cudaStream_t s);

// compatibility mode: the element-wise saturating accumulation of the reference's fused backward with
// a fixed row order; dw_buf / db_buf are [ln_saturate_groups(rows, d), d] floats
int ln_saturate_groups(int rows, int d);
void ln_saturate(const void* dy, const void* x, const float* mean, const float* rstd, float* dw_buf, float* db_buf,
                 void* dgamma, void* dbeta, int rows, int d, int dt, int pdt, float C, float clamp, cudaStream_t s);

// ---- tcgen05 / TMEM / TMA kernels (bf16 / fp16, aligned shapes) ---------------------------------
struct TcPlan {
  bool ok;          // shapes admit the tensor-core path
  int algo;         // FDP_NORM_DIRECT or FDP_NORM_GRAM
  size_t ws_bytes;  // extra workspace: split-K parking area, then the pre-scaled G if needed
  size_t split_bytes;
  int nparts;       // norm partials per sample
  bool scaled_epilogue;  // clip factors applied per sample in the GEMM epilogue, no pre-scale pass
  bool short_seq;        // T < SHORT_SEQ: norms by simt_norm_gram_small, clipped sum over the pre-scaled G
  // fp32 inputs: G and X are first split into high and low bf16 halves ([rows, 2n] each, behind the
  // parking area in the workspace), and every contraction runs as three bf16 products
  bool split3;
  size_t split3_g_bytes, split3_x_bytes;
};
TcPlan tc_plan(int B, int T, int n_in, int n_out, int dt, int norm_algo);
// fp32 [rows, n] -> bf16 [rows, 2n]: high halves, then low halves (x - hi rounded to bf16)
int tc_split3(const void* src, void* dst, size_t rows, int n, cudaStream_t s);
// With pl.split3, G and X are the split matrices and dt is FDP_BF16.
int tc_norms(const void* G, const void* X, float* partials, int* dev_status, int B, int T, int n_in,
             int n_out, int dt, const TcPlan& pl, cudaStream_t s);
// Gs[r,:] = factors[r / T] * G[r,:]
int tc_prescale(const void* G, const float* factors, void* Gs, int B, int T, int n_out, int dt,
                cudaStream_t s);
// Where the scaled epilogue of the clipped-sum GEMM takes its clip factors from: `factors` (device,
// computed by an earlier kernel), or -- factors == nullptr -- the norm pass's partial sums, reduced
// inside the GEMM kernel (tc_fused_factors_ok(B) must hold); the kernel then also fills
// norms_out / factors_out (each may be null).
struct TcFactorSource {
  const float* factors;
  const float* norm_partials; int nparts; float C, clamp;
  float* norms_out; float* factors_out;
};
bool tc_fused_factors_ok(int B);
// dW = inv_div * sum_b c_b G_b^T X_b + noise over K = B*T.  fs == nullptr: Gs is the pre-scaled copy;
// otherwise Gs is G itself and c_b is applied per sample in the epilogue.
int tc_clipped_wgrad(const void* Gs, const void* X, const TcFactorSource* fs, float* split_ws,
                     void* dW, int* dev_status, int B, int T, int n_in, int n_out, int dt, int out_dt,
                     int layout, float inv_div, NoiseKey nk, cudaStream_t s, int terms = 1);
// test aid: one warp waits `limit_cycles` on a barrier nobody arrives on and reports the timeout
int tc_wait_selftest(int* status, long long limit_cycles, cudaStream_t s);
bool tc_dgrad_ok(int rows, int n_in, int n_out, int dt);
// fp32 product Y[rows, N] = A[rows, K] * W (+ bias) as three bf16 tensor-core products over operands split
// by tc_split3 (A3 [rows, 2K]; W3 [K, 2N] if w_kn, else [N, 2K]); workspace for the two split copies
bool tc_gemm3_ok(int rows, int K, int N);
size_t tc_gemm3_ws_bytes(int rows, int K, int N);
int tc_gemm3(const void* A3, const void* W3, const void* bias, void* Y, int* dev_status, int rows, int K, int N,
             int out_dt, bool w_kn, cudaStream_t s);
int tc_fwd(const void* X, const void* W, const void* bias, void* Y, int* dev_status, int rows, int n_in,
           int n_out, int dt, int out_dt, int w_layout, cudaStream_t s);
int tc_dgrad(const void* G, const void* W, void* dX, int* dev_status, int rows, int n_in, int n_out,
             int dt, int out_dt, int w_layout, cudaStream_t s);

}  // namespace fdp
