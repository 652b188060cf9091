/*
 * fdp_b200.h -- C ABI of the B200 (sm_100a) DP-SGD backward kernels.
 *
 * Every entry point is `extern "C"`, takes raw device pointers to contiguous row-major
 * tensors, sizes, and the CUDA stream to launch on.  Nothing here allocates device memory,
 * synchronises the host or throws: the caller passes a workspace whose size the matching
 * `*_workspace_bytes` query returns, and reads a status code (0 = FDP_OK, negative = error;
 * `fdp_status_string` names it).  Inputs are never modified.  (The first call of a process pins
 * one 256-byte block of host memory for the asynchronous status described below.)
 *
 * Asynchronous errors: the only device-side failure the kernels can report is a bounded wait that
 * ran out (an mbarrier that never completed within about a second).  The kernel then stops early
 * -- the outputs of that call are undefined -- and records a code in the call's workspace and in a
 * host-visible word of its device.  Like a CUDA asynchronous error it surfaces on a LATER call:
 * every compute entry point first looks at that word (a plain host read, no synchronisation) and
 * returns FDP_ERR_TIMEOUT while it is set; fdp_async_status polls it, fdp_clear_async_status
 * re-arms the device.  A training loop should poll once per step before using the gradients.
 *
 * The comments cite, as file:line inside the FlashDP4Review project, the Python-level
 * interface of the reference that each entry point takes the place of.
 */
#ifndef FDP_B200_H
#define FDP_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* 2: asynchronous status word, SM reservation, saturating LayerNorm mode, FDP_FP32_TENSOR.
 * 3: fdp_dp_params.step_device (appended; earlier fields keep their offsets); FDP_FP32_TENSOR also
 *    accepted in the dtype of fdp_linear_dgrad / fdp_linear_fwd. */
#define FDP_ABI_VERSION 3

typedef void* fdp_stream_t; /* a cudaStream_t */

enum fdp_status {
  FDP_OK = 0,
  FDP_ERR_ARG = -1,       /* null pointer, non-positive size, bad enum */
  FDP_ERR_DTYPE = -2,     /* dtype not supported by this entry point */
  FDP_ERR_SHAPE = -3,     /* shape outside what the kernels cover */
  FDP_ERR_ALIGN = -4,     /* a pointer the chosen kernel needs 16-byte aligned is not (16-bit inputs with
                           * tensor-core shapes; the generic kernels take any naturally aligned pointer) */
  FDP_ERR_WORKSPACE = -5, /* workspace missing or too small */
  FDP_ERR_ARCH = -6,      /* device is not sm_100 */
  FDP_ERR_LAUNCH = -7,    /* CUDA reported a launch/runtime error */
  FDP_ERR_TIMEOUT = -8,   /* a bounded device-side wait ran out, in this or an earlier call (fdp_async_status) */
  FDP_ERR_STATIC_LIMIT = -9 /* fdp_bias_grad_static: the problem needs more scratch than FDP_STATIC_SCRATCH_BYTES */
};

/* number types: supported_acc_dtypes of flashdp/core/utils.py:9-12 (fp32 accumulation for all) */
enum fdp_dtype { FDP_F32 = 0, FDP_BF16 = 1, FDP_F16 = 2 };

/* orientation of the weight gradient: [out,in] for nn.Linear (flashdp/core/linear_clip.py:94-104),
 * [in,out] for transformers Conv1D (flashdp/core/transformers_conv1d_clip.py:22-28) */
enum fdp_layout { FDP_OUT_IN = 0, FDP_IN_OUT = 1 };

/* how the per-sample norms ||G_b^T X_b||_F are obtained */
enum fdp_norm_algo {
  FDP_NORM_AUTO = 0,   /* pick per shape; sequences shorter than 64 rows use the Gram identity on T x T
                        * blocks (for T = 1, i.e. 2-D layer inputs, that is ||g_b|| * ||x_b||) */
  FDP_NORM_DIRECT = 1, /* per-sample GEMM tiles, squared and reduced in the epilogue, never stored */
  FDP_NORM_GRAM = 2,   /* sum_{t,s} (G_b G_b^T)_{ts} (X_b X_b^T)_{ts} */
  FDP_NORM_MASK = 15,
  /* flag, OR-ed into the norm_algo argument of fdp_linear_wgrad and of its workspace query: fp32 inputs
   * with 64-aligned shapes (n_in, n_out and T multiples of 64, at least 128) run on the tensor cores as
   * three bf16 products (x = hi + lo: hi*hi + hi*lo + lo*hi) instead of fp32 FMAs, about six times
   * faster.  The tensor cores add into their fp32 accumulators by truncation, so no accumulator runs
   * longer than a few K stages before it is added, with round-to-nearest, to registers; norms and
   * gradients stay within 1e-5 of float64 like the FMA kernels (the norms then always use the product
   * form: FDP_NORM_GRAM is ignored).  The workspace grows by the size of the inputs (their bf16 halves).
   * Without the flag fp32 inputs keep fp32 FMA arithmetic, the reference's own
   * (flashdp/core/utils.py:9-12: fp32 accumulates in fp32).  The Python layer sets the flag by default
   * (runtime.set_fp32_mode). */
  FDP_FP32_TENSOR = 16
};

/* DP hyper-parameters of one call.  C / clamp_value are the arguments of
 * get_clip_factor_torch (flashdp/core/clip_fn.py:6-8); noise_std is
 * noise_multiplier / sqrt(B_global) (flashdp/layers/linear.py:74-80). */
typedef struct fdp_dp_params {
  float C;
  float clamp_value;
  float noise_std;       /* 0 disables the noise epilogue */
  int32_t batch_divisor; /* the mean is sum/batch_divisor; <=0 means the local batch size B */
  uint64_t seed;         /* Philox key */
  uint32_t param_id;     /* Philox counter word 2: which parameter tensor */
  uint32_t param_id2;    /* second tensor of the call (LayerNorm beta) */
  uint32_t step;         /* Philox counter word 3: training step */
  int32_t noise_rank;    /* this rank draws the noise of element groups g with g % noise_world == noise_rank */
  int32_t noise_world;   /* <=1: this rank draws all of it */
  /* NULL, or a device pointer to a 32-bit counter that the kernels read when they run: the step
   * word is then step + *step_device.  A step captured in a CUDA graph together with a kernel that
   * increments the counter draws fresh noise on every replay; with a host-side step a replay would
   * repeat the captured draw.  No counterpart in the reference (torch.normal advances the device
   * generator's offset, flashdp/layers/linear.py:74-80). */
  const uint32_t* step_device;
} fdp_dp_params;

int fdp_abi_version(void);
const char* fdp_status_string(int status);

/* 0 if device `device` can run the library (compute capability 10.x), else FDP_ERR_ARCH. */
int fdp_check_device(int device);

/* Waits for `stream`, then reports whether a bounded wait ran out: reads the status word at the start
 * of `workspace` (of fdp_linear_wgrad / fdp_linear_dgrad / fdp_linear_fwd; may be NULL) and the
 * device's host-visible word.  Returns FDP_OK, FDP_ERR_TIMEOUT or FDP_ERR_LAUNCH. */
int fdp_device_status(const void* workspace, fdp_stream_t stream);

/* Non-blocking poll / reset of the host-visible status word of `device` (-1: the current device).
 * No counterpart in the reference (its Triton kernels spin without a limit,
 * flashdp/core/layernorm_clip.py:111). */
int fdp_async_status(int device);
int fdp_clear_async_status(int device);

/* Test aid: launches one warp that waits `limit_cycles` GPU clock cycles (clamped to about a second)
 * on a barrier nobody arrives on, so that the wait runs out and the reporting path above is taken:
 * afterwards fdp_device_status(workspace, stream) and fdp_async_status return FDP_ERR_TIMEOUT.
 * The kernel returns normally; nothing faults.  `workspace`: at least 256 bytes. */
int fdp_selftest_wait_timeout(long long limit_cycles, void* workspace, size_t workspace_bytes,
                              fdp_stream_t stream);

/* SMs that the persistent GEMM grids launched after this call leave free (0 = use all); returns the
 * previous value.  The grids otherwise occupy every SM, so a collective kernel (the all-reduce of
 * the gradients in a data-parallel job) launched beside one cannot start before it ends: a caller
 * sets a reservation around the calls it wants to overlap with a collective and clears it after.
 * Process-wide; FDP_TC_RESERVE_SMS in the environment is the initial value.  No counterpart in the
 * reference (single GPU, example/gpt2/train.py:33). */
int fdp_set_sm_reserve(int n);

/* Every compute entry point below opens an NVTX range named after itself (header-only NVTX: nothing
 * happens unless a timeline tool is attached), so a trace shows which call each kernel belongs to. */

/* Stream semantics.  Every entry point only enqueues work on `stream` and returns.  The first kernel
 * of a call is an ordinary launch: it starts after everything the caller enqueued before it.  Later
 * kernels of the same call are programmatic dependent launches (they are scheduled while the
 * previous kernel of the call drains and wait for it before touching memory); whatever the caller
 * enqueues after the call starts, as always, when the call's last kernel has completed.  FDP_PDL=0
 * in the environment makes every launch an ordinary one. */

/* ---- instrumentation (no counterpart in the reference, which only wall-clocks whole functions in
 * RuntimeAutoTuner._measure_time, flashdp/core/utils.py:42-47) ---------------------------------------
 * fdp_launch_count: kernels launched by this library in this process so far.
 * fdp_profile_enable(1): later fdp_linear_wgrad calls record CUDA events on their stream between
 *   their phases; fdp_profile_read waits for the last such call and writes the milliseconds of
 *   {norm pass, clip factors, c_b pre-scale, clipped-sum GEMM} to ms[0..3]; returns 4 or an error. */
unsigned long long fdp_launch_count(void);
int fdp_profile_enable(int on);
int fdp_profile_read(float* ms, int capacity);

/* ---- DP weight gradient of Linear / Conv1D --------------------------------------------------
 * Takes the place of linear_weight_flashdp(input, grad_output, C, clamp_value, tuner)
 * (flashdp/core/linear_clip.py:107-113) together with the `.div_(B)` and the torch.normal noise
 * of its caller (flashdp/layers/linear.py:72-80; flashdp/layers/transformers_conv1d.py:79-87).
 *   G [B,T,n_out], X [B,T,n_in] in `in_dtype`;  dW in `out_dtype`, [n_out,n_in] or [n_in,n_out].
 *   norms_out / factors_out: optional float[B] (per-sample Frobenius norms and clip factors).
 */
size_t fdp_linear_wgrad_workspace_bytes(int B, int T, int n_in, int n_out, int in_dtype,
                                        int norm_algo);
int fdp_linear_wgrad(const void* G, const void* X, void* dW, float* norms_out, float* factors_out,
                     int B, int T, int n_in, int n_out, int in_dtype, int out_dtype, int layout,
                     int norm_algo, const fdp_dp_params* p, void* workspace, size_t workspace_bytes,
                     fdp_stream_t stream);

/* ---- DP bias gradient -------------------------------------------------------------------------
 * Takes the place of linear_bias_grad_clip(grad_output, C, clamp_value)
 * (flashdp/core/linear_clip.py:116-123) plus its caller's noise (flashdp/layers/linear.py:84-92):
 * norm of sample b over its whole T x n_out block, db = sum_b c_b sum_t G[b,t,:] / (divisor*T).
 * G is read once and not written (the reference scales it in place).
 */
size_t fdp_bias_grad_workspace_bytes(int B, int T, int n_out, int in_dtype);
int fdp_bias_grad(const void* G, void* db, float* norms_out, float* factors_out, int B, int T,
                  int n_out, int in_dtype, int out_dtype, const fdp_dp_params* p, void* workspace,
                  size_t workspace_bytes, fdp_stream_t stream);

/* ---- DP bias gradient without a caller workspace ---------------------------------------------
 * No counterpart in the reference.  Same arguments and results as fdp_bias_grad minus the
 * workspace: the partial sums go to a fixed buffer of FDP_STATIC_SCRATCH_BYTES that the library
 * image itself carries in device memory (every GPU that loads the library holds it until exit).
 * It is for callers that cannot allocate device memory: a host binding with no device allocator,
 * a process whose memory pool already owns the whole GPU, or a path that must avoid the
 * device-wide synchronisation of cudaMalloc/cudaFree.  The call itself allocates nothing.
 * Problems that need more than the fixed buffer return FDP_ERR_STATIC_LIMIT and launch nothing
 * (the need equals fdp_bias_grad_workspace_bytes of the same arguments).
 * All calls on a device share the buffer: calls that overlap on the GPU race and must be
 * serialised by the caller; the buffer keeps the previous call's contents, and every call
 * overwrites what it reads, so no clearing is required.
 * The first call on each device resolves the buffer's device address; issue it before starting
 * any stream capture.
 */
#define FDP_STATIC_SCRATCH_BYTES (8u << 20)
int fdp_bias_grad_static(const void* G, void* db, float* norms_out, float* factors_out, int B, int T,
                         int n_out, int in_dtype, int out_dtype, const fdp_dp_params* p,
                         fdp_stream_t stream);

/* ---- input gradient ---------------------------------------------------------------------------
 * `grad_output @ weight` of flashdp/layers/linear.py:62-67 (w_layout FDP_OUT_IN, W [n_out,n_in]) and
 * `grad_output @ weight.t()` of flashdp/layers/transformers_conv1d.py:70-75 (FDP_IN_OUT, W [n_in,n_out]).
 *   G [rows,n_out] and W in `dtype`; dX [rows,n_in] in `out_dtype` (e.g. fp32 when the layer input was
 *   fp32 under bf16 autocast, which saves the cast pass autograd would otherwise add).
 *   fp32 on the tensor cores: pass FDP_F32 | FDP_FP32_TENSOR as `dtype`, to the workspace query and to
 *   the call (also of fdp_linear_fwd).  Where the contracted dimension is a multiple of 64 and rows,
 *   n_in and n_out are at least 128 the product runs as three bf16 products with chained accumulation,
 *   within 1e-5 of float64 and about five times cuBLAS's fp32 GEMM; the workspace then also holds the
 *   bf16 halves of both operands.  Other shapes ignore the flag.
 */
size_t fdp_linear_dgrad_workspace_bytes(int rows, int n_in, int n_out, int dtype);
int fdp_linear_dgrad(const void* G, const void* W, void* dX, int rows, int n_in, int n_out,
                     int dtype, int out_dtype, int w_layout, void* workspace, size_t workspace_bytes,
                     fdp_stream_t stream);

/* ---- forward -----------------------------------------------------------------------------------
 * `input @ weight.t() + bias` of flashdp/layers/linear.py:41-46 (w_layout FDP_OUT_IN, W [n_out,n_in]) and
 * `input @ weight + bias` of flashdp/layers/transformers_conv1d.py:40-43 (FDP_IN_OUT, W [n_in,n_out]).
 *   X [rows,n_in] and W in `dtype`; bias [n_out] in `dtype` or NULL; Y [rows,n_out] in `out_dtype`.
 * The workspace is that of fdp_linear_dgrad (the status word).
 */
int fdp_linear_fwd(const void* X, const void* W, const void* bias, void* Y, int rows, int n_in, int n_out,
                   int dtype, int out_dtype, int w_layout, void* workspace, size_t workspace_bytes,
                   fdp_stream_t stream);

/* ---- LayerNorm ----------------------------------------------------------------------------------
 * fdp_layernorm_fwd: layernorm_fwd_fused(input, weight, bias, eps) (flashdp/core/layernorm_clip.py:201-239):
 *   x,y [rows,d] in `dtype`; gamma,beta [d] in `param_dtype`; mean,rstd float[rows].
 * fdp_layernorm_bwd: dx as in _layer_norm_bwd_dx_fused_clip (flashdp/core/layernorm_clip.py:95-103);
 *   dgamma/dbeta with the per-sample clipping of layernorm_dw_clip / layernorm_db_clip
 *   (flashdp/core/layernorm_clip.py:163-198) and the noise of flashdp/layers/layernorm.py:139-155
 *   (one draw per tensor).  dx, dbeta and the norms outputs may be NULL.
 */
int fdp_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean,
                      float* rstd, int rows, int d, float eps, int dtype, int param_dtype,
                      fdp_stream_t stream);
size_t fdp_layernorm_bwd_workspace_bytes(int B, int T, int d);
int fdp_layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean,
                      const float* rstd, void* dx, void* dgamma, void* dbeta, float* norms_gamma,
                      float* norms_beta, int B, int T, int d, int dtype, int param_dtype,
                      const fdp_dp_params* p, void* workspace, size_t workspace_bytes,
                      fdp_stream_t stream);

/* ---- LayerNorm, compatibility mode --------------------------------------------------------------
 * The dgamma / dbeta of the reference's FUSED backward: _layer_norm_bwd_dx_fused_clip accumulates row
 * r's dy*xhat and dy into buffer r % G under a spin lock, saturating the buffer element by element
 * before every addition but the first -- buf <- partial + buf * min(clamp, C / (|buf| + 1e-10)) --
 * and _layer_norm_bwd_dwdb sums the G buffers (flashdp/core/layernorm_clip.py:109-131, :134-160; G from
 * :261-264).  No division by the batch, no noise (flashdp/layers/layernorm.py:179-203).  In the
 * reference the rows of a buffer are added in lock-acquisition order, so its result varies from run
 * to run; this entry point takes them in increasing row order.  It is not per-sample clipping: use
 * fdp_layernorm_bwd for DP training.  dx comes from fdp_layernorm_bwd.
 *   dy, x [rows,d] in `dtype`; mean, rstd float[rows]; dgamma, dbeta (may be NULL) [d] in `param_dtype`.
 *   The workspace holds the G buffers of both tensors, [G,d] floats each, dgamma's first: a caller may
 *   read them after the call (they are the reference's dw_ / db_).
 */
size_t fdp_layernorm_saturate_workspace_bytes(int rows, int d);
int fdp_layernorm_saturate_groups(int rows, int d);
int fdp_layernorm_bwd_saturate(const void* dy, const void* x, const float* mean, const float* rstd, void* dgamma,
                               void* dbeta, int rows, int d, int dtype, int param_dtype, float C, float clamp_value,
                               void* workspace, size_t workspace_bytes, fdp_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* FDP_B200_H */
