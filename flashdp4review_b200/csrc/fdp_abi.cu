// extern "C" entry points: argument checks, workspace carving, kernel selection.
// No allocation, no host synchronisation (except fdp_device_status), no exceptions.
#include <cstdlib>
#include <atomic>
#include <mutex>

#include <nvtx3/nvToolsExt.h>

#include "fdp_kernels.h"

using namespace fdp;

namespace fdp {
static std::atomic<unsigned long long> g_launches{0};
void note_launch(int n) { g_launches.fetch_add(static_cast<unsigned long long>(n), std::memory_order_relaxed); }
bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("FDP_PDL");
    return e == nullptr || e[0] != '0';
  }();
  return on;
}

// Host-visible status array: one int per device in mapped, pinned host memory (allocated once per
// process; with unified addressing the host pointer is valid on every device).  Kernels store a
// code there when a bounded wait runs out; the host reads it without synchronising anything.
static volatile int* sticky_array() {
  static std::mutex mu;
  static volatile int* arr = nullptr;
  static bool tried = false;
  std::lock_guard<std::mutex> lk(mu);
  if (!tried) {
    tried = true;
    void* p = nullptr;
    if (cudaHostAlloc(&p, 64 * sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess) {
      for (int i = 0; i < 64; ++i) static_cast<int*>(p)[i] = 0;
      arr = static_cast<volatile int*>(p);
    } else {
      cudaGetLastError();
    }
  }
  return arr;
}
int* sticky_status_slot() {
  volatile int* arr = sticky_array();
  int dev = 0;
  if (arr == nullptr || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return nullptr; }
  return const_cast<int*>(arr + dev);
}
}  // namespace fdp

namespace {

// An NVTX range around every compute entry point, so that a timeline tool shows which library call
// a kernel belongs to.  Header-only NVTX: a no-op unless a tool has injected itself into the process.
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
};

bool valid_dtype(int dt) { return dt == FDP_F32 || dt == FDP_BF16 || dt == FDP_F16; }

// compute capability per device, looked up once
int device_cc_major(int dev) {
  static std::mutex mu;
  static int cache[64];
  static bool have[64];
  if (dev < 0 || dev >= 64) return -1;
  std::lock_guard<std::mutex> lk(mu);
  if (!have[dev]) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
      cudaGetLastError();
      return -1;
    }
    cache[dev] = major;
    have[dev] = true;
  }
  return cache[dev];
}

// Is the current device a B200, and has no earlier kernel on it reported a wait that ran out?
int current_device_ok() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return FDP_ERR_LAUNCH; }
  // A host thread that has not made a CUDA call yet (an autograd worker thread running its first
  // backward node, say) has a device ordinal but no context bound to it.  The runtime binds one on
  // demand, the driver entry point that encodes the tensor maps does not and fails.  cudaSetDevice
  // binds the device's primary context to the calling thread; once per thread and device.
  thread_local int bound_dev = -1;
  if (bound_dev != dev) {
    if (cudaSetDevice(dev) != cudaSuccess) { cudaGetLastError(); return FDP_ERR_LAUNCH; }
    bound_dev = dev;
  }
  if (device_cc_major(dev) != 10) return FDP_ERR_ARCH;
  volatile int* arr = sticky_array();
  if (arr != nullptr && dev < 64 && arr[dev] != 0) return FDP_ERR_TIMEOUT;
  return FDP_OK;
}

int check_params(const fdp_dp_params* p) {
  if (p == nullptr) return FDP_ERR_ARG;
  if (!(p->noise_std >= 0.f)) return FDP_ERR_ARG;
  if (p->noise_world > 1 && (p->noise_rank < 0 || p->noise_rank >= p->noise_world)) return FDP_ERR_ARG;
  return FDP_OK;
}

// workspace of fdp_linear_wgrad: [status word | norms | factors | partials | tensor-core extra]
struct WgradWs {
  int* status; float* norms; float* factors; float* partials; void* tc_extra;
  size_t bytes; int nparts; TcPlan tc;
  bool short_seq;   // norms by the small Gram kernel (T < SHORT_SEQ unless the caller asked for the direct norm)
};
WgradWs wgrad_ws(void* base, int B, int T, int n_in, int n_out, int dt, int norm_algo) {
  WgradWs w;
  w.tc = tc_plan(B, T, n_in, n_out, dt, norm_algo);
  w.short_seq = T < SHORT_SEQ && (norm_algo & FDP_NORM_MASK) != FDP_NORM_DIRECT;
  w.nparts = w.tc.ok ? w.tc.nparts : (w.short_seq ? 1 : simt_norm_tiles(n_in, n_out));
  Carver c(base);
  w.status = c.take<int>(64);
  w.norms = c.take<float>(B);
  w.factors = c.take<float>(B);
  w.partials = c.take<float>(static_cast<size_t>(B) * w.nparts);
  w.tc_extra = c.take<char>(w.tc.ok ? w.tc.ws_bytes : 0);
  w.bytes = c.off;
  return w;
}

// Optional phase timing of fdp_linear_wgrad: CUDA events recorded on the caller's stream between
// the phases (norm pass | clip factors | c_b pre-scale | clipped-sum GEMM).  Off by default.
struct PhaseProfile {
  std::mutex mu;
  bool on = false;
  bool have_events = false;
  bool recorded = false;
  cudaEvent_t ev[5];
} g_prof;

void prof_mark(int i, cudaStream_t s) {
  if (!g_prof.on) return;
  std::lock_guard<std::mutex> lk(g_prof.mu);
  if (g_prof.on && g_prof.have_events) {
    cudaEventRecord(g_prof.ev[i], s);
    if (i == 4) g_prof.recorded = true;
  }
}

}  // namespace

extern "C" {

unsigned long long fdp_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int fdp_profile_enable(int on) {
  std::lock_guard<std::mutex> lk(g_prof.mu);
  if (on && !g_prof.have_events) {
    for (int i = 0; i < 5; ++i)
      if (cudaEventCreate(&g_prof.ev[i]) != cudaSuccess) { cudaGetLastError(); return FDP_ERR_LAUNCH; }
    g_prof.have_events = true;
  }
  g_prof.on = on != 0;
  g_prof.recorded = false;
  return FDP_OK;
}

int fdp_profile_read(float* ms, int capacity) {
  std::lock_guard<std::mutex> lk(g_prof.mu);
  if (ms == nullptr || capacity < 4) return FDP_ERR_ARG;
  if (!g_prof.have_events || !g_prof.recorded) return FDP_ERR_ARG;
  if (cudaEventSynchronize(g_prof.ev[4]) != cudaSuccess) { cudaGetLastError(); return FDP_ERR_LAUNCH; }
  for (int i = 0; i < 4; ++i)
    if (cudaEventElapsedTime(&ms[i], g_prof.ev[i], g_prof.ev[i + 1]) != cudaSuccess) { cudaGetLastError(); return FDP_ERR_LAUNCH; }
  return 4;
}

int fdp_abi_version(void) { return FDP_ABI_VERSION; }

const char* fdp_status_string(int status) {
  switch (status) {
    case FDP_OK: return "ok";
    case FDP_ERR_ARG: return "invalid argument";
    case FDP_ERR_DTYPE: return "unsupported dtype";
    case FDP_ERR_SHAPE: return "unsupported shape";
    case FDP_ERR_ALIGN: return "pointer not 16-byte aligned";
    case FDP_ERR_WORKSPACE: return "workspace missing or too small";
    case FDP_ERR_ARCH: return "device is not sm_100 (B200)";
    case FDP_ERR_LAUNCH: return "CUDA launch/runtime error";
    case FDP_ERR_TIMEOUT: return "a bounded device-side wait ran out (results of that call are undefined; fdp_clear_async_status re-arms the device)";
    case FDP_ERR_STATIC_LIMIT: return "problem needs more scratch than the library's fixed buffer (FDP_STATIC_SCRATCH_BYTES)";
    default: return "unknown status";
  }
}

int fdp_check_device(int device) { return device_cc_major(device) == 10 ? FDP_OK : FDP_ERR_ARCH; }

int fdp_device_status(const void* workspace, fdp_stream_t stream) {
  int h = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (workspace != nullptr)
    FDP_CUDA_OK(cudaMemcpyAsync(&h, workspace, sizeof(int), cudaMemcpyDeviceToHost, s));
  FDP_CUDA_OK(cudaStreamSynchronize(s));
  if (h != 0) return FDP_ERR_TIMEOUT;
  return fdp_async_status(-1);
}

int fdp_async_status(int device) {
  if (device < 0 && cudaGetDevice(&device) != cudaSuccess) { cudaGetLastError(); return FDP_ERR_LAUNCH; }
  if (device < 0 || device >= 64) return FDP_ERR_ARG;
  volatile int* arr = fdp::sticky_array();
  return (arr != nullptr && arr[device] != 0) ? FDP_ERR_TIMEOUT : FDP_OK;
}

int fdp_clear_async_status(int device) {
  if (device < 0 && cudaGetDevice(&device) != cudaSuccess) { cudaGetLastError(); return FDP_ERR_LAUNCH; }
  if (device < 0 || device >= 64) return FDP_ERR_ARG;
  volatile int* arr = fdp::sticky_array();
  if (arr != nullptr) arr[device] = 0;
  return FDP_OK;
}

int fdp_set_sm_reserve(int n) { return sm_reserve_exchange(n); }

int fdp_selftest_wait_timeout(long long limit_cycles, void* workspace, size_t workspace_bytes, fdp_stream_t stream) {
  if (workspace == nullptr || workspace_bytes < 256 || !aligned16(workspace)) return FDP_ERR_WORKSPACE;
  int st = current_device_ok();
  if (st != FDP_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  FDP_CUDA_OK(cudaMemsetAsync(workspace, 0, sizeof(int), s));
  return tc_wait_selftest(static_cast<int*>(workspace), limit_cycles, s);
}

// ---- weight gradient ------------------------------------------------------------------------------
size_t fdp_linear_wgrad_workspace_bytes(int B, int T, int n_in, int n_out, int in_dtype,
                                        int norm_algo) {
  if (B <= 0 || T <= 0 || n_in <= 0 || n_out <= 0 || !valid_dtype(in_dtype)) return 0;
  return wgrad_ws(nullptr, B, T, n_in, n_out, in_dtype, norm_algo).bytes;
}

int fdp_linear_wgrad(const void* G, const void* X, void* dW, float* norms_out, float* factors_out,
                     int B, int T, int n_in, int n_out, int in_dtype, int out_dtype, int layout,
                     int norm_algo, const fdp_dp_params* p, void* workspace, size_t workspace_bytes,
                     fdp_stream_t stream) {
  NvtxRange nvtx_range("fdp_linear_wgrad");
  if (G == nullptr || X == nullptr || dW == nullptr) return FDP_ERR_ARG;
  if (B <= 0 || T <= 0 || n_in <= 0 || n_out <= 0) return FDP_ERR_ARG;
  if (layout != FDP_OUT_IN && layout != FDP_IN_OUT) return FDP_ERR_ARG;
  if (norm_algo < 0 || (norm_algo & ~(FDP_NORM_MASK | FDP_FP32_TENSOR)) != 0 || (norm_algo & FDP_NORM_MASK) > FDP_NORM_GRAM)
    return FDP_ERR_ARG;
  if (!valid_dtype(in_dtype) || !valid_dtype(out_dtype)) return FDP_ERR_DTYPE;
  if (static_cast<long long>(B) * T >= (1ll << 31) / 2) return FDP_ERR_SHAPE;   // row indices are 32-bit
  int st = check_params(p);
  if (st != FDP_OK) return st;
  if ((st = current_device_ok()) != FDP_OK) return st;
  if (workspace == nullptr) return FDP_ERR_WORKSPACE;
  WgradWs w = wgrad_ws(workspace, B, T, n_in, n_out, in_dtype, norm_algo);
  if (workspace_bytes < w.bytes || !aligned16(workspace)) return FDP_ERR_WORKSPACE;
  // the tensor-core path moves 16-byte vectors (TMA, vector stores); the generic kernels load and
  // store single elements and take any naturally aligned pointer
  if (w.tc.ok && (!aligned16(G) || !aligned16(X) || !aligned16(dW))) return FDP_ERR_ALIGN;

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int div = p->batch_divisor > 0 ? p->batch_divisor : B;
  const float inv_div = 1.0f / static_cast<float>(div);
  const NoiseKey nk = make_noise_key(p, p->param_id);
  // the status word: cleared by the first tensor-core launch of the call itself, or here when the call
  // starts with a kernel that does not know it
  if (!w.tc.ok || w.short_seq) FDP_CUDA_OK(cudaMemsetAsync(w.status, 0, sizeof(int), s));

  // the scaled epilogue of the clipped-sum GEMM reduces the norm partials itself: no clip-factor launch
  const bool fused_factors = w.tc.ok && w.tc.scaled_epilogue && tc_fused_factors_ok(B);
  prof_mark(0, s);
  // fp32 inputs on the tensor cores: split G and X into bf16 halves first, then run as bf16
  const void* Gt = G;
  const void* Xt = X;
  int tdt = in_dtype;
  if (w.tc.ok && w.tc.split3) {
    char* sg = static_cast<char*>(w.tc_extra) + w.tc.split_bytes;
    char* sx = sg + w.tc.split3_g_bytes;
    if ((st = tc_split3(G, sg, static_cast<size_t>(B) * T, n_out, s)) != FDP_OK) return st;
    if ((st = tc_split3(X, sx, static_cast<size_t>(B) * T, n_in, s)) != FDP_OK) return st;
    Gt = sg; Xt = sx; tdt = FDP_BF16;
  }
  if (w.short_seq) {
    simt_norm_gram_small(G, X, w.partials, B, T, n_in, n_out, in_dtype, s);
  } else if (w.tc.ok) {
    if ((st = tc_norms(Gt, Xt, w.partials, w.status, B, T, n_in, n_out, tdt, w.tc, s)) != FDP_OK) return st;
  } else {
    w.nparts = simt_norm_direct(G, X, w.partials, B, T, n_in, n_out, in_dtype, norm_algo & FDP_NORM_MASK, s);
  }
  prof_mark(1, s);
  if (!fused_factors)
    clip_factors(w.partials, w.nparts, B, p->C, p->clamp_value, w.norms, w.factors, norms_out, factors_out, s);
  prof_mark(2, s);
  if (w.tc.ok) {
    float* split_ws = static_cast<float*>(w.tc_extra);
    char* gs = static_cast<char*>(w.tc_extra) + w.tc.split_bytes;
    if (!w.tc.scaled_epilogue) {
      if ((st = tc_prescale(G, w.factors, gs, B, T, n_out, in_dtype, s)) != FDP_OK) return st;
    }
    prof_mark(3, s);
    TcFactorSource fs{};
    if (fused_factors) {
      fs.norm_partials = w.partials; fs.nparts = w.nparts; fs.C = p->C; fs.clamp = p->clamp_value;
      fs.norms_out = norms_out; fs.factors_out = factors_out;
    } else {
      fs.factors = w.factors;
    }
    if ((st = tc_clipped_wgrad(w.tc.scaled_epilogue ? Gt : gs, Xt, w.tc.scaled_epilogue ? &fs : nullptr, split_ws,
                               dW, w.status, B, T, n_in, n_out, tdt, out_dtype, layout, inv_div, nk,
                               s, w.tc.split3 ? 3 : 1)) != FDP_OK) return st;
  } else {
    prof_mark(3, s);
    simt_clipped_wgrad(G, X, w.factors, dW, B, T, n_in, n_out, in_dtype, out_dtype, layout, inv_div, nk, s);
  }
  prof_mark(4, s);
  FDP_LAUNCH_OK();
  return FDP_OK;
}

// ---- bias gradient ----------------------------------------------------------------------------------
size_t fdp_bias_grad_workspace_bytes(int B, int T, int n_out, int in_dtype) {
  if (B <= 0 || T <= 0 || n_out <= 0 || !valid_dtype(in_dtype)) return 0;
  const GstatsPlan pl = gstats_plan(B, T, n_out, in_dtype);
  Carver c(nullptr);
  c.take<float>(B);                                                      // factors
  c.take<float>(static_cast<size_t>(B) * pl.row_chunks * pl.col_chunks); // sq partials
  c.take<float>(static_cast<size_t>(B) * pl.row_chunks * n_out);         // column-sum partials
  return c.off;
}

int fdp_bias_grad(const void* G, void* db, float* norms_out, float* factors_out, int B, int T,
                  int n_out, int in_dtype, int out_dtype, const fdp_dp_params* p, void* workspace,
                  size_t workspace_bytes, fdp_stream_t stream) {
  NvtxRange nvtx_range("fdp_bias_grad");
  if (G == nullptr || db == nullptr) return FDP_ERR_ARG;
  if (B <= 0 || T <= 0 || n_out <= 0) return FDP_ERR_ARG;
  if (static_cast<long long>(B) * T >= (1ll << 31) / 2) return FDP_ERR_SHAPE;   // row indices are 32-bit
  if (!valid_dtype(in_dtype) || !valid_dtype(out_dtype)) return FDP_ERR_DTYPE;
  int st = check_params(p);
  if (st != FDP_OK) return st;
  if ((st = current_device_ok()) != FDP_OK) return st;
  if (workspace == nullptr || !aligned16(workspace) ||
      workspace_bytes < fdp_bias_grad_workspace_bytes(B, T, n_out, in_dtype))
    return FDP_ERR_WORKSPACE;
  const GstatsPlan pl = gstats_plan(B, T, n_out, in_dtype);
  Carver c(workspace);
  float* factors = c.take<float>(B);
  float* sq_part = c.take<float>(static_cast<size_t>(B) * pl.row_chunks * pl.col_chunks);
  float* colsum_part = c.take<float>(static_cast<size_t>(B) * pl.row_chunks * n_out);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int div = p->batch_divisor > 0 ? p->batch_divisor : B;
  // mean over the B*T rows (flashdp/core/linear_clip.py:122)
  const float inv_div = 1.0f / (static_cast<float>(div) * static_cast<float>(T));
  gstats(G, colsum_part, sq_part, B, T, n_out, in_dtype, pl, s);
  bias_clip_finalize(colsum_part, sq_part, pl.row_chunks * pl.col_chunks, p->C, p->clamp_value, factors, norms_out,
                     factors_out, db, B, n_out, pl.row_chunks, out_dtype, inv_div, make_noise_key(p, p->param_id), s);
  FDP_LAUNCH_OK();
  return FDP_OK;
}

// ---- input gradient ---------------------------------------------------------------------------------
// fp32 with FDP_FP32_TENSOR in `dtype`: whether the product [rows, K] x [K, N] takes the three-product path
static bool gemm3_wanted(int dtype, int rows, int K, int N) {
  return dtype == (FDP_F32 | FDP_FP32_TENSOR) && tc_gemm3_ok(rows, K, N);
}

size_t fdp_linear_dgrad_workspace_bytes(int rows, int n_in, int n_out, int dtype) {
  // the status word, then the split copies of the two operands when fp32 runs on the tensor cores
  // (K = n_out, N = n_in; the forward product queries with the two exchanged)
  return 256 + (gemm3_wanted(dtype, rows, n_out, n_in) ? tc_gemm3_ws_bytes(rows, n_out, n_in) : 0);
}

// Y[rows, N] = A[rows, K] * W (+ bias), fp32 in and out, as three bf16 products: split, then one GEMM
static int gemm3_call(const void* A, const void* W, const void* bias, void* Y, int rows, int K, int N, int out_dtype,
                      bool w_kn, void* workspace, size_t workspace_bytes, cudaStream_t s) {
  if (workspace_bytes < 256 + tc_gemm3_ws_bytes(rows, K, N)) return FDP_ERR_WORKSPACE;
  int* status = static_cast<int*>(workspace);
  char* a3 = static_cast<char*>(workspace) + 256;
  char* w3 = a3 + ((static_cast<size_t>(rows) * K * 4 + 255) & ~static_cast<size_t>(255));
  FDP_CUDA_OK(cudaMemsetAsync(status, 0, sizeof(int), s));
  int st;
  if ((st = tc_split3(A, a3, static_cast<size_t>(rows), K, s)) != FDP_OK) return st;
  // W is [K, N] (w_kn) or [N, K]: either way its rows are split along their own columns
  if ((st = tc_split3(W, w3, static_cast<size_t>(w_kn ? K : N), w_kn ? N : K, s)) != FDP_OK) return st;
  return tc_gemm3(a3, w3, bias, Y, status, rows, K, N, out_dtype, w_kn, s);
}

int fdp_linear_dgrad(const void* G, const void* W, void* dX, int rows, int n_in, int n_out,
                     int dtype, int out_dtype, int w_layout, void* workspace, size_t workspace_bytes,
                     fdp_stream_t stream) {
  NvtxRange nvtx_range("fdp_linear_dgrad");
  if (G == nullptr || W == nullptr || dX == nullptr) return FDP_ERR_ARG;
  if (rows <= 0 || n_in <= 0 || n_out <= 0) return FDP_ERR_ARG;
  if (w_layout != FDP_OUT_IN && w_layout != FDP_IN_OUT) return FDP_ERR_ARG;
  const bool want3 = gemm3_wanted(dtype, rows, n_out, n_in);
  if ((dtype & FDP_FP32_TENSOR) != 0 && (dtype & ~FDP_FP32_TENSOR) == FDP_F32) dtype = FDP_F32;
  if (!valid_dtype(dtype) || !valid_dtype(out_dtype)) return FDP_ERR_DTYPE;
  int st = current_device_ok();
  if (st != FDP_OK) return st;
  if (workspace == nullptr || workspace_bytes < 256 || !aligned16(workspace)) return FDP_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int* status = static_cast<int*>(workspace);
  if (want3 && aligned16(G) && aligned16(W) && aligned16(dX)) {
    // dX = G [rows, n_out] * W: W is [n_out, n_in] = [K, N] for nn.Linear, [n_in, n_out] = [N, K] for Conv1D
    if ((st = gemm3_call(G, W, nullptr, dX, rows, n_out, n_in, out_dtype, w_layout == FDP_OUT_IN, workspace,
                         workspace_bytes, s)) != FDP_OK) return st;
  } else if (tc_dgrad_ok(rows, n_in, n_out, dtype) && aligned16(G) && aligned16(W) && aligned16(dX)) {
    if ((st = tc_dgrad(G, W, dX, status, rows, n_in, n_out, dtype, out_dtype, w_layout, s)) != FDP_OK) return st;
  } else {
    FDP_CUDA_OK(cudaMemsetAsync(status, 0, sizeof(int), s));
    simt_dgrad(G, W, dX, rows, n_in, n_out, dtype, out_dtype, w_layout, s);
  }
  FDP_LAUNCH_OK();
  return FDP_OK;
}

// ---- forward --------------------------------------------------------------------------------------------
int fdp_linear_fwd(const void* X, const void* W, const void* bias, void* Y, int rows, int n_in, int n_out,
                   int dtype, int out_dtype, int w_layout, void* workspace, size_t workspace_bytes,
                   fdp_stream_t stream) {
  NvtxRange nvtx_range("fdp_linear_fwd");
  if (X == nullptr || W == nullptr || Y == nullptr) return FDP_ERR_ARG;
  if (rows <= 0 || n_in <= 0 || n_out <= 0) return FDP_ERR_ARG;
  if (w_layout != FDP_OUT_IN && w_layout != FDP_IN_OUT) return FDP_ERR_ARG;
  const bool want3 = gemm3_wanted(dtype, rows, n_in, n_out);
  if ((dtype & FDP_FP32_TENSOR) != 0 && (dtype & ~FDP_FP32_TENSOR) == FDP_F32) dtype = FDP_F32;
  if (!valid_dtype(dtype) || !valid_dtype(out_dtype)) return FDP_ERR_DTYPE;
  int st = current_device_ok();
  if (st != FDP_OK) return st;
  if (workspace == nullptr || workspace_bytes < 256 || !aligned16(workspace)) return FDP_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int* status = static_cast<int*>(workspace);
  if (want3 && aligned16(X) && aligned16(W) && aligned16(Y) && (bias == nullptr || aligned16(bias))) {
    // Y = X [rows, n_in] * W^T: W is [n_out, n_in] = [N, K] for nn.Linear, [n_in, n_out] = [K, N] for Conv1D
    if ((st = gemm3_call(X, W, bias, Y, rows, n_in, n_out, out_dtype, w_layout == FDP_IN_OUT, workspace,
                         workspace_bytes, s)) != FDP_OK) return st;
  } else
  // same shape rules as the input gradient with the roles of n_in and n_out exchanged
  if (tc_dgrad_ok(rows, n_out, n_in, dtype) && aligned16(X) && aligned16(W) && aligned16(Y)) {
    if ((st = tc_fwd(X, W, bias, Y, status, rows, n_in, n_out, dtype, out_dtype, w_layout, s)) != FDP_OK) return st;
  } else {
    FDP_CUDA_OK(cudaMemsetAsync(status, 0, sizeof(int), s));
    simt_fwd(X, W, bias, Y, rows, n_in, n_out, dtype, out_dtype, w_layout, s);
  }
  FDP_LAUNCH_OK();
  return FDP_OK;
}

// ---- LayerNorm ------------------------------------------------------------------------------------------
int fdp_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean,
                      float* rstd, int rows, int d, float eps, int dtype, int param_dtype,
                      fdp_stream_t stream) {
  NvtxRange nvtx_range("fdp_layernorm_fwd");
  if (x == nullptr || gamma == nullptr || beta == nullptr || y == nullptr || mean == nullptr || rstd == nullptr)
    return FDP_ERR_ARG;
  if (rows <= 0 || d <= 0) return FDP_ERR_ARG;
  if (!valid_dtype(dtype) || !valid_dtype(param_dtype)) return FDP_ERR_DTYPE;
  int st = current_device_ok();
  if (st != FDP_OK) return st;
  ln_fwd(x, gamma, beta, y, mean, rstd, rows, d, eps, dtype, param_dtype, static_cast<cudaStream_t>(stream));
  FDP_LAUNCH_OK();
  return FDP_OK;
}

size_t fdp_layernorm_bwd_workspace_bytes(int B, int T, int d) {
  if (B <= 0 || T <= 0 || d <= 0) return 0;
  // the query has no dtype: take the larger chunk count of the 32-bit and the 16-bit plan
  const int c32 = ln_plan(B, T, d, FDP_F32).chunks, c16 = ln_plan(B, T, d, FDP_BF16).chunks;
  const int chunks = c32 > c16 ? c32 : c16;
  Carver c(nullptr);
  c.take<float>(static_cast<size_t>(2) * B * ln_sumsq_parts(d)); // partial sums of squares
  c.take<float>(2 * B);                                          // factors
  c.take<float>(static_cast<size_t>(2) * B * chunks * d);        // partials, both tensors
  return c.off;
}

int fdp_layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean,
                      const float* rstd, void* dx, void* dgamma, void* dbeta, float* norms_gamma,
                      float* norms_beta, int B, int T, int d, int dtype, int param_dtype,
                      const fdp_dp_params* p, void* workspace, size_t workspace_bytes,
                      fdp_stream_t stream) {
  NvtxRange nvtx_range("fdp_layernorm_bwd");
  if (dy == nullptr || x == nullptr || gamma == nullptr || mean == nullptr || rstd == nullptr || dgamma == nullptr)
    return FDP_ERR_ARG;
  if (B <= 0 || T <= 0 || d <= 0) return FDP_ERR_ARG;
  if (!valid_dtype(dtype) || !valid_dtype(param_dtype)) return FDP_ERR_DTYPE;
  if (d > 8192 || static_cast<long long>(B) * T >= (1ll << 31) / 2) return FDP_ERR_SHAPE;
  int st = check_params(p);
  if (st != FDP_OK) return st;
  if ((st = current_device_ok()) != FDP_OK) return st;
  if (workspace == nullptr || !aligned16(workspace) ||
      workspace_bytes < fdp_layernorm_bwd_workspace_bytes(B, T, d))
    return FDP_ERR_WORKSPACE;
  const LnPlan pl = ln_plan(B, T, d, dtype);
  Carver c(workspace);
  float* sumsq = c.take<float>(static_cast<size_t>(2) * B * ln_sumsq_parts(d));
  float* factors = c.take<float>(2 * B);
  float* part = c.take<float>(static_cast<size_t>(2) * B * pl.chunks * d);
  float* dg_part = part;
  float* db_part = part + static_cast<size_t>(B) * pl.chunks * d;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int div = p->batch_divisor > 0 ? p->batch_divisor : B;
  const float inv_div = 1.0f / static_cast<float>(div);
  ln_bwd(dy, x, gamma, mean, rstd, dx, dg_part, db_part, B, T, d, dtype, param_dtype, pl, s);
  ln_psgrad_reduce(part, sumsq, B, pl.chunks, d, s);
  // norms over d (one per sample and tensor), clip factors, mean over the batch, noise
  ln_clip_finalize(part, sumsq, ln_sumsq_parts(d), p->C, p->clamp_value, factors, norms_gamma, norms_beta, dgamma,
                   dbeta, B, pl.chunks, d, param_dtype, inv_div, make_noise_key(p, p->param_id),
                   make_noise_key(p, p->param_id2), s);
  FDP_LAUNCH_OK();
  return FDP_OK;
}

size_t fdp_layernorm_saturate_workspace_bytes(int rows, int d) {
  if (rows <= 0 || d <= 0) return 0;
  return static_cast<size_t>(2) * ln_saturate_groups(rows, d) * d * sizeof(float);
}

int fdp_layernorm_saturate_groups(int rows, int d) { return (rows <= 0 || d <= 0) ? 0 : ln_saturate_groups(rows, d); }

int fdp_layernorm_bwd_saturate(const void* dy, const void* x, const float* mean, const float* rstd, void* dgamma,
                               void* dbeta, int rows, int d, int dtype, int param_dtype, float C, float clamp_value,
                               void* workspace, size_t workspace_bytes, fdp_stream_t stream) {
  NvtxRange nvtx_range("fdp_layernorm_bwd_saturate");
  if (dy == nullptr || x == nullptr || mean == nullptr || rstd == nullptr || dgamma == nullptr) return FDP_ERR_ARG;
  if (rows <= 0 || d <= 0) return FDP_ERR_ARG;
  if (!valid_dtype(dtype) || !valid_dtype(param_dtype)) return FDP_ERR_DTYPE;
  int st = current_device_ok();
  if (st != FDP_OK) return st;
  if (workspace == nullptr || !aligned16(workspace) || workspace_bytes < fdp_layernorm_saturate_workspace_bytes(rows, d))
    return FDP_ERR_WORKSPACE;
  float* dw_buf = static_cast<float*>(workspace);
  float* db_buf = dw_buf + static_cast<size_t>(ln_saturate_groups(rows, d)) * d;
  ln_saturate(dy, x, mean, rstd, dw_buf, db_buf, dgamma, dbeta, rows, d, dtype, param_dtype, C, clamp_value,
              static_cast<cudaStream_t>(stream));
  FDP_LAUNCH_OK();
  return FDP_OK;
}

}  // extern "C"
