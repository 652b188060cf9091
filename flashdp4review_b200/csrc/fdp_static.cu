// fdp_bias_grad_static: the DP bias gradient for callers that have no way to hand over a
// workspace.  Same kernels as fdp_bias_grad; the partial sums live in a fixed buffer that is
// part of the library image instead of in caller memory.
//
// Who needs this: a host that binds the C ABI without a device allocator of its own (a thin cgo /
// JNI / ctypes caller that only receives input and output buffers from its framework), a training
// loop whose memory pool has reserved the whole GPU so that a raw cudaMalloc from a plug-in would
// fail, and code on a latency-critical path where the device-wide synchronisation implied by
// cudaMalloc / cudaFree is not acceptable.  This entry point calls no cudaMalloc, cudaFree or any
// allocating routine.
//
// What it costs: FDP_STATIC_SCRATCH_BYTES of device memory on every GPU that loads the library,
// held until the process exits.  Problems whose partial sums need more are refused with
// FDP_ERR_STATIC_LIMIT (nothing is launched).
//
// Sharing: all calls on a device use the same buffer, and it keeps whatever the previous call
// left in it.  That is harmless for correctness here because every word a call reads was written
// by that same call first (there is no accumulate-into-zero step, so nothing needs clearing), but
// two calls that overlap on the GPU (different streams, or different host threads without
// ordering) race on it: serialise them.
//
// Set-up: the first call on each device looks up the device address of the buffer
// (cudaGetSymbolAddress, with that device current) and caches it; make that first call before
// any stream capture begins.
#include <mutex>

#include "fdp_kernels.h"

using namespace fdp;

// In host code the name of a __device__ array is only a handle for the symbol, not a device
// address; kernels get the address obtained below.
static __device__ __align__(256) unsigned char g_static_scratch[FDP_STATIC_SCRATCH_BYTES];

namespace {

// device address of g_static_scratch on the current device (looked up once per device)
int static_scratch(void** out) {
  static std::mutex mu;
  static void* ptr[64];
  static bool have[64];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return FDP_ERR_LAUNCH; }
  std::lock_guard<std::mutex> lk(mu);
  if (!have[dev]) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) { cudaGetLastError(); return FDP_ERR_LAUNCH; }
    if (major != 10) return FDP_ERR_ARCH;
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) { cudaGetLastError(); return FDP_ERR_LAUNCH; }
    ptr[dev] = p;
    have[dev] = true;
  }
  *out = ptr[dev];
  return FDP_OK;
}

bool ok_dtype(int dt) { return dt == FDP_F32 || dt == FDP_BF16 || dt == FDP_F16; }

}  // namespace

extern "C" int fdp_bias_grad_static(const void* G, void* db, float* norms_out, float* factors_out, int B,
                                    int T, int n_out, int in_dtype, int out_dtype, const fdp_dp_params* p,
                                    fdp_stream_t stream) {
  if (G == nullptr || db == nullptr || p == nullptr) return FDP_ERR_ARG;
  if (B <= 0 || T <= 0 || n_out <= 0) return FDP_ERR_ARG;
  if (static_cast<long long>(B) * T >= (1ll << 31) / 2) return FDP_ERR_SHAPE;   // row indices are 32-bit
  if (!ok_dtype(in_dtype) || !ok_dtype(out_dtype)) return FDP_ERR_DTYPE;
  if (!(p->noise_std >= 0.f)) return FDP_ERR_ARG;
  if (p->noise_world > 1 && (p->noise_rank < 0 || p->noise_rank >= p->noise_world)) return FDP_ERR_ARG;
  // the same carve-up as fdp_bias_grad, checked against the fixed capacity before anything runs
  const size_t need = fdp_bias_grad_workspace_bytes(B, T, n_out, in_dtype);
  if (need == 0 || need > static_cast<size_t>(FDP_STATIC_SCRATCH_BYTES)) return FDP_ERR_STATIC_LIMIT;
  void* scratch = nullptr;
  const int st = static_scratch(&scratch);
  if (st != FDP_OK) return st;

  const GstatsPlan pl = gstats_plan(B, T, n_out, in_dtype);
  Carver c(scratch);
  float* factors = c.take<float>(B);
  float* sq_part = c.take<float>(static_cast<size_t>(B) * pl.row_chunks * pl.col_chunks);
  float* colsum_part = c.take<float>(static_cast<size_t>(B) * pl.row_chunks * n_out);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int div = p->batch_divisor > 0 ? p->batch_divisor : B;
  const float inv_div = 1.0f / (static_cast<float>(div) * static_cast<float>(T));
  gstats(G, colsum_part, sq_part, B, T, n_out, in_dtype, pl, s);
  bias_clip_finalize(colsum_part, sq_part, pl.row_chunks * pl.col_chunks, p->C, p->clamp_value, factors, norms_out,
                     factors_out, db, B, n_out, pl.row_chunks, out_dtype, inv_div, make_noise_key(p, p->param_id), s);
  FDP_LAUNCH_OK();
  return FDP_OK;
}
