// Shared device helpers: number-type conversion, Philox noise, block reductions, workspace carving.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <mutex>

#include "../../include/fdp_b200.h"

namespace fdp {

// ---- number types ------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// One 16-byte vector <-> its 16/sizeof(T) values as fp32.  A bf16 value is the upper half of the
// fp32 with the same value, so a pair unpacks with one shift and one mask; packing rounds two
// values at a time (cvt.rn.bf16x2.f32 / cvt.rn.f16x2.f32).  The HBM-bound kernels are limited by
// instruction issue, not bandwidth, which is why the element-at-a-time conversions are avoided.
template <typename T> __device__ __forceinline__ void unpack16(const uint4& r, float* f);
template <> __device__ __forceinline__ void unpack16<float>(const uint4& r, float* f) {
  f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
}
template <> __device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& r, float* f) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    f[2 * k] = __uint_as_float(w[k] << 16);
    f[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
  }
}
template <> __device__ __forceinline__ void unpack16<__half>(const uint4& r, float* f) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
    f[2 * k] = p.x; f[2 * k + 1] = p.y;
  }
}
template <typename T> __device__ __forceinline__ uint4 pack16(const float* f);
template <> __device__ __forceinline__ uint4 pack16<float>(const float* f) {
  return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
}
template <> __device__ __forceinline__ uint4 pack16<__nv_bfloat16>(const float* f) {
  uint32_t w[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
    w[k] = *reinterpret_cast<const uint32_t*>(&p);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
template <> __device__ __forceinline__ uint4 pack16<__half>(const float* f) {
  uint32_t w[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const __half2 p = __floats2half2_rn(f[2 * k], f[2 * k + 1]);
    w[k] = *reinterpret_cast<const uint32_t*>(&p);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

__host__ __device__ inline size_t dtype_size(int dt) { return dt == FDP_F32 ? 4 : 2; }

// store one fp32 value as `dt` at element index i of a type-erased output
__device__ __forceinline__ void store_as(void* out, int dt, size_t i, float v) {
  if (dt == FDP_F32) reinterpret_cast<float*>(out)[i] = v;
  else if (dt == FDP_BF16) reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(out)[i] = __float2half_rn(v);
}
__device__ __forceinline__ float load_as(const void* in, int dt, size_t i) {
  if (dt == FDP_F32) return reinterpret_cast<const float*>(in)[i];
  if (dt == FDP_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(in)[i]);
  return __half2float(reinterpret_cast<const __half*>(in)[i]);
}

// ---- clip factor: min(clamp_value, C / (norm + 1e-10))  (flashdp/core/clip_fn.py:6-8) -----
__device__ __forceinline__ float clip_factor(float norm, float C, float clamp_value) {
  return fminf(clamp_value, C / (norm + 1e-10f));
}

// ---- Philox4x32-10 + Box-Muller -----------------------------------------------------------
// Element i of a tensor uses counter (i>>2 lo, i>>2 hi, param_id, step), key (seed lo, seed hi).
// Words (0,1) give the cos/sin pair of lanes 0/1, words (2,3) that of lanes 2/3; a word w maps
// to the uniform ((w>>9)+0.5)*2^-23, exact in fp32.
struct NoiseKey {
  uint32_t k0, k1, param_id, step;
  float std;
  int rank, world;  // element group g is drawn by the rank with g % world == rank
  const uint32_t* step_dev;  // null, or a device counter added to `step` when the kernel runs
};

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                              uint32_t k0, uint32_t k1, uint32_t r[4]) {
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  r[0] = c0; r[1] = c1; r[2] = c2; r[3] = c3;
}

__device__ __forceinline__ void box_muller(uint32_t w0, uint32_t w1, float& zc, float& zs) {
  float u1 = (static_cast<float>(w0 >> 9) + 0.5f) * 1.1920928955078125e-07f;  // 2^-23
  float u2 = (static_cast<float>(w1 >> 9) + 0.5f) * 1.1920928955078125e-07f;
  float rad = sqrtf(-2.0f * logf(u1));
  float s, c;
  sincospif(2.0f * u2, &s, &c);
  zc = rad * c; zs = rad * s;
}

// four standard normals of element group g (elements 4g..4g+3); zero when another rank owns g
__device__ __forceinline__ void noise_group(const NoiseKey& nk, uint64_t g, float z[4]) {
  if (nk.world > 1 && static_cast<int>(g % static_cast<uint64_t>(nk.world)) != nk.rank) {
    z[0] = z[1] = z[2] = z[3] = 0.f;
    return;
  }
  uint32_t r[4];
  const uint32_t step = nk.step_dev != nullptr ? nk.step + __ldg(nk.step_dev) : nk.step;
  philox4x32_10(static_cast<uint32_t>(g), static_cast<uint32_t>(g >> 32), nk.param_id, step,
                nk.k0, nk.k1, r);
  box_muller(r[0], r[1], z[0], z[1]);
  box_muller(r[2], r[3], z[2], z[3]);
  z[0] *= nk.std; z[1] *= nk.std; z[2] *= nk.std; z[3] *= nk.std;
}
// the noise of a single element (recomputes the group; used where elements are visited singly)
__device__ __forceinline__ float noise_at(const NoiseKey& nk, uint64_t i) {
  float z[4];
  noise_group(nk, i >> 2, z);
  return z[i & 3];
}

inline NoiseKey make_noise_key(const fdp_dp_params* p, uint32_t param_id) {
  NoiseKey nk;
  nk.k0 = static_cast<uint32_t>(p->seed & 0xFFFFFFFFu);
  nk.k1 = static_cast<uint32_t>(p->seed >> 32);
  nk.param_id = param_id;
  nk.step = p->step;
  nk.std = p->noise_std;
  nk.world = p->noise_world > 1 ? p->noise_world : 1;
  nk.rank = p->noise_world > 1 ? p->noise_rank : 0;
  nk.step_dev = p->step_device;
  return nk;
}

// ---- reductions ------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// sum over a block of up to 1024 threads; result valid in every thread; fixed order
__device__ __forceinline__ float block_sum(float v, float* smem32) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem32[w] = v;
  __syncthreads();
  float t = (lane < nw) ? smem32[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

// ---- workspace carving -------------------------------------------------------------------------
struct Carver {
  char* base; size_t off;
  explicit Carver(void* b) : base(reinterpret_cast<char*>(b)), off(0) {}
  template <typename T> T* take(size_t n) {
    T* p = reinterpret_cast<T*>(base + off);
    off += (n * sizeof(T) + 255) & ~static_cast<size_t>(255);
    return p;
  }
};

// Opt a kernel in to more than 48 KiB of dynamic shared memory, once per device.  `done` and `mu`
// are statics of the caller (one set per kernel).
template <typename K>
inline bool smem_opt_in(bool (&done)[64], std::mutex& mu, K kernel, size_t bytes) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return false; }
  std::lock_guard<std::mutex> lk(mu);
  if (!done[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    done[dev] = true;
  }
  return true;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

#define FDP_CUDA_OK(expr) do { if ((expr) != cudaSuccess) { cudaGetLastError(); return FDP_ERR_LAUNCH; } } while (0)
#define FDP_LAUNCH_OK() do { if (cudaPeekAtLastError() != cudaSuccess) { cudaGetLastError(); return FDP_ERR_LAUNCH; } } while (0)

}  // namespace fdp
