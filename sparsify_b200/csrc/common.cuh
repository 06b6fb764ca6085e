// Shared helpers for the libsparsecoder kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/sparsecoder.h"

namespace sc {

// Records the message returned by sc_last_error(); returns `status`.
int fail(int status, const char* fmt, ...);

// SMs the persistent kernels leave free (sc_set_reserved_sms), e.g. for a
// communication library's kernels that have to run beside them.
int reserved_sms();

// Form of the tensor-core encoder (sc_set_cta_pairs): -1 chosen per shape (default), 0 one CTA
// per tile, 1 CTA pairs.
int cta_pairs_mode();

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// Checks the launch of the kernel just enqueued (no synchronisation).
#define SC_CHECK_LAUNCH(name)                                                    \
  do {                                                                           \
    cudaError_t e__ = cudaGetLastError();                                        \
    if (e__ != cudaSuccess)                                                      \
      return sc::fail(SC_ERR_CUDA, "%s: launch failed: %s", name,                \
                      cudaGetErrorString(e__));                                  \
  } while (0)

#define SC_CUDA(call)                                                            \
  do {                                                                           \
    cudaError_t e__ = (call);                                                    \
    if (e__ != cudaSuccess)                                                      \
      return sc::fail(SC_ERR_CUDA, "%s failed: %s", #call,                       \
                      cudaGetErrorString(e__));                                  \
  } while (0)

#define SC_REQUIRE(cond, ...)                                                    \
  do {                                                                           \
    if (!(cond)) return sc::fail(SC_ERR_INVALID, __VA_ARGS__);                   \
  } while (0)

inline bool valid_dtype(int dt) { return dt == SC_F32 || dt == SC_BF16; }
inline size_t dtype_size(int dt) { return dt == SC_BF16 ? 2 : 4; }
inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// ---- device helpers -------------------------------------------------------

// Loads four consecutive elements starting at p (16-byte aligned for float,
// 8-byte aligned for bf16) and widens them to fp32.
template <typename T>
__device__ __forceinline__ float4 load4(const T* p);

template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
  return __ldg(reinterpret_cast<const float4*>(p));
}

template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
  float4 r;
  r.x = __uint_as_float(raw.x << 16);
  r.y = __uint_as_float(raw.x & 0xffff0000u);
  r.z = __uint_as_float(raw.y << 16);
  r.w = __uint_as_float(raw.y & 0xffff0000u);
  return r;
}

template <typename T>
__device__ __forceinline__ float load1(const T* p);
template <>
__device__ __forceinline__ float load1<float>(const float* p) { return __ldg(p); }
template <>
__device__ __forceinline__ float load1<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum over a thread block of up to 1024 threads; result valid in every thread.
// `scratch` is at least 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // protects scratch against a previous use
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

}  // namespace sc
