// Weight-sized passes of the optimiser step: decoder row normalisation, removal
// of the gradient component parallel to each decoder row, Adam, and the refresh
// of the bf16 shadow copy used by the tensor-core encoder and the gathers. One
// CTA per row keeps the row's reductions and its update in a single pass.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kRowThreads = 256;

__global__ void __launch_bounds__(kRowThreads)
normalize_rows_kernel(float* __restrict__ W, int64_t D, float eps,
                      __nv_bfloat16* __restrict__ shadow) {
  __shared__ float scratch[33];
  float* row = W + (int64_t)blockIdx.x * D;
  float ss = 0.f;
  for (int64_t c = threadIdx.x; c < D; c += blockDim.x) { float v = row[c]; ss = fmaf(v, v, ss); }
  ss = sc::block_sum(ss, scratch);
  const float denom = sqrtf(ss) + eps;
  for (int64_t c = threadIdx.x; c < D; c += blockDim.x) {
    float v = row[c] / denom;
    row[c] = v;
    if (shadow != nullptr) shadow[(int64_t)blockIdx.x * D + c] = __float2bfloat16_rn(v);
  }
}

struct AdamArgs {
  float lr, beta1, beta2, eps;
  float bc1;       // 1 - beta1^step
  float bc2_sqrt;  // sqrt(1 - beta2^step)
};

// torch.optim.Adam (single-tensor formulation):
//   m = lerp(m, g, 1-beta1); v = beta2 v + (1-beta2) g^2
//   p -= (lr / bc1) * m / (sqrt(v) / sqrt(bc2) + eps)
__device__ __forceinline__ float adam_update(float p, float g, float& m, float& v,
                                             const AdamArgs& a) {
  m = m + (g - m) * (1.f - a.beta1);
  v = v * a.beta2 + (1.f - a.beta2) * g * g;
  const float denom = sqrtf(v) / a.bc2_sqrt + a.eps;
  return p - (a.lr / a.bc1) * (m / denom);
}

__global__ void __launch_bounds__(kRowThreads)
adam_rows_project_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m,
                         float* __restrict__ v, int64_t D, AdamArgs a,
                         __nv_bfloat16* __restrict__ shadow) {
  __shared__ float scratch[33];
  const int64_t off = (int64_t)blockIdx.x * D;
  float dot = 0.f;
  for (int64_t c = threadIdx.x; c < D; c += blockDim.x) dot = fmaf(g[off + c], p[off + c], dot);
  dot = sc::block_sum(dot, scratch);
  for (int64_t c = threadIdx.x; c < D; c += blockDim.x) {
    const float pc = p[off + c];
    const float gc = g[off + c] - dot * pc;
    g[off + c] = gc;
    float mc = m[off + c], vc = v[off + c];
    const float pn = adam_update(pc, gc, mc, vc, a);
    p[off + c] = pn; m[off + c] = mc; v[off + c] = vc;
    if (shadow != nullptr) shadow[off + c] = __float2bfloat16_rn(pn);
  }
}

__global__ void __launch_bounds__(256)
adam_flat_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                 float* __restrict__ v, int64_t total, AdamArgs a,
                 __nv_bfloat16* __restrict__ shadow) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    float mc = m[i], vc = v[i];
    const float pn = adam_update(p[i], g[i], mc, vc, a);
    p[i] = pn; m[i] = mc; v[i] = vc;
    if (shadow != nullptr) shadow[i] = __float2bfloat16_rn(pn);
  }
}

__global__ void __launch_bounds__(256)
cast_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16_rn(src[i]);
}

int flat_grid(int64_t total) {
  int64_t b = (total + 255) / 256;
  const int64_t cap = 148 * 32;
  return (int)(b < cap ? (b > 0 ? b : 1) : cap);
}

}  // namespace

extern "C" int sc_normalize_rows(float* W, int64_t M, int64_t D, float eps, void* shadow_bf16,
                                 void* stream) {
  SC_REQUIRE(M > 0 && D > 0 && M <= 0x7fffffffLL, "sc_normalize_rows: bad shape");
  SC_REQUIRE(W != nullptr, "sc_normalize_rows: null pointer");
  normalize_rows_kernel<<<(unsigned)M, kRowThreads, 0, sc::as_stream(stream)>>>(
      W, D, eps, static_cast<__nv_bfloat16*>(shadow_bf16));
  SC_CHECK_LAUNCH("sc_normalize_rows");
  return SC_OK;
}

extern "C" int sc_adam_rows(float* p, float* g, float* m, float* v, int64_t M, int64_t D,
                            float lr, float beta1, float beta2, float eps, int64_t step,
                            int project, void* shadow_bf16, void* stream) {
  SC_REQUIRE(M > 0 && D > 0 && M <= 0x7fffffffLL, "sc_adam_rows: bad shape");
  SC_REQUIRE(p && g && m && v, "sc_adam_rows: null pointer");
  SC_REQUIRE(step >= 1, "sc_adam_rows: step counts from 1, got %lld", (long long)step);
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps;
  a.bc1 = (float)(1.0 - pow((double)beta1, (double)step));
  a.bc2_sqrt = (float)sqrt(1.0 - pow((double)beta2, (double)step));
  cudaStream_t st = sc::as_stream(stream);
  __nv_bfloat16* shadow = static_cast<__nv_bfloat16*>(shadow_bf16);
  if (project) {
    adam_rows_project_kernel<<<(unsigned)M, kRowThreads, 0, st>>>(p, g, m, v, D, a, shadow);
  } else {
    adam_flat_kernel<<<flat_grid(M * D), 256, 0, st>>>(p, g, m, v, M * D, a, shadow);
  }
  SC_CHECK_LAUNCH("sc_adam_rows");
  return SC_OK;
}

extern "C" int sc_cast_bf16(const float* src, void* dst_bf16, int64_t n, void* stream) {
  SC_REQUIRE(n >= 0, "sc_cast_bf16: bad size");
  if (n == 0) return SC_OK;
  SC_REQUIRE(src && dst_bf16, "sc_cast_bf16: null pointer");
  cast_bf16_kernel<<<flat_grid(n), 256, 0, sc::as_stream(stream)>>>(
      src, static_cast<__nv_bfloat16*>(dst_bf16), n);
  SC_CHECK_LAUNCH("sc_cast_bf16");
  return SC_OK;
}
