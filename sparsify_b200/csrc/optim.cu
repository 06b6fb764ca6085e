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

// g[m,:] -= (g[m,:] . w[m,:]) w[m,:]: the second pass re-reads the row from L1/L2.
__global__ void __launch_bounds__(kRowThreads)
project_rows_kernel(float* __restrict__ g, const float* __restrict__ w, int64_t D) {
  __shared__ float scratch[33];
  const int64_t off = (int64_t)blockIdx.x * D;
  float dot = 0.f;
  for (int64_t c = threadIdx.x; c < D; c += blockDim.x) dot = fmaf(g[off + c], w[off + c], dot);
  dot = sc::block_sum(dot, scratch);
  for (int64_t c = threadIdx.x; c < D; c += blockDim.x) g[off + c] -= dot * w[off + c];
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

// ---- vectorised variants (D % 4 == 0, 16-byte aligned rows) --------------------
// A row of up to 256 * 4 * NV floats is held in registers, so the row-wise
// reductions cost no second pass over global memory.

__device__ __forceinline__ void store_bf16x4(__nv_bfloat16* dst, float4 v) {
  uint2 packed;
  packed.x = sc::pack_bf16x2(v.x, v.y);
  packed.y = sc::pack_bf16x2(v.z, v.w);
  *reinterpret_cast<uint2*>(dst) = packed;
}

template <int NV>
__global__ void __launch_bounds__(kRowThreads)
normalize_rows_vec_kernel(float* __restrict__ W, int64_t D, float eps, __nv_bfloat16* __restrict__ shadow) {
  __shared__ float scratch[33];
  const int64_t off = (int64_t)blockIdx.x * D;
  float4 w[NV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int64_t c = ((int64_t)i * kRowThreads + threadIdx.x) * 4;
    if (c < D) {
      w[i] = *reinterpret_cast<const float4*>(W + off + c);
      ss += w[i].x * w[i].x + w[i].y * w[i].y + w[i].z * w[i].z + w[i].w * w[i].w;
    }
  }
  ss = sc::block_sum(ss, scratch);
  const float denom = sqrtf(ss) + eps;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int64_t c = ((int64_t)i * kRowThreads + threadIdx.x) * 4;
    if (c < D) {
      float4 o = make_float4(w[i].x / denom, w[i].y / denom, w[i].z / denom, w[i].w / denom);
      *reinterpret_cast<float4*>(W + off + c) = o;
      if (shadow != nullptr) store_bf16x4(shadow + off + c, o);
    }
  }
}

template <int NV>
__global__ void __launch_bounds__(kRowThreads)
adam_rows_project_vec_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, int64_t D, AdamArgs a, __nv_bfloat16* __restrict__ shadow) {
  __shared__ float scratch[33];
  const int64_t off = (int64_t)blockIdx.x * D;
  float4 pw[NV], gw[NV];
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int64_t c = ((int64_t)i * kRowThreads + threadIdx.x) * 4;
    if (c < D) {
      pw[i] = *reinterpret_cast<const float4*>(p + off + c);
      gw[i] = __ldcs(reinterpret_cast<const float4*>(g + off + c));
      dot += gw[i].x * pw[i].x + gw[i].y * pw[i].y + gw[i].z * pw[i].z + gw[i].w * pw[i].w;
    }
  }
  dot = sc::block_sum(dot, scratch);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int64_t c = ((int64_t)i * kRowThreads + threadIdx.x) * 4;
    if (c < D) {
      float4 mw = *reinterpret_cast<const float4*>(m + off + c);
      float4 vw = *reinterpret_cast<const float4*>(v + off + c);
      float4 gp = make_float4(gw[i].x - dot * pw[i].x, gw[i].y - dot * pw[i].y, gw[i].z - dot * pw[i].z,
                              gw[i].w - dot * pw[i].w);
      float4 pn;
      pn.x = adam_update(pw[i].x, gp.x, mw.x, vw.x, a);
      pn.y = adam_update(pw[i].y, gp.y, mw.y, vw.y, a);
      pn.z = adam_update(pw[i].z, gp.z, mw.z, vw.z, a);
      pn.w = adam_update(pw[i].w, gp.w, mw.w, vw.w, a);
      *reinterpret_cast<float4*>(p + off + c) = pn;
      *reinterpret_cast<float4*>(g + off + c) = gp;
      *reinterpret_cast<float4*>(m + off + c) = mw;
      *reinterpret_cast<float4*>(v + off + c) = vw;
      if (shadow != nullptr) store_bf16x4(shadow + off + c, pn);
    }
  }
}

__global__ void __launch_bounds__(256)
adam_flat_vec_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                     float* __restrict__ v, int64_t total4, AdamArgs a, __nv_bfloat16* __restrict__ shadow) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total4;
       i += (int64_t)gridDim.x * blockDim.x) {
    float4 pw = reinterpret_cast<const float4*>(p)[i];
    const float4 gw = __ldcs(reinterpret_cast<const float4*>(g) + i);
    float4 mw = reinterpret_cast<const float4*>(m)[i];
    float4 vw = reinterpret_cast<const float4*>(v)[i];
    pw.x = adam_update(pw.x, gw.x, mw.x, vw.x, a);
    pw.y = adam_update(pw.y, gw.y, mw.y, vw.y, a);
    pw.z = adam_update(pw.z, gw.z, mw.z, vw.z, a);
    pw.w = adam_update(pw.w, gw.w, mw.w, vw.w, a);
    reinterpret_cast<float4*>(p)[i] = pw;
    reinterpret_cast<float4*>(m)[i] = mw;
    reinterpret_cast<float4*>(v)[i] = vw;
    if (shadow != nullptr) store_bf16x4(shadow + i * 4, pw);
  }
}

// Schedule-free wrapper around sign descent, one fused elementwise pass. The
// parameter buffer holds y (where the gradient was taken), `z` the base
// optimiser's iterate. x is recovered from y and z, z takes the sign step, x
// moves towards the new z by the averaging weight c, and y is re-extrapolated:
//   x  = y + (1 - 1/beta)(z - y);  z' = z - lr sign(g);
//   x' = x + c (z' - x);           y' = x' + (1 - beta)(z' - x').
struct SignumArgs { float lr, beta, c; };

__device__ __forceinline__ float signum_sf_update(float y, float& z, float g, const SignumArgs a) {
  const float x = y + (1.f - 1.f / a.beta) * (z - y);
  const float sgn = (g > 0.f) ? 1.f : ((g < 0.f) ? -1.f : 0.f);
  z = z - a.lr * sgn;
  const float xn = x + a.c * (z - x);
  return xn + (1.f - a.beta) * (z - xn);
}

__global__ void __launch_bounds__(256)
signum_sf_vec_kernel(float4* __restrict__ p, float4* __restrict__ z, const float4* __restrict__ g,
                     int64_t n4, SignumArgs a, __nv_bfloat16* __restrict__ shadow) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4;
       i += (int64_t)gridDim.x * blockDim.x) {
    float4 y = p[i], zz = z[i];
    const float4 gg = g[i];
    y.x = signum_sf_update(y.x, zz.x, gg.x, a);
    y.y = signum_sf_update(y.y, zz.y, gg.y, a);
    y.z = signum_sf_update(y.z, zz.z, gg.z, a);
    y.w = signum_sf_update(y.w, zz.w, gg.w, a);
    p[i] = y;
    z[i] = zz;
    if (shadow != nullptr) store_bf16x4(shadow + 4 * i, y);
  }
}

__global__ void __launch_bounds__(256)
signum_sf_kernel(float* __restrict__ p, float* __restrict__ z, const float* __restrict__ g, int64_t n,
                 SignumArgs a, __nv_bfloat16* __restrict__ shadow) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    float zz = z[i];
    const float y = signum_sf_update(p[i], zz, g[i], a);
    p[i] = y;
    z[i] = zz;
    if (shadow != nullptr) shadow[i] = __float2bfloat16_rn(y);
  }
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
  cudaStream_t st = sc::as_stream(stream);
  __nv_bfloat16* shadow = static_cast<__nv_bfloat16*>(shadow_bf16);
  const bool vec = D % 4 == 0 && sc::aligned(W, 16) && (shadow == nullptr || sc::aligned(shadow, 8));
  if (vec && D <= 1024) normalize_rows_vec_kernel<1><<<(unsigned)M, kRowThreads, 0, st>>>(W, D, eps, shadow);
  else if (vec && D <= 2048) normalize_rows_vec_kernel<2><<<(unsigned)M, kRowThreads, 0, st>>>(W, D, eps, shadow);
  else if (vec && D <= 4096) normalize_rows_vec_kernel<4><<<(unsigned)M, kRowThreads, 0, st>>>(W, D, eps, shadow);
  else normalize_rows_kernel<<<(unsigned)M, kRowThreads, 0, st>>>(W, D, eps, shadow);
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
  const bool al = sc::aligned(p, 16) && sc::aligned(g, 16) && sc::aligned(m, 16) && sc::aligned(v, 16) &&
                  (shadow == nullptr || sc::aligned(shadow, 8));
  if (project) {
    const bool vec = al && D % 4 == 0;
    if (vec && D <= 1024) adam_rows_project_vec_kernel<1><<<(unsigned)M, kRowThreads, 0, st>>>(p, g, m, v, D, a, shadow);
    else if (vec && D <= 2048) adam_rows_project_vec_kernel<2><<<(unsigned)M, kRowThreads, 0, st>>>(p, g, m, v, D, a, shadow);
    else if (vec && D <= 4096) adam_rows_project_vec_kernel<4><<<(unsigned)M, kRowThreads, 0, st>>>(p, g, m, v, D, a, shadow);
    else adam_rows_project_kernel<<<(unsigned)M, kRowThreads, 0, st>>>(p, g, m, v, D, a, shadow);
  } else if (al && (M * D) % 4 == 0) {
    adam_flat_vec_kernel<<<flat_grid(M * D / 4), 256, 0, st>>>(p, g, m, v, M * D / 4, a, shadow);
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

extern "C" int sc_signum_schedulefree(float* p, float* z, const float* g, int64_t n, float lr,
                                      float momentum, float ckp1, void* shadow_bf16, void* stream) {
  SC_REQUIRE(n >= 0, "sc_signum_schedulefree: bad size");
  if (n == 0) return SC_OK;
  SC_REQUIRE(p && z && g, "sc_signum_schedulefree: null pointer");
  SC_REQUIRE(momentum > 0.f && momentum <= 1.f, "sc_signum_schedulefree: momentum %g outside (0, 1]", (double)momentum);
  SignumArgs a;
  a.lr = lr; a.beta = momentum; a.c = ckp1;
  __nv_bfloat16* shadow = static_cast<__nv_bfloat16*>(shadow_bf16);
  cudaStream_t st = sc::as_stream(stream);
  const bool vec = n % 4 == 0 && sc::aligned(p, 16) && sc::aligned(z, 16) && sc::aligned(g, 16) &&
                   (shadow == nullptr || sc::aligned(shadow, 8));
  if (vec)
    signum_sf_vec_kernel<<<flat_grid(n / 4), 256, 0, st>>>(reinterpret_cast<float4*>(p), reinterpret_cast<float4*>(z),
                                                          reinterpret_cast<const float4*>(g), n / 4, a, shadow);
  else
    signum_sf_kernel<<<flat_grid(n), 256, 0, st>>>(p, z, g, n, a, shadow);
  SC_CHECK_LAUNCH("sc_signum_schedulefree");
  return SC_OK;
}

extern "C" int sc_project_rows(float* g, const float* w, int64_t M, int64_t D, void* stream) {
  SC_REQUIRE(M >= 0 && D > 0 && M <= 0x7fffffffLL, "sc_project_rows: bad shape");
  if (M == 0) return SC_OK;
  SC_REQUIRE(g && w, "sc_project_rows: null pointer");
  project_rows_kernel<<<(unsigned)M, kRowThreads, 0, sc::as_stream(stream)>>>(g, w, D);
  SC_CHECK_LAUNCH("sc_project_rows");
  return SC_OK;
}
