// Elementwise passes of the Muon step around the Newton-Schulz products
// (sparsify/muon.py:43-181): momentum + Nesterov + bf16 cast + Frobenius norm in
// one pass, the normalisation fused with the transpose that the iteration
// needs anyway, and weight decay + update + bf16 copy in one pass.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kMomentumBlocks = 148 * 8;

// torch.lerp(a, b, w): the two forms torch switches between at w = 0.5.
__device__ __forceinline__ float torch_lerp(float a, float b, float w) {
  return w < 0.5f ? a + w * (b - a) : b - (b - a) * (1.f - w);
}

__device__ __forceinline__ float bf16_round(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// buf = lerp(buf, g, 1 - beta); u = nesterov ? lerp(g, buf, beta) : buf; out = bf16(u);
// partial[block] = sum of out^2 (of the rounded values, as a norm of the bf16 tensor sees them).
__global__ void __launch_bounds__(256)
muon_momentum_kernel(const float* __restrict__ g, float* __restrict__ buf, int64_t n, float beta,
                     int nesterov, __nv_bfloat16* __restrict__ out, float* __restrict__ partial) {
  __shared__ float scratch[33];
  float ss = 0.f;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float gi = g[i];
    const float b = torch_lerp(buf[i], gi, 1.f - beta);
    buf[i] = b;
    const float u = nesterov ? torch_lerp(gi, b, beta) : b;
    const __nv_bfloat16 r = __float2bfloat16_rn(u);
    out[i] = r;
    const float rf = __bfloat162float(r);
    ss = fmaf(rf, rf, ss);
  }
  ss = sc::block_sum(ss, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = ss;
}

__global__ void __launch_bounds__(256)
muon_momentum_vec_kernel(const float4* __restrict__ g, float4* __restrict__ buf, int64_t n4, float beta,
                         int nesterov, uint2* __restrict__ out, float* __restrict__ partial) {
  __shared__ float scratch[33];
  float ss = 0.f;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float4 gi = g[i];
    float4 b = buf[i];
    b.x = torch_lerp(b.x, gi.x, 1.f - beta); b.y = torch_lerp(b.y, gi.y, 1.f - beta);
    b.z = torch_lerp(b.z, gi.z, 1.f - beta); b.w = torch_lerp(b.w, gi.w, 1.f - beta);
    buf[i] = b;
    float4 u = b;
    if (nesterov) {
      u.x = torch_lerp(gi.x, b.x, beta); u.y = torch_lerp(gi.y, b.y, beta);
      u.z = torch_lerp(gi.z, b.z, beta); u.w = torch_lerp(gi.w, b.w, beta);
    }
    uint2 pk;
    pk.x = sc::pack_bf16x2(u.x, u.y);
    pk.y = sc::pack_bf16x2(u.z, u.w);
    out[i] = pk;
    const float r0 = __uint_as_float(pk.x << 16), r1 = __uint_as_float(pk.x & 0xffff0000u);
    const float r2 = __uint_as_float(pk.y << 16), r3 = __uint_as_float(pk.y & 0xffff0000u);
    ss = fmaf(r0, r0, ss); ss = fmaf(r1, r1, ss); ss = fmaf(r2, r2, ss); ss = fmaf(r3, r3, ss);
  }
  ss = sc::block_sum(ss, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = ss;
}

__global__ void __launch_bounds__(1024)
sum_fixed_kernel(const float* __restrict__ partial, int n, float* __restrict__ out) {
  __shared__ float scratch[33];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) acc += partial[i];
  acc = sc::block_sum(acc, scratch);
  if (threadIdx.x == 0) *out = acc;
}

// X / (||X||_F + 1e-7) as torch evaluates it on a bf16 tensor (norm rounded to bf16, the sum
// with 1e-7 rounded to bf16, the quotient rounded to bf16), written in the input's
// orientation and / or transposed. 32x32 tiles through shared memory.
__global__ void __launch_bounds__(256)
scale_transpose_kernel(const __nv_bfloat16* __restrict__ in, int64_t R, int64_t C, const float* __restrict__ sumsq,
                       __nv_bfloat16* __restrict__ out_s, __nv_bfloat16* __restrict__ out_t) {
  __shared__ __nv_bfloat16 tile[32][33];
  float denom = 1.f;
  if (sumsq != nullptr) denom = bf16_round(bf16_round(sqrtf(*sumsq)) + 1e-7f);
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
  for (int i = ty; i < 32; i += 8) {
    if (r0 + i < R && c0 + tx < C) {
      const __nv_bfloat16 v = __float2bfloat16_rn(__bfloat162float(in[(r0 + i) * C + c0 + tx]) / denom);
      tile[i][tx] = v;
      if (out_s != nullptr) out_s[(r0 + i) * C + c0 + tx] = v;
    }
  }
  if (out_t == nullptr) return;
  __syncthreads();
  for (int i = ty; i < 32; i += 8)
    if (c0 + i < C && r0 + tx < R) out_t[(c0 + i) * R + r0 + tx] = tile[tx][i];
}

// p = p * decay - alpha * upd, optional bf16 copy of the result.
__global__ void __launch_bounds__(256)
muon_apply_kernel(float* __restrict__ p, const __nv_bfloat16* __restrict__ upd, int64_t n, float decay,
                  float alpha, __nv_bfloat16* __restrict__ shadow) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float v = p[i] * decay - alpha * __bfloat162float(upd[i]);
    p[i] = v;
    if (shadow != nullptr) shadow[i] = __float2bfloat16_rn(v);
  }
}

__global__ void __launch_bounds__(256)
muon_apply_vec_kernel(float4* __restrict__ p, const uint2* __restrict__ upd, int64_t n4, float decay,
                      float alpha, uint2* __restrict__ shadow) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4;
       i += (int64_t)gridDim.x * blockDim.x) {
    float4 v = p[i];
    const uint2 u = upd[i];
    v.x = v.x * decay - alpha * __uint_as_float(u.x << 16);
    v.y = v.y * decay - alpha * __uint_as_float(u.x & 0xffff0000u);
    v.z = v.z * decay - alpha * __uint_as_float(u.y << 16);
    v.w = v.w * decay - alpha * __uint_as_float(u.y & 0xffff0000u);
    p[i] = v;
    if (shadow != nullptr) {
      uint2 pk;
      pk.x = sc::pack_bf16x2(v.x, v.y);
      pk.y = sc::pack_bf16x2(v.z, v.w);
      shadow[i] = pk;
    }
  }
}

int flat_blocks(int64_t total) {
  const int64_t b = (total + 255) / 256;
  return (int)(b < 148 * 16 ? (b > 0 ? b : 1) : 148 * 16);
}

}  // namespace

extern "C" size_t sc_muon_workspace_bytes(void) { return (size_t)kMomentumBlocks * sizeof(float); }

extern "C" int sc_muon_momentum(const float* g, float* buf, int64_t n, float beta, int nesterov,
                                void* out_bf16, float* sumsq, void* ws, size_t ws_bytes, void* stream) {
  SC_REQUIRE(n > 0, "sc_muon_momentum: bad size");
  SC_REQUIRE(g && buf && out_bf16 && sumsq && ws, "sc_muon_momentum: null pointer");
  SC_REQUIRE(beta >= 0.f && beta < 1.f, "sc_muon_momentum: momentum %g outside [0, 1)", (double)beta);
  if (ws_bytes < sc_muon_workspace_bytes())
    return sc::fail(SC_ERR_WORKSPACE, "sc_muon_momentum: workspace %zu < %zu", ws_bytes, sc_muon_workspace_bytes());
  float* partial = static_cast<float*>(ws);
  cudaStream_t st = sc::as_stream(stream);
  const bool vec = n % 4 == 0 && sc::aligned(g, 16) && sc::aligned(buf, 16) && sc::aligned(out_bf16, 8);
  if (vec)
    muon_momentum_vec_kernel<<<kMomentumBlocks, 256, 0, st>>>(reinterpret_cast<const float4*>(g),
        reinterpret_cast<float4*>(buf), n / 4, beta, nesterov, static_cast<uint2*>(out_bf16), partial);
  else
    muon_momentum_kernel<<<kMomentumBlocks, 256, 0, st>>>(g, buf, n, beta, nesterov,
        static_cast<__nv_bfloat16*>(out_bf16), partial);
  SC_CHECK_LAUNCH("sc_muon_momentum");
  sum_fixed_kernel<<<1, 1024, 0, st>>>(partial, kMomentumBlocks, sumsq);
  SC_CHECK_LAUNCH("sc_muon_momentum(sum)");
  return SC_OK;
}

extern "C" int sc_scale_transpose_bf16(const void* in, int64_t R, int64_t C, const float* sumsq,
                                       void* out_scaled, void* out_t, void* stream) {
  SC_REQUIRE(R > 0 && C > 0 && in && (out_scaled || out_t), "sc_scale_transpose_bf16: bad arguments");
  SC_REQUIRE((R + 31) / 32 <= 65535, "sc_scale_transpose_bf16: too many rows for one launch");
  dim3 grid((unsigned)((C + 31) / 32), (unsigned)((R + 31) / 32));
  scale_transpose_kernel<<<grid, 256, 0, sc::as_stream(stream)>>>(
      static_cast<const __nv_bfloat16*>(in), R, C, sumsq, static_cast<__nv_bfloat16*>(out_scaled),
      static_cast<__nv_bfloat16*>(out_t));
  SC_CHECK_LAUNCH("sc_scale_transpose_bf16");
  return SC_OK;
}

extern "C" int sc_muon_apply(float* p, const void* upd_bf16, int64_t n, float decay, float alpha,
                             void* shadow_bf16, void* stream) {
  SC_REQUIRE(n > 0 && p && upd_bf16, "sc_muon_apply: bad arguments");
  cudaStream_t st = sc::as_stream(stream);
  const bool vec = n % 4 == 0 && sc::aligned(p, 16) && sc::aligned(upd_bf16, 8) &&
                   (shadow_bf16 == nullptr || sc::aligned(shadow_bf16, 8));
  if (vec)
    muon_apply_vec_kernel<<<flat_blocks(n / 4), 256, 0, st>>>(reinterpret_cast<float4*>(p),
        static_cast<const uint2*>(upd_bf16), n / 4, decay, alpha, static_cast<uint2*>(shadow_bf16));
  else
    muon_apply_kernel<<<flat_blocks(n), 256, 0, st>>>(p, static_cast<const __nv_bfloat16*>(upd_bf16), n, decay,
        alpha, static_cast<__nv_bfloat16*>(shadow_bf16));
  SC_CHECK_LAUNCH("sc_muon_apply");
  return SC_OK;
}
