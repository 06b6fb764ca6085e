// Sparse weight gradients and the optimiser step in one pass.
//
// One CTA per latent m. It walks the latent's CSR segment like
// rows_accumulate, but keeps both gradient rows (decoder: sum acts * grad_out,
// encoder: sum grad_acts * x') in registers and applies them at once:
//   encoder row: Adam, bf16 shadow refresh;
//   decoder row: removal of the gradient component parallel to the row, Adam,
//                row normalisation for the next forward, bf16 shadow refresh.
// The two [M,D] gradients are therefore never written to or read from HBM, and
// the separate projection and normalisation passes disappear. Valid when no
// other consumer needs the dense gradients (single process, no accumulation).
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kThreads = 256;
// float4 groups per thread (template parameter NV): 4 for rows of up to 4096 floats (64
// registers, four CTAs per SM), 8 for rows of up to 8192 (two CTAs per SM)

struct Hp {
  float lr, beta1, beta2, eps, bc1, bc2_sqrt;
};

__device__ __forceinline__ float adam1(float p, float g, float& m, float& v, const Hp& a) {
  m = m + (g - m) * (1.f - a.beta1);
  v = v * a.beta2 + (1.f - a.beta2) * g * g;
  const float denom = sqrtf(v) / a.bc2_sqrt + a.eps;
  return p - (a.lr / a.bc1) * (m / denom);
}

__device__ __forceinline__ void store_bf16x4(__nv_bfloat16* dst, float4 v) {
  uint2 packed;
  packed.x = sc::pack_bf16x2(v.x, v.y);
  packed.y = sc::pack_bf16x2(v.z, v.w);
  *reinterpret_cast<uint2*>(dst) = packed;
}

struct Args {
  const int32_t* row_ptr;
  const int32_t* entries;
  const float* coefA;
  const float* coefB;
  const float* extraA;       // optional dense gradient rows added to the decoder gradient
  const int32_t* extra_rank; // [M]: row of extraA for latent m, or -1
  float *pA, *mA, *vA, *pB, *mB, *vB;
  __nv_bfloat16 *shadowA, *shadowB;
  int64_t D, M;
  int k;
  int projectA, normalizeA;
  int parts;  // bit 0: decoder (A), bit 1: encoder (B)
  float norm_eps;
  Hp hpA, hpB;
};

// Asks L2 to fetch `bytes` (a multiple of 16, 16-byte aligned) starting at p; no
// register or shared-memory destination, nothing to wait for.
__device__ __forceinline__ void prefetch_l2(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// sum over the CSR segment [lo, hi) of coef[e] * vec[e / k, cols of this thread]
template <typename T, int kNV>
__device__ __forceinline__ void gather_rows(const int32_t* __restrict__ entries, int32_t lo, int32_t hi, int k,
                                            const float* __restrict__ coef, const T* __restrict__ vec, int64_t D,
                                            float4 (&g)[kNV]) {
#pragma unroll
  for (int c = 0; c < kNV; ++c) g[c] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
  for (int32_t p = lo; p < hi; ++p) {
    const int32_t e = entries[p];
    const float cf = coef[e];
    const T* r = vec + (int64_t)(e / k) * D;
#pragma unroll
    for (int c = 0; c < kNV; ++c) {
      const int col = (c * kThreads + threadIdx.x) * 4;
      if (col < D) {
        const float4 x = sc::load4<T>(r + col);
        g[c].x = fmaf(cf, x.x, g[c].x); g[c].y = fmaf(cf, x.y, g[c].y);
        g[c].z = fmaf(cf, x.z, g[c].z); g[c].w = fmaf(cf, x.w, g[c].w);
      }
    }
  }
}

// The two matrices are handled one after the other (encoder, then decoder) so that
// only one gradient row is live at a time: 64 registers, four CTAs per SM.
template <typename TA, typename TB, int kNV>
__global__ void __launch_bounds__(kThreads, kNV == 4 ? 4 : 2)
rows_adam_kernel(const TA* __restrict__ vecA, const TB* __restrict__ vecB, const Args a) {
  __shared__ float scratch[33];
  const int64_t D = a.D;
  const bool doA = (a.parts & 1) != 0, doB = (a.parts & 2) != 0;
  // one CTA per latent, or (grid smaller than M) a persistent CTA striding over the latents
  for (int64_t m = blockIdx.x; m < a.M; m += gridDim.x) {
    const int64_t off = m * D;
#ifndef SC_NO_L2_PREFETCH
    // The parameter and moment rows are needed only after the gather below, whose loads
    // depend on one another (row_ptr -> entries -> rows): start them towards L2 now, so
    // that the three 4*D-byte streams travel while the gather waits for its own data.
    if (threadIdx.x < 6) {
      const int t = threadIdx.x;
      const float* row = t == 0 ? a.pB : t == 1 ? a.mB : t == 2 ? a.vB : t == 3 ? a.pA : t == 4 ? a.mA : a.vA;
      if (t < 3 ? doB : doA) prefetch_l2(row + off, (uint32_t)(D * sizeof(float)));
    }
#endif
    const int32_t lo = a.row_ptr[m], hi = a.row_ptr[m + 1];
    float4 g[kNV];

    if (doB) {  // ---- encoder row: Adam ----
      gather_rows<TB, kNV>(a.entries, lo, hi, a.k, a.coefB, vecB, D, g);
#pragma unroll
      for (int c = 0; c < kNV; ++c) {
        const int col = (c * kThreads + threadIdx.x) * 4;
        if (col < D) {
          float4 pw = *reinterpret_cast<const float4*>(a.pB + off + col);
          float4 mw = *reinterpret_cast<const float4*>(a.mB + off + col);
          float4 vw = *reinterpret_cast<const float4*>(a.vB + off + col);
          pw.x = adam1(pw.x, g[c].x, mw.x, vw.x, a.hpB);
          pw.y = adam1(pw.y, g[c].y, mw.y, vw.y, a.hpB);
          pw.z = adam1(pw.z, g[c].z, mw.z, vw.z, a.hpB);
          pw.w = adam1(pw.w, g[c].w, mw.w, vw.w, a.hpB);
          *reinterpret_cast<float4*>(a.pB + off + col) = pw;
          *reinterpret_cast<float4*>(a.mB + off + col) = mw;
          *reinterpret_cast<float4*>(a.vB + off + col) = vw;
          if (a.shadowB != nullptr) store_bf16x4(a.shadowB + off + col, pw);
        }
      }
    }
    if (!doA) continue;

    // ---- decoder row: project, Adam, normalise ----
    gather_rows<TA, kNV>(a.entries, lo, hi, a.k, a.coefA, vecA, D, g);
    if (a.extraA != nullptr) {
      const int32_t r = a.extra_rank[m];
      if (r >= 0) {
#pragma unroll
        for (int c = 0; c < kNV; ++c) {
          const int col = (c * kThreads + threadIdx.x) * 4;
          if (col < D) {
            const float4 x = *reinterpret_cast<const float4*>(a.extraA + (int64_t)r * D + col);
            g[c].x += x.x; g[c].y += x.y; g[c].z += x.z; g[c].w += x.w;
          }
        }
      }
    }
    float4 pw[kNV];
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < kNV; ++c) {
      const int col = (c * kThreads + threadIdx.x) * 4;
      if (col < D) {
        pw[c] = *reinterpret_cast<const float4*>(a.pA + off + col);
        dot += g[c].x * pw[c].x + g[c].y * pw[c].y + g[c].z * pw[c].z + g[c].w * pw[c].w;
      }
    }
    if (a.projectA) dot = sc::block_sum(dot, scratch);
    else dot = 0.f;
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < kNV; ++c) {
      const int col = (c * kThreads + threadIdx.x) * 4;
      if (col < D) {
        float4 mw = *reinterpret_cast<const float4*>(a.mA + off + col);
        float4 vw = *reinterpret_cast<const float4*>(a.vA + off + col);
        const float4 gp = make_float4(g[c].x - dot * pw[c].x, g[c].y - dot * pw[c].y,
                                      g[c].z - dot * pw[c].z, g[c].w - dot * pw[c].w);
        pw[c].x = adam1(pw[c].x, gp.x, mw.x, vw.x, a.hpA);
        pw[c].y = adam1(pw[c].y, gp.y, mw.y, vw.y, a.hpA);
        pw[c].z = adam1(pw[c].z, gp.z, mw.z, vw.z, a.hpA);
        pw[c].w = adam1(pw[c].w, gp.w, mw.w, vw.w, a.hpA);
        *reinterpret_cast<float4*>(a.mA + off + col) = mw;
        *reinterpret_cast<float4*>(a.vA + off + col) = vw;
        ss += pw[c].x * pw[c].x + pw[c].y * pw[c].y + pw[c].z * pw[c].z + pw[c].w * pw[c].w;
      }
    }
    if (a.normalizeA) ss = sc::block_sum(ss, scratch);
    const float denom = sqrtf(ss) + a.norm_eps;  // same division as sc_normalize_rows
#pragma unroll
    for (int c = 0; c < kNV; ++c) {
      const int col = (c * kThreads + threadIdx.x) * 4;
      if (col < D) {
        float4 o = pw[c];
        if (a.normalizeA) o = make_float4(o.x / denom, o.y / denom, o.z / denom, o.w / denom);
        *reinterpret_cast<float4*>(a.pA + off + col) = o;
        if (a.shadowA != nullptr) store_bf16x4(a.shadowA + off + col, o);
      }
    }
  }
}

Hp make_hp(const sc_adam_hparams* h) {
  Hp o;
  o.lr = h->lr; o.beta1 = h->beta1; o.beta2 = h->beta2; o.eps = h->eps;
  o.bc1 = (float)(1.0 - pow((double)h->beta1, (double)h->step));
  o.bc2_sqrt = (float)sqrt(1.0 - pow((double)h->beta2, (double)h->step));
  return o;
}

}  // namespace

extern "C" int sc_rows_adam(const int32_t* row_ptr, const int32_t* entries, int k, const float* coefA,
                            const void* vecA, int vecA_dtype, const float* coefB, const void* vecB,
                            int vecB_dtype, int64_t M, int64_t D, float* pA, float* mA, float* vA,
                            void* shadowA_bf16, int projectA, int normalizeA, float norm_eps,
                            const sc_adam_hparams* hpA, float* pB, float* mB, float* vB,
                            void* shadowB_bf16, const sc_adam_hparams* hpB, const float* extraA,
                            const int32_t* extra_rank, int parts, int max_ctas, void* stream) {
  SC_REQUIRE(M > 0 && D > 0 && k > 0 && M <= 0x7fffffffLL, "sc_rows_adam: bad shape");
  SC_REQUIRE(parts >= 1 && parts <= 3, "sc_rows_adam: parts must be 1 (decoder), 2 (encoder) or 3 (both)");
  SC_REQUIRE(row_ptr && entries && coefA && vecA && coefB && vecB && pA && mA && vA && pB && mB && vB && hpA && hpB,
             "sc_rows_adam: null pointer");
  SC_REQUIRE(sc::valid_dtype(vecA_dtype) && sc::valid_dtype(vecB_dtype), "sc_rows_adam: bad dtype");
  SC_REQUIRE(hpA->step >= 1 && hpB->step >= 1, "sc_rows_adam: step counts from 1");
  if (D % 4 != 0 || D > (int64_t)kThreads * 4 * 8)
    return sc::fail(SC_ERR_UNSUPPORTED, "sc_rows_adam: D=%lld must be a multiple of 4 and at most %d",
                    (long long)D, kThreads * 4 * 8);
  const void* ptrs[] = {vecA, vecB, pA, mA, vA, pB, mB, vB};
  for (const void* q : ptrs) SC_REQUIRE(sc::aligned(q, 16), "sc_rows_adam: pointers must be 16-byte aligned");
  Args a;
  a.row_ptr = row_ptr; a.entries = entries; a.coefA = coefA; a.coefB = coefB;
  a.pA = pA; a.mA = mA; a.vA = vA; a.pB = pB; a.mB = mB; a.vB = vB;
  a.shadowA = static_cast<__nv_bfloat16*>(shadowA_bf16);
  a.shadowB = static_cast<__nv_bfloat16*>(shadowB_bf16);
  SC_REQUIRE((extraA == nullptr) == (extra_rank == nullptr), "sc_rows_adam: extraA and extra_rank go together");
  SC_REQUIRE(extraA == nullptr || sc::aligned(extraA, 16), "sc_rows_adam: extraA must be 16-byte aligned");
  a.extraA = extraA; a.extra_rank = extra_rank;
  a.parts = parts;
  a.M = M;
  a.D = D; a.k = k; a.projectA = projectA; a.normalizeA = normalizeA; a.norm_eps = norm_eps;
  a.hpA = make_hp(hpA); a.hpB = make_hp(hpB);
  cudaStream_t st = sc::as_stream(stream);
  dim3 grid((unsigned)(max_ctas > 0 && max_ctas < M ? max_ctas : M)), block(kThreads);
  using bf16 = __nv_bfloat16;
#define SC_LAUNCH_RA(TA, TB)                                                                          \
  do {                                                                                                \
    if (D <= (int64_t)kThreads * 16)                                                                  \
      rows_adam_kernel<TA, TB, 4><<<grid, block, 0, st>>>((const TA*)vecA, (const TB*)vecB, a);       \
    else                                                                                              \
      rows_adam_kernel<TA, TB, 8><<<grid, block, 0, st>>>((const TA*)vecA, (const TB*)vecB, a);       \
  } while (0)
  if (vecA_dtype == SC_F32 && vecB_dtype == SC_F32) SC_LAUNCH_RA(float, float);
  else if (vecA_dtype == SC_F32) SC_LAUNCH_RA(float, bf16);
  else if (vecB_dtype == SC_F32) SC_LAUNCH_RA(bf16, float);
  else SC_LAUNCH_RA(bf16, bf16);
#undef SC_LAUNCH_RA
  SC_CHECK_LAUNCH("sc_rows_adam");
  return SC_OK;
}
