// Per-latent row accumulate: the sparse weight gradients of one training step.
//
// One CTA per latent m. Its CSR segment lists the (token, slot) pairs that
// selected m; the CTA sums coef * vec[token,:] over the segment in fp32 and
// writes the full row of the gradient (zeros when the latent did not fire), so
// the [M,D] gradient needs no separate zero fill and no atomics, and the sum
// order is fixed by the CSR. The decoder gradient (A) and the encoder gradient
// (B) share the segment walk; a bias gradient is the plain sum of the coefficients.
#include "common.cuh"

namespace {

constexpr int kAccThreads = 256;
constexpr int kNch = 4;  // 4-wide column groups per thread per sweep

template <typename TA, typename TB, bool HAS_B>
__global__ void __launch_bounds__(kAccThreads)
rows_accumulate_kernel(const int32_t* __restrict__ row_ptr, const int32_t* __restrict__ entries,
                       int k, const float* __restrict__ coefA, const TA* __restrict__ vecA,
                       float* __restrict__ gradA, float* __restrict__ gbiasA,
                       const float* __restrict__ coefB, const TB* __restrict__ vecB,
                       float* __restrict__ gradB, float* __restrict__ gbiasB, int64_t D,
                       int64_t lat_begin) {
  const int64_t m = lat_begin + blockIdx.x;
  const int32_t lo = row_ptr[m], hi = row_ptr[m + 1];

  if (gbiasA != nullptr && threadIdx.x == 0) {
    float s = 0.f;
    for (int32_t p = lo; p < hi; ++p) s += coefA[entries[p]];
    gbiasA[m] = s;
  }
  if (HAS_B && gbiasB != nullptr && threadIdx.x == 32) {
    float s = 0.f;
    for (int32_t p = lo; p < hi; ++p) s += coefB[entries[p]];
    gbiasB[m] = s;
  }

  const int64_t sweep = (int64_t)kAccThreads * 4 * kNch;
  for (int64_t base = 0; base < D; base += sweep) {
    float4 accA[kNch], accB[kNch];
    int64_t col[kNch];
#pragma unroll
    for (int c = 0; c < kNch; ++c) {
      accA[c] = make_float4(0.f, 0.f, 0.f, 0.f);
      accB[c] = make_float4(0.f, 0.f, 0.f, 0.f);
      col[c] = base + ((int64_t)c * kAccThreads + threadIdx.x) * 4;
    }
#pragma unroll 2
    for (int32_t p = lo; p < hi; ++p) {
      const int32_t e = entries[p];
      const int64_t n = e / k;
      const float ca = coefA[e];
      const TA* ra = vecA + n * D;
      float cb = 0.f;
      const TB* rb = nullptr;
      if (HAS_B) { cb = coefB[e]; rb = vecB + n * D; }
#pragma unroll
      for (int c = 0; c < kNch; ++c) {
        if (col[c] < D) {
          float4 a = sc::load4<TA>(ra + col[c]);
          accA[c].x = fmaf(ca, a.x, accA[c].x);
          accA[c].y = fmaf(ca, a.y, accA[c].y);
          accA[c].z = fmaf(ca, a.z, accA[c].z);
          accA[c].w = fmaf(ca, a.w, accA[c].w);
          if (HAS_B) {
            float4 b = sc::load4<TB>(rb + col[c]);
            accB[c].x = fmaf(cb, b.x, accB[c].x);
            accB[c].y = fmaf(cb, b.y, accB[c].y);
            accB[c].z = fmaf(cb, b.z, accB[c].z);
            accB[c].w = fmaf(cb, b.w, accB[c].w);
          }
        }
      }
    }
#pragma unroll
    for (int c = 0; c < kNch; ++c) {
      if (col[c] < D) {
        __stcs(reinterpret_cast<float4*>(gradA + m * D + col[c]), accA[c]);
        if (HAS_B) __stcs(reinterpret_cast<float4*>(gradB + m * D + col[c]), accB[c]);
      }
    }
  }
}

// out[m] = sum of coef[e] over the CSR entries e of latent m
__global__ void __launch_bounds__(256)
segment_sum_kernel(const int32_t* __restrict__ row_ptr, const int32_t* __restrict__ entries,
                   const float* __restrict__ coef, int64_t M, float* __restrict__ out) {
  const int64_t m = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (m >= M) return;
  float s = 0.f;
  for (int32_t p = row_ptr[m]; p < row_ptr[m + 1]; ++p) s += coef[entries[p]];
  out[m] = s;
}

template <typename TA, typename TB>
int launch(const int32_t* row_ptr, const int32_t* entries, int k, const float* coefA,
           const void* vecA, float* gradA, float* gbiasA, const float* coefB, const void* vecB,
           float* gradB, float* gbiasB, int64_t D, int64_t lat_begin, int64_t nlat, cudaStream_t st) {
  dim3 grid((unsigned)nlat), block(kAccThreads);
  if (gradB != nullptr) {
    rows_accumulate_kernel<TA, TB, true><<<grid, block, 0, st>>>(
        row_ptr, entries, k, coefA, static_cast<const TA*>(vecA), gradA, gbiasA, coefB,
        static_cast<const TB*>(vecB), gradB, gbiasB, D, lat_begin);
  } else {
    rows_accumulate_kernel<TA, TB, false><<<grid, block, 0, st>>>(
        row_ptr, entries, k, coefA, static_cast<const TA*>(vecA), gradA, gbiasA, nullptr, nullptr,
        nullptr, nullptr, D, lat_begin);
  }
  SC_CHECK_LAUNCH("sc_rows_accumulate");
  return SC_OK;
}

}  // namespace

extern "C" int sc_rows_accumulate(const int32_t* row_ptr, const int32_t* entries, int k,
                                  const float* coefA, const void* vecA, int vecA_dtype,
                                  float* gradA, float* gbiasA, const float* coefB,
                                  const void* vecB, int vecB_dtype, float* gradB, float* gbiasB,
                                  int64_t M, int64_t D, int64_t lat_begin, int64_t lat_end,
                                  void* stream) {
  SC_REQUIRE(M > 0 && D > 0 && k > 0, "sc_rows_accumulate: bad shape");
  SC_REQUIRE(0 <= lat_begin && lat_begin <= lat_end && lat_end <= M,
             "sc_rows_accumulate: latent range [%lld,%lld) outside [0,%lld)", (long long)lat_begin,
             (long long)lat_end, (long long)M);
  if (lat_begin == lat_end) return SC_OK;
  SC_REQUIRE(row_ptr && entries && coefA && vecA && gradA, "sc_rows_accumulate: null pointer");
  SC_REQUIRE(sc::valid_dtype(vecA_dtype), "sc_rows_accumulate: bad vecA dtype");
  SC_REQUIRE(D % 4 == 0, "sc_rows_accumulate: D=%lld must be a multiple of 4", (long long)D);
  SC_REQUIRE(sc::aligned(vecA, 16) && sc::aligned(gradA, 16), "sc_rows_accumulate: A pointers must be 16-byte aligned");
  if (gradB != nullptr) {
    SC_REQUIRE(coefB && vecB && sc::valid_dtype(vecB_dtype), "sc_rows_accumulate: B operands missing");
    SC_REQUIRE(sc::aligned(vecB, 16) && sc::aligned(gradB, 16), "sc_rows_accumulate: B pointers must be 16-byte aligned");
  } else {
    SC_REQUIRE(gbiasB == nullptr, "sc_rows_accumulate: gbiasB needs the B operands");
    vecB_dtype = SC_F32;
  }
  cudaStream_t st = sc::as_stream(stream);
  const int64_t nlat = lat_end - lat_begin;
  SC_REQUIRE(nlat <= 0x7fffffffLL, "sc_rows_accumulate: too many latents in one call");
  using bf16 = __nv_bfloat16;
  if (vecA_dtype == SC_F32 && vecB_dtype == SC_F32)
    return launch<float, float>(row_ptr, entries, k, coefA, vecA, gradA, gbiasA, coefB, vecB, gradB, gbiasB, D, lat_begin, nlat, st);
  if (vecA_dtype == SC_F32 && vecB_dtype == SC_BF16)
    return launch<float, bf16>(row_ptr, entries, k, coefA, vecA, gradA, gbiasA, coefB, vecB, gradB, gbiasB, D, lat_begin, nlat, st);
  if (vecA_dtype == SC_BF16 && vecB_dtype == SC_F32)
    return launch<bf16, float>(row_ptr, entries, k, coefA, vecA, gradA, gbiasA, coefB, vecB, gradB, gbiasB, D, lat_begin, nlat, st);
  return launch<bf16, bf16>(row_ptr, entries, k, coefA, vecA, gradA, gbiasA, coefB, vecB, gradB, gbiasB, D, lat_begin, nlat, st);
}

extern "C" int sc_csr_segment_sum(const int32_t* row_ptr, const int32_t* entries, const float* coef,
                                  int64_t M, float* out, void* stream) {
  SC_REQUIRE(M > 0, "sc_csr_segment_sum: bad shape");
  SC_REQUIRE(row_ptr && entries && coef && out, "sc_csr_segment_sum: null pointer");
  segment_sum_kernel<<<(unsigned)((M + 255) / 256), 256, 0, sc::as_stream(stream)>>>(row_ptr, entries, coef, M, out);
  SC_CHECK_LAUNCH("sc_csr_segment_sum");
  return SC_OK;
}
