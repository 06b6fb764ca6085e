// Shape-generic encoder path: dense pre-activations with fp32 FMA, then an exact
// per-row top-k (radix select) or groupmax over the dense rows. It serves every
// shape and dtype the tensor-core path does not (odd D, fp32 operands, k above
// its list capacity), the public `pre_acts` output, and the AuxK / Multi-TopK
// selections that rank all M pre-activations of a row.
#include "common.cuh"

namespace {

// ---- x' = x - b_dec --------------------------------------------------------
template <typename TI, typename TO>
__global__ void prep_input_kernel(const TI* __restrict__ x, const float* __restrict__ b,
                                  int64_t total, int64_t D, TO* __restrict__ out) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    float v = sc::load1<TI>(x + i);
    if (b != nullptr) v -= __ldg(b + (i % D));
    if constexpr (sizeof(TO) == 2) out[i] = __float2bfloat16_rn(v);
    else out[i] = v;
  }
}

// Row-wise form for D % 4 == 0 and 16-byte aligned rows: four elements per thread, the bias
// slice in registers, no per-element index arithmetic.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
prep_input_rows_kernel(const TI* __restrict__ x, const float* __restrict__ b, int64_t N, int64_t D,
                       TO* __restrict__ out) {
  for (int64_t c0 = (int64_t)threadIdx.x * 4; c0 < D; c0 += 1024) {
    const float4 bb = b != nullptr ? __ldg(reinterpret_cast<const float4*>(b + c0)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int64_t r = blockIdx.x; r < N; r += gridDim.x) {
      float4 v = sc::load4<TI>(x + r * D + c0);
      v.x -= bb.x; v.y -= bb.y; v.z -= bb.z; v.w -= bb.w;
      if constexpr (sizeof(TO) == 2) {
        uint2 pk;
        pk.x = sc::pack_bf16x2(v.x, v.y);
        pk.y = sc::pack_bf16x2(v.z, v.w);
        *reinterpret_cast<uint2*>(out + r * D + c0) = pk;
      } else {
        *reinterpret_cast<float4*>(out + r * D + c0) = v;
      }
    }
  }
}

// ---- dense relu(x W^T + b) ---------------------------------------------------
constexpr int TM = 64, TN = 64, TK = 16;

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256)
preacts_dense_kernel(const TX* __restrict__ x, const TW* __restrict__ W,
                     const float* __restrict__ bias, int64_t N, int64_t D, int64_t M,
                     TO* __restrict__ pre) {
  __shared__ float sx[TK][TM + 1];
  __shared__ float sw[TK][TN + 1];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int64_t row0 = (int64_t)blockIdx.y * TM, col0 = (int64_t)blockIdx.x * TN;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < D; k0 += TK) {
    for (int i = threadIdx.x; i < TM * TK; i += 256) {
      int r = i / TK, c = i % TK;
      int64_t gr = row0 + r, gc = k0 + c;
      sx[c][r] = (gr < N && gc < D) ? sc::load1<TX>(x + gr * D + gc) : 0.f;
    }
    for (int i = threadIdx.x; i < TN * TK; i += 256) {
      int r = i / TK, c = i % TK;
      int64_t gr = col0 + r, gc = k0 + c;
      sw[c][r] = (gr < M && gc < D) ? sc::load1<TW>(W + gr * D + gc) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = sx[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = sw[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int64_t r = row0 + ty * 4 + i;
    if (r >= N) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int64_t c = col0 + tx * 4 + j;
      if (c >= M) continue;
      float v = acc[i][j] + (bias != nullptr ? __ldg(bias + c) : 0.f);
      v = fmaxf(v, 0.f);
      if constexpr (sizeof(TO) == 2) pre[r * M + c] = __float2bfloat16_rn(v);
      else pre[r * M + c] = v;
    }
  }
}

// ---- exact per-row top-k by radix select ------------------------------------
// Keys order like the floats they come from; masked-out columns get key 0,
// below every real value.
__device__ __forceinline__ uint32_t order_key(float v) {
  uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

constexpr int kSelThreads = 512;
constexpr int64_t kSelCacheMax = 40960;  // rows of up to this many columns keep their keys in shared memory

// One CTA per row, four 8-bit digit passes over the row's keys, then one pass that emits.
// Post-ReLU rows are full of equal values (zeros), so every shared-memory atomic is aggregated
// per warp first (threads with the same digit elect one to add their count), and rows that
// fit keep their keys in shared memory, so that global memory is read once.
__global__ void __launch_bounds__(kSelThreads)
topk_rows_kernel(const float* __restrict__ pre, int64_t M, int k,
                 const uint8_t* __restrict__ col_mask, float* __restrict__ top_vals,
                 int64_t* __restrict__ top_idx, __nv_bfloat16* __restrict__ dense_out, int cache_keys) {
  extern __shared__ uint32_t s_keys[];  // [M] when cache_keys
  __shared__ uint32_t hist[256];
  __shared__ uint32_t s_prefix, s_need, s_out, s_eq;
  const float* row = pre + (int64_t)blockIdx.x * M;
  // dense_out != NULL: instead of (values, indices) the row is written back densely as bf16
  // with everything outside its top k set to zero
  float* ov = dense_out == nullptr ? top_vals + (int64_t)blockIdx.x * k : nullptr;
  int64_t* oi = dense_out == nullptr ? top_idx + (int64_t)blockIdx.x * k : nullptr;
  __nv_bfloat16* od = dense_out == nullptr ? nullptr : dense_out + (int64_t)blockIdx.x * M;
  const int lane = threadIdx.x & 31;
  const unsigned lanes_below = (1u << lane) - 1u;

  auto key_at = [&](int64_t c, bool first) -> uint32_t {
    if (cache_keys && !first) return s_keys[c];
    const uint32_t key = (col_mask == nullptr || col_mask[c]) ? order_key(row[c]) : 0u;
    if (cache_keys) s_keys[c] = key;
    return key;
  };

  uint32_t prefix = 0, prefix_mask = 0, need = (uint32_t)k;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int64_t base = 0; base < M; base += blockDim.x) {  // whole warps stay together
      const int64_t c = base + threadIdx.x;
      bool active = false;
      uint32_t digit = 0;
      if (c < M) {
        const uint32_t key = key_at(c, shift == 24);
        active = (key & prefix_mask) == prefix;
        digit = (key >> shift) & 0xffu;
      }
      const unsigned act = __ballot_sync(0xffffffffu, active);
      if (active) {
        const unsigned peers = __match_any_sync(act, digit);
        if (lane == __ffs(peers) - 1) atomicAdd(&hist[digit], (uint32_t)__popc(peers));
      }
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      // Which digit holds the need-th largest key: lane l owns bins 8l .. 8l+7; a suffix scan over the
      // lanes finds the one lane whose bins straddle `need`, which then walks its eight bins.
      uint32_t h[8], mine = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) { h[j] = hist[lane * 8 + j]; mine += h[j]; }
      uint32_t at_or_above = mine;  // becomes the count in this lane's bins and all higher ones
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_down_sync(0xffffffffu, at_or_above, o);
        if (lane + o < 32) at_or_above += t;
      }
      uint32_t cum = at_or_above - mine;  // keys in higher bins than this lane's
      if (cum < need && need <= at_or_above) {
        int d = 7;
        for (; d > 0; --d) {
          if (cum + h[d] >= need) break;
          cum += h[d];
        }
        s_prefix = prefix | ((uint32_t)(lane * 8 + d) << shift);
        s_need = need - cum;  // still to take among keys sharing the longer prefix
      }
    }
    __syncthreads();
    prefix = s_prefix;
    need = s_need;
    prefix_mask |= 0xffu << shift;
    __syncthreads();
  }
  // prefix is now the key of the k-th largest element; `need` of the elements
  // equal to it belong to the result.
  if (threadIdx.x == 0) { s_out = 0; s_eq = 0; }
  __syncthreads();
  for (int64_t base = 0; base < M; base += blockDim.x) {
    const int64_t c = base + threadIdx.x;
    const bool valid = c < M;
    float v = 0.f;
    uint32_t key = 0u;
    if (valid) {
      v = row[c];
      key = cache_keys ? s_keys[c] : ((col_mask == nullptr || col_mask[c]) ? order_key(v) : 0u);
    }
    bool take = valid && key > prefix;
    // ties with the k-th value: one shared counter, advanced once per warp
    const bool eq = valid && key == prefix;
    const unsigned eq_mask = __ballot_sync(0xffffffffu, eq);
    if (eq_mask != 0u) {
      uint32_t first = 0;
      if (lane == __ffs(eq_mask) - 1) first = atomicAdd(&s_eq, (uint32_t)__popc(eq_mask));
      first = __shfl_sync(0xffffffffu, first, __ffs(eq_mask) - 1);
      if (eq) take = first + (uint32_t)__popc(eq_mask & lanes_below) < need;
    }
    if (od != nullptr) {
      if (valid) od[c] = __float2bfloat16_rn(take ? v : 0.f);
    } else {
      const unsigned take_mask = __ballot_sync(0xffffffffu, take);
      if (take_mask != 0u) {
        uint32_t first = 0;
        if (lane == __ffs(take_mask) - 1) first = atomicAdd(&s_out, (uint32_t)__popc(take_mask));
        first = __shfl_sync(0xffffffffu, first, __ffs(take_mask) - 1);
        const uint32_t slot = first + (uint32_t)__popc(take_mask & lanes_below);
        if (take && slot < (uint32_t)k) { ov[slot] = v; oi[slot] = c; }
      }
    }
  }
}

int launch_topk_rows(const float* pre, int64_t N, int64_t M, int k, const uint8_t* col_mask, float* top_vals,
                     int64_t* top_idx, __nv_bfloat16* dense_out, cudaStream_t st) {
  const int cache = M <= kSelCacheMax ? 1 : 0;
  const size_t smem = cache ? (size_t)M * sizeof(uint32_t) : 0;
  if (smem > 48 * 1024)
    SC_CUDA(cudaFuncSetAttribute(topk_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  topk_rows_kernel<<<(unsigned)N, kSelThreads, smem, st>>>(pre, M, k, col_mask, top_vals, top_idx, dense_out, cache);
  return SC_OK;
}

// ---- groupmax ---------------------------------------------------------------
__global__ void __launch_bounds__(256)
groupmax_rows_kernel(const float* __restrict__ pre, int64_t M, int k,
                     float* __restrict__ top_vals, int64_t* __restrict__ top_idx) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int64_t g = M / k;
  const float* row = pre + (int64_t)blockIdx.x * M;
  for (int grp = warp; grp < k; grp += nwarps) {
    float best = -INFINITY;
    int64_t besti = 0x7fffffffffffffffLL;
    for (int64_t c = lane; c < g; c += 32) {
      float v = row[grp * g + c];
      if (v > best || (v == best && c < besti)) { best = v; besti = c; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, o);
      int64_t oi = __shfl_xor_sync(0xffffffffu, besti, o);
      if (ob > best || (ob == best && oi < besti)) { best = ob; besti = oi; }
    }
    if (lane == 0) {
      top_vals[(int64_t)blockIdx.x * k + grp] = best;
      top_idx[(int64_t)blockIdx.x * k + grp] = grp * g + besti;
    }
  }
}

template <typename TX, typename TW>
int launch_dense(const void* x, const void* W, const float* bias, int64_t N, int64_t D,
                 int64_t M, void* pre, int pre_dtype, cudaStream_t st) {
  dim3 grid((unsigned)((M + TN - 1) / TN), (unsigned)((N + TM - 1) / TM)), block(256);
  if (pre_dtype == SC_F32)
    preacts_dense_kernel<TX, TW, float><<<grid, block, 0, st>>>(
        static_cast<const TX*>(x), static_cast<const TW*>(W), bias, N, D, M, static_cast<float*>(pre));
  else
    preacts_dense_kernel<TX, TW, __nv_bfloat16><<<grid, block, 0, st>>>(
        static_cast<const TX*>(x), static_cast<const TW*>(W), bias, N, D, M,
        static_cast<__nv_bfloat16*>(pre));
  SC_CHECK_LAUNCH("sc_preacts_dense");
  return SC_OK;
}

}  // namespace

extern "C" int sc_prep_input(const void* x, int x_dtype, const float* b_dec, int64_t N,
                             int64_t D, void* out, int out_dtype, void* stream) {
  SC_REQUIRE(sc::valid_dtype(x_dtype) && sc::valid_dtype(out_dtype), "sc_prep_input: bad dtype");
  SC_REQUIRE(N >= 0 && D > 0, "sc_prep_input: bad shape");
  if (N == 0) return SC_OK;
  SC_REQUIRE(x && out, "sc_prep_input: null pointer");
  const int64_t total = N * D;
  int blocks = (int)((total + 255) / 256 < 148 * 32 ? (total + 255) / 256 : 148 * 32);
  cudaStream_t st = sc::as_stream(stream);
  using bf16 = __nv_bfloat16;
  const bool rows = D % 4 == 0 && sc::aligned(x, 16) && sc::aligned(out, 16) && (b_dec == nullptr || sc::aligned(b_dec, 16));
  if (rows) blocks = (int)(N < 148 * 16 ? N : 148 * 16);
#define SC_PREP(TI, TO)                                                                                  \
  do {                                                                                                   \
    if (rows) prep_input_rows_kernel<TI, TO><<<blocks, 256, 0, st>>>((const TI*)x, b_dec, N, D, (TO*)out); \
    else prep_input_kernel<TI, TO><<<blocks, 256, 0, st>>>((const TI*)x, b_dec, total, D, (TO*)out);       \
  } while (0)
  if (x_dtype == SC_F32 && out_dtype == SC_F32) SC_PREP(float, float);
  else if (x_dtype == SC_F32) SC_PREP(float, bf16);
  else if (out_dtype == SC_F32) SC_PREP(bf16, float);
  else SC_PREP(bf16, bf16);
#undef SC_PREP
  SC_CHECK_LAUNCH("sc_prep_input");
  return SC_OK;
}

extern "C" int sc_preacts_dense(const void* x, int x_dtype, const void* W, int w_dtype,
                                const float* bias, int64_t N, int64_t D, int64_t M, void* pre,
                                int pre_dtype, void* stream) {
  SC_REQUIRE(sc::valid_dtype(x_dtype) && sc::valid_dtype(w_dtype) && sc::valid_dtype(pre_dtype),
             "sc_preacts_dense: bad dtype");
  SC_REQUIRE(N >= 0 && D > 0 && M > 0, "sc_preacts_dense: bad shape");
  if (N == 0) return SC_OK;
  SC_REQUIRE(x && W && pre, "sc_preacts_dense: null pointer");
  SC_REQUIRE((N + TM - 1) / TM <= 65535, "sc_preacts_dense: N=%lld too large for one launch", (long long)N);
  cudaStream_t st = sc::as_stream(stream);
  using bf16 = __nv_bfloat16;
  if (x_dtype == SC_F32 && w_dtype == SC_F32) return launch_dense<float, float>(x, W, bias, N, D, M, pre, pre_dtype, st);
  if (x_dtype == SC_F32) return launch_dense<float, bf16>(x, W, bias, N, D, M, pre, pre_dtype, st);
  if (w_dtype == SC_F32) return launch_dense<bf16, float>(x, W, bias, N, D, M, pre, pre_dtype, st);
  return launch_dense<bf16, bf16>(x, W, bias, N, D, M, pre, pre_dtype, st);
}

extern "C" int sc_topk_rows(const float* pre, int64_t N, int64_t M, int k,
                            const uint8_t* col_mask, float* top_vals, int64_t* top_idx,
                            void* stream) {
  SC_REQUIRE(N >= 0 && M > 0 && k > 0, "sc_topk_rows: bad shape");
  SC_REQUIRE(k <= M, "sc_topk_rows: k=%d exceeds M=%lld", k, (long long)M);
  if (N == 0) return SC_OK;
  SC_REQUIRE(pre && top_vals && top_idx, "sc_topk_rows: null pointer");
  SC_REQUIRE(N <= 0x7fffffffLL, "sc_topk_rows: N too large");
  int rc = launch_topk_rows(pre, N, M, k, col_mask, top_vals, top_idx, nullptr, sc::as_stream(stream));
  if (rc != SC_OK) return rc;
  SC_CHECK_LAUNCH("sc_topk_rows");
  return SC_OK;
}

extern "C" int sc_topk_mask_rows(const float* pre, int64_t N, int64_t M, int k, const uint8_t* col_mask,
                                 void* out_bf16, void* stream) {
  SC_REQUIRE(N >= 0 && M > 0 && k > 0, "sc_topk_mask_rows: bad shape");
  SC_REQUIRE(k <= M, "sc_topk_mask_rows: k=%d exceeds M=%lld", k, (long long)M);
  if (N == 0) return SC_OK;
  SC_REQUIRE(pre && out_bf16, "sc_topk_mask_rows: null pointer");
  SC_REQUIRE(N <= 0x7fffffffLL, "sc_topk_mask_rows: N too large");
  int rc = launch_topk_rows(pre, N, M, k, col_mask, nullptr, nullptr, static_cast<__nv_bfloat16*>(out_bf16),
                            sc::as_stream(stream));
  if (rc != SC_OK) return rc;
  SC_CHECK_LAUNCH("sc_topk_mask_rows");
  return SC_OK;
}

extern "C" int sc_groupmax_rows(const float* pre, int64_t N, int64_t M, int k, float* top_vals,
                                int64_t* top_idx, void* stream) {
  SC_REQUIRE(N >= 0 && M > 0 && k > 0, "sc_groupmax_rows: bad shape");
  SC_REQUIRE(M % k == 0, "sc_groupmax_rows: M=%lld must be divisible by k=%d", (long long)M, k);
  if (N == 0) return SC_OK;
  SC_REQUIRE(pre && top_vals && top_idx, "sc_groupmax_rows: null pointer");
  groupmax_rows_kernel<<<(unsigned)N, 256, 0, sc::as_stream(stream)>>>(pre, M, k, top_vals, top_idx);
  SC_CHECK_LAUNCH("sc_groupmax_rows");
  return SC_OK;
}
