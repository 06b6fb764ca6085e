// General bf16 GEMM on the 5th-generation tensor cores:
//
//   out[m,n] = act(alpha * sum_k A[m,k] B[n,k] + beta * Cin[m,n] + bias[n])
//
// A [M,K] and B [N,K] are row-major bf16 (both K-major, the layout of every
// product on this path: x W^T, X X^T, A A^T, (B X^T^T) with an explicit
// transpose, x W_skip^T). Same pipeline as the fused encoder: persistent CTA per
// SM, warp 0 feeds a TMA ring (128x64 and 256x64 tiles, 128-byte swizzle), warp
// 1 issues tcgen05.mma into one of two 128x256 fp32 accumulators in tensor
// memory, warps 2-5 drain the other one and write the result rows. Used for
// the dense pre-activations, the skip connection and Muon's Newton-Schulz.
#include "tc.cuh"

namespace {

using namespace sc::tc;

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kStages = 4;
constexpr uint32_t kStageBytes = (BM + BN) * BK * 2;
constexpr int kGroupM = 16;  // row blocks that share a sweep over the column tiles (L2 reuse)

enum { kWaitEmpty = 201, kWaitFull = 202, kWaitTmemEmpty = 203, kWaitTmemFull = 204 };

struct Params {
  void* out;
  const void* cin;
  const float* bias;
  int32_t* status;
  int64_t M, N, K;
  float alpha, beta;
  int out_bf16, cin_bf16, relu;
  int tiles_m, tiles_n;
  int n_tiles;
  int cin_aligned;  // Cin is 16-byte aligned
  int symmetric;  // A and B are the same matrix: tiles wholly below the diagonal are not computed
  void* out_t;    // optional second copy of the result, transposed ([N, M])
};

// Column tile j (256 wide) of a symmetric product needs the row tiles (128 high) that
// reach the diagonal or lie above it: 128 i <= 256 j + 255, i.e. i <= 2 j + 1.
__host__ __device__ __forceinline__ int sym_rows_in_col(int tiles_m, int j) {
  return tiles_m < 2 * j + 2 ? tiles_m : 2 * j + 2;
}

__device__ __forceinline__ void tile_coords(const Params& p, int t, int& tm, int& tn) {
  if (p.symmetric) {
    int j = 0, acc = 0;
    for (;; ++j) {
      const int cnt = sym_rows_in_col(p.tiles_m, j);
      if (t < acc + cnt) break;
      acc += cnt;
    }
    tn = j;
    tm = t - acc;
    return;
  }
  const int per_group = kGroupM * p.tiles_n;
  const int g = t / per_group, rem = t % per_group;
  const int gm = min(kGroupM, p.tiles_m - g * kGroupM);
  tn = rem / gm;
  tm = g * kGroupM + rem % gm;
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const Params p) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)kStages * kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* tfull = bars + 2 * kStages;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  float* tscratch = reinterpret_cast<float*>(smem + (size_t)kStages * kStageBytes + 256);  // 4 x [32][33]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kc_count = (int)((p.K + BK - 1) / BK);
  const int n_tiles = p.n_tiles;

  if (threadIdx.x == 0) {
    prefetch_tensor_map(&tmap_a);
    prefetch_tensor_map(&tmap_b);
    for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull[b], 1); mbar_init(&tempty[b], 4); }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coords(p, t, tm, tn);
        for (int kc = 0; kc < kc_count; ++kc) {
          if (!mbar_wait(&empty[stage], phase ^ 1, p.status, kWaitEmpty)) { ok = false; break; }
          unsigned char* sa = smem + (size_t)stage * kStageBytes;
          mbar_arrive_expect_tx(&full[stage], kStageBytes);
          tma_load_2d(sa, &tmap_a, kc * BK, tm * BM, &full[stage]);
          tma_load_2d(sa + BM * BK * 2, &tmap_b, kc * BK, tn * BN, &full[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN);
      int stage = 0, buf = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&tempty[buf], acc_phase ^ 1, p.status, kWaitTmemEmpty)) break;
        fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)buf * BN;
        for (int kc = 0; kc < kc_count; ++kc) {
          if (!mbar_wait(&full[stage], phase, p.status, kWaitFull)) { ok = false; break; }
          fence_after_sync();
          const uint32_t sa = smem_u32(smem + (size_t)stage * kStageBytes);
          const uint64_t adesc = make_smem_desc_sw128(sa);
          const uint64_t bdesc = make_smem_desc_sw128(sa + BM * BK * 2);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk)
            mma_bf16(d_tmem, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc,
                     (kc | kk) != 0 ? 1u : 0u);
          mma_commit(&empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mma_commit(&tfull[buf]);
        buf ^= 1;
        if (buf == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    int buf = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) {
      int tm, tn;
      tile_coords(p, t, tm, tn);
      const bool ok = __all_sync(0xffffffffu, mbar_wait(&tfull[buf], acc_phase, p.status, kWaitTmemFull));
      if (!ok) break;
      fence_after_sync();
      const int64_t gm = (int64_t)tm * BM + row;
      const int64_t col0 = (int64_t)tn * BN;
      const uint32_t taddr = tmem_base + (uint32_t)buf * BN + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tmem_ld_wait();
        const int64_t gc = col0 + c * 32;
        if (gm >= p.M || gc >= p.N) continue;
        const int valid = (int)min((int64_t)32, p.N - gc);
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = p.alpha * __uint_as_float(r[i]);
        if (p.cin != nullptr && p.beta != 0.f) {
          if (p.cin_bf16) {
            const __nv_bfloat16* cr = static_cast<const __nv_bfloat16*>(p.cin) + gm * p.N + gc;
            if (valid == 32 && (p.N % 8 == 0) && p.cin_aligned) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                const uint4 pk = *reinterpret_cast<const uint4*>(cr + i);
                const uint32_t w[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                  v[i + 2 * h] = fmaf(p.beta, __uint_as_float(w[h] << 16), v[i + 2 * h]);
                  v[i + 2 * h + 1] = fmaf(p.beta, __uint_as_float(w[h] & 0xffff0000u), v[i + 2 * h + 1]);
                }
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (i < valid) v[i] = fmaf(p.beta, __bfloat162float(cr[i]), v[i]);
            }
          } else {
            const float* cr = static_cast<const float*>(p.cin) + gm * p.N + gc;
            if (valid == 32 && (p.N % 4 == 0) && p.cin_aligned) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                const float4 c4 = *reinterpret_cast<const float4*>(cr + i);
                v[i] = fmaf(p.beta, c4.x, v[i]); v[i + 1] = fmaf(p.beta, c4.y, v[i + 1]);
                v[i + 2] = fmaf(p.beta, c4.z, v[i + 2]); v[i + 3] = fmaf(p.beta, c4.w, v[i + 3]);
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (i < valid) v[i] = fmaf(p.beta, cr[i], v[i]);
            }
          }
        }
        if (p.bias != nullptr) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i < valid) v[i] += __ldg(p.bias + gc + i);
        }
        if (p.relu) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = fmaxf(v[i], 0.f);
        }
        if (p.out_bf16) {
          __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(p.out) + gm * p.N + gc;
          if (valid == 32 && (p.N % 8 == 0)) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 pk;
              pk.x = sc::pack_bf16x2(v[i], v[i + 1]); pk.y = sc::pack_bf16x2(v[i + 2], v[i + 3]);
              pk.z = sc::pack_bf16x2(v[i + 4], v[i + 5]); pk.w = sc::pack_bf16x2(v[i + 6], v[i + 7]);
              *reinterpret_cast<uint4*>(orow + i) = pk;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < valid) orow[i] = __float2bfloat16_rn(v[i]);
          }
        } else {
          float* orow = static_cast<float*>(p.out) + gm * p.N + gc;
          if (valid == 32 && (p.N % 4 == 0)) {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              *reinterpret_cast<float4*>(orow + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < valid) orow[i] = v[i];
          }
        }
        // Transposed copies: element (gm, gc+i) also goes to row gc+i, column gm - of `out`
        // itself when the mirrored tile of a symmetric product is one that is not computed,
        // of `out_t` when a transposed result was asked for. For a fixed i the 32 lanes of a
        // warp write 32 consecutive elements.
        void* tdst = p.out_t;
        int64_t ldt = p.M;
        if (p.symmetric && (((gm >> 8) << 8) + 255 < ((gc >> 7) << 7))) { tdst = p.out; ldt = p.N; }
        if (tdst != nullptr) {
          const int64_t gm0 = (int64_t)tm * BM + q * 32;  // first row of this warp
          if (p.out_bf16 && valid == 32 && gm0 + 32 <= p.M && ldt % 8 == 0) {
            // 32x32 block transposed through this warp's scratch: lane L then owns column
            // gc + L and stores its 32 rows as 64 contiguous bytes
            float* sw = tscratch + (warp - 2) * (32 * 33);
#pragma unroll
            for (int i = 0; i < 32; ++i) sw[i * 33 + lane] = v[i];
            __syncwarp();
            __nv_bfloat16* tp = static_cast<__nv_bfloat16*>(tdst) + (gc + lane) * ldt + gm0;
            const float* sr = sw + lane * 33;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 pk;
              pk.x = sc::pack_bf16x2(sr[i], sr[i + 1]); pk.y = sc::pack_bf16x2(sr[i + 2], sr[i + 3]);
              pk.z = sc::pack_bf16x2(sr[i + 4], sr[i + 5]); pk.w = sc::pack_bf16x2(sr[i + 6], sr[i + 7]);
              *reinterpret_cast<uint4*>(tp + i) = pk;
            }
            __syncwarp();
          } else if (p.out_bf16) {
            __nv_bfloat16* tp = static_cast<__nv_bfloat16*>(tdst) + gc * ldt + gm;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < valid) tp[i * ldt] = __float2bfloat16_rn(v[i]);
          } else {
            float* tp = static_cast<float*>(tdst) + gc * ldt + gm;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < valid) tp[i * ldt] = v[i];
          }
        }
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[buf]);
      buf ^= 1;
      if (buf == 0) acc_phase ^= 1;
    }
  }

  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// out[c, r] = in[r, c] for bf16 matrices (32x32 tiles through shared memory).
__global__ void __launch_bounds__(256)
transpose_bf16_kernel(const __nv_bfloat16* __restrict__ in, int64_t R, int64_t C, __nv_bfloat16* __restrict__ out) {
  __shared__ __nv_bfloat16 tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
  for (int i = ty; i < 32; i += 8)
    if (r0 + i < R && c0 + tx < C) tile[i][tx] = in[(r0 + i) * C + c0 + tx];
  __syncthreads();
  for (int i = ty; i < 32; i += 8)
    if (c0 + i < C && r0 + tx < R) out[(c0 + i) * R + r0 + tx] = tile[tx][i];
}

}  // namespace

extern "C" int sc_gemm_bf16_nt(const void* A_bf16, const void* B_bf16, int64_t M, int64_t N, int64_t K,
                               float alpha, float beta, const void* Cin, int cin_dtype, const float* bias,
                               int relu, void* out, int out_dtype, int symmetric, void* out_t,
                               int32_t* status_word, void* stream) {
  SC_REQUIRE(M > 0 && N > 0 && K > 0, "sc_gemm_bf16_nt: bad shape");
  SC_REQUIRE(!symmetric || (A_bf16 == B_bf16 && M == N && out_t == nullptr && bias == nullptr),
             "sc_gemm_bf16_nt: symmetric needs A == B, M == N, no bias and no out_t");
  SC_REQUIRE(out_t == nullptr || (sc::aligned(out_t, 16) && out_t != out), "sc_gemm_bf16_nt: bad out_t");
  SC_REQUIRE(A_bf16 && B_bf16 && out, "sc_gemm_bf16_nt: null pointer");
  SC_REQUIRE(sc::valid_dtype(out_dtype) && (Cin == nullptr || sc::valid_dtype(cin_dtype)), "sc_gemm_bf16_nt: bad dtype");
  SC_REQUIRE(K % 8 == 0, "sc_gemm_bf16_nt: K=%lld must be a multiple of 8 (16-byte row stride for TMA)", (long long)K);
  SC_REQUIRE(sc::aligned(A_bf16, 16) && sc::aligned(B_bf16, 16) && sc::aligned(out, 16),
             "sc_gemm_bf16_nt: operands must be 16-byte aligned");
  SC_REQUIRE(M < (int64_t(1) << 31) && N < (int64_t(1) << 31) && K < (int64_t(1) << 31), "sc_gemm_bf16_nt: dimension too large");
  CUtensorMap tma, tmb;
  int rc = make_tensor_map_bf16(&tma, A_bf16, (uint64_t)M, (uint64_t)K, BM);
  if (rc != SC_OK) return rc;
  rc = make_tensor_map_bf16(&tmb, B_bf16, (uint64_t)N, (uint64_t)K, BN);
  if (rc != SC_OK) return rc;
  Params p;
  p.out = out; p.cin = Cin; p.bias = bias; p.status = status_word;
  p.M = M; p.N = N; p.K = K; p.alpha = alpha; p.beta = beta;
  p.out_bf16 = out_dtype == SC_BF16; p.cin_bf16 = cin_dtype == SC_BF16; p.relu = relu;
  p.tiles_m = (int)((M + BM - 1) / BM);
  p.tiles_n = (int)((N + BN - 1) / BN);
  p.cin_aligned = sc::aligned(Cin, 16) ? 1 : 0;
  p.symmetric = symmetric ? 1 : 0;
  p.out_t = out_t;
  int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
  if (symmetric) {
    tiles = 0;
    for (int j = 0; j < p.tiles_n; ++j) tiles += sym_rows_in_col(p.tiles_m, j);
  }
  SC_REQUIRE(tiles < (int64_t(1) << 31), "sc_gemm_bf16_nt: too many tiles");
  p.n_tiles = (int)tiles;
  const size_t smem = (size_t)kStages * kStageBytes + 256 + 4 * 32 * 33 * sizeof(float) + 1024;
  SC_CUDA(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  sms -= sc::reserved_sms();
  const int grid = (int)(tiles < sms ? tiles : sms);
  gemm_tc_kernel<<<grid, kThreads, smem, sc::as_stream(stream)>>>(tma, tmb, p);
  SC_CHECK_LAUNCH("sc_gemm_bf16_nt");
  return SC_OK;
}

extern "C" int sc_transpose_bf16(const void* in, int64_t R, int64_t C, void* out, void* stream) {
  SC_REQUIRE(R > 0 && C > 0 && in && out, "sc_transpose_bf16: bad arguments");
  SC_REQUIRE((R + 31) / 32 <= 65535, "sc_transpose_bf16: too many rows for one launch");
  dim3 grid((unsigned)((C + 31) / 32), (unsigned)((R + 31) / 32));
  transpose_bf16_kernel<<<grid, 256, 0, sc::as_stream(stream)>>>(
      static_cast<const __nv_bfloat16*>(in), R, C, static_cast<__nv_bfloat16*>(out));
  SC_CHECK_LAUNCH("sc_transpose_bf16");
  return SC_OK;
}
