// Sparse decode as a weighted row gather (embedding bag) and its gradient
// with respect to the per-entry weights.
//
// Forward: one CTA per token; every thread owns a few 4-element column groups
// of the output row and walks the k selected rows of W, so each gathered row is
// read once with fully coalesced 8/16-byte loads and accumulated in fp32 in
// ascending j order (the order of sparsify/xformers.py:22-29).
//
// Backward w.r.t. acts: one CTA per token; the incoming gradient row is staged
// in shared memory once and dotted against each of the k gathered rows.
#include <algorithm>

#include "common.cuh"

namespace {

constexpr int kBagThreads = 256;
constexpr int kBagChunk = 1024;  // entries of one token staged in shared memory at a time

// Stages entries [j0, j0 + kc) of token n; ids outside [0, M) contribute nothing.
__device__ __forceinline__ void stage_entries(const int64_t* __restrict__ idx, const float* __restrict__ acts,
                                              int64_t n, int k, int j0, int kc, int64_t M,
                                              int64_t* s_idx, float* s_act) {
  for (int j = threadIdx.x; j < kc; j += blockDim.x) {
    int64_t r = idx[n * k + j0 + j];
    float a = acts[n * k + j0 + j];
    if (r < 0 || r >= M) { r = 0; a = 0.f; }
    s_idx[j] = r;
    s_act[j] = a;
  }
}

template <typename WT, int VEC>
__global__ void __launch_bounds__(kBagThreads)
bag_fwd_kernel(const int64_t* __restrict__ idx, const float* __restrict__ acts,
               const WT* __restrict__ W, const float* __restrict__ bias, int64_t N,
               int64_t D, int64_t M, int k, float* __restrict__ out) {
  __shared__ int64_t s_idx[kBagChunk];
  __shared__ float s_act[kBagChunk];
  const int64_t n = blockIdx.x;
  const bool one_chunk = k <= kBagChunk;
  if (one_chunk) {
    stage_entries(idx, acts, n, k, 0, k, M, s_idx, s_act);
    __syncthreads();
  }

  constexpr int NCH = 4;  // column groups per thread per sweep
  const int64_t sweep = (int64_t)blockDim.x * VEC * NCH;
  for (int64_t base = 0; base < D; base += sweep) {
    float acc[NCH][VEC];
    int64_t col[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      col[c] = base + ((int64_t)c * blockDim.x + threadIdx.x) * VEC;
#pragma unroll
      for (int v = 0; v < VEC; ++v)
        acc[c][v] = (bias != nullptr && col[c] + v < D) ? __ldg(bias + col[c] + v) : 0.f;
    }
    for (int j0 = 0; j0 < k; j0 += kBagChunk) {
      const int kc = min(kBagChunk, k - j0);
      if (!one_chunk) {
        __syncthreads();
        stage_entries(idx, acts, n, k, j0, kc, M, s_idx, s_act);
        __syncthreads();
      }
#pragma unroll 4
      for (int j = 0; j < kc; ++j) {
        const WT* row = W + s_idx[j] * D;
        const float a = s_act[j];
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          if (col[c] < D) {
            if constexpr (VEC == 4) {
              float4 w = sc::load4<WT>(row + col[c]);
              acc[c][0] = fmaf(a, w.x, acc[c][0]);
              acc[c][1] = fmaf(a, w.y, acc[c][1]);
              acc[c][2] = fmaf(a, w.z, acc[c][2]);
              acc[c][3] = fmaf(a, w.w, acc[c][3]);
            } else {
              acc[c][0] = fmaf(a, sc::load1<WT>(row + col[c]), acc[c][0]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      if (col[c] < D) {
        if constexpr (VEC == 4) {
          *reinterpret_cast<float4*>(out + n * D + col[c]) =
              make_float4(acc[c][0], acc[c][1], acc[c][2], acc[c][3]);
        } else {
          out[n * D + col[c]] = acc[c][0];
        }
      }
    }
  }
}

// Decode fused with the residual: out = bias + sum_j acts W[idx], e = y - out,
// partial[n] = sum_d e^2. Writes whichever of out (fp32), e (fp32), e (bf16) is
// non-null, so the forward needs no separate residual / squared-error / cast pass.
template <typename WT, typename YT>
__global__ void __launch_bounds__(kBagThreads)
decode_residual_kernel(const int64_t* __restrict__ idx, const float* __restrict__ acts,
                       const WT* __restrict__ W, const float* __restrict__ bias, const YT* __restrict__ y,
                       int64_t D, int64_t M, int k, float* __restrict__ out, float* __restrict__ e32,
                       __nv_bfloat16* __restrict__ e16, float* __restrict__ partial) {
  __shared__ int64_t s_idx[kBagChunk];
  __shared__ float s_act[kBagChunk];
  __shared__ float scratch[33];
  const int64_t n = blockIdx.x;
  const bool one_chunk = k <= kBagChunk;
  if (one_chunk) {
    stage_entries(idx, acts, n, k, 0, k, M, s_idx, s_act);
    __syncthreads();
  }
  constexpr int NCH = 4;
  const int64_t sweep = (int64_t)blockDim.x * 4 * NCH;
  float sq = 0.f;
  for (int64_t base = 0; base < D; base += sweep) {
    float4 acc[NCH];
    int64_t col[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      col[c] = base + ((int64_t)c * blockDim.x + threadIdx.x) * 4;
      acc[c] = (bias != nullptr && col[c] < D) ? __ldg(reinterpret_cast<const float4*>(bias + col[c]))
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int j0 = 0; j0 < k; j0 += kBagChunk) {
      const int kc = min(kBagChunk, k - j0);
      if (!one_chunk) {
        __syncthreads();
        stage_entries(idx, acts, n, k, j0, kc, M, s_idx, s_act);
        __syncthreads();
      }
#pragma unroll 4
      for (int j = 0; j < kc; ++j) {
        const WT* row = W + s_idx[j] * D;
        const float a = s_act[j];
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          if (col[c] < D) {
            const float4 w = sc::load4<WT>(row + col[c]);
            acc[c].x = fmaf(a, w.x, acc[c].x); acc[c].y = fmaf(a, w.y, acc[c].y);
            acc[c].z = fmaf(a, w.z, acc[c].z); acc[c].w = fmaf(a, w.w, acc[c].w);
          }
        }
      }
    }
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      if (col[c] < D) {
        const float4 t = sc::load4<YT>(y + n * D + col[c]);
        const float4 e = make_float4(t.x - acc[c].x, t.y - acc[c].y, t.z - acc[c].z, t.w - acc[c].w);
        sq += e.x * e.x + e.y * e.y + e.z * e.z + e.w * e.w;
        if (out != nullptr) *reinterpret_cast<float4*>(out + n * D + col[c]) = acc[c];
        if (e32 != nullptr) *reinterpret_cast<float4*>(e32 + n * D + col[c]) = e;
        if (e16 != nullptr) {
          uint2 pk;
          pk.x = sc::pack_bf16x2(e.x, e.y);
          pk.y = sc::pack_bf16x2(e.z, e.w);
          *reinterpret_cast<uint2*>(e16 + n * D + col[c]) = pk;
        }
      }
    }
  }
  sq = sc::block_sum(sq, scratch);
  if (threadIdx.x == 0) partial[n] = sq;
}

// Decode, residual and the activation gradients' dot products in one pass over the gathered
// rows: besides out / e / sum(e^2) as above, dots[n, j] = e[n] . W[idx[n, j]], which is what
// the backward of the decode needs for d loss / d acts (the gradient of the output is a scalar
// multiple of e). A thread owns VEC columns out of every blockDim.x * VEC; it loads that
// column group of all k (<= KMAX) rows into registers, accumulates the decode, forms e and
// dots it with the very same registers, so every row of W is read from memory once instead
// of once per kernel. W is bf16 (two values per register). The dot uses the residual as it is
// stored: rounded to bf16 when only the bf16 copy is written, so that it agrees with a later
// pass over that copy. Ids outside [0, M) contribute nothing and get a zero dot.
template <int KMAX, int VEC, int TPB, int MINB, typename YT>
__global__ void __launch_bounds__(TPB, MINB)
decode_residual_dots_kernel(const int64_t* __restrict__ idx, const float* __restrict__ acts,
                            const __nv_bfloat16* __restrict__ W, const float* __restrict__ bias,
                            const YT* __restrict__ y, int64_t D, int64_t M, int k, float* __restrict__ out,
                            float* __restrict__ e32, __nv_bfloat16* __restrict__ e16,
                            float* __restrict__ partial, float* __restrict__ dots) {
  static_assert(VEC == 2 || VEC == 4, "two or four bf16 columns per thread");
  constexpr int WORDS = VEC / 2;  // 32-bit registers per row and thread
  constexpr int NW = TPB / 32;
  __shared__ int64_t s_idx[KMAX];
  __shared__ float s_act[KMAX];
  __shared__ float s_part[KMAX][NW + 1];
  __shared__ float scratch[33];
  const int64_t n = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int j = threadIdx.x; j < KMAX; j += blockDim.x) {
    int64_t r = j < k ? idx[n * k + j] : -1;
    float a = j < k ? acts[n * k + j] : 0.f;
    const bool valid = r >= 0 && r < M;
    s_idx[j] = valid ? r : -1;
    s_act[j] = valid ? a : 0.f;
  }
  __syncthreads();
  const bool round_e = e32 == nullptr && e16 != nullptr;
  float dot[KMAX];
#pragma unroll
  for (int j = 0; j < KMAX; ++j) dot[j] = 0.f;
  float sq = 0.f;
  for (int64_t col = (int64_t)threadIdx.x * VEC; col < D; col += (int64_t)blockDim.x * VEC) {
    uint32_t w[KMAX][WORDS];
#pragma unroll
    for (int j = 0; j < KMAX; ++j) {
      const int64_t r = s_idx[j];
      if (r >= 0) {
        if constexpr (VEC == 4) {
          const uint2 q = __ldg(reinterpret_cast<const uint2*>(W + r * D + col));
          w[j][0] = q.x; w[j][1] = q.y;
        } else {
          w[j][0] = __ldg(reinterpret_cast<const uint32_t*>(W + r * D + col));
        }
      } else {
#pragma unroll
        for (int q = 0; q < WORDS; ++q) w[j][q] = 0u;
      }
    }
    float acc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v] = bias != nullptr ? __ldg(bias + col + v) : 0.f;
#pragma unroll
    for (int j = 0; j < KMAX; ++j) {
      const float a = s_act[j];
#pragma unroll
      for (int q = 0; q < WORDS; ++q) {
        acc[2 * q] = fmaf(a, __uint_as_float(w[j][q] << 16), acc[2 * q]);
        acc[2 * q + 1] = fmaf(a, __uint_as_float(w[j][q] & 0xffff0000u), acc[2 * q + 1]);
      }
    }
    float e[VEC];
    if constexpr (VEC == 4) {
      const float4 t = sc::load4<YT>(y + n * D + col);
      e[0] = t.x - acc[0]; e[1] = t.y - acc[1]; e[2] = t.z - acc[2]; e[3] = t.w - acc[3];
    } else {
      e[0] = sc::load1<YT>(y + n * D + col) - acc[0];
      e[1] = sc::load1<YT>(y + n * D + col + 1) - acc[1];
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v) sq = fmaf(e[v], e[v], sq);
    if (out != nullptr) {
#pragma unroll
      for (int v = 0; v < VEC; ++v) out[n * D + col + v] = acc[v];
    }
    if (e32 != nullptr) {
#pragma unroll
      for (int v = 0; v < VEC; ++v) e32[n * D + col + v] = e[v];
    }
    if (e16 != nullptr) {
#pragma unroll
      for (int q = 0; q < WORDS; ++q) {
        const uint32_t pk = sc::pack_bf16x2(e[2 * q], e[2 * q + 1]);
        *reinterpret_cast<uint32_t*>(e16 + n * D + col + 2 * q) = pk;
        if (round_e) {
          e[2 * q] = __uint_as_float(pk << 16);
          e[2 * q + 1] = __uint_as_float(pk & 0xffff0000u);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < KMAX; ++j) {
#pragma unroll
      for (int q = 0; q < WORDS; ++q) {
        dot[j] = fmaf(e[2 * q], __uint_as_float(w[j][q] << 16), dot[j]);
        dot[j] = fmaf(e[2 * q + 1], __uint_as_float(w[j][q] & 0xffff0000u), dot[j]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    const float s = sc::warp_sum(dot[j]);
    if (lane == 0) s_part[j][warp] = s;
  }
  sq = sc::block_sum(sq, scratch);  // contains the barrier that publishes s_part
  if (threadIdx.x == 0) partial[n] = sq;
  for (int j = threadIdx.x; j < k; j += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int q = 0; q < NW; ++q) s += s_part[j][q];
    dots[n * k + j] = s;
  }
}

// Launch shape of decode_residual_dots_kernel for k <= 32: 64 threads, six CTAs per SM (about 170
// registers each) measured fastest - 0.88 ms at 16384 x 32 rows of 8 KB, against 0.91 (128 x 3),
// 1.00 (192 x 2) and 1.17 ms (256 x 2)
constexpr int kDotsThreads = 64;
constexpr int kDotsCtasPerSm = 6;

// Decode (and residual) of bf16 rows with the gathered rows staged in registers: a thread owns
// four columns out of every 4 * TPB and loads that column group of GROUP rows at once (GROUP
// independent 8-byte loads), then accumulates them in ascending j order - the same sums, in the
// same order, as bag_fwd_kernel / decode_residual_kernel, with small CTAs and many loads in
// flight per thread, which is what these gathers of random 8 KB rows run fastest with. y may
// be null (decode only: nothing but `out` is written). Entries are staged in dynamic shared
// memory: (k rounded up to GROUP) * 12 bytes.
template <int GROUP, int TPB, int MINB, typename YT>
__global__ void __launch_bounds__(TPB, MINB)
decode_rows_kernel(const int64_t* __restrict__ idx, const float* __restrict__ acts,
                   const __nv_bfloat16* __restrict__ W, const float* __restrict__ bias,
                   const YT* __restrict__ y, int64_t D, int64_t M, int k, float* __restrict__ out,
                   float* __restrict__ e32, __nv_bfloat16* __restrict__ e16, float* __restrict__ partial) {
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  __shared__ float scratch[33];
  const int kpad = (k + GROUP - 1) / GROUP * GROUP;
  int64_t* s_idx = reinterpret_cast<int64_t*>(dyn_smem);
  float* s_act = reinterpret_cast<float*>(s_idx + kpad);
  const int64_t n = blockIdx.x;
  for (int j = threadIdx.x; j < kpad; j += TPB) {
    int64_t r = j < k ? idx[n * k + j] : -1;
    float a = j < k ? acts[n * k + j] : 0.f;
    const bool valid = r >= 0 && r < M;
    s_idx[j] = valid ? r : -1;
    s_act[j] = valid ? a : 0.f;
  }
  __syncthreads();
  float sq = 0.f;
  for (int64_t col = (int64_t)threadIdx.x * 4; col < D; col += (int64_t)TPB * 4) {
    float4 acc = bias != nullptr ? __ldg(reinterpret_cast<const float4*>(bias + col)) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j0 = 0; j0 < kpad; j0 += GROUP) {
      uint2 w[GROUP];
#pragma unroll
      for (int j = 0; j < GROUP; ++j) {
        const int64_t r = s_idx[j0 + j];
        w[j] = r >= 0 ? __ldg(reinterpret_cast<const uint2*>(W + r * D + col)) : make_uint2(0u, 0u);
      }
#pragma unroll
      for (int j = 0; j < GROUP; ++j) {
        const float a = s_act[j0 + j];
        acc.x = fmaf(a, __uint_as_float(w[j].x << 16), acc.x);
        acc.y = fmaf(a, __uint_as_float(w[j].x & 0xffff0000u), acc.y);
        acc.z = fmaf(a, __uint_as_float(w[j].y << 16), acc.z);
        acc.w = fmaf(a, __uint_as_float(w[j].y & 0xffff0000u), acc.w);
      }
    }
    if (out != nullptr) *reinterpret_cast<float4*>(out + n * D + col) = acc;
    if (y != nullptr) {
      const float4 t = sc::load4<YT>(y + n * D + col);
      const float4 e = make_float4(t.x - acc.x, t.y - acc.y, t.z - acc.z, t.w - acc.w);
      sq += e.x * e.x + e.y * e.y + e.z * e.z + e.w * e.w;
      if (e32 != nullptr) *reinterpret_cast<float4*>(e32 + n * D + col) = e;
      if (e16 != nullptr) {
        uint2 pk;
        pk.x = sc::pack_bf16x2(e.x, e.y);
        pk.y = sc::pack_bf16x2(e.z, e.w);
        *reinterpret_cast<uint2*>(e16 + n * D + col) = pk;
      }
    }
  }
  if (partial != nullptr) {
    sq = sc::block_sum(sq, scratch);
    if (threadIdx.x == 0) partial[n] = sq;
  }
}

// 16 rows at a time, 64 threads, 12 CTAs per SM measured fastest at 16384 x 32 rows of 8 KB (decode
// 0.60 ms, decode + residual 0.64 ms; 32 rows at a time: 0.64 / 0.72 ms; 128 threads: 0.62 / 0.67 ms;
// the kernels with 256 threads and four rows in flight that this replaced: 0.86 / 1.03 ms)
constexpr int kRowsGroup = 16, kRowsThreads = 64, kRowsCtasPerSm = 12;
constexpr int kRowsMaxK = 1024;  // entries of one token staged at once by decode_rows_kernel

template <typename YT>
void launch_decode_rows(const int64_t* idx, const float* acts, const __nv_bfloat16* W, const float* bias,
                        const YT* y, int64_t N, int64_t D, int64_t M, int k, float* out, float* e32,
                        __nv_bfloat16* e16, float* partial, cudaStream_t st) {
  const int kpad = (k + kRowsGroup - 1) / kRowsGroup * kRowsGroup;
  decode_rows_kernel<kRowsGroup, kRowsThreads, kRowsCtasPerSm, YT>
      <<<(unsigned)N, kRowsThreads, (size_t)kpad * 12, st>>>(idx, acts, W, bias, y, D, M, k, out, e32, e16, partial);
}

__global__ void __launch_bounds__(1024)
sum_partials_kernel(const float* __restrict__ partial, int64_t n, float* __restrict__ out) {
  __shared__ float scratch[33];
  float acc = 0.f;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) acc += partial[i];
  acc = sc::block_sum(acc, scratch);
  if (threadIdx.x == 0) *out = acc;
}

template <typename WT, typename GT, int VEC>
__global__ void __launch_bounds__(kBagThreads)
bag_bwd_acts_kernel(const int64_t* __restrict__ idx, const GT* __restrict__ gout,
                    const WT* __restrict__ W, int64_t N, int64_t D, int64_t M, int k,
                    float* __restrict__ gacts) {
  extern __shared__ unsigned char smem_raw[];
  float* s_g = reinterpret_cast<float*>(smem_raw);                 // [Dpad]
  const int64_t Dpad = (D + 3) & ~int64_t(3);
  float* s_part = s_g + Dpad;                                      // [min(k, kBagChunk)][nwarps]
  const int nwarps = blockDim.x >> 5;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t n = blockIdx.x;

  for (int64_t c = threadIdx.x; c < Dpad; c += blockDim.x)
    s_g[c] = c < D ? sc::load1<GT>(gout + n * D + c) : 0.f;
  __syncthreads();

  constexpr int JB = 4;  // rows in flight per iteration
  for (int c0 = 0; c0 < k; c0 += kBagChunk) {
  const int c1 = min(k, c0 + kBagChunk);
  for (int j0 = c0; j0 < c1; j0 += JB) {
    float part[JB];
    const WT* rows[JB];
#pragma unroll
    for (int jj = 0; jj < JB; ++jj) {
      part[jj] = 0.f;
      int64_t r = (j0 + jj < c1) ? idx[n * k + j0 + jj] : -1;
      rows[jj] = (r >= 0 && r < M) ? W + r * D : nullptr;
    }
    for (int64_t c = (int64_t)threadIdx.x * VEC; c < D; c += (int64_t)blockDim.x * VEC) {
#pragma unroll
      for (int jj = 0; jj < JB; ++jj) {
        if (rows[jj] != nullptr) {
          if constexpr (VEC == 4) {
            float4 w = sc::load4<WT>(rows[jj] + c);
            float4 g = *reinterpret_cast<const float4*>(s_g + c);
            part[jj] = fmaf(w.x, g.x, part[jj]);
            part[jj] = fmaf(w.y, g.y, part[jj]);
            part[jj] = fmaf(w.z, g.z, part[jj]);
            part[jj] = fmaf(w.w, g.w, part[jj]);
          } else {
            part[jj] = fmaf(sc::load1<WT>(rows[jj] + c), s_g[c], part[jj]);
          }
        }
      }
    }
#pragma unroll
    for (int jj = 0; jj < JB; ++jj) {
      float s = sc::warp_sum(part[jj]);
      if (lane == 0 && j0 + jj < c1) s_part[(j0 + jj - c0) * nwarps + warp] = s;
    }
  }
  __syncthreads();
  for (int j = c0 + threadIdx.x; j < c1; j += blockDim.x) {
    float s = 0.f;
    for (int w = 0; w < nwarps; ++w) s += s_part[(j - c0) * nwarps + w];
    gacts[n * k + j] = s;
  }
  __syncthreads();
  }
}

}  // namespace

extern "C" int sc_embedding_bag_fwd(const int64_t* idx, const float* acts, const void* W,
                                    int w_dtype, const float* bias, int64_t N, int64_t D,
                                    int64_t M, int k, float* out, void* stream) {
  SC_REQUIRE(sc::valid_dtype(w_dtype), "sc_embedding_bag_fwd: bad w_dtype %d", w_dtype);
  SC_REQUIRE(N >= 0 && D > 0 && M > 0 && k > 0, "sc_embedding_bag_fwd: bad shape N=%lld D=%lld M=%lld k=%d",
             (long long)N, (long long)D, (long long)M, k);
  if (N == 0) return SC_OK;
  SC_REQUIRE(idx && acts && W && out, "sc_embedding_bag_fwd: null pointer");
  SC_REQUIRE(N <= 0x7fffffffLL, "sc_embedding_bag_fwd: N too large");
  const size_t smem = 0;  // the entry staging area is static
  const bool vec = (D % 4 == 0) && sc::aligned(W, 16) && sc::aligned(out, 16) &&
                   (bias == nullptr || sc::aligned(bias, 16));
  dim3 grid((unsigned)N), block(kBagThreads);
  cudaStream_t st = sc::as_stream(stream);
  if (w_dtype == SC_F32) {
    const float* w = static_cast<const float*>(W);
    if (vec) bag_fwd_kernel<float, 4><<<grid, block, smem, st>>>(idx, acts, w, bias, N, D, M, k, out);
    else     bag_fwd_kernel<float, 1><<<grid, block, smem, st>>>(idx, acts, w, bias, N, D, M, k, out);
  } else {
    const __nv_bfloat16* w = static_cast<const __nv_bfloat16*>(W);
    if (vec && k <= kRowsMaxK)
      launch_decode_rows<float>(idx, acts, w, bias, nullptr, N, D, M, k, out, nullptr, nullptr, nullptr, st);
    else if (vec) bag_fwd_kernel<__nv_bfloat16, 4><<<grid, block, smem, st>>>(idx, acts, w, bias, N, D, M, k, out);
    else     bag_fwd_kernel<__nv_bfloat16, 1><<<grid, block, smem, st>>>(idx, acts, w, bias, N, D, M, k, out);
  }
  SC_CHECK_LAUNCH("sc_embedding_bag_fwd");
  return SC_OK;
}

extern "C" int sc_embedding_bag_bwd_acts(const int64_t* idx, const void* grad_out, int g_dtype,
                                         const void* W, int w_dtype, int64_t N, int64_t D,
                                         int64_t M, int k, float* grad_acts, void* stream) {
  SC_REQUIRE(sc::valid_dtype(w_dtype) && sc::valid_dtype(g_dtype), "sc_embedding_bag_bwd_acts: bad dtype");
  SC_REQUIRE(N >= 0 && D > 0 && M > 0 && k > 0, "sc_embedding_bag_bwd_acts: bad shape");
  if (N == 0) return SC_OK;
  SC_REQUIRE(idx && grad_out && W && grad_acts, "sc_embedding_bag_bwd_acts: null pointer");
  SC_REQUIRE(N <= 0x7fffffffLL, "sc_embedding_bag_bwd_acts: N too large");
  const int nwarps = kBagThreads / 32;
  const size_t smem = (size_t)(((D + 3) & ~int64_t(3)) + (int64_t)std::min(k, kBagChunk) * nwarps) * sizeof(float);
  SC_REQUIRE(smem <= 200 * 1024, "sc_embedding_bag_bwd_acts: D=%lld, k=%d need %zu B of shared memory",
             (long long)D, k, smem);
  const bool vec = (D % 4 == 0) && sc::aligned(W, 16);
  dim3 grid((unsigned)N), block(kBagThreads);
  cudaStream_t st = sc::as_stream(stream);
#define SC_LAUNCH_BWD(WT, GT, VEC)                                                          \
  do {                                                                                      \
    auto kern = bag_bwd_acts_kernel<WT, GT, VEC>;                                           \
    if (smem > 48 * 1024)                                                                   \
      SC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    kern<<<grid, block, smem, st>>>(idx, static_cast<const GT*>(grad_out), static_cast<const WT*>(W), N, D, M, k, grad_acts); \
  } while (0)
#define SC_LAUNCH_BWD_G(WT, VEC)                                                            \
  do {                                                                                      \
    if (g_dtype == SC_F32) SC_LAUNCH_BWD(WT, float, VEC); else SC_LAUNCH_BWD(WT, __nv_bfloat16, VEC); \
  } while (0)
  if (w_dtype == SC_F32) {
    if (vec) SC_LAUNCH_BWD_G(float, 4); else SC_LAUNCH_BWD_G(float, 1);
  } else {
    if (vec) SC_LAUNCH_BWD_G(__nv_bfloat16, 4); else SC_LAUNCH_BWD_G(__nv_bfloat16, 1);
  }
#undef SC_LAUNCH_BWD_G
#undef SC_LAUNCH_BWD
  SC_CHECK_LAUNCH("sc_embedding_bag_bwd_acts");
  return SC_OK;
}

extern "C" size_t sc_decode_residual_workspace_bytes(int64_t N) {
  return N > 0 ? (size_t)N * sizeof(float) : 0;
}

extern "C" int sc_decode_residual(const int64_t* idx, const float* acts, const void* W, int w_dtype,
                                  const float* bias, const void* y, int y_dtype, int64_t N, int64_t D,
                                  int64_t M, int k, float* out, float* e_f32, void* e_bf16, float* sse,
                                  void* ws, size_t ws_bytes, void* stream) {
  SC_REQUIRE(sc::valid_dtype(w_dtype) && sc::valid_dtype(y_dtype), "sc_decode_residual: bad dtype");
  SC_REQUIRE(N > 0 && D > 0 && M > 0 && k > 0 && N <= 0x7fffffffLL, "sc_decode_residual: bad shape");
  SC_REQUIRE(idx && acts && W && y && sse && ws, "sc_decode_residual: null pointer");
  SC_REQUIRE(D % 4 == 0, "sc_decode_residual: D=%lld must be a multiple of 4", (long long)D);
  const void* al[] = {W, y, out, e_f32, e_bf16, bias};
  for (const void* q : al) SC_REQUIRE(q == nullptr || sc::aligned(q, 16), "sc_decode_residual: pointers must be 16-byte aligned");
  if (ws_bytes < sc_decode_residual_workspace_bytes(N))
    return sc::fail(SC_ERR_WORKSPACE, "sc_decode_residual: workspace %zu < %zu", ws_bytes,
                    sc_decode_residual_workspace_bytes(N));
  const size_t smem = 0;
  float* partial = static_cast<float*>(ws);
  cudaStream_t st = sc::as_stream(stream);
  dim3 grid((unsigned)N), block(kBagThreads);
  using bf16 = __nv_bfloat16;
  bf16* e16 = static_cast<bf16*>(e_bf16);
#define SC_LAUNCH_DR(WT, YT)                                                                 \
  decode_residual_kernel<WT, YT><<<grid, block, smem, st>>>(idx, acts, static_cast<const WT*>(W), bias, \
      static_cast<const YT*>(y), D, M, k, out, e_f32, e16, partial)
  if (w_dtype == SC_BF16 && k <= kRowsMaxK) {
    if (y_dtype == SC_F32)
      launch_decode_rows<float>(idx, acts, static_cast<const bf16*>(W), bias, static_cast<const float*>(y), N, D, M, k,
                                out, e_f32, e16, partial, st);
    else
      launch_decode_rows<bf16>(idx, acts, static_cast<const bf16*>(W), bias, static_cast<const bf16*>(y), N, D, M, k,
                               out, e_f32, e16, partial, st);
  }
  else if (w_dtype == SC_F32 && y_dtype == SC_F32) SC_LAUNCH_DR(float, float);
  else if (w_dtype == SC_F32) SC_LAUNCH_DR(float, bf16);
  else if (y_dtype == SC_F32) SC_LAUNCH_DR(bf16, float);
  else SC_LAUNCH_DR(bf16, bf16);
#undef SC_LAUNCH_DR
  SC_CHECK_LAUNCH("sc_decode_residual");
  sum_partials_kernel<<<1, 1024, 0, st>>>(partial, N, sse);
  SC_CHECK_LAUNCH("sum_partials");
  return SC_OK;
}

// As sc_decode_residual, and also dots[N, k] = e . W[idx] per selected entry (see the kernel).
// Covers what the training step uses: W in bf16, k <= 32, D a multiple of 4. (With 64 rows in
// registers - two columns per thread - the pass took 2.6-2.9 ms at k = 64 against 1.16 + 1.35 ms
// for the two separate kernels, so wider selections keep those.)
extern "C" int sc_decode_residual_dots(const int64_t* idx, const float* acts, const void* W, int w_dtype,
                                       const float* bias, const void* y, int y_dtype, int64_t N, int64_t D,
                                       int64_t M, int k, float* out, float* e_f32, void* e_bf16, float* sse,
                                       float* dots, void* ws, size_t ws_bytes, void* stream) {
  SC_REQUIRE(sc::valid_dtype(w_dtype) && sc::valid_dtype(y_dtype), "sc_decode_residual_dots: bad dtype");
  SC_REQUIRE(N > 0 && D > 0 && M > 0 && k > 0 && N <= 0x7fffffffLL, "sc_decode_residual_dots: bad shape");
  SC_REQUIRE(idx && acts && W && y && sse && ws && dots, "sc_decode_residual_dots: null pointer");
  if (w_dtype != SC_BF16 || k > 32 || D % 4 != 0)
    return sc::fail(SC_ERR_UNSUPPORTED, "sc_decode_residual_dots: needs bf16 W, k <= 32 and D %% 4 == 0");
  const void* al[] = {W, y, out, e_f32, e_bf16, bias};
  for (const void* q : al) SC_REQUIRE(q == nullptr || sc::aligned(q, 16), "sc_decode_residual_dots: pointers must be 16-byte aligned");
  if (ws_bytes < sc_decode_residual_workspace_bytes(N))
    return sc::fail(SC_ERR_WORKSPACE, "sc_decode_residual_dots: workspace %zu < %zu", ws_bytes,
                    sc_decode_residual_workspace_bytes(N));
  float* partial = static_cast<float*>(ws);
  cudaStream_t st = sc::as_stream(stream);
  dim3 grid((unsigned)N);
  using bf16 = __nv_bfloat16;
  bf16* e16 = static_cast<bf16*>(e_bf16);
  const bf16* w = static_cast<const bf16*>(W);
#define SC_LAUNCH_DRD(KMAX, VEC, TPB, MINB, YT)                                                        \
  decode_residual_dots_kernel<KMAX, VEC, TPB, MINB, YT><<<grid, TPB, 0, st>>>(idx, acts, w, bias,       \
      static_cast<const YT*>(y), D, M, k, out, e_f32, e16, partial, dots)
  if (y_dtype == SC_F32) SC_LAUNCH_DRD(32, 4, kDotsThreads, kDotsCtasPerSm, float);
  else SC_LAUNCH_DRD(32, 4, kDotsThreads, kDotsCtasPerSm, bf16);
#undef SC_LAUNCH_DRD
  SC_CHECK_LAUNCH("sc_decode_residual_dots");
  sum_partials_kernel<<<1, 1024, 0, st>>>(partial, N, sse);
  SC_CHECK_LAUNCH("sum_partials");
  return SC_OK;
}
