// Loss reductions of SparseCoder.forward: total variance of the target and
// squared error, as device scalars (no host synchronisation). All partial sums
// are reduced in a fixed order, so results are run-to-run reproducible.
#include "common.cuh"

namespace {

constexpr int kSlices = 256;               // row slices for the column sums (512: same speed; 1024: slower)
constexpr int kColsumUnroll = 4;           // rows in flight per thread
constexpr int kRedBlocks = 1024;           // partial sums of the flat reductions

// partial[s][d] = sum of w[n] * y[n][d] over the rows n of slice s (w == NULL: 1), D % 4 == 0.
// A CTA owns 1024 consecutive columns (a thread four of them) and walks the rows of its
// slice, so every row is read in 2 KB (bf16) / 4 KB contiguous pieces and a thread's sums
// never leave its registers.
template <typename T>
__global__ void __launch_bounds__(256)
colsum_wide_kernel(const T* __restrict__ y, const float* __restrict__ w, int64_t N, int64_t D,
                   float* __restrict__ partial) {
  const int64_t d = ((int64_t)blockIdx.x * 256 + threadIdx.x) * 4;
  if (d >= D) return;
  const int64_t per = (N + kSlices - 1) / kSlices;
  const int64_t r0 = (int64_t)blockIdx.y * per;
  const int64_t r1 = r0 + per < N ? r0 + per : N;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll kColsumUnroll
  for (int64_t r = r0; r < r1; ++r) {
    const float wr = w != nullptr ? __ldg(w + r) : 1.f;
    const float4 x = sc::load4<T>(y + r * D + d);
    acc.x = fmaf(wr, x.x, acc.x); acc.y = fmaf(wr, x.y, acc.y);
    acc.z = fmaf(wr, x.z, acc.z); acc.w = fmaf(wr, x.w, acc.w);
  }
  *reinterpret_cast<float4*>(partial + (int64_t)blockIdx.y * D + d) = acc;
}

// partial[s][d] = sum of w[n] * y[n][d] over the rows n of slice s (w == NULL: 1).
// VEC = 4: each lane owns four consecutive columns (8/16-byte loads); VEC = 1
// serves widths that are not a multiple of four.
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const T* __restrict__ y, const float* __restrict__ w, int64_t N, int64_t D,
                      float* __restrict__ partial) {
  __shared__ float s_acc[8][32 * VEC + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t d = ((int64_t)blockIdx.x * 32 + lane) * VEC;
  const int64_t per = (N + kSlices - 1) / kSlices;
  const int64_t r0 = (int64_t)blockIdx.y * per;
  const int64_t r1 = r0 + per < N ? r0 + per : N;
  float acc[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
  if (d < D) {
#pragma unroll 4
    for (int64_t r = r0 + warp; r < r1; r += 8) {
      const float wr = w != nullptr ? __ldg(w + r) : 1.f;
      if (wr == 0.f) continue;
      if constexpr (VEC == 4) {
        const float4 x = sc::load4<T>(y + r * D + d);
        acc[0] = fmaf(wr, x.x, acc[0]); acc[1] = fmaf(wr, x.y, acc[1]);
        acc[2] = fmaf(wr, x.z, acc[2]); acc[3] = fmaf(wr, x.w, acc[3]);
      } else {
        acc[0] = fmaf(wr, sc::load1<T>(y + r * D + d), acc[0]);
      }
    }
  }
#pragma unroll
  for (int v = 0; v < VEC; ++v) s_acc[warp][lane * VEC + v] = acc[v];
  __syncthreads();
  for (int c = threadIdx.x; c < 32 * VEC; c += blockDim.x) {
    float t = 0.f;
#pragma unroll
    for (int ww = 0; ww < 8; ++ww) t += s_acc[ww][c];
    const int64_t dd = (int64_t)blockIdx.x * 32 * VEC + c;
    if (dd < D) partial[(int64_t)blockIdx.y * D + dd] = t;
  }
}

template <typename T>
void launch_colsum(const T* y, const float* w, int64_t N, int64_t D, float* partial, cudaStream_t st) {
  if (D % 4 == 0 && sc::aligned(y, 16) && sc::aligned(partial, 16)) {
    dim3 grid((unsigned)((D + 1023) / 1024), kSlices);
    colsum_wide_kernel<T><<<grid, 256, 0, st>>>(y, w, N, D, partial);
  } else {
    dim3 grid((unsigned)((D + 31) / 32), kSlices);
    colsum_partial_kernel<T, 1><<<grid, 256, 0, st>>>(y, w, N, D, partial);
  }
}

// out[d] = scale * sum_s partial[s][d]
__global__ void colsum_finish_kernel(const float* __restrict__ partial, float scale, int64_t D,
                                     float* __restrict__ out) {
  int64_t d = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (d >= D) return;
  float t = 0.f;
  for (int s = 0; s < kSlices; ++s) t += partial[(int64_t)s * D + d];
  out[d] = t * scale;
}

// block partials of sum((a[i] - b[i % D])^2) when BROADCAST, else sum((a[i]-b[i])^2)
template <bool BROADCAST, typename TA = float>
__global__ void __launch_bounds__(256)
sqdiff_partial_kernel(const TA* __restrict__ a, const float* __restrict__ b, int64_t total,
                      int64_t D, float* __restrict__ diff, float* __restrict__ partial) {
  __shared__ float scratch[33];
  float acc = 0.f;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    float e = sc::load1<TA>(a + i) - __ldg(b + (BROADCAST ? i % D : i));
    if (diff != nullptr) diff[i] = e;
    acc = fmaf(e, e, acc);
  }
  acc = sc::block_sum(acc, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}

// Row-wise form of the broadcast case for D % 4 == 0: a block walks whole rows, every thread
// keeps its columns' means in registers (no index arithmetic per element, 8/16-byte loads).
template <typename TA>
__global__ void __launch_bounds__(256)
sqdiff_rows_kernel(const TA* __restrict__ a, const float* __restrict__ mean, int64_t N, int64_t D,
                   float* __restrict__ partial) {
  __shared__ float scratch[33];
  float acc = 0.f;
  for (int64_t c0 = (int64_t)threadIdx.x * 4; c0 < D; c0 += 1024) {
    const float4 mu = __ldg(reinterpret_cast<const float4*>(mean + c0));
#pragma unroll 4
    for (int64_t r = blockIdx.x; r < N; r += gridDim.x) {
      const float4 v = sc::load4<TA>(a + r * D + c0);
      const float ex = v.x - mu.x, ey = v.y - mu.y, ez = v.z - mu.z, ew = v.w - mu.w;
      acc = fmaf(ex, ex, acc); acc = fmaf(ey, ey, acc); acc = fmaf(ez, ez, acc); acc = fmaf(ew, ew, acc);
    }
  }
  acc = sc::block_sum(acc, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}

__global__ void __launch_bounds__(256)
final_sum_kernel(const float* __restrict__ partial, int n, float* __restrict__ out) {
  __shared__ float scratch[33];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) acc += partial[i];
  acc = sc::block_sum(acc, scratch);
  if (threadIdx.x == 0) *out = acc;
}

int flat_blocks(int64_t total) {
  int64_t b = (total + 255) / 256;
  return (int)(b < kRedBlocks ? (b > 0 ? b : 1) : kRedBlocks);
}

}  // namespace

extern "C" size_t sc_loss_workspace_bytes(int64_t D) {
  if (D < 0) return 0;
  return ((size_t)kSlices * D + (size_t)D + kRedBlocks) * sizeof(float);
}

extern "C" int sc_total_variance(const void* y, int y_dtype, int64_t N, int64_t D, float* tv, void* ws,
                                 size_t ws_bytes, void* stream) {
  SC_REQUIRE(N > 0 && D > 0, "sc_total_variance: bad shape");
  SC_REQUIRE(sc::valid_dtype(y_dtype), "sc_total_variance: bad dtype");
  SC_REQUIRE(y && tv && ws, "sc_total_variance: null pointer");
  if (ws_bytes < sc_loss_workspace_bytes(D))
    return sc::fail(SC_ERR_WORKSPACE, "sc_total_variance: workspace %zu < %zu", ws_bytes,
                    sc_loss_workspace_bytes(D));
  cudaStream_t st = sc::as_stream(stream);
  float* partial = static_cast<float*>(ws);
  float* mean = partial + (size_t)kSlices * D;
  float* red = mean + D;
  using bf16 = __nv_bfloat16;
  if (y_dtype == SC_F32) launch_colsum<float>(static_cast<const float*>(y), nullptr, N, D, partial, st);
  else launch_colsum<bf16>(static_cast<const bf16*>(y), nullptr, N, D, partial, st);
  SC_CHECK_LAUNCH("colsum_partial");
  colsum_finish_kernel<<<(unsigned)((D + 255) / 256), 256, 0, st>>>(partial, 1.f / (float)N, D, mean);
  SC_CHECK_LAUNCH("colsum_finish");
  int blocks = flat_blocks(N * D);
  if (D % 4 == 0 && sc::aligned(y, 16)) {
    blocks = (int)(N < kRedBlocks ? N : kRedBlocks);
    if (y_dtype == SC_F32)
      sqdiff_rows_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(y), mean, N, D, red);
    else
      sqdiff_rows_kernel<bf16><<<blocks, 256, 0, st>>>(static_cast<const bf16*>(y), mean, N, D, red);
  } else if (y_dtype == SC_F32) {
    sqdiff_partial_kernel<true, float><<<blocks, 256, 0, st>>>(static_cast<const float*>(y), mean, N * D, D, nullptr, red);
  } else {
    sqdiff_partial_kernel<true, bf16><<<blocks, 256, 0, st>>>(static_cast<const bf16*>(y), mean, N * D, D, nullptr, red);
  }
  SC_CHECK_LAUNCH("sqdiff_partial");
  final_sum_kernel<<<1, 256, 0, st>>>(red, blocks, tv);
  SC_CHECK_LAUNCH("final_sum");
  return SC_OK;
}

extern "C" int sc_sq_err(const float* a, const float* b, int64_t n, float* diff, float* sse,
                         void* ws, size_t ws_bytes, void* stream) {
  SC_REQUIRE(n > 0, "sc_sq_err: bad size");
  SC_REQUIRE(a && b && sse && ws, "sc_sq_err: null pointer");
  if (ws_bytes < kRedBlocks * sizeof(float))
    return sc::fail(SC_ERR_WORKSPACE, "sc_sq_err: workspace %zu < %zu", ws_bytes,
                    kRedBlocks * sizeof(float));
  cudaStream_t st = sc::as_stream(stream);
  float* red = static_cast<float*>(ws);
  const int blocks = flat_blocks(n);
  sqdiff_partial_kernel<false><<<blocks, 256, 0, st>>>(a, b, n, 1, diff, red);
  SC_CHECK_LAUNCH("sqdiff_partial");
  final_sum_kernel<<<1, 256, 0, st>>>(red, blocks, sse);
  SC_CHECK_LAUNCH("final_sum");
  return SC_OK;
}

extern "C" int sc_weighted_colsum(const void* Y, int y_dtype, const float* w, int64_t R, int64_t D,
                                  float* out, void* ws, size_t ws_bytes, void* stream) {
  SC_REQUIRE(R > 0 && D > 0, "sc_weighted_colsum: bad shape");
  SC_REQUIRE(Y && out && ws, "sc_weighted_colsum: null pointer");
  SC_REQUIRE(sc::valid_dtype(y_dtype), "sc_weighted_colsum: bad dtype");
  if (ws_bytes < sc_loss_workspace_bytes(D))
    return sc::fail(SC_ERR_WORKSPACE, "sc_weighted_colsum: workspace %zu < %zu", ws_bytes,
                    sc_loss_workspace_bytes(D));
  cudaStream_t st = sc::as_stream(stream);
  float* partial = static_cast<float*>(ws);
  if (y_dtype == SC_F32) launch_colsum<float>(static_cast<const float*>(Y), w, R, D, partial, st);
  else launch_colsum<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(Y), w, R, D, partial, st);
  SC_CHECK_LAUNCH("colsum_partial");
  colsum_finish_kernel<<<(unsigned)((D + 255) / 256), 256, 0, st>>>(partial, 1.f, D, out);
  SC_CHECK_LAUNCH("colsum_finish");
  return SC_OK;
}
