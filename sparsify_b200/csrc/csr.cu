// Latent-major CSR of the [N,k] top-k index matrix.
//
// count (atomic histogram) -> exclusive scan -> slot fill (atomic cursors) ->
// per-latent sort of the claimed slots, so that the entries of each latent
// come out in ascending flat position n*k+j whatever order the atomics ran in:
// a warp per latent for segments of up to kSortMax entries, and a second small
// launch that sorts the (rare) longer segments in place, one CTA per segment.
#include <mutex>

#include "common.cuh"

namespace {

constexpr int kSortMax = 2048;

__global__ void csr_count_kernel(const int64_t* __restrict__ idx, int64_t total, int64_t M,
                                 int32_t* __restrict__ counts) {
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
       e += (int64_t)gridDim.x * blockDim.x) {
    int64_t m = idx[e];
    if (m >= 0 && m < M) atomicAdd(&counts[m], 1);
  }
}

// Exclusive scan of counts[0..M) into row_ptr[0..M] (also seeds cursor = row_ptr)
// in three small launches: per-tile sums, a scan of the tile sums by one CTA,
// and the per-tile scans with their offsets.
constexpr int kScanTile = 1024;  // elements per CTA (256 threads x 4)

__global__ void __launch_bounds__(256)
scan_tile_sums_kernel(const int32_t* __restrict__ counts, int64_t M, int32_t* __restrict__ tile_sums) {
  __shared__ int32_t s_warp[8];
  const int64_t base = (int64_t)blockIdx.x * kScanTile + threadIdx.x * 4;
  int32_t v = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) v += base + i < M ? counts[base + i] : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) s_warp[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    int32_t t = 0;
    for (int w = 0; w < 8; ++w) t += s_warp[w];
    tile_sums[blockIdx.x] = t;
  }
}

// In-place exclusive scan of tile_sums[0..n) by one CTA; writes the total to *total.
__global__ void __launch_bounds__(1024)
scan_tile_offsets_kernel(int32_t* __restrict__ tile_sums, int n, int32_t* __restrict__ total) {
  __shared__ int32_t s_warp[32];
  __shared__ int32_t s_carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  for (int base = 0; base < n; base += 1024) {
    const int i = base + threadIdx.x;
    const int32_t v = i < n ? tile_sums[i] : 0;
    int32_t incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t y = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += y;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int32_t w = s_warp[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int32_t y = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += y;
      }
      s_warp[lane] = w;
    }
    __syncthreads();
    const int32_t carry = s_carry;
    const int32_t excl = carry + incl - v + (warp > 0 ? s_warp[warp - 1] : 0);
    if (i < n) tile_sums[i] = excl;
    __syncthreads();
    if (threadIdx.x == 1023) s_carry = carry + s_warp[31];
    __syncthreads();
  }
  if (threadIdx.x == 0) *total = s_carry;
}

__global__ void __launch_bounds__(256)
scan_tiles_kernel(const int32_t* __restrict__ counts, int64_t M, const int32_t* __restrict__ tile_offsets,
                  int32_t* __restrict__ row_ptr, int32_t* __restrict__ cursor) {
  __shared__ int32_t s_warp[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t base = (int64_t)blockIdx.x * kScanTile + threadIdx.x * 4;
  int32_t c[4];
  int32_t v = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) { c[i] = base + i < M ? counts[base + i] : 0; v += c[i]; }
  int32_t incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int32_t y = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += y;
  }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  int32_t before = tile_offsets[blockIdx.x] + incl - v;
  for (int w = 0; w < warp; ++w) before += s_warp[w];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (base + i < M) { row_ptr[base + i] = before; cursor[base + i] = before; }
    before += c[i];
  }
}

// counts -> row_ptr[0..M], cursor[0..M); tile_sums holds ceil(M / kScanTile) ints.
int launch_scan(const int32_t* counts, int64_t M, int32_t* row_ptr, int32_t* cursor, int32_t* tile_sums,
                cudaStream_t st) {
  const int tiles = (int)((M + kScanTile - 1) / kScanTile);
  scan_tile_sums_kernel<<<tiles, 256, 0, st>>>(counts, M, tile_sums);
  SC_CHECK_LAUNCH("scan_tile_sums");
  scan_tile_offsets_kernel<<<1, 1024, 0, st>>>(tile_sums, tiles, row_ptr + M);
  SC_CHECK_LAUNCH("scan_tile_offsets");
  scan_tiles_kernel<<<tiles, 256, 0, st>>>(counts, M, tile_sums, row_ptr, cursor);
  SC_CHECK_LAUNCH("scan_tiles");
  return SC_OK;
}

__global__ void csr_fill_kernel(const int64_t* __restrict__ idx, int64_t total, int64_t M,
                                int32_t* __restrict__ cursor, int32_t* __restrict__ entries) {
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
       e += (int64_t)gridDim.x * blockDim.x) {
    int64_t m = idx[e];
    if (m >= 0 && m < M) {
      int32_t pos = atomicAdd(&cursor[m], 1);
      entries[pos] = (int32_t)e;
    }
  }
}

// One warp per latent; segments of 2..32 entries sort in registers, segments up
// to kSortMax in a per-warp shared-memory buffer (bitonic network).
// Longer segments are queued: *long_count = how many, long_ids[0 .. long_cap) their latents
// (the histogram and cursor arrays, dead by then, serve as the queue).
constexpr int kSortWarps = 4;
__global__ void __launch_bounds__(kSortWarps * 32)
csr_sort_kernel(const int32_t* __restrict__ row_ptr, int64_t M, int32_t* __restrict__ entries,
                int32_t* __restrict__ long_count, int32_t* __restrict__ long_ids, int32_t long_cap) {
  __shared__ int32_t s_buf[kSortWarps][kSortMax];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t m = (int64_t)blockIdx.x * kSortWarps + warp;
  if (m >= M) return;
  const int32_t lo = row_ptr[m], len = row_ptr[m + 1] - lo;
  if (len > kSortMax) {
    if (lane == 0) {
      const int32_t slot = atomicAdd(long_count, 1);
      if (slot < long_cap) long_ids[slot] = (int32_t)m;
    }
    return;
  }
  if (len <= 1) return;
  if (len <= 32) {
    int32_t v = lane < len ? entries[lo + lane] : 0x7fffffff;
    for (int size = 2; size <= 32; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        int32_t o = __shfl_xor_sync(0xffffffffu, v, stride);
        bool up = (lane & size) == 0;          // ascending block?
        bool lower = (lane & stride) == 0;     // lower partner keeps min when ascending
        bool keep_min = (up == lower);
        v = keep_min ? min(v, o) : max(v, o);
      }
    }
    if (lane < len) entries[lo + lane] = v;
    return;
  }
  int32_t* buf = s_buf[warp];
  int n2 = 64;
  while (n2 < len) n2 <<= 1;
  for (int i = lane; i < n2; i += 32) buf[i] = i < len ? entries[lo + i] : 0x7fffffff;
  __syncwarp();
  for (int size = 2; size <= n2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = lane; i < n2 / 2; i += 32) {
        int a = 2 * i - (i & (stride - 1));  // index with bit `stride` clear
        int b = a + stride;
        bool up = (a & size) == 0;
        int32_t x = buf[a], y = buf[b];
        if ((x > y) == up) { buf[a] = y; buf[b] = x; }
      }
      __syncwarp();
    }
  }
  for (int i = lane; i < len; i += 32) entries[lo + i] = buf[i];
}

// Sorts the queued long segments in place in global memory, one CTA per segment: a bitonic
// network in its all-ascending form (the first step of every merge pairs i with i ^ (size-1),
// the others i with i ^ stride), which sorts any length as if the tail were padded with
// +infinity - a pair whose upper index lies beyond the segment is simply left alone.
__global__ void __launch_bounds__(1024)
csr_sort_long_kernel(const int32_t* __restrict__ row_ptr, int32_t* __restrict__ entries,
                     const int32_t* __restrict__ long_count, const int32_t* __restrict__ long_ids,
                     int32_t long_cap) {
  const int32_t n_long = min(*long_count, long_cap);
  for (int32_t w = blockIdx.x; w < n_long; w += gridDim.x) {
    const int32_t m = long_ids[w];
    const int32_t lo = row_ptr[m], len = row_ptr[m + 1] - lo;
    int32_t* seg = entries + lo;
    int64_t n2 = 1;
    while (n2 < len) n2 <<= 1;
    for (int64_t size = 2; size <= n2; size <<= 1) {
      for (int64_t stride = size >> 1; stride > 0; stride >>= 1) {
        for (int64_t i = threadIdx.x; i < n2 / 2; i += blockDim.x) {
          const int64_t a = 2 * i - (i & (stride - 1));                     // bit `stride` clear
          const int64_t b = (stride == (size >> 1)) ? (a ^ (size - 1)) : (a + stride);
          if (b < len) {
            const int32_t x = seg[a], y = seg[b];
            if (x > y) { seg[a] = y; seg[b] = x; }
          }
        }
        __syncthreads();
      }
    }
  }
}

// count -> scan -> fill -> sort with the three scratch arrays given (counts, cursor: M ints
// each; tile_sums: ceil(M / kScanTile) ints).
int build_csr(const int64_t* idx, int64_t N, int k, int64_t M, int32_t* row_ptr, int32_t* entries,
              int32_t* counts, int32_t* cursor, int32_t* tile_sums, cudaStream_t st) {
  const int64_t total = N * k;
  // scratch keeps whatever an earlier call left: the histogram must start at zero
  SC_CUDA(cudaMemsetAsync(counts, 0, (size_t)M * sizeof(int32_t), st));
  if (total == 0) return launch_scan(counts, M, row_ptr, cursor, tile_sums, st);
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  csr_count_kernel<<<blocks, 256, 0, st>>>(idx, total, M, counts);
  SC_CHECK_LAUNCH("csr_count");
  int rc = launch_scan(counts, M, row_ptr, cursor, tile_sums, st);
  if (rc != SC_OK) return rc;
  csr_fill_kernel<<<blocks, 256, 0, st>>>(idx, total, M, cursor, entries);
  SC_CHECK_LAUNCH("csr_fill");
  // histogram and cursors are dead now: counts[0] counts the long segments, cursor[0..M) lists them
  int32_t* long_count = counts;
  int32_t* long_ids = cursor;
  const int32_t long_cap = (int32_t)M;
  SC_CUDA(cudaMemsetAsync(long_count, 0, sizeof(int32_t), st));
  csr_sort_kernel<<<(unsigned)((M + kSortWarps - 1) / kSortWarps), kSortWarps * 32, 0, st>>>(
      row_ptr, M, entries, long_count, long_ids, long_cap);
  SC_CHECK_LAUNCH("csr_sort");
  if (total > kSortMax) {  // otherwise no segment can be long
    const int64_t most = total / kSortMax;
    csr_sort_long_kernel<<<(unsigned)(most < 64 ? most : 64), 1024, 0, st>>>(row_ptr, entries, long_count, long_ids,
                                                                            long_cap);
    SC_CHECK_LAUNCH("csr_sort_long");
  }
  return SC_OK;
}

}  // namespace

extern "C" size_t sc_csr_workspace_bytes(int64_t M) {
  if (M < 0) return 0;
  // counts[M] + cursor[M] + tile sums of the scan, each padded to 256 bytes
  size_t one = (((size_t)M * sizeof(int32_t)) + 255) & ~size_t(255);
  size_t tiles = ((((size_t)M + kScanTile - 1) / kScanTile) * sizeof(int32_t) + 255) & ~size_t(255);
  return 2 * one + tiles;
}

extern "C" int sc_csr_build(const int64_t* idx, int64_t N, int k, int64_t M, int32_t* row_ptr,
                            int32_t* entries, void* ws, size_t ws_bytes, void* stream) {
  SC_REQUIRE(N >= 0 && k > 0 && M > 0, "sc_csr_build: bad shape N=%lld k=%d M=%lld",
             (long long)N, k, (long long)M);
  SC_REQUIRE(row_ptr && ws, "sc_csr_build: null pointer");
  // Flat positions are stored as int32 (sparsify/xformers.py:156 has the same bound).
  SC_REQUIRE(N * (int64_t)k < (int64_t(1) << 31), "sc_csr_build: N*k must be below 2^31");
  if (ws_bytes < sc_csr_workspace_bytes(M))
    return sc::fail(SC_ERR_WORKSPACE, "sc_csr_build: workspace %zu < %zu", ws_bytes,
                    sc_csr_workspace_bytes(M));
  cudaStream_t st = sc::as_stream(stream);
  const size_t one = (((size_t)M * sizeof(int32_t)) + 255) & ~size_t(255);
  int32_t* counts = static_cast<int32_t*>(ws);
  int32_t* cursor = reinterpret_cast<int32_t*>(static_cast<char*>(ws) + one);
  int32_t* tile_sums = reinterpret_cast<int32_t*>(static_cast<char*>(ws) + 2 * one);
  SC_REQUIRE(N * (int64_t)k == 0 || (idx && entries), "sc_csr_build: null pointer");
  return build_csr(idx, N, k, M, row_ptr, entries, counts, cursor, tile_sums, st);
}

// ---------------------------------------------------------------------------
// sc_csr_build_noalloc: the same CSR build for callers that cannot obtain
// device memory for the scratch (see include/sparsecoder.h). The scratch lives
// in a fixed array that is part of the library image on every GPU.
namespace {

constexpr int64_t kNoAllocMaxLatents = 262144;  // 2 x 1 MiB of counters
static __device__ __align__(256) unsigned char g_csr_scratch[(2 * kNoAllocMaxLatents + kNoAllocMaxLatents / kScanTile) * sizeof(int32_t)];

constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
void* g_scratch_ptr[kMaxDevices] = {};  // device address of g_csr_scratch, per device

// Resolves the device address of the static scratch for the current device.
// In host code the symbol name is only a handle: the address a kernel may use
// has to come from cudaGetSymbolAddress, once per device, with that device
// current.
int scratch_for_current_device(void** out) {
  int dev = -1;
  SC_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return sc::fail(SC_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    SC_CUDA(cudaGetSymbolAddress(&p, g_csr_scratch));
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return SC_OK;
}

}  // namespace

extern "C" int sc_csr_build_noalloc(const int64_t* idx, int64_t N, int k, int64_t M, int32_t* row_ptr,
                                    int32_t* entries, void* stream) {
  SC_REQUIRE(N >= 0 && k > 0 && M > 0, "sc_csr_build_noalloc: bad shape N=%lld k=%d M=%lld",
             (long long)N, k, (long long)M);
  if (M > kNoAllocMaxLatents)
    return sc::fail(SC_ERR_TOO_LARGE, "sc_csr_build_noalloc: M=%lld exceeds the built-in scratch (max %lld latents)",
                    (long long)M, (long long)kNoAllocMaxLatents);
  SC_REQUIRE(row_ptr != nullptr, "sc_csr_build_noalloc: null pointer");
  SC_REQUIRE(N * (int64_t)k < (int64_t(1) << 31), "sc_csr_build_noalloc: N*k must be below 2^31");
  void* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != SC_OK) return rc;
  cudaStream_t st = sc::as_stream(stream);
  int32_t* counts = static_cast<int32_t*>(scratch);
  int32_t* cursor = counts + kNoAllocMaxLatents;
  int32_t* tile_sums = cursor + kNoAllocMaxLatents;
  // every call shares the one array; build_csr clears what has to start at zero
  SC_REQUIRE(N * (int64_t)k == 0 || (idx && entries), "sc_csr_build_noalloc: null pointer");
  return build_csr(idx, N, k, M, row_ptr, entries, counts, cursor, tile_sums, st);
}
