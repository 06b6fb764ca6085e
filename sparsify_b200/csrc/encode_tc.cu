// Fused encoder forward on the 5th-generation tensor cores.
//
//   pre[n,m] = relu(sum_d x[n,d] W[m,d] + b[m]),   top-k per row
//
// A persistent CTA per SM walks work units (128-token row block x strip of
// consecutive 256-latent tiles). Warp 0 streams 128x64 / 256x64 bf16 tiles of x
// and W into a shared-memory ring with TMA, warp 1 issues tcgen05.mma into one
// of two 128x256 fp32 accumulators in tensor memory, and warps 2-5 drain the
// other accumulator: bias, ReLU and a running top-k list per row held in shared
// memory, so the epilogue of tile t overlaps the MMAs of tile t+1 and the N x M
// matrix never reaches HBM. Each (row, strip) emits k candidates; a second
// kernel merges the strips of a row into the final k.
//
// A second form of the same kernel (sc_set_cta_pairs) lets two CTAs on the SMs of one
// TPC work as a pair (tcgen05 cta_group::2) on a 256-token row block: each loads its
// own 128 rows of x and its own half of the W tile with its own TMA loads, the even
// CTA issues 256x256x16 MMAs for both, and each drains its own 128 accumulator rows,
// so that an SM stages 32 KB per k-chunk instead of 48 KB. Measured on B200 at
// d=4096, 131072 latents, 16384 tokens, back to back under the 1000 W power cap: the
// pair form needs 4 % fewer SM cycles but more energy per launch (15.3 J against
// 14.0 J), the clock settles lower (1147 against 1312 MHz) and the launch takes 15.5 ms
// against 14.2 ms - so the one-CTA form is the default for k = 32. Wide lists (k = 64,
// k = 128 for Multi-TopK) leave the one-CTA form fewer than four 48 KB stages; there the
// pair form is chosen, see make_plan. Results are identical.
//
// A per-row lower bound on the k-th largest value (`tau`) is published after
// every finished strip and read at the start of later strips of the same rows:
// values not above it cannot be among the row's top k, which removes most list
// insertions after the first wave of units.
#include "tc.cuh"

#include <stdlib.h>

namespace {

using namespace sc::tc;

constexpr int BM = 128;   // tokens per tile (TMEM lanes)
constexpr int BN = 256;   // latents per tile (TMEM columns per accumulator)
constexpr int BK = 64;    // bf16 per 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
// bytes one CTA stages per k-chunk: its 128 rows of x plus its share of the W tile (all 256
// rows alone, 128 as one of a pair)
constexpr uint32_t stage_bytes(int cg) { return (uint32_t)(BM + BN / cg) * BK * 2; }  // 48 / 32 KiB
constexpr int kMaxK = 128;
constexpr int kRowGroupRows = 4096;  // rows whose units run together (L2 footprint of x: 32 MB at d=4096)

struct Plan {
  int cg;         // CTAs per work unit: 1, or 2 (a pair sharing 256-row blocks)
  int n_rb;       // row blocks (of 128 * cg rows)
  int n_ct;       // column tiles
  int n_strips;   // strips per row block
  int stages;     // smem ring depth
  int units;      // n_rb * n_strips
  size_t smem;    // dynamic shared memory bytes
  size_t off_lists_val, off_lists_idx, off_gmin, off_gpos, off_bias, off_bars;
};

// Status codes written to the device status word by a wait that gave up.
enum { kWaitEmpty = 101, kWaitFull = 102, kWaitTmemEmpty = 103, kWaitTmemFull = 104 };

struct Params {
  const float* bias;
  float* cand_vals;     // [N][n_strips][k]
  int32_t* cand_idx;    // [N][n_strips][k]
  float* tau;           // [N]
  int32_t* status;
  int64_t N, D, M;
  int k, n_rb, n_ct, n_strips, stages, units;
  int row_group;  // row blocks (of 128 rows per CTA of the unit) per scheduling group
  // groupmax mode (group_cols > 0): the M columns form k groups of group_cols consecutive
  // latents and every row keeps the largest post-ReLU value of each group; results go
  // straight to gm_vals / gm_idx ([N, k]), strips hold whole groups, no lists, no merge.
  int group_cols;
  float* gm_vals;
  int64_t* gm_idx;
#ifdef SC_DIAG
  int debug;  // diagnostics build only: bit 0 = epilogue only drains (no bias / top-k work), bit 3 = reads the accumulator only, bit 4 = stops after the threshold mask
#endif
  uint32_t off_lists_val, off_lists_idx, off_gmin, off_gpos, off_bias, off_bars;
};

__device__ __forceinline__ void decode_unit(const Params& p, int u, int& rb, int& strip, int& t0, int& t1) {
  const int per_group = p.row_group * p.n_strips;
  const int g = u / per_group, rem = u % per_group;
  const int rg = min(p.row_group, p.n_rb - g * p.row_group);
  strip = rem / rg;
  rb = g * p.row_group + rem % rg;
  t0 = (int)(((int64_t)strip * p.n_ct) / p.n_strips);
  t1 = (int)(((int64_t)(strip + 1) * p.n_ct) / p.n_strips);
}

// Per-row running top-k list, owned by one thread (the row's TMEM lane) and
// kept in shared memory column-wise - entry j of row r at l_val[j * 128 + r] -
// so that the 32 rows of a warp touch 32 different banks. Entries are grouped
// by eight with each group's minimum cached (g_val / g_pos), so replacing the
// row minimum rescans one group and the group minima instead of all k
// entries. While the list still has free slots, values are appended without
// any scan. Lanes of a warp with a candidate in the same column run this
// together (plain SIMT divergence, no cross-lane traffic). Out of line: it is
// called from 32 unrolled sites.
struct RowState {
  float thr;      // smallest value in the row's list (-1 while it has free slots)
  float thr_cmp;  // what a raw pre-activation must exceed to enter the list
  int minpos;     // position of the smallest value
  int cnt;        // filled entries (== k once the list is full)
};

constexpr int kGroup = 8;

// v[i] for a run-time i: a five-level select tree (registers cannot be indexed).
__device__ __forceinline__ float pick32(const float (&v)[32], int i) {
  float a[16], b[8], c[4], d[2];
#pragma unroll
  for (int j = 0; j < 16; ++j) a[j] = (i & 1) ? v[2 * j + 1] : v[2 * j];
#pragma unroll
  for (int j = 0; j < 8; ++j) b[j] = (i & 2) ? a[2 * j + 1] : a[2 * j];
#pragma unroll
  for (int j = 0; j < 4; ++j) c[j] = (i & 4) ? b[2 * j + 1] : b[2 * j];
#pragma unroll
  for (int j = 0; j < 2; ++j) d[j] = (i & 8) ? c[2 * j + 1] : c[2 * j];
  return (i & 16) ? d[1] : d[0];
}

// Minimum of group g (entries g*8 .. g*8+7, those below k) with its position.
// All eight loads are issued before the first comparison.
__device__ __forceinline__ void group_min(const float* lv, int k, int g, float& best, int& pos) {
  float x[kGroup];
#pragma unroll
  for (int j = 0; j < kGroup; ++j) {
    const int e = g * kGroup + j;
    x[j] = e < k ? lv[e * BM] : INFINITY;
  }
  best = x[0];
  pos = g * kGroup;
#pragma unroll
  for (int j = 1; j < kGroup; ++j)
    if (x[j] < best) { best = x[j]; pos = g * kGroup + j; }
}

// The list is full: overwrite its minimum with (v, rel_col), refresh the cached
// minimum of the touched group and find the new row minimum among the G groups.
template <int G>
__device__ __forceinline__ RowState replace_min(float* lv, uint16_t* li, float* gv, uint16_t* gp, int k,
                                                int groups, float v, uint16_t rel_col, float tau, RowState st) {
  const int g = st.minpos / kGroup;
  float gm[G];
#pragma unroll
  for (int i = 0; i < G; ++i) gm[i] = i < groups ? gv[i * BM] : INFINITY;  // independent of the rescan
  lv[st.minpos * BM] = fmaxf(v, 0.f);
  li[st.minpos * BM] = rel_col;
  float best; int pos;
  group_min(lv, k, g, best, pos);
  gv[g * BM] = best;
  gp[g * BM] = (uint16_t)pos;
  float rbest = INFINITY;
  int rg = 0;
#pragma unroll
  for (int i = 0; i < G; ++i) {
    const float x = (i == g) ? best : gm[i];
    if (x < rbest) { rbest = x; rg = i; }
  }
  st.thr = rbest;
  st.minpos = (rg == g) ? pos : (int)gp[rg * BM];
  st.thr_cmp = fmaxf(rbest, tau);
  return st;
}

__device__ __noinline__ RowState list_insert(float* lv, uint16_t* li, float* gv, uint16_t* gp, int k, float v,
                                             uint16_t rel_col, float tau, RowState st) {
  const int groups = (k + kGroup - 1) / kGroup;
  if (st.cnt < k) {  // append; on the k-th entry build the group minima
    lv[st.cnt * BM] = fmaxf(v, 0.f);
    li[st.cnt * BM] = rel_col;
    if (++st.cnt < k) return st;
    float rbest = INFINITY;
    int rpos = 0;
    for (int g = 0; g < groups; ++g) {
      float best; int pos;
      group_min(lv, k, g, best, pos);
      gv[g * BM] = best;
      gp[g * BM] = (uint16_t)pos;
      if (best < rbest) { rbest = best; rpos = pos; }
    }
    st.thr = rbest;
    st.minpos = rpos;
    st.thr_cmp = fmaxf(rbest, tau);
    return st;
  }
  if (groups <= 4) return replace_min<4>(lv, li, gv, gp, k, groups, v, rel_col, tau, st);
  if (groups <= 8) return replace_min<8>(lv, li, gv, gp, k, groups, v, rel_col, tau, st);
  return replace_min<16>(lv, li, gv, gp, k, groups, v, rel_col, tau, st);
}

__global__ void init_tau_kernel(float* tau, int64_t n) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < n) tau[i] = -1.f;
}

// CG = CTAs per work unit. CG == 2: launched as clusters of two CTAs (a pair); rank 0 of the
// cluster is the leader that issues the MMAs and owns the `full` and `tempty` barriers that
// both CTAs signal; `empty` and `tfull` exist in both CTAs and the leader's commits reach both.
template <int CG>
__global__ void __launch_bounds__(kThreads, 1)
encode_topk_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                      const Params p) {
  constexpr uint32_t kStageBytes = stage_bytes(CG);
  extern __shared__ unsigned char smem_dyn[];
  // 1024-byte alignment for the swizzled tiles (the same offset in both CTAs of a pair: the
  // dynamic shared memory of a kernel starts at the same address in every CTA)
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  float* l_val = reinterpret_cast<float*>(smem + p.off_lists_val);         // [128][k]
  uint16_t* l_idx = reinterpret_cast<uint16_t*>(smem + p.off_lists_idx);   // [128][k]
  float* s_bias = reinterpret_cast<float*>(smem + p.off_bias);             // [4 warps][256]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.off_bars);
  uint64_t* full = bars;                    // [stages]
  uint64_t* empty = bars + p.stages;        // [stages]
  uint64_t* tfull = bars + 2 * p.stages;    // [2]
  uint64_t* tempty = tfull + 2;             // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kc_count = (int)((p.D + BK - 1) / BK);
  const uint32_t cta_rank = CG == 2 ? cluster_ctarank() : 0u;   // position inside the pair
  const bool leader = cta_rank == 0;
  const int unit0 = CG == 2 ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int unit_stride = CG == 2 ? (int)(gridDim.x >> 1) : (int)gridDim.x;

  if (threadIdx.x == 0) {
    prefetch_tensor_map(&tmap_x);
    prefetch_tensor_map(&tmap_w);
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull[b], 1); mbar_init(&tempty[b], 4 * CG); }
    fence_barrier_init();
  }
  if (warp == 1) {
    if constexpr (CG == 2) { tmem_alloc_pair(tmem_slot, 512); tmem_relinquish_pair(); }
    else { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  }
  fence_before_sync();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync();  // the peer's barriers and tensor memory are ready too
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (one per CTA; each loads only its own operands) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
#ifdef SC_DIAG
      long long wait_empty = 0;  // debug bit 2
#endif
      for (int u = unit0; u < p.units && ok; u += unit_stride) {
        int rb, strip, t0, t1;
        decode_unit(p, u, rb, strip, t0, t1);
        for (int t = t0; t < t1 && ok; ++t) {
          for (int kc = 0; kc < kc_count; ++kc) {
#ifdef SC_DIAG
            const long long w2 = clock64();
#endif
            if (!mbar_wait(&empty[stage], phase ^ 1, p.status, kWaitEmpty)) { ok = false; break; }
#ifdef SC_DIAG
            wait_empty += clock64() - w2;
#endif
            unsigned char* sa = smem + (size_t)stage * kStageBytes;
            unsigned char* sb = sa + BM * BK * 2;
            if constexpr (CG == 2) {
              // the bytes of both CTAs are counted on the leader's barrier, which its MMA thread waits on
              if (leader) mbar_arrive_expect_tx(&full[stage], 2 * kStageBytes);
              const uint32_t bar = map_to_cta(smem_u32(&full[stage]), 0);
              tma_load_2d_pair(sa, &tmap_x, kc * BK, (rb * 2 + (int)cta_rank) * BM, bar);
              tma_load_2d_pair(sb, &tmap_w, kc * BK, t * BN + (int)cta_rank * (BN / 2), bar);
            } else {
              mbar_arrive_expect_tx(&full[stage], kStageBytes);
              tma_load_2d(sa, &tmap_x, kc * BK, rb * BM, &full[stage]);
              tma_load_2d(sb, &tmap_w, kc * BK, t * BN, &full[stage]);
            }
            if (++stage == p.stages) { stage = 0; phase ^= 1; }
          }
        }
      }
#ifdef SC_DIAG
      if ((p.debug & 4) && p.status != nullptr && blockIdx.x == 0) p.status[6] = (int)(wait_empty >> 10);
#endif
      if constexpr (CG == 2) {
        // Stay until the leader's last commits have reached this CTA's `empty` barriers: a CTA of
        // a pair must not leave while its peer can still signal its shared memory.
        for (int i = 0; i < p.stages && ok; ++i) {
          if (!mbar_wait(&empty[stage], phase ^ 1, p.status, kWaitEmpty)) ok = false;
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (the leader's, for both CTAs of a pair) ----------------
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc_bf16(BM * CG, BN);
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
#ifdef SC_DIAG
      long long wait_tmem = 0, wait_full = 0, issue_time = 0;  // debug bit 2
      const long long t_begin = clock64();
#endif
      for (int u = unit0; u < p.units && ok; u += unit_stride) {
        int rb, strip, t0, t1;
        decode_unit(p, u, rb, strip, t0, t1);
        for (int t = t0; t < t1 && ok; ++t) {
#ifdef SC_DIAG
          const long long w0 = clock64();
#endif
          if constexpr (CG == 2) {
            if (!mbar_wait_cluster(&tempty[buf], acc_phase ^ 1, p.status, kWaitTmemEmpty)) { ok = false; break; }
          } else {
            if (!mbar_wait(&tempty[buf], acc_phase ^ 1, p.status, kWaitTmemEmpty)) { ok = false; break; }
          }
#ifdef SC_DIAG
          wait_tmem += clock64() - w0;
#endif
          fence_after_sync();
          const uint32_t d_tmem = tmem_base + (uint32_t)buf * BN;
          for (int kc = 0; kc < kc_count; ++kc) {
#ifdef SC_DIAG
            const long long w1 = clock64();
#endif
            if (!mbar_wait(&full[stage], phase, p.status, kWaitFull)) { ok = false; break; }
#ifdef SC_DIAG
            wait_full += clock64() - w1;
#endif
            fence_after_sync();
            const uint32_t sa = smem_u32(smem + (size_t)stage * kStageBytes);
            const uint64_t adesc = make_smem_desc_sw128(sa);
            const uint64_t bdesc = make_smem_desc_sw128(sa + BM * BK * 2);
#ifdef SC_DIAG
            const long long w3 = clock64();
#endif
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk) {
              // 32 bytes per K step inside the 128-byte swizzle row
              if constexpr (CG == 2)
                mma_bf16_pair(d_tmem, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc,
                              (kc | kk) != 0 ? 1u : 0u);
              else
                mma_bf16(d_tmem, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc,
                         (kc | kk) != 0 ? 1u : 0u);
            }
            // frees the stage (in both CTAs of a pair) once these MMAs have read it
            if constexpr (CG == 2) mma_commit_pair(&empty[stage], 3);
            else mma_commit(&empty[stage]);
#ifdef SC_DIAG
            issue_time += clock64() - w3;
#endif
            if (++stage == p.stages) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          // accumulator complete (each CTA of a pair drains its own 128 rows)
          if constexpr (CG == 2) mma_commit_pair(&tfull[buf], 3);
          else mma_commit(&tfull[buf]);
          buf ^= 1;
          if (buf == 0) acc_phase ^= 1;
        }
      }
#ifdef SC_DIAG
      if ((p.debug & 4) && p.status != nullptr && blockIdx.x == 0) {
        // kilo-cycles of SM 0's MMA thread: total, waiting for a free accumulator, waiting for operands
        p.status[3] = (int)((clock64() - t_begin) >> 10);
        p.status[4] = (int)(wait_tmem >> 10);
        p.status[5] = (int)(wait_full >> 10);
        p.status[7] = (int)(issue_time >> 10);  // inside the MMA and commit instructions
      }
#endif
    }
  } else {
    // ---------------- epilogue: bias + ReLU + running top-k ----------------
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;          // row inside the tile
    const int k = p.k;
    float* lv = l_val + row;                // this row's list: lv[j * BM], li[j * BM]
    uint16_t* li = l_idx + row;
    float* gv = reinterpret_cast<float*>(smem + p.off_gmin) + row;            // group minima
    uint16_t* gp = reinterpret_cast<uint16_t*>(smem + p.off_gpos) + row;
    float* sb = s_bias + (warp - 2) * BN;   // this warp's copy of the tile's bias
    int buf = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    // the leader's `tempty` barrier as the peer CTA addresses it
    const uint32_t tempty_leader0 = CG == 2 ? map_to_cta(smem_u32(&tempty[0]), 0) : 0u;
    const uint32_t tempty_leader1 = CG == 2 ? map_to_cta(smem_u32(&tempty[1]), 0) : 0u;
    for (int u = unit0; u < p.units && ok; u += unit_stride) {
      int rb, strip, t0, t1;
      decode_unit(p, u, rb, strip, t0, t1);
      const int64_t grow = ((int64_t)rb * CG + cta_rank) * BM + row;
      const int64_t strip_col0 = (int64_t)t0 * BN;
      RowState st;
      st.thr = -1.f; st.minpos = 0; st.cnt = 0;
      float published = -1.f;  // last bound this thread pushed to p.tau
#ifdef SC_DIAG
      unsigned n_ins = 0, n_cols = 0;  // debug bit 1
#endif
      // rows past N are padding: an infinite bound keeps them out of the lists
      float tau = (grow < p.N && p.group_cols == 0) ? __ldcg(p.tau + grow) : INFINITY;
      // Threshold the raw (pre-ReLU) value is compared with: max(thr, tau), or
      // -inf while that is still negative (list not full and no bound known), so
      // that every value, clamped to >= 0 on insertion, is taken.
      st.thr_cmp = tau < 0.f ? -INFINITY : tau;
      // groupmax state: current group, position inside it, best value so far and its offset
      int gm_group = 0, gm_pos = 0, gm_arg = 0;
      float gm_best = -1.f;
      if (p.group_cols > 0) {
        gm_group = (int)(strip_col0 / p.group_cols);
        gm_pos = (int)(strip_col0 % p.group_cols);
      }

      for (int t = t0; t < t1 && ok; ++t) {
        __syncwarp();
        for (int c = lane; c < BN; c += 32) {
          const int64_t col = (int64_t)t * BN + c;
          sb[c] = (col < p.M) ? __ldg(p.bias + col) : 0.f;
        }
        __syncwarp();

        ok = __all_sync(0xffffffffu, mbar_wait(&tfull[buf], acc_phase, p.status, kWaitTmemFull));
        if (!ok) break;
        fence_after_sync();
        const int64_t tile_col0 = (int64_t)t * BN;
        const int ncols = (int)min((int64_t)BN, p.M - tile_col0);
        const uint32_t taddr = tmem_base + (uint32_t)buf * BN + ((uint32_t)(q * 32) << 16);
#ifdef SC_DIAG
        const int n_chunks = (p.debug & 1) ? 0 : BN / 32;
#else
        constexpr int n_chunks = BN / 32;
#endif
#pragma unroll 1
        for (int c = 0; c < n_chunks; ++c) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
#ifdef SC_DIAG
          if (p.debug & 8) {  // accumulator read only
            unsigned acc = 0;
#pragma unroll
            for (int i = 0; i < 32; ++i) acc ^= r[i];
            if (acc == 0x7fc12345u) ++n_cols;
            continue;
          }
#endif
          // Pass 1 (full ILP): add the bias and mark the columns that beat this
          // row's threshold as it stood at chunk start.
          float v[32];
          const float4* sb4 = reinterpret_cast<const float4*>(sb + c * 32);
#pragma unroll
          for (int i4 = 0; i4 < 8; ++i4) {
            const float4 b4 = sb4[i4];
            v[4 * i4 + 0] = __uint_as_float(r[4 * i4 + 0]) + b4.x;
            v[4 * i4 + 1] = __uint_as_float(r[4 * i4 + 1]) + b4.y;
            v[4 * i4 + 2] = __uint_as_float(r[4 * i4 + 2]) + b4.z;
            v[4 * i4 + 3] = __uint_as_float(r[4 * i4 + 3]) + b4.w;
          }
          const int valid = ncols - c * 32;  // columns of this chunk inside the matrix
          if (p.group_cols > 0) {
            // a chunk of 32 columns lies inside one group (group_cols % 32 == 0)
            if (valid <= 0) continue;
            float best = fmaxf(v[0], 0.f);
            int bi = 0;
#pragma unroll
            for (int i = 1; i < 32; ++i) {
              const float xv = fmaxf(v[i], 0.f);
              if (i < valid && xv > best) { best = xv; bi = i; }  // strict: ties keep the lowest index
            }
            if (best > gm_best) { gm_best = best; gm_arg = gm_pos + bi; }
            gm_pos += 32;
            if (gm_pos >= p.group_cols) {
              if (grow < p.N) {
                p.gm_vals[grow * k + gm_group] = gm_best;
                p.gm_idx[grow * k + gm_group] = (int64_t)gm_group * p.group_cols + gm_arg;
              }
              ++gm_group; gm_pos = 0; gm_best = -1.f;
            }
            continue;
          }
          unsigned m = 0;
#pragma unroll
          for (int i = 0; i < 32; ++i) m |= (v[i] > st.thr_cmp ? 1u : 0u) << i;
          if (valid < 32) m &= valid <= 0 ? 0u : ((1u << valid) - 1u);
#ifdef SC_DIAG
          if (p.debug & 16) {  // bias and threshold mask only: no candidate is walked or inserted
            n_cols += __popc(m);
            continue;
          }
#endif
          // Pass 2: every row walks its own marked columns (ascending), so the loop
          // runs as often as the busiest row has candidates, not once per marked column.
          const uint16_t rel0 = (uint16_t)(tile_col0 - strip_col0 + c * 32);
          while (__any_sync(0xffffffffu, m != 0)) {
#ifdef SC_DIAG
            ++n_cols;
#endif
            if (m != 0) {
              const int i = __ffs(m) - 1;
              m &= m - 1;
              const float val = pick32(v, i);
              if (val > st.thr_cmp) {
                if (st.cnt + 1 < k) {  // free slots left: append in line
                  lv[st.cnt * BM] = fmaxf(val, 0.f);
                  li[st.cnt * BM] = (uint16_t)(rel0 + i);
                  ++st.cnt;
                } else {
                  st = list_insert(lv, li, gv, gp, k, val, (uint16_t)(rel0 + i), tau, st);
                }
#ifdef SC_DIAG
                ++n_ins;
#endif
              }
            }
          }
        }
        // Exchange the row's lower bound with the CTAs working on other strips of
        // the same rows: push ours when it grew, pull theirs for the next tile.
        if (grow < p.N && p.group_cols == 0) {
          if (st.cnt == k && st.thr > published) {
            atomicMax(reinterpret_cast<int*>(p.tau + grow), __float_as_int(st.thr));
            published = st.thr;
          }
          tau = fmaxf(tau, __ldcg(p.tau + grow));
          if (st.cnt == k) st.thr_cmp = fmaxf(st.thr, tau);
          else st.thr_cmp = tau < 0.f ? -INFINITY : tau;
        }
        // accumulator drained
        fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if (CG == 2 && !leader) mbar_arrive_cluster(buf ? tempty_leader1 : tempty_leader0);
          else mbar_arrive(&tempty[buf]);
        }
        buf ^= 1;
        if (buf == 0) acc_phase ^= 1;
      }
      if (!ok) break;
#ifdef SC_DIAG
      if ((p.debug & 2) && p.status != nullptr) {  // status[1] = insertions, status[2] = visited columns
        atomicAdd(p.status + 1, (int)n_ins);
        if (lane == 0) atomicAdd(p.status + 2, (int)n_cols);
      }
#endif
      // write this strip's candidates and publish the row's lower bound
      if (grow < p.N && p.group_cols == 0) {
        float* cv = p.cand_vals + (grow * p.n_strips + strip) * k;
        int32_t* ci = p.cand_idx + (grow * p.n_strips + strip) * k;
        for (int j = 0; j < k; ++j) {
          const bool used = j < st.cnt;
          cv[j] = used ? lv[j * BM] : -1.f;
          ci[j] = used ? (int32_t)(strip_col0 + li[j * BM]) : -1;
        }
        if (st.cnt == k && st.thr > published)
          atomicMax(reinterpret_cast<int*>(p.tau + grow), __float_as_int(st.thr));
      }
    }
  }


  // teardown: nobody's tensor or shared memory is touched by the peer any more
  fence_before_sync();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync();
  fence_after_sync();
  if (warp == 1) {
    if constexpr (CG == 2) tmem_dealloc_pair(tmem_base, 512);
    else tmem_dealloc(tmem_base, 512);
  }
}

// ---- merge: final k of a row from its n_strips*k candidates --------------------
// One warp per row. Candidates with value < 0 are empty slots. Output is in
// descending value (ties: ascending index), so it does not depend on the order
// in which the lists were filled.
//
// Keys are 64-bit: value bits in the high word (values are >= 0), inverted index in the
// low word, so a larger key is the better candidate, keys of real candidates are distinct
// and non-zero, and 0 stands for an empty slot. Every strip's list becomes a chunk of
// kp = 2^ceil(log2 k) keys in shared memory; each chunk is sorted (descending) by a bitonic
// network, then chunks are merged pairwise keeping only the better kp of each pair:
// max(A[i], B[kp-1-i]) is a bitonic sequence holding them, which log2(kp) compare-exchange
// steps sort again. After log2(chunks) rounds chunk 0 is the row's top kp.
__device__ __forceinline__ void cmp_swap_desc(unsigned long long* keys, int i, int j, bool desc) {
  const unsigned long long x = keys[i], y = keys[j];
  const bool swap = desc ? x < y : x > y;
  keys[i] = swap ? y : x;
  keys[j] = swap ? x : y;
}

__global__ void __launch_bounds__(128)
topk_merge_kernel(const float* __restrict__ cand_vals, const int32_t* __restrict__ cand_idx, int64_t N,
                  int n_strips, int k, int kp, int chunks, float* __restrict__ top_vals,
                  int64_t* __restrict__ top_idx) {
  extern __shared__ unsigned long long s_keys[];  // [warps][chunks * kp]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t n = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
  if (n >= N) return;
  const int P = chunks * kp;
  unsigned long long* keys = s_keys + (size_t)warp * P;
  const float* cv = cand_vals + n * (int64_t)n_strips * k;
  const int32_t* ci = cand_idx + n * (int64_t)n_strips * k;
  for (int t = lane; t < P; t += 32) {
    const int c = t / kp, j = t - c * kp;
    unsigned long long key = 0ull;
    if (c < n_strips && j < k) {
      const float v = cv[c * k + j];
      if (v >= 0.f)
        key = ((unsigned long long)__float_as_uint(v) << 32) |
              (unsigned long long)(0xffffffffu - (uint32_t)ci[c * k + j]);
    }
    keys[t] = key;
  }
  __syncwarp();
  // every chunk sorted descending
  for (int size = 2; size <= kp; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = lane; t < (P >> 1); t += 32) {
        const int i = ((t & ~(stride - 1)) << 1) | (t & (stride - 1));
        const bool desc = size == kp || (i & size) == 0;
        cmp_swap_desc(keys, i, i + stride, desc);
      }
      __syncwarp();
    }
  }
  // pairwise merges that keep the better kp keys of two chunks in the first of them
  for (int step = 1; step < chunks; step <<= 1) {
    const int pairs = chunks / (2 * step);
    for (int t = lane; t < pairs * kp; t += 32) {
      const int m = t / kp, i = t - m * kp;
      unsigned long long* A = keys + (size_t)(2 * step * m) * kp;
      const unsigned long long* B = A + (size_t)step * kp;
      const unsigned long long x = A[i], y = B[kp - 1 - i];
      A[i] = x > y ? x : y;
    }
    __syncwarp();
    for (int stride = kp >> 1; stride > 0; stride >>= 1) {
      for (int t = lane; t < pairs * (kp >> 1); t += 32) {
        const int m = t / (kp >> 1), u = t - m * (kp >> 1);
        const int i = ((u & ~(stride - 1)) << 1) | (u & (stride - 1));
        cmp_swap_desc(keys + (size_t)(2 * step * m) * kp, i, i + stride, true);
      }
      __syncwarp();
    }
  }
  for (int r = lane; r < k; r += 32) {
    const unsigned long long best = keys[r];
    if (best != 0ull) {
      top_vals[n * k + r] = __uint_as_float((uint32_t)(best >> 32));
      top_idx[n * k + r] = (int64_t)(0xffffffffu - (uint32_t)(best & 0xffffffffu));
    } else {  // fewer than k candidates: cannot happen when M >= k
      top_vals[n * k + r] = 0.f;
      top_idx[n * k + r] = 0;
    }
  }
}

int make_plan(int64_t N, int64_t D, int64_t M, int k, Plan* pl, int group_cols = 0) {
  const int kl = group_cols > 0 ? 1 : k;  // groupmax keeps no lists
  const size_t lists_val = (size_t)BM * kl * sizeof(float);
  const size_t lists_idx = (size_t)BM * kl * sizeof(uint16_t);
  const size_t groups = (size_t)(kl + 7) / 8;
  const size_t gmin = groups * BM * sizeof(float), gpos = groups * BM * sizeof(uint16_t);
  const size_t fixed = lists_val + lists_idx + gmin + gpos + 4 * BN * sizeof(float) + 256 /*barriers*/ + 1024 /*align*/;
  const size_t smem_limit = 227 * 1024;
  // Form: forced by sc_set_cta_pairs, else chosen by what the lists leave for the operand ring.
  // With four 48 KB stages (k up to ~40) the one-CTA form is the faster one under the power
  // cap; wider lists leave it three stages (k = 64) or two (k = 128), and the pair form, whose
  // stages are 32 KB, then wins: 14.0 against 15.2 ms at k = 64, 16.3 against 21.6 ms at k = 128
  // (d = 4096, 131072 latents, 16384 tokens).
  const int mode = sc::cta_pairs_mode();
  const int single_stages = fixed + stage_bytes(1) <= smem_limit ? (int)((smem_limit - fixed) / stage_bytes(1)) : 0;
  const int cg = mode == 1 ? 2 : mode == 0 ? 1 : (single_stages < 4 ? 2 : 1);
  pl->cg = cg;
  pl->n_rb = (int)((N + BM * cg - 1) / (BM * cg));
  pl->n_ct = (int)((M + BN - 1) / BN);
  // groupmax with groups of whole tiles: a strip must hold whole groups, i.e. the strip count
  // divides the group count k
  const bool whole_groups = group_cols >= BN;
  // Strips per row block: the fewest (longest strips, fewest list insertions)
  // that keep the persistent grid (one CTA, or one CTA pair, per work unit) busy; strips
  // hold at most 255 tiles so that a strip-relative column fits 16 bits.
  const int sms = (148 - sc::reserved_sms()) / cg;
  int min_strips = (pl->n_ct + 254) / 255;
  int best = -1;
  double best_eff = -1.0;
  for (int s = min_strips; s <= pl->n_ct; ++s) {
    if (whole_groups && (s > k || k % s != 0)) continue;
    const long units = (long)pl->n_rb * s;
    const long waves = (units + sms - 1) / sms;
    const double eff = (double)units / (double)(waves * sms);
    if (eff > best_eff + 1e-9) { best_eff = eff; best = s; }
    if (eff >= 0.97) { best = s; break; }
    if (pl->n_ct / s < 4 && best_eff > 0) break;  // do not shred strips below 4 tiles for balance
  }
  pl->n_strips = best < 1 ? 1 : best;
  pl->units = pl->n_rb * pl->n_strips;
  const size_t stage = stage_bytes(cg);
  if (fixed + 2 * stage > smem_limit) return SC_ERR_UNSUPPORTED;
  int stages = (int)((smem_limit - fixed) / stage);
  if (stages > 8) stages = 8;
#ifdef SC_MAX_STAGES
  if (stages > SC_MAX_STAGES) stages = SC_MAX_STAGES;  // diagnostics builds: sensitivity to the ring depth
#endif
  pl->stages = stages;
  pl->off_lists_val = (size_t)stages * stage;
  pl->off_lists_idx = pl->off_lists_val + lists_val;
  pl->off_gmin = pl->off_lists_idx + lists_idx;
  pl->off_gpos = pl->off_gmin + gmin;
  pl->off_bias = pl->off_gpos + gpos;
  pl->off_bars = pl->off_bias + 4 * BN * sizeof(float);
  pl->smem = pl->off_bars + 256 + 1024;
  return SC_OK;
}

// Launches the persistent kernel: one CTA per SM, as clusters of two for the pair form.
int launch_encoder(const Plan& pl, const CUtensorMap& tmx, const CUtensorMap& tmw, const Params& p,
                   cudaStream_t st, const char* what) {
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  sms -= sc::reserved_sms();
  if (pl.cg == 1) {
    SC_CUDA(cudaFuncSetAttribute(encode_topk_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
    const int grid = pl.units < sms ? pl.units : sms;
    encode_topk_tc_kernel<1><<<grid, kThreads, pl.smem, st>>>(tmx, tmw, p);
  } else {
    SC_CUDA(cudaFuncSetAttribute(encode_topk_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
    const int pairs = pl.units < sms / 2 ? pl.units : sms / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    SC_CUDA(cudaLaunchKernelEx(&cfg, encode_topk_tc_kernel<2>, tmx, tmw, p));
  }
  SC_CHECK_LAUNCH(what);
  return SC_OK;
}

size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

}  // namespace

extern "C" size_t sc_encode_topk_workspace_bytes(int64_t N, int64_t D, int64_t M, int k) {
  if (N <= 0 || D <= 0 || M <= 0 || k <= 0 || k > kMaxK) return 0;
  Plan pl;
  if (make_plan(N, D, M, k, &pl) != SC_OK) return 0;
  const size_t cand = (size_t)N * pl.n_strips * k;
  return align256(cand * sizeof(float)) + align256(cand * sizeof(int32_t)) + align256((size_t)N * sizeof(float));
}

extern "C" int sc_encode_topk(const void* x_bf16, const void* W_bf16, const float* bias, int64_t N,
                              int64_t D, int64_t M, int k, float* top_vals, int64_t* top_idx, void* ws,
                              size_t ws_bytes, int32_t* status_word, void* stream) {
  SC_REQUIRE(N >= 0 && D > 0 && M > 0 && k > 0, "sc_encode_topk: bad shape");
  if (N == 0) return SC_OK;
  SC_REQUIRE(x_bf16 && W_bf16 && bias && top_vals && top_idx && ws, "sc_encode_topk: null pointer");
  if (k > kMaxK) return sc::fail(SC_ERR_UNSUPPORTED, "sc_encode_topk: k=%d above %d", k, kMaxK);
  SC_REQUIRE(k <= M, "sc_encode_topk: k=%d exceeds M=%lld", k, (long long)M);
  SC_REQUIRE(D % 8 == 0, "sc_encode_topk: D=%lld must be a multiple of 8 (16-byte row stride for TMA)",
             (long long)D);
  SC_REQUIRE(sc::aligned(x_bf16, 16) && sc::aligned(W_bf16, 16), "sc_encode_topk: operands must be 16-byte aligned");
  SC_REQUIRE(N < (int64_t(1) << 31) && M < (int64_t(1) << 31), "sc_encode_topk: N, M must be below 2^31");
  SC_REQUIRE(sc::aligned(ws, 256), "sc_encode_topk: workspace must be 256-byte aligned");
  Plan pl;
  if (make_plan(N, D, M, k, &pl) != SC_OK)
    return sc::fail(SC_ERR_UNSUPPORTED, "sc_encode_topk: k=%d leaves no room for the operand ring", k);
  const size_t need = sc_encode_topk_workspace_bytes(N, D, M, k);
  if (ws_bytes < need) return sc::fail(SC_ERR_WORKSPACE, "sc_encode_topk: workspace %zu < %zu", ws_bytes, need);

  const size_t cand = (size_t)N * pl.n_strips * k;
  char* w = static_cast<char*>(ws);
  float* cand_vals = reinterpret_cast<float*>(w);
  int32_t* cand_idx = reinterpret_cast<int32_t*>(w + align256(cand * sizeof(float)));
  float* tau = reinterpret_cast<float*>(w + align256(cand * sizeof(float)) + align256(cand * sizeof(int32_t)));

  CUtensorMap tmx, tmw;
  int rc = make_tensor_map_bf16(&tmx, x_bf16, (uint64_t)N, (uint64_t)D, BM);
  if (rc != SC_OK) return rc;
  rc = make_tensor_map_bf16(&tmw, W_bf16, (uint64_t)M, (uint64_t)D, BN / pl.cg);
  if (rc != SC_OK) return rc;

  Params p;
  p.bias = bias; p.cand_vals = cand_vals; p.cand_idx = cand_idx; p.tau = tau; p.status = status_word;
  p.N = N; p.D = D; p.M = M; p.k = k;
  p.row_group = kRowGroupRows / (BM * pl.cg);
#ifdef SC_DIAG
  // diagnostics build (-DSC_DIAG) only: the shipped library reads no environment
  const char* dbg = getenv("SC_ENCODE_DEBUG");
  p.debug = dbg ? atoi(dbg) : 0;
  const char* rg_env = getenv("SC_ENCODE_ROWGROUP");
  if (rg_env && atoi(rg_env) > 0) p.row_group = atoi(rg_env);
#endif
  p.group_cols = 0; p.gm_vals = nullptr; p.gm_idx = nullptr;
  p.n_rb = pl.n_rb; p.n_ct = pl.n_ct; p.n_strips = pl.n_strips; p.stages = pl.stages; p.units = pl.units;
  p.off_lists_val = (uint32_t)pl.off_lists_val; p.off_lists_idx = (uint32_t)pl.off_lists_idx;
  p.off_gmin = (uint32_t)pl.off_gmin; p.off_gpos = (uint32_t)pl.off_gpos;
  p.off_bias = (uint32_t)pl.off_bias; p.off_bars = (uint32_t)pl.off_bars;

  cudaStream_t st = sc::as_stream(stream);
  init_tau_kernel<<<(unsigned)((N + 255) / 256), 256, 0, st>>>(tau, N);
  SC_CHECK_LAUNCH("init_tau");
  rc = launch_encoder(pl, tmx, tmw, p, st, "encode_topk_tc");
  if (rc != SC_OK) return rc;
  int kp = 1, chunks = 1;
  while (kp < k) kp <<= 1;
  while (chunks < pl.n_strips) chunks <<= 1;
  const size_t merge_smem = (size_t)4 * chunks * kp * sizeof(unsigned long long);
  if (merge_smem > 48 * 1024)
    SC_CUDA(cudaFuncSetAttribute(topk_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)merge_smem));
  topk_merge_kernel<<<(unsigned)((N + 3) / 4), 128, merge_smem, st>>>(cand_vals, cand_idx, N, pl.n_strips, k, kp,
                                                                      chunks, top_vals, top_idx);
  SC_CHECK_LAUNCH("topk_merge");
  return SC_OK;
}

extern "C" int sc_encode_groupmax(const void* x_bf16, const void* W_bf16, const float* bias, int64_t N,
                                  int64_t D, int64_t M, int k, float* top_vals, int64_t* top_idx,
                                  int32_t* status_word, void* stream) {
  SC_REQUIRE(N >= 0 && D > 0 && M > 0 && k > 0, "sc_encode_groupmax: bad shape");
  if (N == 0) return SC_OK;
  SC_REQUIRE(x_bf16 && W_bf16 && bias && top_vals && top_idx, "sc_encode_groupmax: null pointer");
  SC_REQUIRE(M % k == 0, "sc_encode_groupmax: M=%lld must be divisible by k=%d", (long long)M, k);
  const int64_t g = M / k;
  if (g % 32 != 0 || !(g % BN == 0 || BN % g == 0) || g >= (int64_t(1) << 31))
    return sc::fail(SC_ERR_UNSUPPORTED, "sc_encode_groupmax: group size %lld must be 32, 64, 128 or a multiple of 256",
                    (long long)g);
  SC_REQUIRE(D % 8 == 0, "sc_encode_groupmax: D=%lld must be a multiple of 8", (long long)D);
  SC_REQUIRE(sc::aligned(x_bf16, 16) && sc::aligned(W_bf16, 16), "sc_encode_groupmax: operands must be 16-byte aligned");
  SC_REQUIRE(N < (int64_t(1) << 31) && M < (int64_t(1) << 31), "sc_encode_groupmax: N, M must be below 2^31");
  Plan pl;
  if (make_plan(N, D, M, k, &pl, (int)g) != SC_OK || pl.n_strips < 1)
    return sc::fail(SC_ERR_UNSUPPORTED, "sc_encode_groupmax: no plan for this shape");
  if (g >= BN && (k % pl.n_strips != 0))
    return sc::fail(SC_ERR_UNSUPPORTED, "sc_encode_groupmax: no strip count divides k=%d", k);
  CUtensorMap tmx, tmw;
  int rc = make_tensor_map_bf16(&tmx, x_bf16, (uint64_t)N, (uint64_t)D, BM);
  if (rc != SC_OK) return rc;
  rc = make_tensor_map_bf16(&tmw, W_bf16, (uint64_t)M, (uint64_t)D, BN / pl.cg);
  if (rc != SC_OK) return rc;
  Params p;
  p.bias = bias; p.cand_vals = nullptr; p.cand_idx = nullptr; p.tau = nullptr; p.status = status_word;
  p.N = N; p.D = D; p.M = M; p.k = k;
#ifdef SC_DIAG
  p.debug = 0;
#endif
  p.row_group = kRowGroupRows / (BM * pl.cg);
  p.group_cols = (int)g; p.gm_vals = top_vals; p.gm_idx = top_idx;
  p.n_rb = pl.n_rb; p.n_ct = pl.n_ct; p.n_strips = pl.n_strips; p.stages = pl.stages; p.units = pl.units;
  p.off_lists_val = (uint32_t)pl.off_lists_val; p.off_lists_idx = (uint32_t)pl.off_lists_idx;
  p.off_gmin = (uint32_t)pl.off_gmin; p.off_gpos = (uint32_t)pl.off_gpos;
  p.off_bias = (uint32_t)pl.off_bias; p.off_bars = (uint32_t)pl.off_bars;
  return launch_encoder(pl, tmx, tmw, p, sc::as_stream(stream), "encode_groupmax_tc");
}
