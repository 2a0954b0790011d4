// Sparse-attention indexer on sm_100a: index scores on tcgen05, and a deterministic top-k row selection.
//
// (1) dsa_index_scores: I[i, j] = sum_h w[i, h] * relu(<q[i, h, :], k[j, :]>) for a block of query rows against the keys a
//     query may see (same sequence, j <= i); -inf elsewhere.  One CTA per (128 queries, 128 keys) tile.  Roles: warps 0-7 =
//     epilogue (row = TMEM lane, warps 0-3 take columns 0-63, warps 4-7 columns 64-127), warp 8 = TMA producer, warp 9 = MMA
//     issuer and TMEM owner.  The key tile stays in shared memory; the heads stream through a ring of query tiles:
//         S_h = Q_h K^T          tcgen05.mma, both operands K-major, accumulator in tensor memory (four buffers)
//         acc += w_h * relu(S_h) epilogue threads, tcgen05.ld of their own row, head weights staged in shared memory
//     so the (heads, queries, keys) intermediate of the eager form never exists.  Tiles no query of which sees a key are
//     filled with -inf without touching the tensor pipe.  Every wait is a bounded mbarrier wait; on a time-out the CTA
//     raises the error word and leaves.
// (2) dsa_topk: per row, the k largest entries as ascending key indices (-1 where fewer than k finite entries exist).
//     Radix select over the order-preserving integer image of the floats (4 passes of 8 bits, histogram in shared
//     memory), then an ordered compaction (block scans), so ties are always broken towards the smaller index: the same
//     input gives the same selection on every run.
// Reference role: src/dataflow_training/kernels/dsa.py (index-score and top-k kernels), eager anchors
// src/dataflow_training/blocks/modules/dsa_forms.py:47-110.
#include <cfloat>

#include "attention_common.cuh"
#include "ops.h"

namespace dfb {
int* gemm_error_word_shared();          // the kernels' common error word (checked by the host after a step)
namespace dsa {

constexpr int BM = 128, BN = 128, UK = 16;
constexpr int CH = 128 * 128;                    // one 128-row x 64-element (128-byte) swizzled chunk: 16 KiB
constexpr int ST = 3;                            // query-tile ring stages
constexpr int EPI_WARPS = 8, THREADS = (EPI_WARPS + 2) * 32;
constexpr int NB = 4;                            // accumulator buffers in tensor memory: the issuer runs up to three heads ahead
constexpr int TMEM_COLS = NB * BN;

struct Bars {
  uint64_t k_full, q_full[ST], q_empty[ST], s_full[NB], s_empty[NB];
  uint32_t tmem_base;
  int abort;
};

struct Params {
  const float* wgt;         // (n, H) fp32
  const int* seg_start;     // (n,) first row of the sequence each row belongs to
  float* out;               // (q1 - q0, ld): out[(i - q0) * ld + (j - key_lo)]
  long long ld;
  int n, H, q0, q1, key_lo;
  int* err;
};

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
index_scores_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k, Params p) {
  constexpr int NCH = D / 64;                    // 64-element chunks per row
  constexpr int TILE = NCH * CH;
  const int row0 = p.q0 + static_cast<int>(blockIdx.y) * BM;
  const int key0 = p.key_lo + static_cast<int>(blockIdx.x) * BN;
  const int row_end = min(row0 + BM, p.q1);
  if (row0 >= p.q1 || key0 >= p.q1) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Does any query of the tile see any key of the tile?  Sequence starts do not decrease with the row index, so the
  // tile's first row has the smallest start and its last row the largest index.
  const bool dead = key0 > row_end - 1 || key0 + BN <= p.seg_start[row0];
  if (dead) {
    if (warp < EPI_WARPS) {
      const int r = row0 + (warp & 3) * 32 + lane;
      if (r < row_end) {
        float* o = p.out + static_cast<long long>(r - p.q0) * p.ld + (key0 - p.key_lo) + (warp >> 2) * 64;
        const int lim = min(64, p.q1 - (key0 + (warp >> 2) * 64));
        for (int c = 0; c < lim; ++c) o[c] = -INFINITY;
      }
    }
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_k = smem;
  uint8_t* s_q = smem + TILE;
  float* s_w = reinterpret_cast<float*>(smem + TILE + ST * TILE);           // (H, 128): head-major, one row per thread
  Bars* bar = reinterpret_cast<Bars*>(smem + TILE + ST * TILE + static_cast<size_t>(p.H) * BM * 4);
  volatile int* abort_flag = &bar->abort;

  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar->k_full, 1);
    for (int s = 0; s < ST; ++s) { ptx::mbar_init(&bar->q_full[s], 1); ptx::mbar_init(&bar->q_empty[s], 1); }
    for (int b = 0; b < NB; ++b) { ptx::mbar_init(&bar->s_full[b], 1); ptx::mbar_init(&bar->s_empty[b], EPI_WARPS); }
    bar->abort = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmap_q);
    ptx::prefetch_tmap(&tmap_k);
  }
  if (warp == EPI_WARPS + 1) {
    ptx::tmem_alloc(&bar->tmem_base, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  // head weights of the tile's rows, transposed: s_w[h * 128 + r]
  for (int e = threadIdx.x; e < p.H * BM; e += THREADS) {
    const int r = e / p.H, h = e - r * p.H;
    s_w[h * BM + r] = row0 + r < p.n ? p.wgt[static_cast<long long>(row0 + r) * p.H + h] : 0.f;
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = bar->tmem_base;

  if (warp == EPI_WARPS) {
    // ------------------------------------------------------------------ TMA producer
    if (ptx::elect_one()) {
      ptx::mbar_expect_tx(&bar->k_full, TILE);
      for (int c = 0; c < NCH; ++c) ptx::tma_load_2d(s_k + c * CH, &tmap_k, &bar->k_full, c * 64, key0);
      for (int h = 0; h < p.H && !*abort_flag; ++h) {
        const int s = h % ST;
        const uint32_t ph = (h / ST) & 1;
        if (!ptx::mbar_wait(&bar->q_empty[s], ph ^ 1, abort_flag)) { bar->abort = 1; atomicExch(p.err, 81); break; }
        ptx::mbar_expect_tx(&bar->q_full[s], TILE);
        for (int c = 0; c < NCH; ++c) ptx::tma_load_2d(s_q + s * TILE + c * CH, &tmap_q, &bar->q_full[s], h * D + c * 64, row0);
      }
    }
  } else if (warp == EPI_WARPS + 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (ptx::elect_one()) {
      constexpr uint32_t idesc = ptx::idesc_bf16_f32(BM, BN, false, false);
      constexpr uint64_t k_step = (UK * 2) >> 4;
      const uint32_t k_addr = ptx::smem_u32(s_k);
      bool ok = ptx::mbar_wait(&bar->k_full, 0, abort_flag);
      if (!ok) { bar->abort = 1; atomicExch(p.err, 82); }
      for (int h = 0; h < p.H && ok; ++h) {
        const int s = h % ST, b = h % NB;
        if (!ptx::mbar_wait(&bar->q_full[s], (h / ST) & 1, abort_flag) || !ptx::mbar_wait(&bar->s_empty[b], ((h / NB) & 1) ^ 1, abort_flag)) {
          bar->abort = 1; atomicExch(p.err, 83); ok = false; break;
        }
        ptx::tc_fence_after();
        const uint32_t q_addr = ptx::smem_u32(s_q + s * TILE);
        const uint32_t tmem_s = tmem_base + b * BN;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          const uint64_t adesc = ptx::desc_kmajor_sw128(q_addr + c * CH), bdesc = ptx::desc_kmajor_sw128(k_addr + c * CH);
#pragma unroll
          for (int k = 0; k < 64 / UK; ++k) ptx::umma_bf16(tmem_s, adesc + k * k_step, bdesc + k * k_step, idesc, (c | k) != 0);
        }
        ptx::umma_commit(&bar->q_empty[s]);
        ptx::umma_commit(&bar->s_full[b]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: own row, 64 columns
    const int quarter = warp & 3, half = warp >> 2;
    const int rl = quarter * 32 + lane;                    // row inside the tile = TMEM lane
    const uint32_t lane_addr = (static_cast<uint32_t>(quarter * 32) << 16) + half * 64;
    float acc[64];
#pragma unroll
    for (int c = 0; c < 64; ++c) acc[c] = 0.f;
    bool ok = true;
    for (int h = 0; h < p.H; ++h) {
      const int b = h % NB;
      if (!ptx::mbar_wait(&bar->s_full[b], (h / NB) & 1, abort_flag)) { bar->abort = 1; atomicExch(p.err, 84); ok = false; break; }
      ptx::tc_fence_after();
      const float w = s_w[h * BM + rl];
      uint32_t v[64];
      ptx::tmem_ld_32x32(tmem_base + lane_addr + b * BN, v);
      ptx::tmem_ld_32x32(tmem_base + lane_addr + b * BN + 32, v + 32);
      ptx::tmem_ld_wait();
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bar->s_empty[b]);
#pragma unroll
      for (int c = 0; c < 64; ++c) acc[c] = fmaf(w, fmaxf(__uint_as_float(v[c]), 0.f), acc[c]);
    }
    const int r = row0 + rl;
    if (ok && r < row_end) {
      const int start = p.seg_start[r];
      const int j0 = key0 + half * 64;
      float* o = p.out + static_cast<long long>(r - p.q0) * p.ld + (j0 - p.key_lo);
      const int lim = min(64, p.q1 - j0);
#pragma unroll
      for (int c = 0; c < 64; ++c)
        if (c < lim) o[c] = (j0 + c <= r && j0 + c >= start) ? acc[c] : -INFINITY;
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == EPI_WARPS + 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------- top-k rows
constexpr int TK_THREADS = 256;

__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);          // larger float <=> larger unsigned key; -inf is the smallest finite image
}

// exclusive scan of one int per thread over the block; returns the thread's prefix and the block total
__device__ __forceinline__ int block_scan(int x, int* warp_sums, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = x;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int y = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += y;
  }
  __syncthreads();                                   // warp_sums may still be read from the previous scan
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  int base = 0;
  total = 0;
#pragma unroll
  for (int w = 0; w < TK_THREADS / 32; ++w) {
    const int s = warp_sums[w];
    if (w < warp) base += s;
    total += s;
  }
  return base + incl - x;
}

__global__ void __launch_bounds__(TK_THREADS)
topk_rows_kernel(const float* __restrict__ scores, long long ld, int cols, int col_base, int k, int* __restrict__ sel, int sel_ld) {
  const float* row = scores + static_cast<long long>(blockIdx.x) * ld;
  int* out = sel + static_cast<long long>(blockIdx.x) * sel_ld;
  __shared__ int hist[256];
  __shared__ int warp_sums[TK_THREADS / 32];
  __shared__ uint32_t s_prefix;
  __shared__ int s_need;
  // threshold key: the k-th largest.  After pass b, ``prefix`` holds its top 8 * (b + 1) bits and ``need`` how many
  // elements with exactly that prefix are still wanted.
  uint32_t prefix = 0;
  int need = min(k, cols);
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    const uint32_t mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int b = threadIdx.x; b < 256; b += TK_THREADS) hist[b] = 0;
    __syncthreads();
    for (int c = threadIdx.x; c < cols; c += TK_THREADS) {
      const uint32_t key = order_key(row[c]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int left = need, b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= left) break;
        left -= hist[b];
      }
      s_prefix = prefix | (static_cast<uint32_t>(b) << shift);
      s_need = left;
    }
    __syncthreads();
    prefix = s_prefix;
    need = s_need;
    __syncthreads();
  }
  // ordered compaction: everything above the threshold, and the first ``need`` entries equal to it
  const uint32_t thr = prefix;
  int run_eq = 0, run_sel = 0;
  const uint32_t dead_key = order_key(-INFINITY);
  for (int c0 = 0; c0 < cols; c0 += TK_THREADS) {
    const int c = c0 + threadIdx.x;
    const uint32_t key = c < cols ? order_key(row[c]) : 0u;
    const int eq = c < cols && key == thr;
    int tot_eq;
    const int eq_rank = run_eq + block_scan(eq, warp_sums, tot_eq);
    const int take = c < cols && key != dead_key && (key > thr || (eq && eq_rank < need));      // -inf is never selected
    int tot_sel;
    const int pos = run_sel + block_scan(take, warp_sums, tot_sel);
    if (take && pos < k) out[pos] = col_base + c;
    run_eq += tot_eq;
    run_sel += tot_sel;
  }
  for (int i = run_sel + threadIdx.x; i < k; i += TK_THREADS) out[i] = -1;
}

template <int D>
static int launch_scores(const void* q, long long ldq, const void* k, long long ldk, const float* wgt, const int* seg_start, float* out,
                         long long ld, int n, int H, int q0, int q1, int key_lo, int* err, cudaStream_t s) {
  CUtensorMap tq, tk;
  if (!fa::make_map(&tq, q, static_cast<uint64_t>(H) * D, n, ldq, BM) || !fa::make_map(&tk, k, D, n, ldk, BN)) return -2;
  constexpr int TILE = (D / 64) * CH;
  const size_t smem = static_cast<size_t>(TILE) * (1 + ST) + static_cast<size_t>(H) * BM * 4 + sizeof(Bars) + 1024 + 64;
  if (smem > 227 * 1024) return -3;
  static bool attr_done[2] = {false, false};
  if (!attr_done[D == 128]) {
    if (cudaFuncSetAttribute(index_scores_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) return -4;
    attr_done[D == 128] = true;
  }
  Params p{wgt, seg_start, out, ld, n, H, q0, q1, key_lo, err ? err : gemm_error_word_shared()};
  dim3 grid((q1 - key_lo + BN - 1) / BN, (q1 - q0 + BM - 1) / BM);
  index_scores_kernel<D><<<grid, THREADS, smem, s>>>(tq, tk, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace dsa

int dsa_index_scores(const void* q, long long ldq, const void* k, long long ldk, const float* wgt, const int* seg_start, float* out,
                     long long ld, int n, int H, int D, int q0, int q1, int key_lo, int* err, cudaStream_t s) {
  if (q1 <= q0 || key_lo < 0 || key_lo > q0 || q1 > n || ld < q1 - key_lo || H < 1) return -1;
  if (D == 128) return dsa::launch_scores<128>(q, ldq, k, ldk, wgt, seg_start, out, ld, n, H, q0, q1, key_lo, err, s);
  if (D == 64) return dsa::launch_scores<64>(q, ldq, k, ldk, wgt, seg_start, out, ld, n, H, q0, q1, key_lo, err, s);
  return -1;
}

int dsa_topk_rows(const float* scores, long long ld, int rows, int cols, int col_base, int k, int* sel, int sel_ld, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (k <= 0 || cols <= 0 || sel_ld < k) return -1;
  dsa::topk_rows_kernel<<<rows, dsa::TK_THREADS, 0, s>>>(scores, ld, cols, col_base, k, sel, sel_ld);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace dfb
