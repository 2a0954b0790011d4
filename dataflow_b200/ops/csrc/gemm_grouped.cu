// Grouped bf16 GEMMs for mixture-of-experts layers on the CTA-pair tcgen05 pipeline, scheduled from DEVICE-side
// expert tables (no host knowledge of how many rows each expert got, hence no host synchronisation).
//
// Rows of the dispatched activations are expert-major and every expert's segment is padded to whole 256-row
// tiles (ops/eager.py::moe_sort), so a row tile belongs to exactly one expert:
//   mode 0  forward / dgrad:  Y[r, :] = X[r, :] * W[e(r)]       (W stored (E, K, N), or (E, N, K) for the transpose)
//           the tile's expert comes from ``tile_expert[row tile]``; -1 marks tiles past the last expert: skipped.
//           B tiles are fetched through a 3-D tensor map whose third coordinate is the expert.
//   mode 1  wgrad:            dW[e] (+)= X_e^T * dY_e            (X (Mp, K), dY (Mp, N), dW (E, K, N))
//           one tile per (expert, 256 x 256 block of dW); the contraction runs over the expert's padded row range
//           ``offsets_pad[e] .. offsets_pad[e + 1]`` read on the device (padding rows are zero: they add nothing);
//           experts with no rows are skipped (the host zero-fills dW when it is not accumulating).
//   mode 0 + GATHER (expert parallelism: the dispatch all-to-all fused into the up-projection): the rows of X do
//           not exist locally yet.  Four extra copy warps per CTA pull them from the ranks that own the tokens
//           (``row_src[r]`` = source rank * tokens_per_rank + token; plain peer loads over NVLink) into the local X,
//           each CTA of a pair filling its own 128 rows of a tile, and bump the tile's arrival counter; the TMA
//           producer of a tile waits for that counter.  Transfer and multiplication overlap tile by tile.
// Pipeline, barriers and the TMA-store epilogue are those of gemm_tcgen05_2sm.cu.  Every wait is bounded.
// Reference role: src/dataflow_training/kernels/moe_grouped_gemm.py:190-339 (Triton, device prefix search).
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "ops.h"
#include "ptx.cuh"

namespace dfb {
namespace gemmg {

constexpr int BM = 256, HALF_M = 128, BN = 256, HALF_N = 128, BK = 64, UK = 16;
constexpr int STAGES = 6;
constexpr int A_BYTES = HALF_M * BK * 2;
constexpr int B_BYTES = HALF_N * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int CHUNK_BYTES = 64 * BK * 2;
constexpr int TMEM_COLS = 512;
constexpr int THREADS = 192;
constexpr int COPY_THREADS = 128;
constexpr int kMaxWorld = 8;
constexpr int EPI_BOX_BYTES = 32 * 128;
constexpr int EPI_BYTES = 4 * 2 * EPI_BOX_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 256;

struct Params {
  int M, N, K;                   // mode 0: M = padded rows; mode 1: M = K_w (rows of dW[e]), K unused
  int E;
  const int* tile_expert;        // mode 0
  const int* offsets_pad;        // mode 1
  int accumulate;                // mode 1: dW += (fetched through the same 3-D map)
  int group_m;
  int* err;
  // GATHER (mode 0): rows pulled from the token owners
  const unsigned char* x_src[kMaxWorld];    // every rank's (tokens_per_rank, K) activations (peer pointers)
  unsigned char* x_dst;                     // local X, (Mp, K)
  const int* row_src;                       // Mp entries: rank * tokens_per_rank + token, or -1 (padding: zero row)
  int tokens_per_rank;
  int rank, world;
  unsigned int* tile_flags;                 // local, one per row tile, zeroed in front of the launch
  unsigned int flag_target;                 // 2: each CTA of a pair fills half a tile
  unsigned int* ready[kMaxWorld];           // rank r's "my activations may be read, launch seq" word
  unsigned int* acks[kMaxWorld];            // rank r's "readers are done with my activations" counter
  unsigned int seq, ack_expect;
  unsigned long long timeout_ns;
  unsigned int* done_ctr;
};

DFB_DEVICE unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
DFB_DEVICE unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
DFB_DEVICE unsigned long long gtimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
template <bool SYS>
DFB_DEVICE bool wait_ge(const unsigned int* p, unsigned int want, unsigned long long timeout_ns, volatile int* abort_flag) {
  unsigned long long t0 = gtimer();
  for (;;) {
    unsigned int v = SYS ? ld_acquire_sys(p) : ld_acquire_gpu(p);
    if (static_cast<int>(v - want) >= 0) return true;
    if (*abort_flag || gtimer() - t0 > timeout_ns) return false;
    __nanosleep(200);
  }
}

struct SharedBarriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t add_full[4][2];
  uint32_t tmem_base;
  int abort;
};

struct Tile { int mb, nb, e, k0, kblocks; };

// MODE 0: tiles over (row tile, column tile), expert looked up; MODE 1: tiles over (expert, row block, column block).
template <int MODE>
DFB_DEVICE bool get_tile(const Params& p, int tile, int m_blocks, int n_blocks, Tile& t) {
  if (MODE == 0) {
    const int gm = p.group_m;
    const int per_group = gm * n_blocks;
    const int g = tile / per_group;
    const int first = g * gm;
    const int rows = min(m_blocks - first, gm);
    const int r = tile - g * per_group;
    t.mb = first + r % rows;
    t.nb = r / rows;
    t.e = p.tile_expert[t.mb];
    t.k0 = 0;
    t.kblocks = (p.K + BK - 1) / BK;
    return t.e >= 0;
  }
  const int per_e = m_blocks * n_blocks;
  t.e = tile / per_e;
  const int r = tile - t.e * per_e;
  t.mb = r % m_blocks;
  t.nb = r / m_blocks;
  t.k0 = p.offsets_pad[t.e];
  t.kblocks = (p.offsets_pad[t.e + 1] - t.k0) / BK;
  return t.kblocks > 0;
}

template <int MODE, bool B_MN, bool GATHER = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS + (GATHER ? COPY_THREADS : 0), 1)
gemm_grouped_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_d, Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + STAGES * STAGE_BYTES;
  SharedBarriers* sb = reinterpret_cast<SharedBarriers*>(epi_smem + EPI_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = ptx::cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const int m_blocks = (p.M + BM - 1) / BM, n_blocks = (p.N + BN - 1) / BN;
  const int num_tiles = (MODE == 0 ? 1 : p.E) * m_blocks * n_blocks;
  volatile int* abort_flag = &sb->abort;
  constexpr bool A_MN = MODE == 1;
  constexpr bool BMN = MODE == 1 ? true : B_MN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { ptx::mbar_init(&sb->full[s], 1); ptx::mbar_init(&sb->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { ptx::mbar_init(&sb->tmem_full[a], 1); ptx::mbar_init(&sb->tmem_empty[a], 8); }
    for (int w = 0; w < 4; ++w) { ptx::mbar_init(&sb->add_full[w][0], 1); ptx::mbar_init(&sb->add_full[w][1], 1); }
    sb->abort = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
    ptx::prefetch_tmap(&tmap_d);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(&sb->tmem_base, TMEM_COLS);
    ptx::tmem_relinquish_pair();
  }
  if (GATHER && blockIdx.x == 0 && threadIdx.x == 0) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.ready[p.rank]), "r"(p.seq) : "memory");
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();
  ptx::tc_fence_after();
  const uint32_t tmem_base = sb->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (ptx::elect_one()) {
      uint32_t it = 0;
      int have_tile = -1;
      for (int tile = cluster_id; tile < num_tiles && !*abort_flag; tile += num_clusters) {
        Tile t;
        if (!get_tile<MODE>(p, tile, m_blocks, n_blocks, t)) continue;
        if (GATHER && t.mb != have_tile) {
          // both halves of this row tile must have landed in the local X
          if (!wait_ge<false>(&p.tile_flags[t.mb], p.flag_target, p.timeout_ns, abort_flag)) {
            sb->abort = 1; atomicExch(p.err, (41 << 8)); break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");
          have_tile = t.mb;
        }
        const int m0 = t.mb * BM + static_cast<int>(cta) * HALF_M;
        const int n0 = t.nb * BN + static_cast<int>(cta) * HALF_N;
        for (int kb = 0; kb < t.kblocks; ++kb, ++it) {
          int s = it % STAGES;
          uint32_t ph = (it / STAGES) & 1;
          if (!ptx::mbar_wait(&sb->empty[s], ph ^ 1, abort_flag)) { sb->abort = 1; atomicExch(p.err, 31); break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sbm = sa + A_BYTES;
          if (cta == 0) ptx::mbar_expect_tx(&sb->full[s], 2 * STAGE_BYTES);
          const int kk = t.k0 + kb * BK;
          if (MODE == 1) {
            // A = X^T: (inner = K_w index, outer = row); B = dY: (inner = N_w index, outer = row)
#pragma unroll
            for (int c = 0; c < HALF_M / 64; ++c) ptx::tma_load_2d_pair(sa + c * CHUNK_BYTES, &tmap_a, &sb->full[s], m0 + c * 64, kk);
#pragma unroll
            for (int c = 0; c < HALF_N / 64; ++c) ptx::tma_load_2d_pair(sbm + c * CHUNK_BYTES, &tmap_b, &sb->full[s], n0 + c * 64, kk);
          } else {
            ptx::tma_load_2d_pair(sa, &tmap_a, &sb->full[s], kk, m0);
            if (B_MN) {
#pragma unroll
              for (int c = 0; c < HALF_N / 64; ++c)
                ptx::tma_load_3d_pair(sbm + c * CHUNK_BYTES, &tmap_b, &sb->full[s], n0 + c * 64, kk, t.e);
            } else {
              ptx::tma_load_3d_pair(sbm, &tmap_b, &sb->full[s], kk, n0, t.e);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (cta == 0 && ptx::elect_one()) {
      constexpr uint32_t idesc = ptx::idesc_bf16_f32(BM, BN, A_MN, BMN);
      uint32_t it = 0, tcount = 0;
      for (int tile = cluster_id; tile < num_tiles && !*abort_flag; tile += num_clusters) {
        Tile t;
        if (!get_tile<MODE>(p, tile, m_blocks, n_blocks, t)) continue;
        int acc = tcount & 1;
        uint32_t aph = (tcount >> 1) & 1;
        ++tcount;
        if (!ptx::mbar_wait(&sb->tmem_empty[acc], aph ^ 1, abort_flag)) { sb->abort = 1; atomicExch(p.err, 32); break; }
        ptx::tc_fence_after();
        uint32_t tmem_d = tmem_base + acc * BN;
        bool failed = false;
        for (int kb = 0; kb < t.kblocks; ++kb, ++it) {
          int s = it % STAGES;
          uint32_t ph = (it / STAGES) & 1;
          if (!ptx::mbar_wait(&sb->full[s], ph, abort_flag)) { sb->abort = 1; atomicExch(p.err, 33); failed = true; break; }
          ptx::tc_fence_after();
          uint32_t a_addr = ptx::smem_u32(smem + s * STAGE_BYTES);
          uint32_t b_addr = a_addr + A_BYTES;
          uint64_t adesc = A_MN ? ptx::desc_mnmajor_sw128(a_addr, CHUNK_BYTES) : ptx::desc_kmajor_sw128(a_addr);
          uint64_t bdesc = BMN ? ptx::desc_mnmajor_sw128(b_addr, CHUNK_BYTES) : ptx::desc_kmajor_sw128(b_addr);
          constexpr uint64_t a_step = (A_MN ? UK * 128 : UK * 2) >> 4;
          constexpr uint64_t b_step = (BMN ? UK * 128 : UK * 2) >> 4;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k)
            ptx::umma_bf16_pair(tmem_d, adesc + k * a_step, bdesc + k * b_step, idesc, (kb | k) != 0);
          ptx::umma_commit_pair(&sb->empty[s], 0x3);
        }
        if (failed) break;
        ptx::umma_commit_pair(&sb->tmem_full[acc], 0x3);
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue: boxes through shared memory + TMA
    const int q = warp & 3;
    uint8_t* my_smem = epi_smem + q * 2 * EPI_BOX_BYTES;
    uint64_t* my_bar = sb->add_full[q];
    const int row_in_cta = static_cast<int>(cta) * HALF_M + q * 32;
    const bool has_add = MODE == 1 && p.accumulate;
    uint32_t cc = 0, tcount = 0;
    for (int tile = cluster_id; tile < num_tiles && !*abort_flag; tile += num_clusters) {
      Tile t;
      if (!get_tile<MODE>(p, tile, m_blocks, n_blocks, t)) continue;
      const int acc = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      ++tcount;
      if (!ptx::mbar_wait(&sb->tmem_full[acc], aph, abort_flag)) { sb->abort = 1; atomicExch(p.err, 34); break; }
      ptx::tc_fence_after();
      const int row0 = t.mb * BM + row_in_cta;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      bool failed = false;
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c, ++cc) {
        const int b = cc & 1;
        uint8_t* buf = my_smem + b * EPI_BOX_BYTES;
        uint8_t* my_row = buf + lane * 128;
        const int col0 = t.nb * BN + c * 64;
        if (has_add) {
          // the gradient block already in memory: fetched into the box, summed in place (this warp owns the box)
          if (lane == 0) {
            ptx::mbar_expect_tx(&my_bar[b], EPI_BOX_BYTES);
            ptx::tma_load_3d(buf, &tmap_d, &my_bar[b], col0, row0, t.e);
          }
        }
        float f[64];
        {
          uint32_t r[32], r2[32];
          ptx::tmem_ld_32x32(taddr + c * 64, r);
          ptx::tmem_ld_32x32(taddr + c * 64 + 32, r2);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) { f[i] = __uint_as_float(r[i]); f[32 + i] = __uint_as_float(r2[i]); }
        }
        if (has_add) {
          if (!ptx::mbar_wait(&my_bar[b], (cc >> 1) & 1, abort_flag)) { sb->abort = 1; atomicExch(p.err, 35); failed = true; break; }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint4 v = *reinterpret_cast<const uint4*>(my_row + ((j ^ (lane & 7)) << 4));
            float tt[8];
            unpack8(*reinterpret_cast<const bf16x8*>(&v), tt);
#pragma unroll
            for (int i = 0; i < 8; ++i) f[j * 8 + i] += tt[i];
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const bf16x8 pk = pack8(f + j * 8);
          *reinterpret_cast<uint4*>(my_row + ((j ^ (lane & 7)) << 4)) = *reinterpret_cast<const uint4*>(&pk);
        }
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          if (col0 < p.N && row0 < p.M) {
            if (MODE == 1) ptx::tma_store_3d(&tmap_d, buf, col0, row0, t.e);
            else ptx::tma_store_2d(&tmap_d, buf, col0, row0);
          }
          ptx::tma_store_commit();
          ptx::tma_store_wait_read<1>();
        }
        __syncwarp();
      }
      if (failed) break;
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(&sb->tmem_empty[acc], 0);
    }
    if (lane == 0) ptx::tma_store_wait<0>();
    __syncwarp();
  } else if (GATHER) {
    // ------------------------------------------------------------------ copy warps: the dispatch all-to-all
    const int t = threadIdx.x - THREADS;                         // 0 .. 127
    const long long row_vecs = static_cast<long long>(p.K) / 8;   // 16-byte vectors per row
    __shared__ int copy_failed;
    __shared__ int srcs[HALF_M];
    if (t == 0) copy_failed = 0;
    asm volatile("bar.sync 2, 128;" ::: "memory");
    // every peer's activations must be final before the first remote row is read
    if (t < p.world && t != p.rank) {
      if (!wait_ge<true>(p.ready[t], p.seq, p.timeout_ns, abort_flag)) { atomicExch(p.err, (42 << 8) | t); copy_failed = 1; }
    }
    asm volatile("bar.sync 2, 128;" ::: "memory");
    // row tiles in the order the GEMM consumes them; this CTA fills its own 128 rows of each
    for (int mb = cluster_id; mb < m_blocks && !copy_failed; mb += num_clusters) {
      if (p.tile_expert[mb] < 0) continue;
      const long long r0 = static_cast<long long>(mb) * BM + static_cast<long long>(cta) * HALF_M;
      srcs[t] = p.row_src[r0 + t];
      asm volatile("bar.sync 2, 128;" ::: "memory");
      uint4* dst = reinterpret_cast<uint4*>(p.x_dst) + r0 * row_vecs;
      const long long n_vec = static_cast<long long>(HALF_M) * row_vecs;
      // sixteen 16-byte loads in flight per thread: a peer load takes microseconds, and 128 threads x 16 x 16 bytes per CTA
      // are what it takes to keep NVLink busy while the GEMM warps of the same CTA multiply
      constexpr int UNR = 16;
      for (long long v = t; v < n_vec; v += UNR * COPY_THREADS) {
        uint4 x[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          const long long vv = v + u * COPY_THREADS;
          x[u] = make_uint4(0, 0, 0, 0);
          if (vv < n_vec) {
            const int row = static_cast<int>(vv / row_vecs);
            const int s = srcs[row];
            if (s >= 0) {
              const int rk = s / p.tokens_per_rank, tok = s - rk * p.tokens_per_rank;
              x[u] = __ldcg(reinterpret_cast<const uint4*>(p.x_src[rk]) + static_cast<long long>(tok) * row_vecs + (vv - row * row_vecs));
            }
          }
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          const long long vv = v + u * COPY_THREADS;
          if (vv < n_vec) dst[vv] = x[u];
        }
      }
      __threadfence();
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (t == 0) atomicAdd(&p.tile_flags[mb], 1u);
    }
    if (copy_failed && t == 0) sb->abort = 1;
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (GATHER) {
    // the last CTA tells every peer that this rank is done reading, then holds the kernel until every peer is done
    // reading this rank's activations
    __shared__ int is_last;
    __threadfence();
    if (threadIdx.x == 0) is_last = (atomicAdd(p.done_ctr, 1u) == gridDim.x - 1);
    __syncthreads();
    if (is_last && threadIdx.x == 0) {
      *p.done_ctr = 0;
      __threadfence_system();
      for (int r = 0; r < p.world; ++r)
        if (r != p.rank) asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.acks[r]), "r"(1u) : "memory");
      if (!wait_ge<true>(p.acks[p.rank], p.ack_expect, p.timeout_ns, abort_flag)) atomicExch(p.err, (43 << 8) | p.rank);
    }
  }
  if (*abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  ptx::cluster_sync();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess) fn = reinterpret_cast<EncodeFn>(p);
  });
  return fn;
}

static bool map2(CUtensorMap* m, const void* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t bi, uint32_t bo) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {bi, bo};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// (E, outer, inner) row-major stack of matrices
static bool map3(CUtensorMap* m, const void* base, uint64_t inner, uint64_t outer, uint64_t e, uint32_t bi, uint32_t bo) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {inner, outer, e};
  cuuint64_t strides[2] = {inner * 2, inner * outer * 2};
  cuuint32_t box[3] = {bi, bo, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace gemmg

int* gemm_error_word_shared();

// Y (Mp, N) = X (Mp, K) * W[expert of the row tile].  ``w_kn`` = 1: W is (E, K, N); 0: W is (E, N, K) (dgrad through the
// transpose).  ``tile_expert``: Mp / 256 device ints.  Mp must be a multiple of 256.
int moe_grouped_mm(const void* X, const void* W, void* Y, const int* tile_expert, int Mp, int N, int K, int E, int w_kn,
                   int num_sms, cudaStream_t stream) {
  using namespace gemmg;
  if (Mp <= 0) return 0;
  if (Mp % BM || N % 8 || K % 8) return -2;
  CUtensorMap ta, tb, td;
  bool ok = map2(&ta, X, K, Mp, K, BK, HALF_M);
  ok = ok && (w_kn ? map3(&tb, W, N, K, E, 64, BK) : map3(&tb, W, K, N, E, BK, HALF_N));
  ok = ok && map2(&td, Y, N, Mp, N, 64, 32);
  if (!ok) return -4;
  Params p{};
  p.M = Mp; p.N = N; p.K = K; p.E = E; p.tile_expert = tile_expert; p.group_m = 4; p.err = gemm_error_word_shared();
  long long tiles = static_cast<long long>(Mp / BM) * ((N + BN - 1) / BN);
  int clusters = num_sms / 2;
  int grid = 2 * static_cast<int>(tiles < clusters ? tiles : clusters);
  auto launch = [&](auto kernel, int idx) {
    static bool configured[2] = {false, false};
    if (!configured[idx]) {
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
      configured[idx] = true;
    }
    kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(ta, tb, td, p);
  };
  if (w_kn) launch(gemm_grouped_kernel<0, true>, 1); else launch(gemm_grouped_kernel<0, false>, 0);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Expert-parallel dispatch fused with the grouped up-projection: like moe_grouped_mm, but the rows of X are pulled
// from the ranks that own the tokens while the GEMM runs.  ``x_src[r]``: rank r's (tokens_per_rank, K) activations
// (peer pointers); ``X``: the local (Mp, K) matrix the kernel fills; ``row_src``: Mp device ints (global token or -1).
int moe_grouped_mm_gather(const unsigned long long* x_src, void* X, const int* row_src, const void* W, void* Y,
                          const int* tile_expert, int Mp, int N, int K, int E, int w_kn, int tokens_per_rank, int rank,
                          int world, unsigned int* tile_flags, const unsigned long long* ready, const unsigned long long* acks,
                          unsigned int launch_seq, double timeout_s, int* err, unsigned int* done_ctr, int num_sms, cudaStream_t stream) {
  using namespace gemmg;
  if (Mp <= 0) return 0;
  if (Mp % BM || N % 8 || K % 8 || world > kMaxWorld) return -2;
  CUtensorMap ta, tb, td;
  bool ok = map2(&ta, X, K, Mp, K, BK, HALF_M);
  ok = ok && (w_kn ? map3(&tb, W, N, K, E, 64, BK) : map3(&tb, W, K, N, E, BK, HALF_N));
  ok = ok && map2(&td, Y, N, Mp, N, 64, 32);
  if (!ok) return -4;
  Params p{};
  p.M = Mp; p.N = N; p.K = K; p.E = E; p.tile_expert = tile_expert; p.group_m = 4; p.err = err;
  for (int r = 0; r < world; ++r) {
    p.x_src[r] = reinterpret_cast<const unsigned char*>(x_src[r]);
    p.ready[r] = reinterpret_cast<unsigned int*>(ready[r]);
    p.acks[r] = reinterpret_cast<unsigned int*>(acks[r]);
  }
  p.x_dst = reinterpret_cast<unsigned char*>(X); p.row_src = row_src; p.tokens_per_rank = tokens_per_rank;
  // arrival counters start from zero every launch (tiles past the last expert are never filled)
  cudaMemsetAsync(tile_flags, 0, sizeof(unsigned int) * (Mp / BM), stream);
  p.rank = rank; p.world = world; p.tile_flags = tile_flags; p.flag_target = 2u;
  p.seq = launch_seq; p.ack_expect = static_cast<unsigned int>(world - 1) * launch_seq;
  p.timeout_ns = static_cast<unsigned long long>(timeout_s * 1e9); p.done_ctr = done_ctr;
  int clusters = num_sms / 2;
  int grid = 2 * clusters;          // every pair takes part in the copy, whatever the tile count
  auto launch = [&](auto kernel, int idx) {
    static bool configured[2] = {false, false};
    if (!configured[idx]) {
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
      configured[idx] = true;
    }
    kernel<<<grid, THREADS + COPY_THREADS, SMEM_BYTES, stream>>>(ta, tb, td, p);
  };
  if (w_kn) launch(gemm_grouped_kernel<0, true, true>, 1); else launch(gemm_grouped_kernel<0, false, true>, 0);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// dW[e] (Kw, N) (+)= X_e^T * dY_e over the rows offsets_pad[e] .. offsets_pad[e + 1] (multiples of 256).
int moe_grouped_wgrad(const void* X, const void* dY, void* dW, const int* offsets_pad, int Mp, int Kw, int N, int E,
                      int accumulate, int num_sms, cudaStream_t stream) {
  using namespace gemmg;
  if (E <= 0) return 0;
  if (Kw % 8 || N % 8) return -2;
  if (!accumulate) {
    cudaError_t rc = cudaMemsetAsync(dW, 0, static_cast<size_t>(E) * Kw * N * 2, stream);     // experts without rows stay zero
    if (rc != cudaSuccess) return -1;
  }
  CUtensorMap ta, tb, td;
  bool ok = map2(&ta, X, Kw, Mp, Kw, 64, BK);
  ok = ok && map2(&tb, dY, N, Mp, N, 64, BK);
  ok = ok && map3(&td, dW, N, Kw, E, 64, 32);
  if (!ok) return -4;
  Params p{};
  p.M = Kw; p.N = N; p.K = 0; p.E = E; p.offsets_pad = offsets_pad; p.accumulate = accumulate; p.group_m = 4;
  p.err = gemm_error_word_shared();
  long long tiles = static_cast<long long>(E) * ((Kw + BM - 1) / BM) * ((N + BN - 1) / BN);
  int clusters = num_sms / 2;
  int grid = 2 * static_cast<int>(tiles < clusters ? tiles : clusters);
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(gemm_grouped_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    configured = true;
  }
  gemm_grouped_kernel<1, true><<<grid, THREADS, SMEM_BYTES, stream>>>(ta, tb, td, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace dfb
