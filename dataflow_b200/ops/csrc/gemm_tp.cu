// Tensor-parallel GEMMs fused with their collective, on the CTA-pair tcgen05 pipeline.
//
//   mode 1, all-gather -> GEMM (column-parallel linear under sequence parallelism):
//       Y[M, N] = concat_r(X_r)[M, K] * W[K, N]; rank r holds the rows X_r, stored in slot r of its own gathered
//       buffer.  Four extra "copy" warps in every CTA pull the peers' row panels over NVLink (plain peer loads)
//       into the other slots, panel by panel in ring order, and bump a per-panel arrival counter; the TMA
//       producer of a tile waits for the counter of the panel its rows come from.  The main loop of the first
//       panels overlaps the transfer of the later ones and every remote row crosses NVLink exactly once.
//   mode 2, GEMM -> reduce-scatter (row-parallel linear under sequence parallelism):
//       Y_r = sum over ranks of partial[M, N] rows of rank r.  The epilogue hands each 32 x 128 B box of a tile
//       to a TMA store aimed at the staging buffer of the rank that owns those rows (peer memory; tiles bound
//       for other ranks are computed first), then releases a per-tile arrival counter on that rank.  When its
//       own tiles are done a CTA pair turns reducer: it waits for the counters of the output tiles it owns, sums
//       the ranks' partials in rank order (fp32), adds the residual and writes the final rows.
//
// Rendezvous words live in a symmetric workspace the group maps into every rank.  All waits are bounded by
// %globaltimer; on expiry the kernel records {phase, peer} in the error word, stops waiting and leaves.
// No TMA load carries a cluster-broadcast qualifier.  The reference has no such kernels (its tensor-parallel
// lane all-reduces through NCCL: src/dataflow_training/model_families/llama3/blocks.py:91-128).
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "ops.h"
#include "ptx.cuh"

namespace dfb {
namespace gemmtp {

constexpr int BM = 256, HALF_M = 128, BN = 256, HALF_N = 128, BK = 64, UK = 16;
constexpr int STAGES = 6;
constexpr int A_BYTES = HALF_M * BK * 2;
constexpr int B_BYTES = HALF_N * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int CHUNK_BYTES = 64 * BK * 2;
constexpr int TMEM_COLS = 512;
constexpr int GEMM_THREADS = 192;
constexpr int COPY_THREADS = 128;
constexpr int THREADS = GEMM_THREADS + COPY_THREADS;
constexpr int EPI_BOX_BYTES = 32 * 128;
constexpr int EPI_BYTES = 4 * 2 * EPI_BOX_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 256;
constexpr int kMaxWorld = 8;

struct Maps { CUtensorMap m[kMaxWorld]; };

struct Params {
  int M, N, K;                  // M: rows of the whole problem (all ranks' rows)
  int mode, rank, world;
  int panel_rows;               // M / world
  int group_m;
  unsigned long long timeout_ns;
  int* err;
  unsigned int* done_ctr;
  // mode 1
  const unsigned char* ag_src[kMaxWorld];   // every rank's rows X_r (peer pointers; own entry is local)
  long long ag_src_ld;                      // leading dimension of X_r in elements
  unsigned char* ag_dst;                    // local gathered A, (M, K) row-major
  unsigned int* ag_flags;                   // local, one per panel: chunks arrived (grows over launches)
  unsigned int ag_target;
  int ag_chunk_rows;
  unsigned int* ready[kMaxWorld];           // rank r's "my rows may be read, launch seq" word
  unsigned int* acks[kMaxWorld];            // rank r's "readers finished my rows" counter
  unsigned int seq, ack_expect;
  // mode 2
  unsigned int* rs_flags[kMaxWorld];        // rank d's per-tile arrival counters
  unsigned int rs_target;
  const unsigned char* rs_stage;            // local staging: [world][panel_rows][N] bf16
  void* D;                                  // final rows of this rank, (panel_rows, N) bf16
  long long ldd;
  const void* addend;                       // optional residual, same shape
  long long ld_add;
  // mode 1 output
  void* Y;                                  // (M, N) bf16, plain epilogue
  long long ldy;
};

struct SharedBarriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort;
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
DFB_DEVICE void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
DFB_DEVICE void red_release_sys_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
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

// Tile order.  mode 1: row blocks rotated so that this rank's own panel comes first and the others follow in
// ring order (the order the copy warps fetch them).  mode 2: the panels of the OTHER ranks first (their tiles
// have to travel), this rank's own panel last.
DFB_DEVICE void tile_coords(const Params& p, int tile, int n_blocks, int& mb, int& nb, int& panel) {
  const int bpp = p.panel_rows / BM;                 // row blocks per panel
  const int per_panel = bpp * n_blocks;
  const int k = tile / per_panel;
  const int r = tile - k * per_panel;
  panel = (p.rank + (p.mode == 2 ? k + 1 : k)) % p.world;
  const int gm = p.group_m < bpp ? p.group_m : bpp;
  const int per_group = gm * n_blocks;
  const int g = r / per_group;
  const int first = g * gm;
  const int rows = (bpp - first) < gm ? (bpp - first) : gm;
  const int q = r - g * per_group;
  mb = panel * bpp + first + q % rows;
  nb = q / rows;
}

template <bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_tp_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_y, const __grid_constant__ Maps stage_maps, Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + STAGES * STAGE_BYTES;
  SharedBarriers* sb = reinterpret_cast<SharedBarriers*>(epi_smem + EPI_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = ptx::cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const int m_blocks = p.M / BM, n_blocks = (p.N + BN - 1) / BN;
  const int num_tiles = m_blocks * n_blocks;
  const int k_blocks = (p.K + BK - 1) / BK;
  volatile int* abort_flag = &sb->abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { ptx::mbar_init(&sb->full[s], 1); ptx::mbar_init(&sb->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { ptx::mbar_init(&sb->tmem_full[a], 1); ptx::mbar_init(&sb->tmem_empty[a], 8); }
    sb->abort = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(&sb->tmem_base, TMEM_COLS);
    ptx::tmem_relinquish_pair();
  }
  // mode 1: tell the peers that this rank's rows may be read (the producing kernel ran earlier on this stream)
  if (p.mode == 1 && blockIdx.x == 0 && threadIdx.x == 0) {
    __threadfence_system();
    st_release_sys(p.ready[p.rank], p.seq);
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
      int have_panel = -1;
      for (int tile = cluster_id; tile < num_tiles && !*abort_flag; tile += num_clusters) {
        int mb, nb, panel;
        tile_coords(p, tile, n_blocks, mb, nb, panel);
        if (p.mode == 1 && panel != have_panel && panel != p.rank) {
          // the rows of this tile come from ``panel``: wait until every chunk of it has landed locally
          if (!wait_ge<false>(&p.ag_flags[panel], p.ag_target, p.timeout_ns, abort_flag)) {
            sb->abort = 1; atomicExch(p.err, (21 << 8) | panel); break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");      // generic-proxy copies -> visible to the TMA loads below
          have_panel = panel;
        }
        const int m0 = mb * BM + static_cast<int>(cta) * HALF_M;
        const int n0 = nb * BN + static_cast<int>(cta) * HALF_N;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          int s = it % STAGES;
          uint32_t ph = (it / STAGES) & 1;
          if (!ptx::mbar_wait(&sb->empty[s], ph ^ 1, abort_flag)) { sb->abort = 1; atomicExch(p.err, 11); break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sbm = sa + A_BYTES;
          if (cta == 0) ptx::mbar_expect_tx(&sb->full[s], 2 * STAGE_BYTES);
          ptx::tma_load_2d_pair(sa, &tmap_a, &sb->full[s], kb * BK, m0);
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < HALF_N / 64; ++c)
              ptx::tma_load_2d_pair(sbm + c * CHUNK_BYTES, &tmap_b, &sb->full[s], n0 + c * 64, kb * BK);
          } else {
            ptx::tma_load_2d_pair(sbm, &tmap_b, &sb->full[s], kb * BK, n0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (cta == 0 && ptx::elect_one()) {
      constexpr uint32_t idesc = ptx::idesc_bf16_f32(BM, BN, false, B_MN);
      uint32_t it = 0, tcount = 0;
      for (int tile = cluster_id; tile < num_tiles && !*abort_flag; tile += num_clusters, ++tcount) {
        int acc = tcount & 1;
        uint32_t aph = (tcount >> 1) & 1;
        if (!ptx::mbar_wait(&sb->tmem_empty[acc], aph ^ 1, abort_flag)) { sb->abort = 1; atomicExch(p.err, 12); break; }
        ptx::tc_fence_after();
        uint32_t tmem_d = tmem_base + acc * BN;
        bool failed = false;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          int s = it % STAGES;
          uint32_t ph = (it / STAGES) & 1;
          if (!ptx::mbar_wait(&sb->full[s], ph, abort_flag)) { sb->abort = 1; atomicExch(p.err, 13); failed = true; break; }
          ptx::tc_fence_after();
          uint32_t a_addr = ptx::smem_u32(smem + s * STAGE_BYTES);
          uint32_t b_addr = a_addr + A_BYTES;
          uint64_t adesc = ptx::desc_kmajor_sw128(a_addr);
          uint64_t bdesc = B_MN ? ptx::desc_mnmajor_sw128(b_addr, CHUNK_BYTES) : ptx::desc_kmajor_sw128(b_addr);
          constexpr uint64_t a_step = (UK * 2) >> 4;
          constexpr uint64_t b_step = (B_MN ? UK * 128 : UK * 2) >> 4;
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
    const int row_in_cta = static_cast<int>(cta) * HALF_M + q * 32;
    uint32_t cc = 0, tcount = 0;
    for (int tile = cluster_id; tile < num_tiles && !*abort_flag; tile += num_clusters, ++tcount) {
      int mb, nb, panel;
      tile_coords(p, tile, n_blocks, mb, nb, panel);
      const int acc = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      if (!ptx::mbar_wait(&sb->tmem_full[acc], aph, abort_flag)) { sb->abort = 1; atomicExch(p.err, 14); break; }
      ptx::tc_fence_after();
      const int row0 = mb * BM + row_in_cta;                    // row of the whole problem
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c, ++cc) {
        uint8_t* buf = my_smem + (cc & 1) * EPI_BOX_BYTES;
        uint8_t* my_row = buf + lane * 128;
        const int col0 = nb * BN + c * 64;
        float f[64];
        {
          uint32_t r[32], r2[32];
          ptx::tmem_ld_32x32(taddr + c * 64, r);
          ptx::tmem_ld_32x32(taddr + c * 64 + 32, r2);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) { f[i] = __uint_as_float(r[i]); f[32 + i] = __uint_as_float(r2[i]); }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const bf16x8 pk = pack8(f + j * 8);
          *reinterpret_cast<uint4*>(my_row + ((j ^ (lane & 7)) << 4)) = *reinterpret_cast<const uint4*>(&pk);
        }
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          if (col0 < p.N) {
            if (p.mode == 2) {
              // rows of panel ``panel`` go to that rank's staging slot for partials from this rank
              ptx::tma_store_2d(&stage_maps.m[panel], buf, col0, row0 - panel * p.panel_rows);
            } else {
              ptx::tma_store_2d(&tmap_y, buf, col0, row0);
            }
          }
          ptx::tma_store_commit();
          ptx::tma_store_wait_read<1>();
        }
        __syncwarp();
      }
      if (p.mode == 2) {
        // every box of this warp's share of the tile has fully landed at the owner before the counter moves
        if (lane == 0) {
          ptx::tma_store_wait<0>();
          ptx::fence_proxy_async();
          __threadfence_system();
          const int bpp = p.panel_rows / BM;
          const int t_in_panel = (mb - panel * bpp) * n_blocks + nb;
          red_release_sys_add(p.rs_flags[panel] + t_in_panel, 1u);
        }
        __syncwarp();
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(&sb->tmem_empty[acc], 0);
    }
    if (lane == 0) ptx::tma_store_wait<0>();
    __syncwarp();
  } else if (p.mode == 1) {
    // ------------------------------------------------------------------ copy warps: all-gather by peer loads
    const int t = threadIdx.x - GEMM_THREADS;                   // 0 .. 127
    const int chunks_per_panel = p.panel_rows / p.ag_chunk_rows;
    const long long row_vecs = static_cast<long long>(p.K) / 8;  // 16-byte vectors per row
    __shared__ int copy_failed;
    if (t == 0) copy_failed = 0;
    asm volatile("bar.sync 2, 128;" ::: "memory");
    // this rank's own rows already sit in their slot of the gathered buffer (that slot IS the buffer peers read),
    // so only the world - 1 remote panels are fetched, in ring order, spread over the CTAs in small chunks
    const int remote_chunks = (p.world - 1) * chunks_per_panel;
    for (int c = blockIdx.x; c < remote_chunks && !copy_failed; c += gridDim.x) {
      const int k = c / chunks_per_panel + 1;
      const int panel = (p.rank + k) % p.world;
      const int r0 = (c - (k - 1) * chunks_per_panel) * p.ag_chunk_rows;
      if (t == 0 && !wait_ge<true>(p.ready[panel], p.seq, p.timeout_ns, abort_flag)) {
        atomicExch(p.err, (22 << 8) | panel);
        copy_failed = 1;
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (copy_failed) break;
      const uint4* src = reinterpret_cast<const uint4*>(p.ag_src[panel]) + static_cast<long long>(r0) * (p.ag_src_ld / 8);
      uint4* dst = reinterpret_cast<uint4*>(p.ag_dst) + (static_cast<long long>(panel) * p.panel_rows + r0) * row_vecs;
      const long long n_vec = static_cast<long long>(p.ag_chunk_rows) * row_vecs;
      const bool dense = p.ag_src_ld == p.K;
      long long v = t;
      // four independent 16-byte peer loads in flight per thread: NVLink latency, not issue rate, is the limit
      for (; v + 3 * COPY_THREADS < n_vec; v += 4 * COPY_THREADS) {
        uint4 x[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const long long vv = v + u * COPY_THREADS;
          const long long row = dense ? 0 : vv / row_vecs;
          x[u] = __ldcg(dense ? src + vv : src + row * (p.ag_src_ld / 8) + (vv - row * row_vecs));
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) dst[v + u * COPY_THREADS] = x[u];
      }
      for (; v < n_vec; v += COPY_THREADS) {
        const long long row = v / row_vecs;
        dst[v] = __ldcg(src + row * (p.ag_src_ld / 8) + (v - row * row_vecs));
      }
      __threadfence();
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (t == 0) {
        const unsigned int prev = atomicAdd(&p.ag_flags[panel], 1u);
        // the chunk that completes a remote panel tells its owner that this rank is done reading it
        if (prev + 1u == p.ag_target) {
          __threadfence_system();
          red_release_sys_add(p.acks[panel], 1u);
        }
      }
    }
    if (copy_failed && t == 0) sb->abort = 1;
  }

  // ------------------------------------------------------------------ teardown (+ mode 2: reduce the owned rows)
  ptx::tc_fence_before();
  __syncthreads();
  if (p.mode == 2 && !*abort_flag) {
    const int bpp = p.panel_rows / BM;
    const int own_tiles = bpp * n_blocks;
    const long long slot_elems = static_cast<long long>(p.panel_rows) * p.N;        // one rank's partial of my rows
    const bf16* stage = reinterpret_cast<const bf16*>(p.rs_stage);
    __shared__ int red_ok;
    for (int tl = cluster_id; tl < own_tiles; tl += num_clusters) {
      if (threadIdx.x == 0) {
        red_ok = wait_ge<true>(p.rs_flags[p.rank] + tl, p.rs_target, p.timeout_ns, abort_flag) ? 1 : 0;
        if (!red_ok) atomicExch(p.err, (23 << 8) | p.rank);
      }
      __syncthreads();
      if (!red_ok) break;
      const int mbl = tl / n_blocks, nbl = tl - mbl * n_blocks;
      const int r_base = mbl * BM + static_cast<int>(cta) * HALF_M;     // row inside my panel
      const int c_base = nbl * BN;
      const int cols = min(BN, p.N - c_base);
      const int vec_per_row = cols / 8;
      for (int v = threadIdx.x; v < HALF_M * vec_per_row; v += THREADS) {
        const int rr = v / vec_per_row, cv = v - rr * vec_per_row;
        const long long off = static_cast<long long>(r_base + rr) * p.N + c_base + cv * 8;
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
        for (int src = 0; src < p.world; ++src) {                       // rank order: deterministic
          float fv[8];
          const uint4 x = __ldcg(reinterpret_cast<const uint4*>(stage + src * slot_elems + off));
          unpack8(*reinterpret_cast<const bf16x8*>(&x), fv);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += fv[i];
        }
        if (p.addend) {
          float fv[8];
          unpack8(ld8(reinterpret_cast<const bf16*>(p.addend) + static_cast<long long>(r_base + rr) * p.ld_add + c_base + cv * 8), fv);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += fv[i];
        }
        st8(reinterpret_cast<bf16*>(p.D) + static_cast<long long>(r_base + rr) * p.ldd + c_base + cv * 8, pack8(acc));
      }
      __syncthreads();
    }
  }
  if (p.mode == 1) {
    // the last CTA holds the kernel until every peer has finished reading this rank's rows
    __shared__ int is_last;
    __threadfence();
    if (threadIdx.x == 0) is_last = (atomicAdd(p.done_ctr, 1u) == gridDim.x - 1);
    __syncthreads();
    if (is_last && threadIdx.x == 0) {
      *p.done_ctr = 0;
      if (!wait_ge<true>(p.acks[p.rank], p.ack_expect, p.timeout_ns, abort_flag)) atomicExch(p.err, (24 << 8) | p.rank);
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

static bool make_map(CUtensorMap* m, const void* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                     uint32_t box_outer) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace gemmtp

// All-gather -> GEMM.  ``x_src[r]``: rank r's rows (panel_rows, K), leading dimension ``x_ld``; ``gathered``: local
// (world * panel_rows, K) buffer the kernel fills; ``W`` stored (K, N) (b_mn = 1) or (N, K).  ``flags``: local
// ``world`` counters; ``ready`` / ``acks``: one word per rank in the symmetric workspace.  ``launch_seq`` counts the
// launches that used these words (1, 2, ...).  Returns 0, or a negative code for shapes the kernel does not take.
int tp_ag_gemm(const unsigned long long* x_src, long long x_ld, void* gathered, const void* W, long long ldw, int b_mn, void* Y,
               long long ldy, int panel_rows, int N, int K, int rank, int world, unsigned int* flags,
               const unsigned long long* ready, const unsigned long long* acks, unsigned int launch_seq, int chunk_rows,
               double timeout_s, int* err, unsigned int* done_ctr, int num_sms, cudaStream_t stream) {
  using namespace gemmtp;
  const int M = panel_rows * world;
  if (world > kMaxWorld || world < 1 || panel_rows % BM || K % 8 || N % 8 || x_ld % 8 || ldw % 8 || ldy % 8) return -2;
  if (chunk_rows <= 0 || panel_rows % chunk_rows) return -2;
  CUtensorMap ta, tb, ty;
  Maps maps{};
  bool ok = make_map(&ta, gathered, K, M, K, BK, HALF_M);
  ok = ok && (b_mn ? make_map(&tb, W, N, K, ldw, 64, BK) : make_map(&tb, W, K, N, ldw, BK, HALF_N));
  ok = ok && make_map(&ty, Y, N, M, ldy, 64, 32);
  if (!ok) return -4;
  for (int i = 0; i < kMaxWorld; ++i) maps.m[i] = ty;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.mode = 1; p.rank = rank; p.world = world; p.panel_rows = panel_rows; p.group_m = 8;
  p.timeout_ns = static_cast<unsigned long long>(timeout_s * 1e9);
  p.err = err; p.done_ctr = done_ctr;
  for (int r = 0; r < world; ++r) {
    p.ag_src[r] = reinterpret_cast<const unsigned char*>(x_src[r]);
    p.ready[r] = reinterpret_cast<unsigned int*>(ready[r]);
    p.acks[r] = reinterpret_cast<unsigned int*>(acks[r]);
  }
  p.ag_src_ld = x_ld; p.ag_dst = reinterpret_cast<unsigned char*>(gathered); p.ag_flags = flags;
  p.ag_chunk_rows = chunk_rows;
  p.ag_target = static_cast<unsigned int>(panel_rows / chunk_rows) * launch_seq;
  p.seq = launch_seq; p.ack_expect = static_cast<unsigned int>(world - 1) * launch_seq;
  p.Y = Y; p.ldy = ldy;
  long long tiles = static_cast<long long>(M / BM) * ((N + BN - 1) / BN);
  int clusters = num_sms / 2;
  int grid = 2 * static_cast<int>(tiles < clusters ? tiles : clusters);
  auto launch = [&](auto kernel, int idx) {
    static bool configured[2] = {false, false};
    if (!configured[idx]) {
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
      configured[idx] = true;
    }
    kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(ta, tb, ty, maps, p);
  };
  if (b_mn) launch(gemm_tp_kernel<true>, 1); else launch(gemm_tp_kernel<false>, 0);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// GEMM -> reduce-scatter.  ``X``: (M, K) local activations with M = world * panel_rows; ``stage[r]``: rank r's staging
// buffer [world][panel_rows][N] bf16 (peer pointers); ``tile_flags[r]``: rank r's per-tile counters
// ((panel_rows / 256) * ceil(N / 256) words).  ``D``: this rank's final rows (panel_rows, N); ``addend`` optional.
int tp_gemm_rs(const void* X, long long ldx, const void* W, long long ldw, int b_mn, void* D, long long ldd, const void* addend,
               long long ld_add, int panel_rows, int N, int K, int rank, int world, const unsigned long long* stage,
               const unsigned long long* tile_flags, unsigned int launch_seq, double timeout_s, int* err,
               unsigned int* done_ctr, int num_sms, cudaStream_t stream) {
  using namespace gemmtp;
  const int M = panel_rows * world;
  if (world > kMaxWorld || world < 1 || panel_rows % BM || K % 8 || N % 8 || ldx % 8 || ldw % 8 || ldd % 8) return -2;
  if (addend && (ld_add % 8)) return -3;
  CUtensorMap ta, tb;
  Maps maps{};
  bool ok = make_map(&ta, X, K, M, ldx, BK, HALF_M);
  ok = ok && (b_mn ? make_map(&tb, W, N, K, ldw, 64, BK) : make_map(&tb, W, K, N, ldw, BK, HALF_N));
  const unsigned long long slot_bytes = static_cast<unsigned long long>(panel_rows) * N * 2;
  for (int r = 0; r < world && ok; ++r) {
    // the slot of rank r's staging buffer that receives partials from THIS rank
    ok = make_map(&maps.m[r], reinterpret_cast<const void*>(stage[r] + static_cast<unsigned long long>(rank) * slot_bytes), N,
                  panel_rows, N, 64, 32);
  }
  if (!ok) return -4;
  for (int r = world; r < kMaxWorld; ++r) maps.m[r] = maps.m[0];
  Params p{};
  p.M = M; p.N = N; p.K = K; p.mode = 2; p.rank = rank; p.world = world; p.panel_rows = panel_rows; p.group_m = 8;
  p.timeout_ns = static_cast<unsigned long long>(timeout_s * 1e9);
  p.err = err; p.done_ctr = done_ctr;
  for (int r = 0; r < world; ++r) p.rs_flags[r] = reinterpret_cast<unsigned int*>(tile_flags[r]);
  p.rs_target = 8u * static_cast<unsigned int>(world) * launch_seq;
  p.rs_stage = reinterpret_cast<const unsigned char*>(stage[rank]);
  p.D = D; p.ldd = ldd; p.addend = addend; p.ld_add = ld_add;
  long long tiles = static_cast<long long>(M / BM) * ((N + BN - 1) / BN);
  int clusters = num_sms / 2;
  int grid = 2 * static_cast<int>(tiles < clusters ? tiles : clusters);
  auto launch = [&](auto kernel, int idx) {
    static bool configured[2] = {false, false};
    if (!configured[idx]) {
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
      configured[idx] = true;
    }
    kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(ta, tb, ta, maps, p);
  };
  if (b_mn) launch(gemm_tp_kernel<true>, 1); else launch(gemm_tp_kernel<false>, 0);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace dfb
