// bf16 GEMM on CTA pairs: D = A * B (+ addend) (+ bias), 256 x 256 output tile per pair of SMs.
//
// With one CTA per tile the 128 x 256 x 16 MMA reads 12 KiB of shared memory every 128 cycles while
// TMA fills the same shared memory at the same rate: the shared-memory port saturates near two
// thirds of tensor peak (measured: tensor pipe 61 % active, l1tex 78 %).  Pairing two SMs on one
// 256-row MMA (tcgen05 cta_group::2) halves both streams per SM: each CTA stages only its own 128
// rows of A and HALF of the tile's B rows, and the pair shares B through the MMA itself.
//
// Cluster of two CTAs along M, persistent over tiles.  Per CTA:
//   warp 0      TMA producer: own A rows + own half of B into a 6-stage ring; transaction bytes of
//               BOTH CTAs are counted on the leader's "full" barrier
//   warp 1      leader only: issues tcgen05.mma.cta_group::2; tcgen05.commit arrives on the
//               "empty" barrier of both CTAs and publishes finished accumulators to both
//   warps 2-5   epilogue for the CTA's own 128 accumulator lanes (two 256-column accumulators in
//               tensor memory, so the epilogue overlaps the next tile's main loop).  Each warp turns
//               its 32 rows into 128-byte-swizzled 32 x 128 B boxes in shared memory and hands them
//               to TMA stores (row-per-thread stores straight to global cost a quarter of the
//               throughput on short-K shapes); an addend (residual / gradient accumulation) is
//               fetched by TMA into the same box one chunk ahead
// No TMA load carries a cluster-broadcast qualifier.  Every wait is bounded.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "ops.h"
#include "ptx.cuh"

namespace dfb {
namespace gemm2 {

constexpr int BM = 256, HALF_M = 128, BN = 256, HALF_N = 128, BK = 64, UK = 16;
constexpr int STAGES = 6;
constexpr int A_BYTES = HALF_M * BK * 2;       // 16 KiB: this CTA's rows of A
constexpr int B_BYTES = HALF_N * BK * 2;       // 16 KiB: this CTA's half of B
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int CHUNK_BYTES = 64 * BK * 2;
constexpr int TMEM_COLS = 512;
constexpr int THREADS = 192;
constexpr int EPI_BOX_BYTES = 32 * 128;       // 32 rows x 128 bytes: one TMA store of one epilogue warp
constexpr int EPI_BYTES = 4 * 2 * EPI_BOX_BYTES;   // four warps, double buffered
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 256;

struct Params {
  int M, N, K;
  void* D;
  const void* addend;
  const void* bias;
  long long ldd, ld_add;
  int d_is_f32, add_is_f32;
  int group_m;
  int tma_epi;                  // epilogue through shared memory + TMA (needs addend dtype == D dtype)
  int* err;
  // fp8 operands: D[m, n] = acc[m, n] * row_scale[m] * col_scale[n] (dequantisation; either may be null = 1)
  const float* row_scale;
  const float* col_scale;
  int a_fmt, b_fmt;             // 0 = e4m3, 1 = e5m2
};

struct SharedBarriers {
  uint64_t full[STAGES];        // used in the leader: both CTAs' TMA bytes land here
  uint64_t empty[STAGES];       // per CTA: stage reusable
  uint64_t tmem_full[2];        // per CTA: accumulator ready
  uint64_t tmem_empty[2];       // used in the leader: both CTAs' epilogues drained the accumulator
  uint64_t add_full[4][2];      // per epilogue warp and box: addend bytes landed
  uint32_t tmem_base;
  int abort;
};

DFB_DEVICE void tile_coords(int tile, int m_blocks, int n_blocks, int group_m, int& mb, int& nb) {
  int per_group = group_m * n_blocks;
  int g = tile / per_group;
  int first = g * group_m;
  int gm = min(m_blocks - first, group_m);
  int r = tile - g * per_group;
  mb = first + r % gm;
  nb = r / gm;
}

// FP8: operands are one byte wide and K-major; a stage holds 128 elements of K (the same 128-byte swizzled rows)
template <bool A_MN, bool B_MN, bool FP8 = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_d, const __grid_constant__ CUtensorMap tmap_add, Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + STAGES * STAGE_BYTES;          // 1024-byte aligned (swizzle atom)
  SharedBarriers* sb = reinterpret_cast<SharedBarriers*>(epi_smem + EPI_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = ptx::cluster_ctarank();            // 0 = leader
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const int m_blocks = (p.M + BM - 1) / BM, n_blocks = (p.N + BN - 1) / BN;
  const int num_tiles = m_blocks * n_blocks;
  constexpr int BKE = FP8 ? 2 * BK : BK;        // elements of K per stage (128 bytes per row either way)
  static_assert(!FP8 || (!A_MN && !B_MN), "fp8 operands are K-major");
  const int k_blocks = (p.K + BKE - 1) / BKE;
  volatile int* abort_flag = &sb->abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { ptx::mbar_init(&sb->full[s], 1); ptx::mbar_init(&sb->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { ptx::mbar_init(&sb->tmem_full[a], 1); ptx::mbar_init(&sb->tmem_empty[a], 8); }
    for (int w = 0; w < 4; ++w) { ptx::mbar_init(&sb->add_full[w][0], 1); ptx::mbar_init(&sb->add_full[w][1], 1); }
    sb->abort = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
    if (p.tma_epi) {
      ptx::prefetch_tmap(&tmap_d);
      if (p.addend) ptx::prefetch_tmap(&tmap_add);
    }
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(&sb->tmem_base, TMEM_COLS);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();                 // both CTAs' barriers exist before anything remote touches them
  ptx::tc_fence_after();
  const uint32_t tmem_base = sb->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (ptx::elect_one()) {
      uint32_t it = 0;
      for (int tile = cluster_id; tile < num_tiles && !*abort_flag; tile += num_clusters) {
        int mb, nb;
        tile_coords(tile, m_blocks, n_blocks, p.group_m, mb, nb);
        const int m0 = mb * BM + static_cast<int>(cta) * HALF_M;
        const int n0 = nb * BN + static_cast<int>(cta) * HALF_N;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          int s = it % STAGES;
          uint32_t ph = (it / STAGES) & 1;
          if (!ptx::mbar_wait(&sb->empty[s], ph ^ 1, abort_flag)) { sb->abort = 1; atomicExch(p.err, 11); break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sbm = sa + A_BYTES;
          if (cta == 0) ptx::mbar_expect_tx(&sb->full[s], 2 * STAGE_BYTES);     // bytes of both CTAs
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < HALF_M / 64; ++c)
              ptx::tma_load_2d_pair(sa + c * CHUNK_BYTES, &tmap_a, &sb->full[s], m0 + c * 64, kb * BK);
          } else {
            ptx::tma_load_2d_pair(sa, &tmap_a, &sb->full[s], kb * BKE, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < HALF_N / 64; ++c)
              ptx::tma_load_2d_pair(sbm + c * CHUNK_BYTES, &tmap_b, &sb->full[s], n0 + c * 64, kb * BK);
          } else {
            ptx::tma_load_2d_pair(sbm, &tmap_b, &sb->full[s], kb * BKE, n0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (cta == 0 && ptx::elect_one()) {
      const uint32_t idesc = FP8 ? ptx::idesc_f8_f32(BM, BN, p.a_fmt, p.b_fmt) : ptx::idesc_bf16_f32(BM, BN, A_MN, B_MN);
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
          uint64_t adesc = A_MN ? ptx::desc_mnmajor_sw128(a_addr, CHUNK_BYTES) : ptx::desc_kmajor_sw128(a_addr);
          uint64_t bdesc = B_MN ? ptx::desc_mnmajor_sw128(b_addr, CHUNK_BYTES) : ptx::desc_kmajor_sw128(b_addr);
          constexpr uint64_t a_step = (A_MN ? UK * 128 : UK * 2) >> 4;
          constexpr uint64_t b_step = (B_MN ? UK * 128 : UK * 2) >> 4;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            // one instruction consumes 32 bytes of K per row in both kinds: 16 bf16 or 32 fp8 elements
            if (FP8) ptx::umma_f8_pair(tmem_d, adesc + k * a_step, bdesc + k * b_step, idesc, (kb | k) != 0);
            else ptx::umma_bf16_pair(tmem_d, adesc + k * a_step, bdesc + k * b_step, idesc, (kb | k) != 0);
          }
          ptx::umma_commit_pair(&sb->empty[s], 0x3);        // both CTAs may refill this stage
        }
        if (failed) break;
        ptx::umma_commit_pair(&sb->tmem_full[acc], 0x3);    // both CTAs' epilogues may drain
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs, own lanes)
    const int q = warp & 3;
    uint32_t tcount = 0;
    if (p.tma_epi) {
      // One box = this warp's 32 rows x 128 bytes of D (64 bf16 or 32 fp32 columns), 128-byte swizzled.
      const int box_cols = p.d_is_f32 ? 32 : 64;
      const int chunks = BN / box_cols;
      uint8_t* my_smem = epi_smem + q * 2 * EPI_BOX_BYTES;
      uint64_t* my_bar = sb->add_full[q];
      const bool has_add = p.addend != nullptr;
      const int row_in_cta = static_cast<int>(cta) * HALF_M + q * 32;
      uint32_t cc = 0;                       // boxes handled by this warp so far (buffer = cc & 1)
      if (has_add && lane == 0 && cluster_id < num_tiles) {
        int mb, nb;
        tile_coords(cluster_id, m_blocks, n_blocks, p.group_m, mb, nb);
        ptx::mbar_expect_tx(&my_bar[0], EPI_BOX_BYTES);
        ptx::tma_load_2d(my_smem, &tmap_add, &my_bar[0], nb * BN, mb * BM + row_in_cta);
      }
      for (int tile = cluster_id; tile < num_tiles && !*abort_flag; tile += num_clusters, ++tcount) {
        int mb, nb;
        tile_coords(tile, m_blocks, n_blocks, p.group_m, mb, nb);
        const int acc = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1;
        if (!ptx::mbar_wait(&sb->tmem_full[acc], aph, abort_flag)) { sb->abort = 1; atomicExch(p.err, 14); break; }
        ptx::tc_fence_after();
        const int row0 = mb * BM + row_in_cta;
        const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
        bool failed = false;
#pragma unroll 1
        for (int c = 0; c < chunks; ++c, ++cc) {
          const int b = cc & 1;
          uint8_t* buf = my_smem + b * EPI_BOX_BYTES;
          uint8_t* my_row = buf + lane * 128;
          const int col0 = nb * BN + c * box_cols;
          float f[64];
          {
            uint32_t r[32];
            ptx::tmem_ld_32x32(taddr + c * box_cols, r);
            if (!p.d_is_f32) {
              uint32_t r2[32];
              ptx::tmem_ld_32x32(taddr + c * box_cols + 32, r2);
              ptx::tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) f[32 + i] = __uint_as_float(r2[i]);
            } else {
              ptx::tmem_ld_wait();
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(r[i]);
          }
          if (FP8) {
            const int row = row0 + lane;
            const float rs = (p.row_scale && row < p.M) ? p.row_scale[row] : 1.f;
#pragma unroll
            for (int i = 0; i < 64; ++i)
              if (i < box_cols) f[i] *= rs * ((p.col_scale && col0 + i < p.N) ? p.col_scale[col0 + i] : 1.f);
          }
          if (p.bias) {
            const bf16* bp = reinterpret_cast<const bf16*>(p.bias) + col0;
#pragma unroll
            for (int i = 0; i < 64; ++i)
              if (i < box_cols && col0 + i < p.N) f[i] += bf2f(bp[i]);
          }
          if (has_add) {
            if (!ptx::mbar_wait(&my_bar[b], (cc >> 1) & 1, abort_flag)) { sb->abort = 1; atomicExch(p.err, 15); failed = true; break; }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint4 v = *reinterpret_cast<const uint4*>(my_row + ((j ^ (lane & 7)) << 4));
              if (p.d_is_f32) {
                f[j * 4] += __uint_as_float(v.x); f[j * 4 + 1] += __uint_as_float(v.y);
                f[j * 4 + 2] += __uint_as_float(v.z); f[j * 4 + 3] += __uint_as_float(v.w);
              } else {
                float t[8];
                unpack8(*reinterpret_cast<const bf16x8*>(&v), t);
#pragma unroll
                for (int i = 0; i < 8; ++i) f[j * 8 + i] += t[i];
              }
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 v;
            if (p.d_is_f32) {
              v = make_uint4(__float_as_uint(f[j * 4]), __float_as_uint(f[j * 4 + 1]), __float_as_uint(f[j * 4 + 2]),
                             __float_as_uint(f[j * 4 + 3]));
            } else {
              const bf16x8 pk = pack8(f + j * 8);
              v = *reinterpret_cast<const uint4*>(&pk);
            }
            *reinterpret_cast<uint4*>(my_row + ((j ^ (lane & 7)) << 4)) = v;
          }
          ptx::fence_proxy_async();          // generic-proxy writes -> visible to the TMA engine
          __syncwarp();
          if (lane == 0) {
            if (col0 < p.N && row0 < p.M) ptx::tma_store_2d(&tmap_d, buf, col0, row0);
            ptx::tma_store_commit();
            ptx::tma_store_wait_read<1>();   // the other box's previous store has left shared memory
            if (has_add) {
              // addend of the next box (same tile, or the first box of this cluster's next tile)
              int nt = tile, nc = c + 1;
              if (nc == chunks) { nt = tile + num_clusters; nc = 0; }
              if (nt < num_tiles) {
                int nmb, nnb;
                tile_coords(nt, m_blocks, n_blocks, p.group_m, nmb, nnb);
                ptx::mbar_expect_tx(&my_bar[b ^ 1], EPI_BOX_BYTES);
                ptx::tma_load_2d(my_smem + (b ^ 1) * EPI_BOX_BYTES, &tmap_add, &my_bar[b ^ 1], nnb * BN + nc * box_cols,
                                 nmb * BM + row_in_cta);
              }
            }
          }
          __syncwarp();
        }
        if (failed) break;
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_cluster(&sb->tmem_empty[acc], 0);
      }
      if (lane == 0) ptx::tma_store_wait<0>();     // every store of this warp has completed before the CTA exits
      __syncwarp();
    } else
    for (int tile = cluster_id; tile < num_tiles && !*abort_flag; tile += num_clusters, ++tcount) {
      int mb, nb;
      tile_coords(tile, m_blocks, n_blocks, p.group_m, mb, nb);
      int acc = tcount & 1;
      uint32_t aph = (tcount >> 1) & 1;
      if (!ptx::mbar_wait(&sb->tmem_full[acc], aph, abort_flag)) { sb->abort = 1; atomicExch(p.err, 14); break; }
      ptx::tc_fence_after();
      const int row = mb * BM + static_cast<int>(cta) * HALF_M + q * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(taddr + c * 32, r);
        ptx::tmem_ld_wait();
        const int col0 = nb * BN + c * 32;
        if (row_ok && col0 < p.N) {
          float f[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(r[i]);
          const int ncol = min(32, p.N - col0);
          if (p.bias) {
            const bf16* bp = reinterpret_cast<const bf16*>(p.bias) + col0;
#pragma unroll
            for (int i = 0; i < 32; ++i) if (i < ncol) f[i] += bf2f(bp[i]);
          }
          if (p.addend) {
            if (p.add_is_f32) {
              const float* ap = reinterpret_cast<const float*>(p.addend) + static_cast<long long>(row) * p.ld_add + col0;
              if (ncol == 32) {
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                  float4 t = *reinterpret_cast<const float4*>(ap + v * 4);
                  f[v * 4] += t.x; f[v * 4 + 1] += t.y; f[v * 4 + 2] += t.z; f[v * 4 + 3] += t.w;
                }
              } else {
                for (int i = 0; i < ncol; ++i) f[i] += ap[i];
              }
            } else {
              const bf16* ap = reinterpret_cast<const bf16*>(p.addend) + static_cast<long long>(row) * p.ld_add + col0;
              if (ncol == 32) {
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                  float t[8];
                  unpack8(ld8(ap + v * 8), t);
#pragma unroll
                  for (int i = 0; i < 8; ++i) f[v * 8 + i] += t[i];
                }
              } else {
                for (int i = 0; i < ncol; ++i) f[i] += bf2f(ap[i]);
              }
            }
          }
          if (p.d_is_f32) {
            float* dp = reinterpret_cast<float*>(p.D) + static_cast<long long>(row) * p.ldd + col0;
            if (ncol == 32) {
#pragma unroll
              for (int v = 0; v < 8; ++v)
                *reinterpret_cast<float4*>(dp + v * 4) = make_float4(f[v * 4], f[v * 4 + 1], f[v * 4 + 2], f[v * 4 + 3]);
            } else {
              for (int i = 0; i < ncol; ++i) dp[i] = f[i];
            }
          } else {
            bf16* dp = reinterpret_cast<bf16*>(p.D) + static_cast<long long>(row) * p.ldd + col0;
            if (ncol == 32) {
#pragma unroll
              for (int v = 0; v < 4; ++v) st8(dp + v * 8, pack8(f + v * 8));
            } else {
              for (int i = 0; i < ncol; ++i) dp[i] = f2bf(f[i]);
            }
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(&sb->tmem_empty[acc], 0);     // the leader owns the accumulator handshake
    }
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);      // let copies still in flight land
  }
  ptx::cluster_sync();                 // neither CTA leaves while its partner may still touch its memory
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
                     uint32_t box_outer, bool f32 = false, bool u8 = false) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * (u8 ? 1 : f32 ? 4 : 2)};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, u8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace gemm2

int* gemm_error_word_shared();

// Same contract as gemm_bf16 (gemm_tcgen05.cu); returns -6 when the shape is better served by the
// single-CTA kernel (too few 256 x 256 tiles), so the caller can fall back.
int gemm_bf16_2sm(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn, void* D, long long ldd,
                  int d_is_f32, const void* addend, long long ld_add, int add_is_f32, const void* bias, int M, int N, int K,
                  int num_sms, cudaStream_t stream) {
  using namespace gemm2;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return -5;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -2;
  if ((ldd % (d_is_f32 ? 4 : 8)) || (reinterpret_cast<uintptr_t>(D) & 15)) return -3;
  if (addend && ((ld_add % (add_is_f32 ? 4 : 8)) || (reinterpret_cast<uintptr_t>(addend) & 15))) return -3;
  long long tiles = static_cast<long long>((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int clusters = num_sms / 2;
  if (tiles < clusters) return -6;
  CUtensorMap ta, tb;
  bool ok = a_mn ? make_map(&ta, A, M, K, lda, 64, BK) : make_map(&ta, A, K, M, lda, BK, HALF_M);
  ok = ok && (b_mn ? make_map(&tb, B, N, K, ldb, 64, BK) : make_map(&tb, B, K, N, ldb, BK, HALF_N));
  // epilogue through TMA when the addend (if any) has D's element type; otherwise direct stores
  const bool tma_epi = !addend || (add_is_f32 != 0) == (d_is_f32 != 0);
  CUtensorMap td, tadd;
  if (tma_epi) {
    const uint32_t bc = d_is_f32 ? 32 : 64;
    ok = ok && make_map(&td, D, N, M, ldd, bc, 32, d_is_f32 != 0);
    ok = ok && make_map(&tadd, addend ? addend : D, N, M, addend ? ld_add : ldd, bc, 32, d_is_f32 != 0);
  } else {
    td = ta; tadd = ta;
  }
  if (!ok) return -4;
  Params p;
  p.M = M; p.N = N; p.K = K;
  p.D = D; p.addend = addend; p.bias = bias;
  p.ldd = ldd; p.ld_add = ld_add; p.d_is_f32 = d_is_f32; p.add_is_f32 = add_is_f32;
  p.group_m = 16;
  p.tma_epi = tma_epi ? 1 : 0;
  p.err = gemm_error_word_shared();
  p.row_scale = nullptr; p.col_scale = nullptr; p.a_fmt = 0; p.b_fmt = 0;
  int grid = 2 * static_cast<int>(tiles < clusters ? tiles : clusters);
  auto launch = [&](auto kernel, int idx) {
    static bool configured[4] = {false, false, false, false};
    if (!configured[idx]) {
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
      configured[idx] = true;
    }
    kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(ta, tb, td, tadd, p);
  };
  const int lay = (a_mn ? 2 : 0) + (b_mn ? 1 : 0);
  switch (lay) {
    case 3: launch(gemm2_bf16_kernel<true, true>, 3); break;
    case 2: launch(gemm2_bf16_kernel<true, false>, 2); break;
    case 1: launch(gemm2_bf16_kernel<false, true>, 1); break;
    default: launch(gemm2_bf16_kernel<false, false>, 0); break;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// fp8 GEMM with dequantising epilogue: D (M, N) bf16 or fp32 = (A (M, K) fp8  x  B (N, K)^T fp8) * row_scale[m] * col_scale[n]
// (+ bias) (+ addend).  Both operands K-major (rows of K contiguous), K a multiple of 16, leading dimensions multiples of 16.
int gemm_fp8_2sm(const void* A, long long lda, int a_fmt, const void* B, long long ldb, int b_fmt, void* D, long long ldd, int d_is_f32,
                 const float* row_scale, const float* col_scale, const void* addend, long long ld_add, const void* bias, int M, int N,
                 int K, int num_sms, cudaStream_t stream) {
  using namespace gemm2;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return -5;
  if ((lda % 16) || (ldb % 16) || (K % 16) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -2;
  if ((ldd % (d_is_f32 ? 4 : 8)) || (reinterpret_cast<uintptr_t>(D) & 15)) return -3;
  if (addend && ((ld_add % (d_is_f32 ? 4 : 8)) || (reinterpret_cast<uintptr_t>(addend) & 15))) return -3;
  long long tiles = static_cast<long long>((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int clusters = num_sms / 2;
  CUtensorMap ta, tb, td, tadd;
  bool ok = make_map(&ta, A, K, M, lda, 2 * BK, HALF_M, false, true) && make_map(&tb, B, K, N, ldb, 2 * BK, HALF_N, false, true);
  const uint32_t bc = d_is_f32 ? 32 : 64;
  ok = ok && make_map(&td, D, N, M, ldd, bc, 32, d_is_f32 != 0);
  ok = ok && make_map(&tadd, addend ? addend : D, N, M, addend ? ld_add : ldd, bc, 32, d_is_f32 != 0);
  if (!ok) return -4;
  Params p;
  p.M = M; p.N = N; p.K = K;
  p.D = D; p.addend = addend; p.bias = bias;
  p.ldd = ldd; p.ld_add = ld_add; p.d_is_f32 = d_is_f32; p.add_is_f32 = d_is_f32;
  p.group_m = 16;
  p.tma_epi = 1;
  p.err = gemm_error_word_shared();
  p.row_scale = row_scale; p.col_scale = col_scale; p.a_fmt = a_fmt; p.b_fmt = b_fmt;
  int grid = 2 * static_cast<int>(tiles < clusters ? tiles : clusters);
  static bool configured = false;
  auto kernel = gemm2_bf16_kernel<false, false, true>;
  if (!configured) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    configured = true;
  }
  kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(ta, tb, td, tadd, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace dfb
