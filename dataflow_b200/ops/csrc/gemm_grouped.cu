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
};

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

template <int MODE, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
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
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();
  ptx::tc_fence_after();
  const uint32_t tmem_base = sb->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (ptx::elect_one()) {
      uint32_t it = 0;
      for (int tile = cluster_id; tile < num_tiles && !*abort_flag; tile += num_clusters) {
        Tile t;
        if (!get_tile<MODE>(p, tile, m_blocks, n_blocks, t)) continue;
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
  } else {
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
  }

  ptx::tc_fence_before();
  __syncthreads();
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
