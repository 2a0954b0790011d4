// bf16 GEMM on the 5th-generation tensor cores: D = A * B (+ addend) (+ bias).
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer  - cp.async.bulk.tensor tiles (128-byte swizzle) into a 4-stage
//                               shared-memory ring, completion by mbarrier transaction bytes
//   warp 1      MMA issuer    - one elected thread issues tcgen05.mma (M128 x N256 x K16, bf16 in,
//                               fp32 accumulate in tensor memory); tcgen05.commit frees ring stages
//                               and publishes finished accumulators
//   warps 2-5   epilogue      - tcgen05.ld the accumulator (TMEM -> registers), add the optional
//                               addend / bias in fp32, round once, 16-byte stores
// Two 256-column accumulators in tensor memory let the epilogue of tile i overlap the main loop of
// tile i+1.  Both operands may be K-major or MN-major in global memory (the MN-major case is loaded
// as 64-wide chunks and described to the tensor core with the MN-major descriptor form), which
// covers forward (x * W), input gradient (dy * W^T) and weight gradient (x^T * dy) without copies.
// Every barrier wait is bounded; on expiry the kernel raises ``*err`` and leaves after releasing its
// tensor memory.
//
// Replaces the reference's cuBLAS calls behind its linear seam (src/dataflow_training/blocks/linear.py:58-90).
#include <cuda.h>

#include <cstdlib>

#include <mutex>

#include "common.cuh"
#include "ops.h"
#include "ptx.cuh"

namespace dfb {

namespace gemm {

// MT = number of 128-row MMA sub-tiles a CTA stacks along M.  MT = 1: 128 x 256 tile, two TMEM
// accumulators (the epilogue of one tile overlaps the main loop of the next).  MT = 2: 256 x 256
// tile, both sub-tiles share every B stage (1.5x fewer shared-memory fill bytes per FLOP, which is
// what bounds the kernel when operands stream from L2), one accumulator set.
constexpr int SUB_M = 128, BN = 256, BK = 64, UK = 16;
constexpr int MAX_STAGES = 4;
constexpr int SUB_A_BYTES = SUB_M * BK * 2;    // 16 KiB
constexpr int B_BYTES = BN * BK * 2;           // 32 KiB
constexpr int CHUNK_BYTES = 64 * BK * 2;       // one 64-wide MN-major chunk: 8 KiB
constexpr int TMEM_COLS = 512;
constexpr int THREADS = 192;
template <int MT> struct Cfg {
  static constexpr int BM = SUB_M * MT;
  static constexpr int A_BYTES = SUB_A_BYTES * MT;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = MT == 1 ? 4 : 3;
  static constexpr int ACCS = MT == 1 ? 2 : 1;           // accumulator sets in tensor memory
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
};

struct Params {
  int M, N, K;
  void* D;               // output (bf16 or fp32), row-major, leading dimension ldd
  const void* addend;    // optional, same shape as D (may alias D: accumulate)
  const void* bias;      // optional bf16 (N)
  long long ldd, ld_add;
  int d_is_f32, add_is_f32;
  int group_m;
  int* err;
};

struct SharedBarriers {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
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

template <bool A_MN, bool B_MN, int MT>
__global__ void __launch_bounds__(THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, Params p) {
  constexpr int BM = Cfg<MT>::BM, A_BYTES = Cfg<MT>::A_BYTES, STAGE_BYTES = Cfg<MT>::STAGE_BYTES;
  constexpr int STAGES = Cfg<MT>::STAGES, ACCS = Cfg<MT>::ACCS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SharedBarriers* sb = reinterpret_cast<SharedBarriers*>(smem + STAGES * STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_blocks = (p.M + BM - 1) / BM, n_blocks = (p.N + BN - 1) / BN;
  const int num_tiles = m_blocks * n_blocks;
  const int k_blocks = (p.K + BK - 1) / BK;
  volatile int* abort_flag = &sb->abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { ptx::mbar_init(&sb->full[s], 1); ptx::mbar_init(&sb->empty[s], 1); }
    for (int a = 0; a < ACCS; ++a) { ptx::mbar_init(&sb->tmem_full[a], 1); ptx::mbar_init(&sb->tmem_empty[a], 4); }
    sb->abort = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&sb->tmem_base, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = sb->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (ptx::elect_one()) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x) {
        int mb, nb;
        tile_coords(tile, m_blocks, n_blocks, p.group_m, mb, nb);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          int s = it % STAGES;
          uint32_t ph = (it / STAGES) & 1;
          if (!ptx::mbar_wait(&sb->empty[s], ph ^ 1, abort_flag)) { sb->abort = 1; atomicExch(p.err, 1); break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sbm = sa + A_BYTES;
          ptx::mbar_expect_tx(&sb->full[s], STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              ptx::tma_load_2d(sa + c * CHUNK_BYTES, &tmap_a, &sb->full[s], mb * BM + c * 64, kb * BK);
          } else {
#pragma unroll
            for (int t = 0; t < MT; ++t)
              ptx::tma_load_2d(sa + t * SUB_A_BYTES, &tmap_a, &sb->full[s], kb * BK, mb * BM + t * SUB_M);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              ptx::tma_load_2d(sbm + c * CHUNK_BYTES, &tmap_b, &sb->full[s], nb * BN + c * 64, kb * BK);
          } else {
            ptx::tma_load_2d(sbm, &tmap_b, &sb->full[s], kb * BK, nb * BN);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (ptx::elect_one()) {
      constexpr uint32_t idesc = ptx::idesc_bf16_f32(SUB_M, BN, A_MN, B_MN);
      uint32_t it = 0, tcount = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x, ++tcount) {
        int acc = ACCS == 2 ? (tcount & 1) : 0;
        uint32_t aph = ACCS == 2 ? ((tcount >> 1) & 1) : (tcount & 1);
        if (!ptx::mbar_wait(&sb->tmem_empty[acc], aph ^ 1, abort_flag)) { sb->abort = 1; atomicExch(p.err, 2); break; }
        ptx::tc_fence_after();
        uint32_t tmem_d = tmem_base + acc * BN;
        bool failed = false;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          int s = it % STAGES;
          uint32_t ph = (it / STAGES) & 1;
          if (!ptx::mbar_wait(&sb->full[s], ph, abort_flag)) { sb->abort = 1; atomicExch(p.err, 3); failed = true; break; }
          ptx::tc_fence_after();
          uint32_t a_addr = ptx::smem_u32(smem + s * STAGE_BYTES);
          uint32_t b_addr = a_addr + A_BYTES;
          uint64_t adesc = A_MN ? ptx::desc_mnmajor_sw128(a_addr, CHUNK_BYTES) : ptx::desc_kmajor_sw128(a_addr);
          uint64_t bdesc = B_MN ? ptx::desc_mnmajor_sw128(b_addr, CHUNK_BYTES) : ptx::desc_kmajor_sw128(b_addr);
          constexpr uint64_t a_step = (A_MN ? UK * 128 : UK * 2) >> 4;   // bytes per K=16 step, in 16-byte units
          constexpr uint64_t b_step = (B_MN ? UK * 128 : UK * 2) >> 4;
          // an MN-major A sub-tile is two 64-wide chunks further on; a K-major one is SUB_A_BYTES further on
          constexpr uint64_t a_sub = (A_MN ? 2 * CHUNK_BYTES : SUB_A_BYTES) >> 4;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k)
#pragma unroll
            for (int t = 0; t < MT; ++t)
              ptx::umma_bf16(tmem_d + t * BN, adesc + t * a_sub + k * a_step, bdesc + k * b_step, idesc, (kb | k) != 0);
          ptx::umma_commit(&sb->empty[s]);          // stage reusable once these MMAs have read it
        }
        if (failed) break;
        ptx::umma_commit(&sb->tmem_full[acc]);      // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;                         // TMEM lane quarter this warp may read
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x, ++tcount) {
      int mb, nb;
      tile_coords(tile, m_blocks, n_blocks, p.group_m, mb, nb);
      int acc = ACCS == 2 ? (tcount & 1) : 0;
      uint32_t aph = ACCS == 2 ? ((tcount >> 1) & 1) : (tcount & 1);
      if (!ptx::mbar_wait(&sb->tmem_full[acc], aph, abort_flag)) { sb->abort = 1; atomicExch(p.err, 4); break; }
      ptx::tc_fence_after();
#pragma unroll 1
      for (int t = 0; t < MT; ++t) {
      const int row = mb * BM + t * SUB_M + q * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (acc + t) * BN + (static_cast<uint32_t>(q * 32) << 16);
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
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&sb->tmem_empty[acc]);
    }
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // give copies that may still be in flight time to land before shared memory is released
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------- host side
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

// 2D bf16 map: ``inner`` contiguous elements, ``outer`` rows ``ld`` elements apart.
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

}  // namespace gemm

static int* gemm_error_word() {
  static int* word = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    cudaMalloc(&word, sizeof(int));
    cudaMemset(word, 0, sizeof(int));
  });
  return word;
}

int* gemm_error_word_shared() { return gemm_error_word(); }

int gemm_bf16_2sm(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn, void* D, long long ldd,
                  int d_is_f32, const void* addend, long long ld_add, int add_is_f32, const void* bias, int M, int N, int K,
                  int num_sms, cudaStream_t stream);

int gemm_bf16_last_error() {
  int v = 0;
  cudaMemcpy(&v, gemm_error_word(), sizeof(int), cudaMemcpyDeviceToHost);
  return v;
}

// a_mn / b_mn: operand is MN-major in memory (A stored as (K, M) row-major; B stored as (K, N) row-major).
// Otherwise K-major (A stored (M, K), B stored (N, K)).  Returns 0 on success.
// 0: default path; 1 / 2: single-CTA kernel with that M stacking; 3: CTA-pair kernel (falls back when too few tiles)
static int g_gemm_mt_override = 0;
// DFB_GEMM_PATH in the environment picks the default path of the process (read once)
static int g_gemm_default_path = getenv("DFB_GEMM_PATH") ? atoi(getenv("DFB_GEMM_PATH")) : 3;
void gemm_bf16_set_mt(int mt) { g_gemm_mt_override = mt; }
void gemm_bf16_set_default_path(int path) { g_gemm_default_path = path; }

int gemm_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn, void* D, long long ldd,
              int d_is_f32, const void* addend, long long ld_add, int add_is_f32, const void* bias, int M, int N, int K,
              int num_sms, cudaStream_t stream) {
  using namespace gemm;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return -5;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -2;
  if ((ldd % (d_is_f32 ? 4 : 8)) || (reinterpret_cast<uintptr_t>(D) & 15)) return -3;
  if (addend && ((ld_add % (add_is_f32 ? 4 : 8)) || (reinterpret_cast<uintptr_t>(addend) & 15))) return -3;
  const int path = g_gemm_mt_override ? g_gemm_mt_override : g_gemm_default_path;
  if (path == 3) {
    int rc = gemm_bf16_2sm(A, lda, a_mn, B, ldb, b_mn, D, ldd, d_is_f32, addend, ld_add, add_is_f32, bias, M, N, K, num_sms, stream);
    if (rc != -6) return rc;            // -6: too few pair tiles, use the single-CTA kernel below
  }
  CUtensorMap ta, tb;
  bool ok = a_mn ? make_map(&ta, A, M, K, lda, 64, BK) : make_map(&ta, A, K, M, lda, BK, SUB_M);
  ok = ok && (b_mn ? make_map(&tb, B, N, K, ldb, 64, BK) : make_map(&tb, B, K, N, ldb, BK, BN));
  if (!ok) return -4;
  Params p;
  p.M = M; p.N = N; p.K = K;
  p.D = D; p.addend = addend; p.bias = bias;
  p.ldd = ldd; p.ld_add = ld_add; p.d_is_f32 = d_is_f32; p.add_is_f32 = add_is_f32;
  p.err = gemm_error_word();
  const long long n_blocks = (N + BN - 1) / BN;
  const long long tiles2 = ((M + 255) / 256) * n_blocks;
  // stack two M sub-tiles when that still leaves every SM at least two tiles of work
  // measured on B200: the stacked variant loses more to its un-overlapped epilogue than it gains, so it is opt-in
  (void)tiles2;
  int mt = path == 2 ? 2 : 1;
  const int bm = SUB_M * mt;
  p.group_m = mt == 2 ? 8 : 16;
  long long tiles = ((M + bm - 1) / bm) * n_blocks;
  int grid = static_cast<int>(tiles < num_sms ? tiles : num_sms);
  auto launch = [&](auto kernel, int smem, int idx) {
    static bool configured[8] = {false, false, false, false, false, false, false, false};
    if (!configured[idx]) {
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      configured[idx] = true;
    }
    kernel<<<grid, THREADS, smem, stream>>>(ta, tb, p);
  };
  const int lay = (a_mn ? 2 : 0) + (b_mn ? 1 : 0);
  if (mt == 2) {
    constexpr int smem = Cfg<2>::SMEM_BYTES;
    switch (lay) {
      case 3: launch(gemm_bf16_kernel<true, true, 2>, smem, 7); break;
      case 2: launch(gemm_bf16_kernel<true, false, 2>, smem, 6); break;
      case 1: launch(gemm_bf16_kernel<false, true, 2>, smem, 5); break;
      default: launch(gemm_bf16_kernel<false, false, 2>, smem, 4); break;
    }
  } else {
    constexpr int smem = Cfg<1>::SMEM_BYTES;
    switch (lay) {
      case 3: launch(gemm_bf16_kernel<true, true, 1>, smem, 3); break;
      case 2: launch(gemm_bf16_kernel<true, false, 1>, smem, 2); break;
      case 1: launch(gemm_bf16_kernel<false, true, 1>, smem, 1); break;
      default: launch(gemm_bf16_kernel<false, false, 1>, smem, 0); break;
    }
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace dfb
