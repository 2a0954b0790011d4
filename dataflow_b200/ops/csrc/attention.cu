// Causal varlen flash attention, forward, on tcgen05 (head_dim 128, bf16, GQA).
//
// One CTA per (128-row query tile, head, sequence).  Roles: warp 0 = TMA producer, warp 1 = MMA issuer (and TMEM owner),
// warps 2-5 = softmax: one thread per query row.  Per 128-key tile j
//     S(j)  = Q K_j^T            tcgen05.mma, both operands K-major from shared memory, accumulator in TMEM (two buffers)
//     softmax reads S(j) from TMEM (tcgen05.ld, its own lane = its own row): running max / sum in registers, P(j) as bf16
//            into shared memory in the 128-byte swizzled K-major layout the next MMA wants
//     O    += P(j) V_j           tcgen05.mma, V MN-major straight from its (keys, d) rows, O accumulates in TMEM
// The exponent base m of a row is only raised when the row maximum outgrows it by more than 2^8 (then O is rescaled in
// tensor memory, tcgen05.ld / st, after the previous P V has finished); otherwise probabilities simply use the older,
// slightly smaller base — exact in the final quotient O / l, and the common tile costs one pass over S and no read of O.
// S(j+1) and P V(j-1) run on the tensor pipe while the softmax of tile j runs on the ALUs.  K, V and P tiles are
// double-buffered.  Every wait is a bounded mbarrier wait: on a timeout the CTA raises the error word and leaves.
// Output: out (tokens, heads, 128) bf16 and lse (heads, tokens) fp32 = log sum exp(scale * s), the statistics the backward
// (library lane) consumes.
// Reference role: src/dataflow_training/kernels/flash.py:59-172 (aten varlen flash attention forward).
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "ops.h"
#include "ptx.cuh"

namespace dfb {
namespace fa {

constexpr int BM = 128, BN = 128, D = 128, UK = 16;
constexpr int CH = 128 * 128;                    // one 128-row x 64-element (128-byte) swizzled chunk: 16 KiB
constexpr int TILE = 2 * CH;                     // a 128 x 128 bf16 tile
constexpr int OFF_Q = 0, OFF_K = TILE, OFF_V = 3 * TILE, OFF_P = 5 * TILE, OFF_BAR = 7 * TILE;
constexpr int SMEM_BYTES = 7 * TILE + 256 + 1024;
constexpr float kRescaleGap = 8.f;               // log2 units the row maximum may run ahead of the exponent base
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr float kNegBig = -1e30f;

struct Bars {
  uint64_t q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[2], s_empty[2], p_full[2], pv_done[2];
  uint32_t tmem_base;
  int abort;
};

struct Params {
  const int* cu_seqlens;
  bf16* out;            // (T, hq, 128)
  float* lse;           // (hq, T)
  long long out_row_stride;     // elements between tokens in ``out``
  int T, hq, hkv;
  float sl2;            // scale * log2(e)
  int* err;
};

DFB_DEVICE float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, Params p) {
  const int seg = blockIdx.z, h = blockIdx.y;
  const int seg_start = p.cu_seqlens[seg];
  const int seg_len = p.cu_seqlens[seg + 1] - seg_start;
  const int n_qt = (seg_len + BM - 1) / BM;
  const int qt = n_qt - 1 - static_cast<int>(blockIdx.x);        // heavy tiles first
  if (qt < 0) return;                                            // the whole CTA leaves before any barrier or TMEM exists
  const int n_kv = qt + 1;
  const int kvh = h / (p.hq / p.hkv);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Bars* bar = reinterpret_cast<Bars*>(smem + OFF_BAR);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &bar->abort;

  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar->q_full, 1);
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&bar->k_full[b], 1); ptx::mbar_init(&bar->v_full[b], 1);
      ptx::mbar_init(&bar->k_empty[b], 1); ptx::mbar_init(&bar->v_empty[b], 1);
      ptx::mbar_init(&bar->s_full[b], 1); ptx::mbar_init(&bar->s_empty[b], 4);
    }
    for (int b = 0; b < 2; ++b) { ptx::mbar_init(&bar->p_full[b], 4); ptx::mbar_init(&bar->pv_done[b], 1); }
    bar->abort = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmap_q);
    ptx::prefetch_tmap(&tmap_k);
    ptx::prefetch_tmap(&tmap_v);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&bar->tmem_base, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = bar->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (ptx::elect_one()) {
      const int row0 = seg_start + qt * BM;
      ptx::mbar_expect_tx(&bar->q_full, TILE);
      for (int c = 0; c < 2; ++c) ptx::tma_load_2d(smem + OFF_Q + c * CH, &tmap_q, &bar->q_full, h * D + c * 64, row0);
      for (int j = 0; j < n_kv && !*abort_flag; ++j) {
        const int b = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int key0 = seg_start + j * BN;
        if (!ptx::mbar_wait(&bar->k_empty[b], ph ^ 1, abort_flag)) { bar->abort = 1; atomicExch(p.err, 61); break; }
        ptx::mbar_expect_tx(&bar->k_full[b], TILE);
        for (int c = 0; c < 2; ++c)
          ptx::tma_load_2d(smem + OFF_K + b * TILE + c * CH, &tmap_k, &bar->k_full[b], kvh * D + c * 64, key0);
        if (!ptx::mbar_wait(&bar->v_empty[b], ph ^ 1, abort_flag)) { bar->abort = 1; atomicExch(p.err, 62); break; }
        ptx::mbar_expect_tx(&bar->v_full[b], TILE);
        // V as the MN-major operand of P V: per 64-key block, two 64-column chunks of (64 keys x 128 bytes)
        for (int kb = 0; kb < 2; ++kb)
          for (int c = 0; c < 2; ++c)
            ptx::tma_load_2d(smem + OFF_V + b * TILE + kb * CH + c * (CH / 2), &tmap_v, &bar->v_full[b], kvh * D + c * 64, key0 + kb * 64);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (ptx::elect_one()) {
      constexpr uint32_t idesc_s = ptx::idesc_bf16_f32(BM, BN, false, false);
      constexpr uint32_t idesc_pv = ptx::idesc_bf16_f32(BM, D, false, true);
      constexpr uint64_t k_step = (UK * 2) >> 4;             // K-major operand: 16 elements = 32 bytes along the row
      constexpr uint64_t mn_step = (UK * 128) >> 4;          // MN-major operand: 16 k-rows of 128 bytes
      const uint32_t q_addr = ptx::smem_u32(smem + OFF_Q), p_addr = ptx::smem_u32(smem + OFF_P);
      bool ok = ptx::mbar_wait(&bar->q_full, 0, abort_flag);
      if (!ok) { bar->abort = 1; atomicExch(p.err, 63); }
      for (int j = 0; j <= n_kv && ok; ++j) {
        if (j < n_kv) {
          const int b = j & 1;
          const uint32_t ph = (j >> 1) & 1;
          if (!ptx::mbar_wait(&bar->k_full[b], ph, abort_flag) || !ptx::mbar_wait(&bar->s_empty[b], ph ^ 1, abort_flag)) {
            bar->abort = 1; atomicExch(p.err, 64); ok = false; break;
          }
          ptx::tc_fence_after();
          const uint32_t k_addr = ptx::smem_u32(smem + OFF_K + b * TILE);
          const uint32_t tmem_s = tmem_base + b * BN;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const uint64_t adesc = ptx::desc_kmajor_sw128(q_addr + c * CH), bdesc = ptx::desc_kmajor_sw128(k_addr + c * CH);
#pragma unroll
            for (int k = 0; k < 64 / UK; ++k) ptx::umma_bf16(tmem_s, adesc + k * k_step, bdesc + k * k_step, idesc_s, (c | k) != 0);
          }
          ptx::umma_commit(&bar->k_empty[b]);
          ptx::umma_commit(&bar->s_full[b]);
        }
        if (j >= 1) {
          const int jj = j - 1, b = jj & 1;
          const uint32_t ph = (jj >> 1) & 1;
          if (!ptx::mbar_wait(&bar->p_full[b], ph, abort_flag) || !ptx::mbar_wait(&bar->v_full[b], ph, abort_flag)) {
            bar->abort = 1; atomicExch(p.err, 65); ok = false; break;
          }
          ptx::tc_fence_after();
          const uint32_t v_addr = ptx::smem_u32(smem + OFF_V + b * TILE);
          const uint32_t tmem_o = tmem_base + 2 * BN;
#pragma unroll
          for (int kb = 0; kb < 2; ++kb) {
            const uint64_t adesc = ptx::desc_kmajor_sw128(p_addr + b * TILE + kb * CH);
            const uint64_t bdesc = ptx::desc_mnmajor_sw128(v_addr + kb * CH, CH / 2);
#pragma unroll
            for (int k = 0; k < 64 / UK; ++k)
              ptx::umma_bf16(tmem_o, adesc + k * k_step, bdesc + k * mn_step, idesc_pv, (jj | kb | k) != 0);
          }
          ptx::umma_commit(&bar->v_empty[b]);
          ptx::umma_commit(&bar->pv_done[b]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + output: one thread per query row
    const int q4 = warp & 3;
    const int r = q4 * 32 + lane;                 // row inside the tile == TMEM lane
    const int qi = qt * BM + r;                   // row inside the sequence
    const uint32_t lane_base = static_cast<uint32_t>(q4 * 32) << 16;
    const uint32_t t_o = tmem_base + 2 * BN + lane_base;
    float m = kNegBig, l = 0.f;                   // exponent base (log2 units) and the row sum relative to it
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int b = j & 1;
      // waits are made warp-uniform: the tensor-memory loads below are warp-wide instructions
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bar->s_full[b], (j >> 1) & 1, abort_flag))) { bar->abort = 1; atomicExch(p.err, 66); ok = false; break; }
      ptx::tc_fence_after();
      const uint32_t t_s = tmem_base + b * BN + lane_base;
      float t[BN];
#pragma unroll
      for (int c = 0; c < 4; ++c) ptx::tmem_ld_32x32(t_s + c * 32, reinterpret_cast<uint32_t*>(t) + c * 32);
      ptx::tmem_ld_wait();
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bar->s_empty[b]);          // S(j) is in registers: its buffer may take S(j + 2)
      float mx = kNegBig;
      if (j == n_kv - 1) {                        // the diagonal tile (it also holds the end of the sequence)
        const int key_base = j * BN;
#pragma unroll
        for (int i = 0; i < BN; ++i) {
          const int kj = key_base + i;
          t[i] = (kj > qi || kj >= seg_len) ? kNegBig : t[i] * p.sl2;
          mx = fmaxf(mx, t[i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < BN; ++i) { t[i] *= p.sl2; mx = fmaxf(mx, t[i]); }
      }
      // raise the exponent base only when the maximum ran away from it (always on the first tile); the decision is taken
      // per warp because rescaling O touches tensor memory with warp-wide instructions
      const bool raise = j == 0 || mx > m + kRescaleGap;
      if (__any_sync(0xffffffffu, raise)) {
        const float m_new = fmaxf(m, mx);
        if (j > 0) {
          // O must be complete up to tile j - 1 and no P V may be in flight while it is rescaled
          if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bar->pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag))) {
            bar->abort = 1; atomicExch(p.err, 67); ok = false; break;
          }
          ptx::tc_fence_after();
          const float alpha = ex2(m - m_new);
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t v[32];
            ptx::tmem_ld_32x32(t_o + c * 32, v);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            ptx::tmem_st_32x32(t_o + c * 32, v);
          }
          ptx::tmem_st_wait();
          l *= alpha;
        }
        m = m_new;
      }
      // P(j) goes to the buffer P V(j - 2) read: that product must be finished
      if (j >= 2) {
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bar->pv_done[b], ((j - 2) >> 1) & 1, abort_flag))) {
          bar->abort = 1; atomicExch(p.err, 68); ok = false; break;
        }
      }
      uint8_t* p_row = smem + OFF_P + b * TILE + r * 128;
      float rowsum = 0.f;
#pragma unroll
      for (int g = 0; g < BN / 8; ++g) {
        float pr[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) { pr[i] = ex2(t[g * 8 + i] - m); rowsum += pr[i]; }
        const bf16x8 pk = pack8(pr);
        // key g*8 .. g*8+7: chunk g / 8 (64 keys each), 16-byte vector g % 8 inside the 128-byte row, XOR-swizzled by the row
        *reinterpret_cast<uint4*>(p_row + (g >> 3) * CH + (((g & 7) ^ (r & 7)) << 4)) = *reinterpret_cast<const uint4*>(&pk);
      }
      l += rowsum;
      ptx::fence_proxy_async();           // the MMA reads P through the async proxy
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bar->p_full[b]);
    }
    if (ok) {
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bar->pv_done[(n_kv - 1) & 1], ((n_kv - 1) >> 1) & 1, abort_flag))) {
        bar->abort = 1; atomicExch(p.err, 69); ok = false;
      }
    }
    if (ok) {
      ptx::tc_fence_after();
      const float inv = 1.f / l;
      const long long tok = seg_start + qi;
      bf16* dst = p.out + tok * p.out_row_stride + static_cast<long long>(h) * D;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        ptx::tmem_ld_32x32(t_o + c * 32, v);
        ptx::tmem_ld_wait();
        if (qi < seg_len) {
          float o[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __uint_as_float(v[i]) * inv;
#pragma unroll
          for (int g = 0; g < 4; ++g) st8(dst + c * 32 + g * 8, pack8(o + g * 8));
        }
      }
      if (qi < seg_len) p.lse[static_cast<long long>(h) * p.T + tok] = (m + log2f(l)) * 0.6931471805599453f;
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) ptx::tmem_dealloc(tmem_base, TMEM_COLS);
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

// (tokens, heads * 128) bf16 with ``ld`` elements between tokens; boxes of 64 columns x ``box_rows`` tokens
static bool make_map(CUtensorMap* m, const void* base, uint64_t cols, uint64_t rows, uint64_t ld, uint32_t box_rows) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace fa

int* gemm_error_word_shared();

// q (T, hq, 128), k / v (T, hkv, 128): row strides in elements (views into a packed qkv are fine); out (T, hq, 128);
// lse (hq, T) fp32; cu_seqlens: nseg + 1 device ints.  Returns -2 for unsupported shapes or alignment.
int flash_fwd_sm100(const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv, void* out, long long ldo,
                    float* lse, const int* cu_seqlens, int nseg, int max_seqlen, int T, int hq, int hkv, int head_dim, float scale,
                    cudaStream_t stream) {
  using namespace fa;
  if (head_dim != D || hq % hkv || nseg <= 0 || T <= 0) return -2;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8)) return -2;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out)) & 15) return -2;
  CUtensorMap tq, tk, tv;
  bool ok = make_map(&tq, q, static_cast<uint64_t>(hq) * D, T, ldq, BM) && make_map(&tk, k, static_cast<uint64_t>(hkv) * D, T, ldk, BN) &&
            make_map(&tv, v, static_cast<uint64_t>(hkv) * D, T, ldv, 64);
  if (!ok) return -4;
  Params p;
  p.cu_seqlens = cu_seqlens; p.out = reinterpret_cast<bf16*>(out); p.lse = lse; p.out_row_stride = ldo;
  p.T = T; p.hq = hq; p.hkv = hkv; p.sl2 = scale * 1.4426950408889634f; p.err = gemm_error_word_shared();
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    configured = true;
  }
  dim3 grid((max_seqlen + BM - 1) / BM, hq, nseg);
  flash_fwd_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace dfb
