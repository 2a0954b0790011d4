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
#include <cstdlib>

#include "attention_common.cuh"
#include "ops.h"

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

}  // namespace fa


// ============================================================================ two query tiles per CTA
// The kernel above keeps the tensor pipe waiting for its single softmax warpgroup and moves P through shared memory.  This one
// gives a CTA TWO 128-row query tiles (256 consecutive queries of one head) and one softmax warpgroup per tile, and keeps P
// in tensor memory: a softmax thread pulls its row of S out of tensor memory, exponentiates it and stores it back over the
// same columns as packed bf16 pairs; the P V product takes that as its A operand straight from tensor memory.  Shared
// memory then carries only Q, K and V (the operand reads of the tensor pipe and the P round trip were what bounded the
// kernel above), and the tensor pipe works on one tile while the ALUs work on the other:
//     tensor pipe:  S0(0) S1(0) | O0 += P0(0) V_0, S0(1) | O1 += P1(0) V_0, S1(1) | O0 += P0(1) V_1, S0(2) | ...
// Tensor memory: S0/P0 | S1/P1 | O0 | O1, 128 columns each.  Shared memory: Q0, Q1 and a ring of four K / V tiles (K_j, V_j
// alternate).  The exponent base is raised lazily as in the kernel above.
namespace fa2 {

constexpr int BM = 128, BN = 128, D = 128, UK = 16;
constexpr int CH = 128 * 128;                    // one 128-row x 64-element (128-byte) swizzled chunk: 16 KiB
constexpr int TILE = 2 * CH;
constexpr int KV_SLOTS = 4;
constexpr int OFF_Q = 0, OFF_KV = 2 * TILE, OFF_BAR = OFF_KV + KV_SLOTS * TILE;
constexpr int SMEM_BYTES = OFF_BAR + 512 + 1024;
constexpr float kRescaleGap = 8.f;
constexpr int THREADS = 384;                     // warpgroup 0: TMA warp, MMA warp, two idle; warpgroups 1 / 2: softmax of query tile 0 / 1
// Register budgets after the role split: a warpgroup that asks for more (setmaxnreg.inc) can only take what warpgroups of the
// same CTA gave back, and blocks until it gets it.  Launched with 168 each (12 warps), the control warpgroup returns
// (168 - 48) x 128 registers and the two softmax warpgroups take (216 - 168) x 256.
constexpr int kLaunchRegs = 168, kCtrlRegs = 48, kSoftmaxRegs = 216;
static_assert((kLaunchRegs - kCtrlRegs) * 128 >= (kSoftmaxRegs - kLaunchRegs) * 256, "setmaxnreg.inc would wait forever");
constexpr int TMEM_COLS = 512;
constexpr float kNegBig = -1e30f;

struct Bars {
  uint64_t q_full[2], kv_full[KV_SLOTS], kv_empty[KV_SLOTS], s_full[2], p_half[2], p_full[2], pv_done[2];
  uint32_t tmem_base;
  int abort;
};

using fa::Params;
using fa::ex2;

#define DFB_FA_FAIL(code) do { bar->abort = 1; atomicExch(p.err, (code)); } while (0)

// kTrace: CTA (0, 0, 0) records clock64() stamps of its first 32 key tiles into ``trace`` — per tile 8 slots for each of
// three observers (softmax thread 0 of either query tile, the MMA thread).  A profiling aid: the regular launch passes false.
constexpr int kTraceTiles = 32, kTraceSlots = 8;
#define DFB_STAMP(who, j, slot)                                                                                       \
  do { if (kTrace && trace_on && (j) < kTraceTiles) trace[((who) * kTraceTiles + (j)) * kTraceSlots + (slot)] = clock64(); } while (0)

template <bool kTrace>
__global__ void __launch_bounds__(THREADS, 1)
flash_fwd2_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, Params p, long long* trace) {
  const bool trace_on = kTrace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
  const int seg = blockIdx.y, h = blockIdx.x;
  const int seg_start = p.cu_seqlens[seg];
  const int seg_len = p.cu_seqlens[seg + 1] - seg_start;
  const int n_pairs = (seg_len + 2 * BM - 1) / (2 * BM);
  const int pt = n_pairs - 1 - static_cast<int>(blockIdx.z);      // the grid's slowest index: the heaviest pairs of every head first
  if (pt < 0) return;                                            // the whole CTA leaves before any barrier or TMEM exists
  const bool has1 = (2 * pt + 1) * BM < seg_len;                 // does the second query tile hold any row of the sequence
  const int n0 = 2 * pt + 1, n1 = has1 ? 2 * pt + 2 : 0;         // key tiles each query tile attends to
  const int n_tot = has1 ? n1 : n0;
  const int kvh = h / (p.hq / p.hkv);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Bars* bar = reinterpret_cast<Bars*>(smem + OFF_BAR);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &bar->abort;

  if (threadIdx.x == 0) {
    for (int t = 0; t < 2; ++t) {
      ptx::mbar_init(&bar->q_full[t], 1);
      ptx::mbar_init(&bar->s_full[t], 1);
      ptx::mbar_init(&bar->p_half[t], 4); ptx::mbar_init(&bar->p_full[t], 4); ptx::mbar_init(&bar->pv_done[t], 1);
    }
    for (int b = 0; b < KV_SLOTS; ++b) { ptx::mbar_init(&bar->kv_full[b], 1); ptx::mbar_init(&bar->kv_empty[b], 1); }
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
  // register budgets: the softmax threads hold a whole row of scores (128 registers) plus what they are computing, the
  // control warps need little; each role branch opens with its own setmaxnreg

  if (warp < 4) {
   ptx::setmaxnreg_dec<kCtrlRegs>();
   if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (ptx::elect_one()) {
      for (int t = 0; t < (has1 ? 2 : 1); ++t) {
        const int row0 = seg_start + (2 * pt + t) * BM;
        ptx::mbar_expect_tx(&bar->q_full[t], TILE);
        for (int c = 0; c < 2; ++c) ptx::tma_load_2d(smem + OFF_Q + t * TILE + c * CH, &tmap_q, &bar->q_full[t], h * D + c * 64, row0);
      }
      // loads alternate K_0, V_0, K_1, V_1, ...: load L goes to ring slot L % KV_SLOTS
      for (int L = 0; L < 2 * n_tot && !*abort_flag; ++L) {
        const int slot = L % KV_SLOTS, use = L / KV_SLOTS, j = L >> 1;
        const int key0 = seg_start + j * BN;
        if (use > 0 && !ptx::mbar_wait(&bar->kv_empty[slot], (use - 1) & 1, abort_flag)) { DFB_FA_FAIL(71); break; }
        uint8_t* dst = smem + OFF_KV + slot * TILE;
        ptx::mbar_expect_tx(&bar->kv_full[slot], TILE);
        if ((L & 1) == 0) {
          for (int c = 0; c < 2; ++c) ptx::tma_load_2d(dst + c * CH, &tmap_k, &bar->kv_full[slot], kvh * D + c * 64, key0);
        } else {
          // V as the MN-major operand of P V: per 64-key block, two 64-column chunks of (64 keys x 128 bytes)
          for (int kb = 0; kb < 2; ++kb)
            for (int c = 0; c < 2; ++c)
              ptx::tma_load_2d(dst + kb * CH + c * (CH / 2), &tmap_v, &bar->kv_full[slot], kvh * D + c * 64, key0 + kb * 64);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (ptx::elect_one()) {
      constexpr uint32_t idesc_s = ptx::idesc_bf16_f32(BM, BN, false, false);
      constexpr uint32_t idesc_pv = ptx::idesc_bf16_f32(BM, D, false, true);
      constexpr uint64_t k_step = (UK * 2) >> 4;             // K-major operand: 16 elements = 32 bytes along the row
      constexpr uint64_t mn_step = (UK * 128) >> 4;          // MN-major operand: 16 k-rows of 128 bytes
      const uint32_t q_addr = ptx::smem_u32(smem + OFF_Q), kv_addr = ptx::smem_u32(smem + OFF_KV);
      bool ok = ptx::mbar_wait(&bar->q_full[0], 0, abort_flag) && (!has1 || ptx::mbar_wait(&bar->q_full[1], 0, abort_flag));
      if (!ok) DFB_FA_FAIL(73);
      auto issue_s = [&](int t, int j) {                    // S_t(j) = Q_t K_j^T into the tile's S / P columns
        const uint32_t k_addr = kv_addr + ((2 * j) % KV_SLOTS) * TILE, tmem_s = tmem_base + t * BN;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const uint64_t adesc = ptx::desc_kmajor_sw128(q_addr + t * TILE + c * CH), bdesc = ptx::desc_kmajor_sw128(k_addr + c * CH);
#pragma unroll
          for (int k = 0; k < 64 / UK; ++k) ptx::umma_bf16(tmem_s, adesc + k * k_step, bdesc + k * k_step, idesc_s, (c | k) != 0);
        }
        ptx::umma_commit(&bar->s_full[t]);
      };
      if (ok) {
        if (!ptx::mbar_wait(&bar->kv_full[0], 0, abort_flag)) { DFB_FA_FAIL(74); ok = false; }
      }
      if (ok) {
        ptx::tc_fence_after();
        issue_s(0, 0);
        if (has1) issue_s(1, 0);
        ptx::umma_commit(&bar->kv_empty[0]);
      }
      for (int j = 0; j < n_tot && ok; ++j) {
        const int Lv = 2 * j + 1, vslot = Lv % KV_SLOTS, Lk = 2 * j + 2, kslot = Lk % KV_SLOTS;
        const bool next = j + 1 < n_tot;
        if (!ptx::mbar_wait(&bar->kv_full[vslot], (Lv / KV_SLOTS) & 1, abort_flag) ||
            (next && !ptx::mbar_wait(&bar->kv_full[kslot], (Lk / KV_SLOTS) & 1, abort_flag))) { DFB_FA_FAIL(76); ok = false; break; }
        const uint32_t v_addr = kv_addr + vslot * TILE;
        for (int t = 0; t < 2 && ok; ++t) {
          const int nt = t ? n1 : n0;
          if (j >= nt) continue;
          DFB_STAMP(2, j, 4 * t + 0);
          const uint32_t tmem_o = tmem_base + (2 + t) * BN, tmem_p = tmem_base + t * BN;
          // P arrives in two halves of 64 keys: the product over the first runs while the second is exponentiated
#pragma unroll
          for (int kb = 0; kb < 2; ++kb) {
            if (!ptx::mbar_wait(kb ? &bar->p_full[t] : &bar->p_half[t], j & 1, abort_flag)) { DFB_FA_FAIL(77); ok = false; break; }
            if (kb == 0) DFB_STAMP(2, j, 4 * t + 1);
            ptx::tc_fence_after();
            const uint64_t bdesc = ptx::desc_mnmajor_sw128(v_addr + kb * CH, CH / 2);
#pragma unroll
            for (int k = 0; k < 64 / UK; ++k)
              ptx::umma_bf16_ts(tmem_o, tmem_p + (kb * 4 + k) * (UK / 2), bdesc + k * mn_step, idesc_pv, (j | kb | k) != 0);
          }
          if (!ok) break;
          ptx::umma_commit(&bar->pv_done[t]);
          if (j + 1 < nt) issue_s(t, j + 1);                 // ordered behind the product that read P_t(j) from the same columns
          DFB_STAMP(2, j, 4 * t + 2);
        }
        if (!ok) break;
        ptx::umma_commit(&bar->kv_empty[vslot]);
        if (next) ptx::umma_commit(&bar->kv_empty[kslot]);
      }
    }
   }
  } else {
    ptx::setmaxnreg_inc<kSoftmaxRegs>();
    // ------------------------------------------------------------------ softmax + output: one thread per query row
    const int t = (warp - 4) >> 2;                // query tile of this warpgroup
    const int q4 = warp & 3;                      // the quarter of tensor-memory lanes this warp may touch
    const int r = q4 * 32 + lane;                 // row inside the tile == TMEM lane
    const int n_kv = t ? n1 : n0;
    const int qi = (2 * pt + t) * BM + r;         // row inside the sequence
    const uint32_t lane_base = static_cast<uint32_t>(q4 * 32) << 16;
    const uint32_t t_s = tmem_base + t * BN + lane_base;
    const uint32_t t_o = tmem_base + (2 + t) * BN + lane_base;
    float m = kNegBig, l = 0.f;                   // exponent base (log2 units, scaled) and the row sum relative to it
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      // waits are made warp-uniform: the tensor-memory loads below are warp-wide instructions
      const bool me = trace_on && (threadIdx.x & 127) == 0;
#define DFB_STAMP_S(slot) do { if (kTrace && me && j < kTraceTiles) trace[(t * kTraceTiles + j) * kTraceSlots + (slot)] = clock64(); } while (0)
      DFB_STAMP_S(0);
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bar->s_full[t], j & 1, abort_flag))) { DFB_FA_FAIL(78); ok = false; break; }
      DFB_STAMP_S(1);
      ptx::tc_fence_after();
      float sc[BN];
#pragma unroll
      for (int c = 0; c < 4; ++c) ptx::tmem_ld_32x32(t_s + c * 32, reinterpret_cast<uint32_t*>(sc) + c * 32);
      ptx::tmem_ld_wait();
      DFB_STAMP_S(2);
      float mx = kNegBig;
      if (j == n_kv - 1) {                        // the diagonal tile (it also holds the end of the sequence)
        const int key_base = j * BN;
#pragma unroll
        for (int i = 0; i < BN; ++i) {
          const int kj = key_base + i;
          if (kj > qi || kj >= seg_len) sc[i] = kNegBig;
        }
      }
      {                                           // four independent chains instead of one of 128 dependent maxima
        float m0 = sc[0], m1 = sc[1], m2 = sc[2], m3 = sc[3];
#pragma unroll
        for (int i = 4; i < BN; i += 4) { m0 = fmaxf(m0, sc[i]); m1 = fmaxf(m1, sc[i + 1]); m2 = fmaxf(m2, sc[i + 2]); m3 = fmaxf(m3, sc[i + 3]); }
        mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      }
      mx *= p.sl2;                                // the scale is positive: the maximum commutes with it
      const bool raise = j == 0 || mx > m + kRescaleGap;
      if (__any_sync(0xffffffffu, raise)) {
        const float m_new = fmaxf(m, mx);
        if (j > 0) {
          // O must be complete up to tile j - 1 and no P V may be in flight while it is rescaled
          if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bar->pv_done[t], (j - 1) & 1, abort_flag))) { DFB_FA_FAIL(79); ok = false; break; }
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
      DFB_STAMP_S(3);
      // P(j) goes back over the columns S(j) came from (this thread already holds its whole row), 64 keys per store
      const float neg_m = -m;
      float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;
#pragma unroll
      for (int hc = 0; hc < 2; ++hc) {
        uint32_t pk[32];
        // sixteen elements at a time, one kind of instruction after the other: the sixteen exponentials are in flight
        // together instead of each waiting for its own multiply-add
#pragma unroll
        for (int i0 = 0; i0 < 64; i0 += 16) {
          float e[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) e[i] = fmaf(sc[hc * 64 + i0 + i], p.sl2, neg_m);
#pragma unroll
          for (int i = 0; i < 16; ++i) e[i] = (i & 3) == 3 ? fa::ex2_poly(e[i]) : ex2(e[i]);   // a quarter on the FMA pipe
#pragma unroll
          for (int i = 0; i < 16; i += 4) { r0 += e[i]; r1 += e[i + 1]; r2 += e[i + 2]; r3 += e[i + 3]; }
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            __nv_bfloat162 b2 = __floats2bfloat162_rn(e[i], e[i + 1]);
            pk[(i0 + i) >> 1] = *reinterpret_cast<uint32_t*>(&b2);
          }
        }
        ptx::tmem_st_32x32(t_s + hc * 32, pk);
        if (hc == 0) {
          ptx::tmem_st_wait();
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&bar->p_half[t]);
        }
      }
      l += (r0 + r1) + (r2 + r3);
      DFB_STAMP_S(4);
      ptx::tmem_st_wait();
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bar->p_full[t]);
      DFB_STAMP_S(5);
    }
    if (ok && n_kv > 0) {
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bar->pv_done[t], (n_kv - 1) & 1, abort_flag))) { DFB_FA_FAIL(81); ok = false; }
    }
    if (ok && n_kv > 0) {
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

}  // namespace fa2

int* gemm_error_word_shared();

// q (T, hq, 128), k / v (T, hkv, 128): row strides in elements (views into a packed qkv are fine); out (T, hq, 128);
// lse (hq, T) fp32; cu_seqlens: nseg + 1 device ints.  Returns -2 for unsupported shapes or alignment.
int flash_fwd_sm100(const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv, void* out, long long ldo,
                    float* lse, const int* cu_seqlens, int nseg, int max_seqlen, int T, int hq, int hkv, int head_dim, float scale,
                    cudaStream_t stream, long long* trace) {
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
  static const bool one_tile = [] { const char* e = getenv("DATAFLOW_FLASH_ONE_TILE"); return e && e[0] == '1'; }();
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    cudaFuncSetAttribute(fa2::flash_fwd2_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, fa2::SMEM_BYTES);
    cudaFuncSetAttribute(fa2::flash_fwd2_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, fa2::SMEM_BYTES);
    configured = true;
  }
  if (one_tile) {
    dim3 grid((max_seqlen + BM - 1) / BM, hq, nseg);
    flash_fwd_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(tq, tk, tv, p);
  } else {
    dim3 grid(hq, nseg, (max_seqlen + 2 * BM - 1) / (2 * BM));
    if (trace) fa2::flash_fwd2_kernel<true><<<grid, fa2::THREADS, fa2::SMEM_BYTES, stream>>>(tq, tk, tv, p, trace);
    else fa2::flash_fwd2_kernel<false><<<grid, fa2::THREADS, fa2::SMEM_BYTES, stream>>>(tq, tk, tv, p, nullptr);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace dfb
