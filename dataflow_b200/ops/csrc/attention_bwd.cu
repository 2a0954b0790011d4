// Causal varlen flash attention, backward, on tcgen05 (head_dim 128, bf16, GQA).  Deterministic: no atomics, every
// output element has one writer and a fixed summation order.
//
// Three launches:
//   flash_bwd_prep   : per (token, head) the pair (lse * log2 e, delta = sum_d dO * O) the two kernels below read.
//   flash_bwd_dkdv   : one CTA per 128-key tile and KV head; loops over the query heads of the group and their 64-row
//                      query tiles i from the diagonal to the end of the sequence, everything transposed so that keys are
//                      the accumulator rows (tensor-memory lanes):
//                          S^T = K Q_i^T, dP^T = V dO_i^T         (two buffers of 64 columns each, both operands in shared memory)
//                          P^T = exp2(S^T * scale * log2 e - lse2),  dS^T = P^T * (dP^T - delta)
//                                                                 -> packed bf16 pairs stored back over the columns they came from
//                          dV += P^T dO_i,  dK += dS^T Q_i        (A operand straight from tensor memory; Q_i / dO_i read
//                                                                  MN-major from the shared-memory tiles that fed S^T / dP^T)
//                      dK and dV of a KV head sum over the whole group inside tensor memory: GQA needs no second pass.
//   flash_bwd_dq     : one CTA per 128-row query tile and head; loops over 64-key tiles j up to the diagonal:
//                          S = Q K_j^T, dP = dO V_j^T;  dS -> packed bf16 over dP's columns;  dQ += dS K_j
// The scores are recomputed twice (once per kernel): seven products per tile pair instead of five, in exchange for no
// atomics and no fp32 dQ buffer.  Roles per CTA: warp 0 TMA producer, warp 1 MMA issuer (one thread), then two groups of
// eight math warps that take alternate tiles (a thread owns one accumulator row and 32 of the tile's 64 columns), so two
// tiles are in flight: while one group exponentiates, the tensor pipe runs the other group's products.  Register budgets
// are rebalanced with setmaxnreg.  Every wait is a bounded mbarrier wait: on a timeout the CTA raises the error word and leaves.
// Reference role: src/dataflow_training/blocks/ops.py:242 (flash_bwd), kernels/flash.py:59-172 (aten / FA3 backward).
#include <cstdlib>

#include "attention_common.cuh"
#include "ops.h"

namespace dfb {

int* gemm_error_word_shared();

namespace fab {

constexpr int D = 128, UK = 16;
constexpr int CH = 128 * 128;                    // 128 rows x 128 bytes: one swizzled chunk of a 128-row tile
constexpr int TILE = 2 * CH;                     // 128 x 128 bf16
constexpr int CH64 = 64 * 128;                   // one chunk of a 64-row tile
constexpr int TILE64 = 2 * CH64;                 // 64 x 128 bf16
constexpr int THREADS = 640;                     // warpgroup 0: producer warp, MMA warp, two idle; warpgroups 1-2 / 3-4: math group 0 / 1
constexpr int TMEM_COLS = 512;
constexpr float kBig = 1e30f;
// Register budgets after the role split.  A warpgroup that asks for more (setmaxnreg.inc) can only take what warpgroups of
// the SAME CTA gave back (setmaxnreg.dec) — the pool is what the CTA was launched with — and blocks until it gets it, so the
// books must balance: launched with kLaunchRegs each, the control warpgroup returns (kLaunchRegs - kCtrlRegs) x 128
// registers and the four math warpgroups take (kMathRegs - kLaunchRegs) x 512.
constexpr int kLaunchRegs = 96, kCtrlRegs = 40, kMathRegs = 104;
static_assert((kLaunchRegs - kCtrlRegs) * 128 >= (kMathRegs - kLaunchRegs) * 512, "setmaxnreg.inc would wait forever");
constexpr uint64_t k_step = (UK * 2) >> 4;       // K-major operand: 16 elements = 32 bytes along the row
constexpr uint64_t mn_step = (UK * 128) >> 4;    // MN-major operand: 16 k-rows of 128 bytes

using fa::ex2;

struct Params {
  const int* cu_seqlens;
  const float2* ld2;            // (hq, T): (lse * log2 e, delta)
  bf16 *dq, *dk, *dv;
  long long lddq, lddk, lddv;   // elements between tokens
  int T, hq, hkv;
  float scale, sl2;             // softmax scale and scale * log2 e
  int* err;
};

#define DFB_FAB_FAIL(code) do { bar->abort = 1; atomicExch(p.err, (code)); } while (0)

// ---------------------------------------------------------------------------------------------------- prep
// one warp per (token, head): delta = sum_d dO * O
__global__ void __launch_bounds__(256) flash_bwd_prep_kernel(const bf16* __restrict__ o, long long ldo, const bf16* __restrict__ dout,
                                                             long long lddo, const float* __restrict__ lse, float2* __restrict__ ld2,
                                                             int T, int hq) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= T * hq) return;
  const int tok = w / hq, h = w - tok * hq;
  const uint2 a = *reinterpret_cast<const uint2*>(o + tok * ldo + h * D + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(dout + tok * lddo + h * D + lane * 4);
  const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x)), a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
  const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.x)), b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.y));
  float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
  s = warp_sum(s);
  if (lane == 0) ld2[static_cast<long long>(h) * T + tok] = make_float2(lse[static_cast<long long>(h) * T + tok] * 1.4426950408889634f, s);
}

// What a math thread does with its 32 scores and 32 dP values: 16 at a time, one kind of instruction after the other, so
// that the sixteen exponentials are in flight together.  ``dead(c)`` says which columns are masked out.
template <bool kMasked, bool kWantP, typename LseFn, typename DeadFn>
DFB_DEVICE void prob_and_ds(const float* s, const float* dp, float sl2, LseFn lse_delta, DeadFn dead, uint32_t* pp, uint32_t* pd) {
#pragma unroll
  for (int c0 = 0; c0 < 32; c0 += 16) {
    float e[16], d[16];
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      const float2 ld = lse_delta(c0 + c);
      e[c] = fmaf(s[c0 + c], sl2, -ld.x);
      d[c] = dp[c0 + c] - ld.y;
    }
#pragma unroll
    for (int c = 0; c < 16; ++c) e[c] = ex2(e[c]);
    if (kMasked) {
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const bool z = dead(c0 + c);
        e[c] = z ? 0.f : e[c];
        d[c] = z ? 0.f : d[c];               // whatever the masked product held (rows of another sequence) must not reach dS
      }
    }
#pragma unroll
    for (int c = 0; c < 16; ++c) d[c] *= e[c];
#pragma unroll
    for (int c = 0; c < 16; c += 2) {
      if (kWantP) {
        __nv_bfloat162 a2 = __floats2bfloat162_rn(e[c], e[c + 1]);
        pp[(c0 + c) >> 1] = *reinterpret_cast<uint32_t*>(&a2);
      }
      __nv_bfloat162 d2 = __floats2bfloat162_rn(d[c], d[c + 1]);
      pd[(c0 + c) >> 1] = *reinterpret_cast<uint32_t*>(&d2);
    }
  }
}

// column of the k-th 16-element slice of a packed 64-element row that two threads wrote, 16 columns each, at the start of
// their own 32-column halves
DFB_DEVICE uint32_t packed_col(int k) { return static_cast<uint32_t>((k >> 1) * 32 + (k & 1) * 8); }

// ---------------------------------------------------------------------------------------------------- dQ
namespace dq {

constexpr int KS = 4, VS = 4;
constexpr int OFF_Q = 0, OFF_DO = TILE, OFF_K = 2 * TILE, OFF_V = OFF_K + KS * TILE64, OFF_BAR = OFF_V + VS * TILE64;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;

struct Bars {
  uint64_t q_full, k_full[KS], k_empty[KS], v_full[VS], v_empty[VS], sdp_full[2], ds_full[2], acc_done;
  uint32_t tmem_base;
  int abort;
};

__global__ void __launch_bounds__(THREADS, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                    const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v, Params p) {
  const int seg = blockIdx.y, h = blockIdx.x;
  const int seg_start = p.cu_seqlens[seg];
  const int seg_len = p.cu_seqlens[seg + 1] - seg_start;
  const int n_qt = (seg_len + 127) / 128;
  const int qt = n_qt - 1 - static_cast<int>(blockIdx.z);        // the grid's slowest index: heavy tiles of every head first
  if (qt < 0) return;
  const int n_kv = min(2 * qt + 2, (seg_len + 63) / 64);         // 64-key tiles up to the diagonal
  const int kvh = h / (p.hq / p.hkv);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Bars* bar = reinterpret_cast<Bars*>(smem + OFF_BAR);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &bar->abort;

  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar->q_full, 1);
    for (int b = 0; b < KS; ++b) { ptx::mbar_init(&bar->k_full[b], 1); ptx::mbar_init(&bar->k_empty[b], 1); }
    for (int b = 0; b < VS; ++b) { ptx::mbar_init(&bar->v_full[b], 1); ptx::mbar_init(&bar->v_empty[b], 1); }
    for (int b = 0; b < 2; ++b) { ptx::mbar_init(&bar->sdp_full[b], 1); ptx::mbar_init(&bar->ds_full[b], 8); }
    ptx::mbar_init(&bar->acc_done, 1);
    bar->abort = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmap_q); ptx::prefetch_tmap(&tmap_do); ptx::prefetch_tmap(&tmap_k); ptx::prefetch_tmap(&tmap_v);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&bar->tmem_base, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = bar->tmem_base;
  const uint32_t tmem_s = tmem_base, tmem_dp = tmem_base + 128, tmem_dq = tmem_base + 256;

  if (warp < 4) {
    ptx::setmaxnreg_dec<kCtrlRegs>();
    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0) {
        const int row0 = seg_start + qt * 128;
        ptx::mbar_expect_tx(&bar->q_full, 2 * TILE);
        for (int c = 0; c < 2; ++c) {
          ptx::tma_load_2d(smem + OFF_Q + c * CH, &tmap_q, &bar->q_full, h * D + c * 64, row0);
          ptx::tma_load_2d(smem + OFF_DO + c * CH, &tmap_do, &bar->q_full, h * D + c * 64, row0);
        }
        for (int j = 0; j < n_kv && !*abort_flag; ++j) {
          const int kb = j % KS, ku = j / KS, vb = j % VS, vu = j / VS;
          const int key0 = seg_start + j * 64;
          if (ku > 0 && !ptx::mbar_wait(&bar->k_empty[kb], (ku - 1) & 1, abort_flag)) { DFB_FAB_FAIL(91); break; }
          ptx::mbar_expect_tx(&bar->k_full[kb], TILE64);
          for (int c = 0; c < 2; ++c) ptx::tma_load_2d(smem + OFF_K + kb * TILE64 + c * CH64, &tmap_k, &bar->k_full[kb], kvh * D + c * 64, key0);
          if (vu > 0 && !ptx::mbar_wait(&bar->v_empty[vb], (vu - 1) & 1, abort_flag)) { DFB_FAB_FAIL(92); break; }
          ptx::mbar_expect_tx(&bar->v_full[vb], TILE64);
          for (int c = 0; c < 2; ++c) ptx::tma_load_2d(smem + OFF_V + vb * TILE64 + c * CH64, &tmap_v, &bar->v_full[vb], kvh * D + c * 64, key0);
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------------ MMA issuer
      if (lane == 0) {
        constexpr uint32_t idesc_s = ptx::idesc_bf16_f32(128, 64, false, false);
        constexpr uint32_t idesc_acc = ptx::idesc_bf16_f32(128, 128, false, true);
        const uint32_t q_addr = ptx::smem_u32(smem + OFF_Q), do_addr = ptx::smem_u32(smem + OFF_DO);
        bool ok = ptx::mbar_wait(&bar->q_full, 0, abort_flag);
        if (!ok) DFB_FAB_FAIL(93);
        auto issue_sdp = [&](int j) -> bool {                 // S(j) = Q K_j^T, dP(j) = dO V_j^T into buffer j & 1
          const int kb = j % KS, vb = j % VS, b = j & 1;
          if (!ptx::mbar_wait(&bar->k_full[kb], (j / KS) & 1, abort_flag) || !ptx::mbar_wait(&bar->v_full[vb], (j / VS) & 1, abort_flag)) return false;
          ptx::tc_fence_after();
          const uint32_t k_addr = ptx::smem_u32(smem + OFF_K + kb * TILE64), v_addr = ptx::smem_u32(smem + OFF_V + vb * TILE64);
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const uint64_t adesc = ptx::desc_kmajor_sw128(q_addr + c * CH), bdesc = ptx::desc_kmajor_sw128(k_addr + c * CH64);
#pragma unroll
            for (int k = 0; k < 4; ++k) ptx::umma_bf16(tmem_s + b * 64, adesc + k * k_step, bdesc + k * k_step, idesc_s, (c | k) != 0);
          }
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const uint64_t adesc = ptx::desc_kmajor_sw128(do_addr + c * CH), bdesc = ptx::desc_kmajor_sw128(v_addr + c * CH64);
#pragma unroll
            for (int k = 0; k < 4; ++k) ptx::umma_bf16(tmem_dp + b * 64, adesc + k * k_step, bdesc + k * k_step, idesc_s, (c | k) != 0);
          }
          ptx::umma_commit(&bar->v_empty[vb]);
          ptx::umma_commit(&bar->sdp_full[b]);
          return true;
        };
        if (ok && !(issue_sdp(0) && (n_kv < 2 || issue_sdp(1)))) { DFB_FAB_FAIL(94); ok = false; }
        for (int j = 0; j < n_kv && ok; ++j) {
          const int b = j & 1, kb = j % KS;
          if (!ptx::mbar_wait(&bar->ds_full[b], (j >> 1) & 1, abort_flag)) { DFB_FAB_FAIL(95); ok = false; break; }
          ptx::tc_fence_after();
          // K_j once more, now as the MN-major operand: 64-column chunks CH64 apart, keys 128 bytes apart; dS from tensor memory
          const uint64_t b_k = ptx::desc_mnmajor_sw128(ptx::smem_u32(smem + OFF_K + kb * TILE64), CH64);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            ptx::umma_bf16_ts(tmem_dq, tmem_dp + b * 64 + packed_col(k), b_k + k * mn_step, idesc_acc, (j | k) != 0);
          ptx::umma_commit(&bar->k_empty[kb]);
          if (j + 2 < n_kv && !issue_sdp(j + 2)) { DFB_FAB_FAIL(94); ok = false; break; }   // ordered behind the product that read dS(j)
        }
        if (ok) ptx::umma_commit(&bar->acc_done);
      }
    }
  } else {
    ptx::setmaxnreg_inc<kMathRegs>();
    // ------------------------------------------------------------------ math warps: query row r, keys [hh * 32, hh * 32 + 32) of every second tile
    const int mw = warp - 4, grp = mw >> 3, hh = (mw >> 2) & 1;
    const int q4 = warp & 3;
    const int r = q4 * 32 + lane;
    const int qi = qt * 128 + r;
    const bool row_ok = qi < seg_len;
    const uint32_t lane_base = static_cast<uint32_t>(q4 * 32) << 16;
    float2 ld = make_float2(kBig, 0.f);
    if (row_ok) ld = p.ld2[static_cast<long long>(h) * p.T + seg_start + qi];
    bool ok = true;
    for (int j = grp; j < n_kv && ok; j += 2) {
      const int b = grp;
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bar->sdp_full[b], (j >> 1) & 1, abort_flag))) { DFB_FAB_FAIL(96); ok = false; break; }
      ptx::tc_fence_after();
      float s[32], dp[32];
      const uint32_t col = lane_base + b * 64 + hh * 32;
      ptx::tmem_ld_32x32(tmem_s + col, reinterpret_cast<uint32_t*>(s));
      ptx::tmem_ld_32x32(tmem_dp + col, reinterpret_cast<uint32_t*>(dp));
      ptx::tmem_ld_wait();
      uint32_t pd[16];
      const int key_base = j * 64 + hh * 32;
      auto lse_delta = [&](int) { return ld; };
      if (j >= 2 * qt || !row_ok)                   // the two tiles on the diagonal (they also hold the end of the sequence)
        prob_and_ds<true, false>(s, dp, p.sl2, lse_delta, [&](int c) { return key_base + c > qi || key_base + c >= seg_len || !row_ok; }, nullptr, pd);
      else
        prob_and_ds<false, false>(s, dp, p.sl2, lse_delta, [&](int) { return false; }, nullptr, pd);
      ptx::tmem_st_32x16(tmem_dp + col, pd);         // dS(j) as packed pairs over the first half of this thread's own dP columns
      ptx::tmem_st_wait();
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bar->ds_full[b]);
    }
    if (ok && !__all_sync(0xffffffffu, ptx::mbar_wait(&bar->acc_done, 0, abort_flag))) { DFB_FAB_FAIL(98); ok = false; }
    if (ok) {
      ptx::tc_fence_after();
      const int quarter = grp * 2 + hh;             // 32 of the 128 output columns per thread
      bf16* dst = p.dq + (seg_start + qi) * p.lddq + static_cast<long long>(h) * D + quarter * 32;
      uint32_t v[32];
      ptx::tmem_ld_32x32(tmem_dq + lane_base + quarter * 32, v);
      ptx::tmem_ld_wait();
      if (row_ok) {
        float o[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __uint_as_float(v[i]) * p.scale;
#pragma unroll
        for (int g = 0; g < 4; ++g) st8(dst + g * 8, pack8(o + g * 8));
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) ptx::tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace dq

// ---------------------------------------------------------------------------------------------------- dK, dV
namespace dkv {

constexpr int STAGES = 4;
constexpr int OFF_K = 0, OFF_V = TILE, OFF_QDO = 2 * TILE;            // stage s: Q_i at OFF_QDO + s * 2 * TILE64, dO_i right behind it
constexpr int OFF_LD = OFF_QDO + STAGES * 2 * TILE64;
constexpr int OFF_BAR = OFF_LD + STAGES * 64 * 8;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;

struct Bars {
  uint64_t kv_full, qdo_full[STAGES], qdo_empty[STAGES], sdp_full[2], pds_full[2], acc_done;
  uint32_t tmem_base;
  int abort;
};

// kTrace: CTA (0, 0, 0) records clock64() stamps of its first 32 tiles into ``trace`` — per tile 8 slots for each of three
// observers (thread 0 of either math group, the MMA thread).  A profiling aid: the regular launch passes false.
constexpr int kTraceTiles = 32, kTraceSlots = 8;
#define DFB_BSTAMP(who, it, slot)                                                                                       \
  do { if (kTrace && trace_on && (it) < kTraceTiles) trace[((who) * kTraceTiles + (it)) * kTraceSlots + (slot)] = clock64(); } while (0)

template <bool kTrace>
__global__ void __launch_bounds__(THREADS, 1)
flash_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                      const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v, Params p, long long* trace) {
  const bool trace_on = kTrace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
  const int seg = blockIdx.y, kvh = blockIdx.x;
  const int seg_start = p.cu_seqlens[seg];
  const int seg_len = p.cu_seqlens[seg + 1] - seg_start;
  const int jt = blockIdx.z;                                     // the grid's slowest index; key tile 0 has the longest loop and goes first
  if (jt * 128 >= seg_len) return;
  const int G = p.hq / p.hkv;
  const int i0 = 2 * jt, per = (seg_len + 63) / 64 - i0;         // 64-row query tiles from the diagonal to the end
  const int n_it = G * per;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Bars* bar = reinterpret_cast<Bars*>(smem + OFF_BAR);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &bar->abort;

  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar->kv_full, 1);
    for (int s = 0; s < STAGES; ++s) { ptx::mbar_init(&bar->qdo_full[s], 2); ptx::mbar_init(&bar->qdo_empty[s], 1); }
    for (int b = 0; b < 2; ++b) { ptx::mbar_init(&bar->sdp_full[b], 1); ptx::mbar_init(&bar->pds_full[b], 8); }
    ptx::mbar_init(&bar->acc_done, 1);
    bar->abort = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmap_q); ptx::prefetch_tmap(&tmap_do); ptx::prefetch_tmap(&tmap_k); ptx::prefetch_tmap(&tmap_v);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&bar->tmem_base, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = bar->tmem_base;
  const uint32_t tmem_st = tmem_base, tmem_dpt = tmem_base + 128, tmem_dv = tmem_base + 256, tmem_dk = tmem_base + 384;

  if (warp < 4) {
    ptx::setmaxnreg_dec<kCtrlRegs>();
    if (warp == 0) {
      // ------------------------------------------------------------------ producer: TMA by lane 0, (lse2, delta) staging by the whole warp
      if (lane == 0) {
        const int key0 = seg_start + jt * 128;
        ptx::mbar_expect_tx(&bar->kv_full, 2 * TILE);
        for (int c = 0; c < 2; ++c) {
          ptx::tma_load_2d(smem + OFF_K + c * CH, &tmap_k, &bar->kv_full, kvh * D + c * 64, key0);
          ptx::tma_load_2d(smem + OFF_V + c * CH, &tmap_v, &bar->kv_full, kvh * D + c * 64, key0);
        }
      }
      bool ok = true;
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it % STAGES, use = it / STAGES;
        const int g = it / per, i = i0 + it - g * per, h = kvh * G + g;
        if (use > 0 && !__all_sync(0xffffffffu, ptx::mbar_wait(&bar->qdo_empty[st], (use - 1) & 1, abort_flag))) { DFB_FAB_FAIL(101); ok = false; break; }
        if (__any_sync(0xffffffffu, *abort_flag != 0)) break;
        if (lane == 0) {
          uint8_t* dst = smem + OFF_QDO + st * 2 * TILE64;
          const int row0 = seg_start + i * 64;
          ptx::mbar_expect_tx(&bar->qdo_full[st], 2 * TILE64);
          for (int c = 0; c < 2; ++c) {
            ptx::tma_load_2d(dst + c * CH64, &tmap_q, &bar->qdo_full[st], h * D + c * 64, row0);
            ptx::tma_load_2d(dst + TILE64 + c * CH64, &tmap_do, &bar->qdo_full[st], h * D + c * 64, row0);
          }
        }
        float2* ld = reinterpret_cast<float2*>(smem + OFF_LD + st * 64 * 8);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int q = lane + u * 32, qi = i * 64 + q;
          ld[q] = qi < seg_len ? p.ld2[static_cast<long long>(h) * p.T + seg_start + qi] : make_float2(kBig, 0.f);
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&bar->qdo_full[st]);
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------------ MMA issuer
      if (lane == 0) {
        constexpr uint32_t idesc_s = ptx::idesc_bf16_f32(128, 64, false, false);
        constexpr uint32_t idesc_acc = ptx::idesc_bf16_f32(128, 128, false, true);
        const uint32_t k_addr = ptx::smem_u32(smem + OFF_K), v_addr = ptx::smem_u32(smem + OFF_V);
        bool ok = ptx::mbar_wait(&bar->kv_full, 0, abort_flag);
        if (!ok) DFB_FAB_FAIL(102);
        auto issue_sdp = [&](int it) -> bool {              // S^T(it) = K Q_i^T, dP^T(it) = V dO_i^T into buffer it & 1
          const int st = it % STAGES, b = it & 1;
          if (!ptx::mbar_wait(&bar->qdo_full[st], (it / STAGES) & 1, abort_flag)) return false;
          ptx::tc_fence_after();
          const uint32_t q_addr = ptx::smem_u32(smem + OFF_QDO + st * 2 * TILE64), do_addr = q_addr + TILE64;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const uint64_t adesc = ptx::desc_kmajor_sw128(k_addr + c * CH), bdesc = ptx::desc_kmajor_sw128(q_addr + c * CH64);
#pragma unroll
            for (int k = 0; k < 4; ++k) ptx::umma_bf16(tmem_st + b * 64, adesc + k * k_step, bdesc + k * k_step, idesc_s, (c | k) != 0);
          }
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const uint64_t adesc = ptx::desc_kmajor_sw128(v_addr + c * CH), bdesc = ptx::desc_kmajor_sw128(do_addr + c * CH64);
#pragma unroll
            for (int k = 0; k < 4; ++k) ptx::umma_bf16(tmem_dpt + b * 64, adesc + k * k_step, bdesc + k * k_step, idesc_s, (c | k) != 0);
          }
          ptx::umma_commit(&bar->sdp_full[b]);
          return true;
        };
        if (ok && !(issue_sdp(0) && (n_it < 2 || issue_sdp(1)))) { DFB_FAB_FAIL(103); ok = false; }
        for (int it = 0; it < n_it && ok; ++it) {
          const int st = it % STAGES, b = it & 1;
          DFB_BSTAMP(2, it, 0);
          if (!ptx::mbar_wait(&bar->pds_full[b], (it >> 1) & 1, abort_flag)) { DFB_FAB_FAIL(104); ok = false; break; }
          DFB_BSTAMP(2, it, 1);
          ptx::tc_fence_after();
          const uint32_t q_addr = ptx::smem_u32(smem + OFF_QDO + st * 2 * TILE64), do_addr = q_addr + TILE64;
          // Q_i / dO_i once more, as MN-major operands: 64-column chunks CH64 apart, queries 128 bytes apart; P^T and dS^T
          // come straight from tensor memory
          const uint64_t b_do = ptx::desc_mnmajor_sw128(do_addr, CH64), b_q = ptx::desc_mnmajor_sw128(q_addr, CH64);
#pragma unroll
          for (int k = 0; k < 4; ++k) ptx::umma_bf16_ts(tmem_dv, tmem_st + b * 64 + packed_col(k), b_do + k * mn_step, idesc_acc, (it | k) != 0);
#pragma unroll
          for (int k = 0; k < 4; ++k) ptx::umma_bf16_ts(tmem_dk, tmem_dpt + b * 64 + packed_col(k), b_q + k * mn_step, idesc_acc, (it | k) != 0);
          ptx::umma_commit(&bar->qdo_empty[st]);
          DFB_BSTAMP(2, it, 2);
          if (it + 2 < n_it && !issue_sdp(it + 2)) { DFB_FAB_FAIL(103); ok = false; break; }   // ordered behind the products that read buffer b
          DFB_BSTAMP(2, it, 3);
        }
        if (ok) ptx::umma_commit(&bar->acc_done);
      }
    }
  } else {
    ptx::setmaxnreg_inc<kMathRegs>();
    // ------------------------------------------------------------------ math warps: key row r, queries [hh * 32, hh * 32 + 32) of every second tile
    const int mw = warp - 4, grp = mw >> 3, hh = (mw >> 2) & 1;
    const int q4 = warp & 3;
    const int r = q4 * 32 + lane;
    const int kj = jt * 128 + r;
    const bool row_ok = kj < seg_len;
    const uint32_t lane_base = static_cast<uint32_t>(q4 * 32) << 16;
    bool ok = true;
    for (int it = grp; it < n_it && ok; it += 2) {
      const int st = it % STAGES, b = grp;
      const int g = it / per, i = i0 + it - g * per;
      const bool me = trace_on && (threadIdx.x & 255) == 128;          // thread 0 of the group's first warp
#define DFB_BSTAMP_M(slot) do { if (kTrace && me && it < kTraceTiles) trace[(grp * kTraceTiles + it) * kTraceSlots + (slot)] = clock64(); } while (0)
      DFB_BSTAMP_M(0);
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bar->sdp_full[b], (it >> 1) & 1, abort_flag) &&
                                       ptx::mbar_wait(&bar->qdo_full[st], (it / STAGES) & 1, abort_flag))) { DFB_FAB_FAIL(105); ok = false; break; }
      ptx::tc_fence_after();
      float s[32], dp[32];
      const uint32_t col = lane_base + b * 64 + hh * 32;
      ptx::tmem_ld_32x32(tmem_st + col, reinterpret_cast<uint32_t*>(s));
      ptx::tmem_ld_32x32(tmem_dpt + col, reinterpret_cast<uint32_t*>(dp));
      DFB_BSTAMP_M(1);
      ptx::tmem_ld_wait();
      DFB_BSTAMP_M(2);
      const float2* ld = reinterpret_cast<const float2*>(smem + OFF_LD + st * 64 * 8) + hh * 32;
      uint32_t pp[16], pd[16];
      const int q_base = i * 64 + hh * 32;
      auto lse_delta = [&](int c) { return ld[c]; };
      // queries past the end of the sequence carry lse2 = 1e30: their probabilities are exactly zero without a mask
      if (i < i0 + 2 || !row_ok)                    // tiles that touch the diagonal; key rows past the end of the sequence
        prob_and_ds<true, true>(s, dp, p.sl2, lse_delta, [&](int c) { return kj > q_base + c || !row_ok; }, pp, pd);
      else
        prob_and_ds<false, true>(s, dp, p.sl2, lse_delta, [&](int) { return false; }, pp, pd);
      // P^T and dS^T as packed pairs over the first half of this thread's own S^T / dP^T columns
      DFB_BSTAMP_M(3);
      ptx::tmem_st_32x16(tmem_st + col, pp);
      ptx::tmem_st_32x16(tmem_dpt + col, pd);
      ptx::tmem_st_wait();
      DFB_BSTAMP_M(4);
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bar->pds_full[b]);
      DFB_BSTAMP_M(5);
    }
    if (ok && !__all_sync(0xffffffffu, ptx::mbar_wait(&bar->acc_done, 0, abort_flag))) { DFB_FAB_FAIL(107); ok = false; }
    if (ok) {
      ptx::tc_fence_after();
      const int quarter = grp * 2 + hh;             // 32 of the 128 output columns per thread
      const long long tok = seg_start + kj;
      bf16* dv_dst = p.dv + tok * p.lddv + static_cast<long long>(kvh) * D + quarter * 32;
      bf16* dk_dst = p.dk + tok * p.lddk + static_cast<long long>(kvh) * D + quarter * 32;
      uint32_t v[32], k[32];
      ptx::tmem_ld_32x32(tmem_dv + lane_base + quarter * 32, v);
      ptx::tmem_ld_32x32(tmem_dk + lane_base + quarter * 32, k);
      ptx::tmem_ld_wait();
      if (row_ok) {
        float o[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __uint_as_float(v[i]);
#pragma unroll
        for (int g4 = 0; g4 < 4; ++g4) st8(dv_dst + g4 * 8, pack8(o + g4 * 8));
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __uint_as_float(k[i]) * p.scale;
#pragma unroll
        for (int g4 = 0; g4 < 4; ++g4) st8(dk_dst + g4 * 8, pack8(o + g4 * 8));
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) ptx::tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace dkv
}  // namespace fab

// q, o, dout, dq: (T, hq, 128); k, v, dk, dv: (T, hkv, 128); row strides in elements (views into packed buffers are fine);
// lse (hq, T) fp32 from the forward; ld2: scratch of hq * T float2; cu_seqlens: nseg + 1 device ints.
// Returns -2 for unsupported shapes or alignment.
int flash_bwd_sm100(const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv, const void* o, long long ldo,
                    const void* dout, long long lddo, const float* lse, void* dq, long long lddq, void* dk, long long lddk, void* dv,
                    long long lddv, void* ld2, const int* cu_seqlens, int nseg, int max_seqlen, int T, int hq, int hkv, int head_dim,
                    float scale, cudaStream_t stream, long long* trace) {
  using namespace fab;
  if (head_dim != D || hkv <= 0 || hq % hkv || nseg <= 0 || T <= 0 || max_seqlen <= 0) return -2;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 4) || (lddo % 8) || (lddq % 8) || (lddk % 8) || (lddv % 8)) return -2;
  const uintptr_t all = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                        reinterpret_cast<uintptr_t>(dout) | reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) |
                        reinterpret_cast<uintptr_t>(dv);
  if ((all & 15) || (reinterpret_cast<uintptr_t>(o) & 7) || (reinterpret_cast<uintptr_t>(ld2) & 7)) return -2;
  CUtensorMap tq, tdo, tk, tv, tq64, tdo64, tk64, tv64;
  const uint64_t qc = static_cast<uint64_t>(hq) * D, kc = static_cast<uint64_t>(hkv) * D;
  bool ok = fa::make_map(&tq, q, qc, T, ldq, 128) && fa::make_map(&tdo, dout, qc, T, lddo, 128) && fa::make_map(&tk, k, kc, T, ldk, 128) &&
            fa::make_map(&tv, v, kc, T, ldv, 128) && fa::make_map(&tq64, q, qc, T, ldq, 64) && fa::make_map(&tdo64, dout, qc, T, lddo, 64) &&
            fa::make_map(&tk64, k, kc, T, ldk, 64) && fa::make_map(&tv64, v, kc, T, ldv, 64);
  if (!ok) return -4;
  Params p;
  p.cu_seqlens = cu_seqlens; p.ld2 = reinterpret_cast<const float2*>(ld2);
  p.dq = reinterpret_cast<bf16*>(dq); p.dk = reinterpret_cast<bf16*>(dk); p.dv = reinterpret_cast<bf16*>(dv);
  p.lddq = lddq; p.lddk = lddk; p.lddv = lddv;
  p.T = T; p.hq = hq; p.hkv = hkv; p.scale = scale; p.sl2 = scale * 1.4426950408889634f; p.err = gemm_error_word_shared();
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(dq::flash_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dq::SMEM_BYTES);
    cudaFuncSetAttribute(dkv::flash_bwd_dkdv_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, dkv::SMEM_BYTES);
    cudaFuncSetAttribute(dkv::flash_bwd_dkdv_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, dkv::SMEM_BYTES);
    configured = true;
  }
  const long long warps = static_cast<long long>(T) * hq;
  flash_bwd_prep_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const bf16*>(o), ldo, reinterpret_cast<const bf16*>(dout), lddo, lse, reinterpret_cast<float2*>(ld2), T, hq);
  const int n_t = (max_seqlen + 127) / 128;
  if (trace) dkv::flash_bwd_dkdv_kernel<true><<<dim3(hkv, nseg, n_t), THREADS, dkv::SMEM_BYTES, stream>>>(tq64, tdo64, tk, tv, p, trace);
  else dkv::flash_bwd_dkdv_kernel<false><<<dim3(hkv, nseg, n_t), THREADS, dkv::SMEM_BYTES, stream>>>(tq64, tdo64, tk, tv, p, nullptr);
  dq::flash_bwd_dq_kernel<<<dim3(hq, nseg, n_t), THREADS, dq::SMEM_BYTES, stream>>>(tq, tdo, tk64, tv64, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace dfb
