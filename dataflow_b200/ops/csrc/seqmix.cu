// Small sequence-mixing kernels of the linear-attention and latent-attention families (memory bound; one pass each):
//   l2norm            y = x * rsqrt(sum x^2 + eps) over the last dim, forward and backward
//   gated rmsnorm     y = x * rstd * w * silu(g), forward and backward (dw as per-block partials, summed by the host op)
//   causal conv + silu depthwise convolution of width <= 4 along tokens that never crosses a segment start, then SiLU;
//                     forward and backward (dw as per-block partials)
//   sigmoid no-aux router  sigmoid scores, selection on score + bias inside the best groups of experts (a group's rank is
//                     the sum of its two best biased scores), weights from the unbiased scores, normalised and scaled
// bf16 storage, fp32 math, deterministic reductions.
// Reference role: src/dataflow_training/blocks/ops.py:509-623 (DeltaNet helpers), moe/forms.py (sigmoid_noaux_tc).
#include <float.h>

#include "common.cuh"
#include "ops.h"

namespace dfb {
namespace {

constexpr int kMaxD = 512;             // widest row the per-warp kernels take (16 values per lane)
constexpr int kMaxPer = 8;             // experts per lane in the router (E <= 256)
constexpr int kMaxK = 16;

DFB_DEVICE float silu(float x) { return x / (1.f + __expf(-x)); }
DFB_DEVICE float dsilu(float x) {
  float s = 1.f / (1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}

// ------------------------------------------------------------------------------------------------ l2norm
__global__ void l2norm_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, float* __restrict__ rstd, long long rows, int D, float eps) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const bf16* xr = x + row * D;
  float v[kMaxD / 32], s = 0.f;
  const int per = (D + 31) / 32;
  for (int j = 0; j < per; ++j) {
    int c = j * 32 + lane;
    v[j] = c < D ? bf2f(xr[c]) : 0.f;
    s += v[j] * v[j];
  }
  s = warp_sum(s);
  const float r = rsqrtf(s + eps);
  for (int j = 0; j < per; ++j) {
    int c = j * 32 + lane;
    if (c < D) y[row * D + c] = f2bf(v[j] * r);
  }
  if (lane == 0 && rstd) rstd[row] = r;
}

__global__ void l2norm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const float* __restrict__ rstd,
                                  bf16* __restrict__ dx, long long rows, int D) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float xv[kMaxD / 32], gv[kMaxD / 32], dot = 0.f;
  const int per = (D + 31) / 32;
  for (int j = 0; j < per; ++j) {
    int c = j * 32 + lane;
    xv[j] = c < D ? bf2f(x[row * D + c]) : 0.f;
    gv[j] = c < D ? bf2f(dy[row * D + c]) : 0.f;
    dot += xv[j] * gv[j];
  }
  dot = warp_sum(dot);
  const float r = rstd[row], r3 = r * r * r;
  for (int j = 0; j < per; ++j) {
    int c = j * 32 + lane;
    if (c < D) dx[row * D + c] = f2bf(r * gv[j] - xv[j] * r3 * dot);
  }
}

// ------------------------------------------------------------------------------------------------ gated rmsnorm
__global__ void gated_rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ g, const bf16* __restrict__ w,
                                         bf16* __restrict__ y, float* __restrict__ rstd, long long rows, int D, float eps) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float v[kMaxD / 32], s = 0.f;
  const int per = (D + 31) / 32;
  for (int j = 0; j < per; ++j) {
    int c = j * 32 + lane;
    v[j] = c < D ? bf2f(x[row * D + c]) : 0.f;
    s += v[j] * v[j];
  }
  s = warp_sum(s);
  const float r = rsqrtf(s / D + eps);
  for (int j = 0; j < per; ++j) {
    int c = j * 32 + lane;
    if (c < D) {
      // the normalised value is rounded to storage precision before the gate, as the two-op reference does
      float n = bf2f(f2bf(v[j] * r)) * bf2f(w[c]);
      y[row * D + c] = f2bf(bf2f(f2bf(n)) * bf2f(f2bf(silu(bf2f(g[row * D + c])))));
    }
  }
  if (lane == 0) rstd[row] = r;
}

// one block = 8 warps walking rows with a grid stride; dw partial per block
__global__ void gated_rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ g,
                                         const bf16* __restrict__ w, const float* __restrict__ rstd, bf16* __restrict__ dx,
                                         bf16* __restrict__ dg, float* __restrict__ dw_partial, long long rows, int D) {
  __shared__ float acc[8][kMaxD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per = (D + 31) / 32;
  float dwl[kMaxD / 32];
  for (int j = 0; j < per; ++j) dwl[j] = 0.f;
  for (long long row = blockIdx.x * 8LL + warp; row < rows; row += gridDim.x * 8LL) {
    const float r = rstd[row];
    float xv[kMaxD / 32], dn[kMaxD / 32], dot = 0.f;
    for (int j = 0; j < per; ++j) {
      int c = j * 32 + lane;
      xv[j] = dn[j] = 0.f;
      if (c < D) {
        float gy = bf2f(dy[row * D + c]), gg = bf2f(g[row * D + c]), wc = bf2f(w[c]);
        xv[j] = bf2f(x[row * D + c]);
        float nrm = xv[j] * r;
        dg[row * D + c] = f2bf(gy * nrm * wc * dsilu(gg));
        float d_n = gy * silu(gg);                 // gradient at (x * rstd * w)
        dwl[j] += d_n * nrm;
        dn[j] = d_n * wc;                          // gradient at (x * rstd)
        dot += dn[j] * xv[j];
      }
    }
    dot = warp_sum(dot);
    const float k = r * r * r / D;
    for (int j = 0; j < per; ++j) {
      int c = j * 32 + lane;
      if (c < D) dx[row * D + c] = f2bf(r * dn[j] - xv[j] * k * dot);
    }
  }
  for (int j = 0; j < per; ++j) {
    int c = j * 32 + lane;
    if (c < D) acc[warp][c] = dwl[j];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float s = 0.f;
    for (int q = 0; q < 8; ++q) s += acc[q][c];
    dw_partial[static_cast<long long>(blockIdx.x) * D + c] = s;
  }
}

// ------------------------------------------------------------------------------------------------ causal conv + silu
__global__ void conv_silu_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const int* __restrict__ seg_start,
                                     bf16* __restrict__ y, long long n, int C, int W) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= n * C) return;
  const long long t = i / C;
  const int c = static_cast<int>(i - t * C);
  const int s0 = seg_start[t];
  float acc = 0.f;
  for (int j = 0; j < W; ++j) {
    long long src = t - (W - 1 - j);
    if (src >= s0) acc += bf2f(x[src * C + c]) * bf2f(w[c * W + j]);
  }
  y[i] = f2bf(silu(bf2f(f2bf(acc))));
}

// dx and the per-block partial of dw; block = 256 channels-major threads over a chunk of ``rows_per_block`` tokens
__global__ void conv_silu_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                                     const int* __restrict__ seg_start, bf16* __restrict__ dx, float* __restrict__ dw_partial,
                                     long long n, int C, int W, int rows_per_block) {
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const long long t0 = static_cast<long long>(blockIdx.x) * rows_per_block;
  const long long t1 = min(t0 + rows_per_block, n);
  float wv[4], dwl[4] = {0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < W; ++j) wv[j] = bf2f(w[c * W + j]);
  auto dpre_at = [&](long long u) -> float {           // gradient at the convolution output of token u
    const int s0 = seg_start[u];
    float pre = 0.f;
    for (int j = 0; j < W; ++j) {
      long long src = u - (W - 1 - j);
      if (src >= s0) pre += bf2f(x[src * C + c]) * wv[j];
    }
    return bf2f(dy[u * C + c]) * dsilu(bf2f(f2bf(pre)));
  };
  for (long long t = t0; t < t1; ++t) {
    // dx[t] gathers from the outputs t .. t + W - 1 that lie in the same segment
    float g = 0.f;
    for (int j = 0; j < W; ++j) {
      long long u = t + (W - 1 - j);
      if (u < n && seg_start[u] <= t) g += wv[j] * dpre_at(u);
    }
    dx[t * C + c] = f2bf(g);
    // dw from output t
    const float dp = dpre_at(t);
    const int s0 = seg_start[t];
    for (int j = 0; j < W; ++j) {
      long long src = t - (W - 1 - j);
      if (src >= s0) dwl[j] += dp * bf2f(x[src * C + c]);
    }
  }
  for (int j = 0; j < W; ++j) dw_partial[(static_cast<long long>(blockIdx.x) * C + c) * W + j] = dwl[j];
}

// ------------------------------------------------------------------------------------------------ sigmoid no-aux router
DFB_DEVICE void warp_argmax2(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, v, o);
    int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

__global__ void router_sigmoid_noaux_kernel(const bf16* __restrict__ logits, const float* __restrict__ bias, float* __restrict__ route_w,
                                            int* __restrict__ route_ids, int t, int E, int K, int n_group, int topk_group, float scaling) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= t) return;
  __shared__ float s_sel[8][256];
  float* sel = s_sel[(threadIdx.x >> 5) & 7];
  const int per = (E + 31) / 32;
  float score[kMaxPer];
  for (int j = 0; j < per; ++j) {
    int e = j * 32 + lane;
    score[j] = e < E ? 1.f / (1.f + __expf(-bf2f(logits[static_cast<long long>(warp) * E + e]))) : 0.f;
    if (e < E) sel[e] = score[j] + bias[e];
  }
  __syncwarp();
  if (n_group > 1) {
    const int gs = E / n_group;
    // lane g ranks group g by the sum of its two best biased scores
    float rank = -FLT_MAX;
    if (lane < n_group) {
      float a = -FLT_MAX, b = -FLT_MAX;
      for (int e = lane * gs; e < (lane + 1) * gs; ++e) {
        float v = sel[e];
        if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
      }
      rank = gs > 1 ? a + b : a;
    }
    unsigned keep = 0;
    for (int k = 0; k < topk_group; ++k) {
      float bv = rank;
      int bi = lane < n_group ? lane : 0x7fffffff;
      if (lane >= n_group) bv = -FLT_MAX;
      warp_argmax2(bv, bi);
      keep |= 1u << bi;
      if (lane == bi) rank = -FLT_MAX;
    }
    __syncwarp();
    for (int j = 0; j < per; ++j) {
      int e = j * 32 + lane;
      if (e < E && !((keep >> (e / gs)) & 1u)) sel[e] = -FLT_MAX;
    }
    __syncwarp();
  }
  float wsel[kMaxK];
  int isel[kMaxK];
  float total = 0.f;
  for (int k = 0; k < K; ++k) {
    float bv = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int j = 0; j < per; ++j) {
      int e = j * 32 + lane;
      if (e < E && (sel[e] > bv || (sel[e] == bv && e < bi))) { bv = sel[e]; bi = e; }
    }
    warp_argmax2(bv, bi);
    // the weight is the UNBIASED score of the winner
    float sc = __shfl_sync(0xffffffffu, score[bi >> 5], bi & 31);
    wsel[k] = sc; isel[k] = bi; total += sc;
    if ((bi & 31) == lane) sel[bi] = -FLT_MAX;
    __syncwarp();
  }
  if (lane == 0) {
    for (int k = 0; k < K; ++k) {
      route_w[static_cast<long long>(warp) * K + k] = wsel[k] / (total + 1e-20f) * scaling;
      route_ids[static_cast<long long>(warp) * K + k] = isel[k];
    }
  }
}

}  // namespace

int l2norm_fwd(const void* x, void* y, float* rstd, long long rows, int D, float eps, cudaStream_t s) {
  if (D > kMaxD) return -2;
  if (rows) l2norm_fwd_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, s>>>((const bf16*)x, (bf16*)y, rstd, rows, D, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
int l2norm_bwd(const void* dy, const void* x, const float* rstd, void* dx, long long rows, int D, cudaStream_t s) {
  if (D > kMaxD) return -2;
  if (rows) l2norm_bwd_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, s>>>((const bf16*)dy, (const bf16*)x, rstd, (bf16*)dx, rows, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
int gated_rmsnorm_fwd(const void* x, const void* g, const void* w, void* y, float* rstd, long long rows, int D, float eps, cudaStream_t s) {
  if (D > kMaxD) return -2;
  if (rows) gated_rmsnorm_fwd_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, s>>>((const bf16*)x, (const bf16*)g, (const bf16*)w,
                                                                                          (bf16*)y, rstd, rows, D, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
int gated_rmsnorm_bwd(const void* dy, const void* x, const void* g, const void* w, const float* rstd, void* dx, void* dg,
                      float* dw_partial, int blocks, long long rows, int D, cudaStream_t s) {
  if (D > kMaxD) return -2;
  gated_rmsnorm_bwd_kernel<<<blocks, 256, 0, s>>>((const bf16*)dy, (const bf16*)x, (const bf16*)g, (const bf16*)w, rstd, (bf16*)dx,
                                                  (bf16*)dg, dw_partial, rows, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
int conv_silu_fwd(const void* x, const void* w, const int* seg_start, void* y, long long n, int C, int W, cudaStream_t s) {
  if (W > 4) return -2;
  const long long total = n * C;
  if (total) conv_silu_fwd_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>((const bf16*)x, (const bf16*)w, seg_start, (bf16*)y, n, C, W);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
int conv_silu_bwd(const void* dy, const void* x, const void* w, const int* seg_start, void* dx, float* dw_partial, int row_blocks,
                  int rows_per_block, long long n, int C, int W, cudaStream_t s) {
  if (W > 4) return -2;
  dim3 grid(row_blocks, (C + 127) / 128);
  conv_silu_bwd_kernel<<<grid, 128, 0, s>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, seg_start, (bf16*)dx, dw_partial, n, C, W,
                                            rows_per_block);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
int router_sigmoid_noaux(const void* logits, const float* bias, float* route_w, int* route_ids, int t, int E, int K, int n_group,
                         int topk_group, float scaling, cudaStream_t s) {
  if (E > 256 || K > kMaxK || n_group > 32 || (n_group > 1 && E % n_group)) return -2;
  if (t) router_sigmoid_noaux_kernel<<<(t + 7) / 8, 256, 0, s>>>((const bf16*)logits, bias, route_w, route_ids, t, E, K, n_group, topk_group, scaling);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace dfb
