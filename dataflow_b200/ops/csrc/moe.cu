// Mixture-of-experts routing and data movement kernels (sm_100a).
//
//   moe_topk_softmax   one warp per token: top-k over E <= 1024 logits with the smallest-index tie-break, softmax over
//                      the selection (mode 0) or selection of softmax probabilities (mode 1); fp32 math end to end
//   moe_router_bwd     d(logits) rows from d(route weights), both modes
//   moe_dispatch       xp[r] = x[row_src[r]], zero rows where row_src < 0 (the padding of the expert-major layout)
//   moe_combine        y[t] = base[t] + sum_k w[t,k] * yp[row_of[t,k]]   (fp32 accumulate, one rounding)
//   moe_dispatch_bwd   dx[t] (+)= sum_k dxp[row_of[t,k]]
//   moe_scale_rows     xp[row_of[t,k]] *= w[t,k]
//   moe_rowdot         out[t,k] = <a[row_of[t,k]], b[row_of[t,k]]>
//
// Semantics follow the reference ops (src/dataflow_training/kernels/moe_router.py:181-316,
// kernels/moe_dispatch.py:63-235); the row tables address the padded layout of ops/eager.py::moe_sort.
#include <cfloat>

#include "common.cuh"
#include "ops.h"

namespace dfb {

constexpr int kMaxTopK = 16;
constexpr int kMaxPerLane = 32;      // E <= 1024

template <typename T>
DFB_DEVICE float load_f(const T* p);
template <>
DFB_DEVICE float load_f<float>(const float* p) { return *p; }
template <>
DFB_DEVICE float load_f<bf16>(const bf16* p) { return bf2f(*p); }

// (value, index) argmax across the warp; ties -> smaller index
DFB_DEVICE void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, v, o);
    int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}
template <typename T>
__global__ void moe_topk_softmax_kernel(const T* __restrict__ logits, float* __restrict__ route_w, int* __restrict__ route_ids,
                                        int t, int E, int K, int mode) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= t) return;
  const T* row = logits + static_cast<long long>(warp) * E;
  float v[kMaxPerLane];
  const int per = (E + 31) / 32;
#pragma unroll 1
  for (int j = 0; j < per; ++j) {
    int e = j * 32 + lane;
    v[j] = e < E ? load_f(row + e) : -FLT_MAX;
  }
  if (mode == 1) {            // probabilities over all experts first
    float mx = -FLT_MAX;
    for (int j = 0; j < per; ++j) mx = fmaxf(mx, v[j]);
    mx = warp_max(mx);
    float s = 0.f;
    for (int j = 0; j < per; ++j) {
      int e = j * 32 + lane;
      v[j] = e < E ? __expf(v[j] - mx) : -FLT_MAX;
      if (e < E) s += v[j];
    }
    s = warp_sum(s);
    for (int j = 0; j < per; ++j) if (j * 32 + lane < E) v[j] /= s;
  }
  float sel_v[kMaxTopK];
  int sel_i[kMaxTopK];
  for (int k = 0; k < K; ++k) {
    float bv = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int j = 0; j < per; ++j) {
      int e = j * 32 + lane;
      if (e < E && (v[j] > bv || (v[j] == bv && e < bi))) { bv = v[j]; bi = e; }
    }
    warp_argmax(bv, bi);
    sel_v[k] = bv; sel_i[k] = bi;
    if ((bi & 31) == lane) v[bi >> 5] = -FLT_MAX;        // remove the winner
  }
  if (lane == 0) {
    if (mode == 0) {
      float mx = sel_v[0], s = 0.f;
      for (int k = 0; k < K; ++k) { sel_v[k] = __expf(sel_v[k] - mx); s += sel_v[k]; }
      for (int k = 0; k < K; ++k) sel_v[k] /= s;
    }
    for (int k = 0; k < K; ++k) {
      route_w[static_cast<long long>(warp) * K + k] = sel_v[k];
      route_ids[static_cast<long long>(warp) * K + k] = sel_i[k];
    }
  }
}

template <typename T>
__global__ void moe_router_bwd_kernel(const float* __restrict__ dprob, const float* __restrict__ route_w,
                                      const int* __restrict__ route_ids, const T* __restrict__ logits,
                                      float* __restrict__ dlogits, int t, int E, int K, int mode) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= t) return;
  const long long rk = static_cast<long long>(warp) * K, re = static_cast<long long>(warp) * E;
  if (mode == 0) {
    float dot = 0.f;
    for (int k = 0; k < K; ++k) dot += route_w[rk + k] * dprob[rk + k];
    for (int e = lane; e < E; e += 32) dlogits[re + e] = 0.f;
    __syncwarp();
    if (lane < K) dlogits[re + route_ids[rk + lane]] = route_w[rk + lane] * (dprob[rk + lane] - dot);
  } else {
    float mx = -FLT_MAX;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, load_f(logits + re + e));
    mx = warp_max(mx);
    float s = 0.f;
    for (int e = lane; e < E; e += 32) s += __expf(load_f(logits + re + e) - mx);
    s = warp_sum(s);
    float dot = 0.f;          // sum_k dp_k P[c_k]; route_w holds P[c_k] in this mode
    for (int k = 0; k < K; ++k) dot += dprob[rk + k] * route_w[rk + k];
    for (int e = lane; e < E; e += 32) dlogits[re + e] = -(__expf(load_f(logits + re + e) - mx) / s) * dot;
    __syncwarp();
    if (lane < K) dlogits[re + route_ids[rk + lane]] += dprob[rk + lane] * route_w[rk + lane];
  }
}

// one block of 128 threads per row (d / 8 16-byte vectors strided over the block)
__global__ void moe_dispatch_kernel(const bf16* __restrict__ x, const int* __restrict__ row_src, bf16* __restrict__ xp,
                                    int d, long long ldx) {
  const long long r = blockIdx.x;
  const int src = row_src[r];
  const int nvec = d >> 3;
  uint4* dst = reinterpret_cast<uint4*>(xp + r * d);
  if (src < 0) {
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) dst[v] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* s = reinterpret_cast<const uint4*>(x + static_cast<long long>(src) * ldx);
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) dst[v] = s[v];
}

template <bool WEIGHTED>
__global__ void moe_gather_sum_kernel(const bf16* __restrict__ base, const bf16* __restrict__ yp, const float* __restrict__ w,
                                      const int* __restrict__ row_of, bf16* __restrict__ out, int d, int K, int accumulate) {
  const long long t = blockIdx.x;
  const int nvec = d >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int k = 0; k < K; ++k) {
      const long long r = row_of[t * K + k];
      float f[8];
      unpack8(ld8(yp + r * d + v * 8), f);
      const float wk = WEIGHTED ? w[t * K + k] : 1.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += wk * f[i];
    }
    if (base) {
      float f[8];
      unpack8(ld8(base + t * d + v * 8), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
    if (accumulate) {
      float f[8];
      unpack8(ld8(out + t * d + v * 8), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
    st8(out + t * d + v * 8, pack8(acc));
  }
}

__global__ void moe_scale_rows_kernel(bf16* __restrict__ xp, const float* __restrict__ w, const int* __restrict__ row_of, int d) {
  const long long slot = blockIdx.x;
  const long long r = row_of[slot];
  const float s = w[slot];
  for (int v = threadIdx.x; v < (d >> 3); v += blockDim.x) {
    float f[8];
    unpack8(ld8(xp + r * d + v * 8), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] *= s;
    st8(xp + r * d + v * 8, pack8(f));
  }
}

__global__ void moe_rowdot_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, const int* __restrict__ row_of,
                                  float* __restrict__ out, int d) {
  const long long slot = blockIdx.x;
  const long long r = row_of[slot];
  float acc = 0.f;
  for (int v = threadIdx.x; v < (d >> 3); v += blockDim.x) {
    float fa[8], fb[8];
    unpack8(ld8(a + r * d + v * 8), fa);
    unpack8(ld8(b + r * d + v * 8), fb);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += fa[i] * fb[i];
  }
  __shared__ float red[4];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) s += red[i];
    out[slot] = s;
  }
}

// ---------------------------------------------------------------------------- host entry points
int moe_topk_softmax(const void* logits, int logits_f32, float* route_w, int* route_ids, int t, int E, int K, int mode,
                     cudaStream_t s) {
  if (E > 32 * kMaxPerLane || K > kMaxTopK || K > E) return -2;
  if (t == 0) return 0;
  int blocks = (t * 32 + 255) / 256;
  if (logits_f32) moe_topk_softmax_kernel<float><<<blocks, 256, 0, s>>>((const float*)logits, route_w, route_ids, t, E, K, mode);
  else moe_topk_softmax_kernel<bf16><<<blocks, 256, 0, s>>>((const bf16*)logits, route_w, route_ids, t, E, K, mode);
  return 0;
}

int moe_router_bwd(const float* dprob, const float* route_w, const int* route_ids, const void* logits, int logits_f32,
                   float* dlogits, int t, int E, int K, int mode, cudaStream_t s) {
  if (K > 32) return -2;
  if (t == 0) return 0;
  int blocks = (t * 32 + 255) / 256;
  if (logits_f32) moe_router_bwd_kernel<float><<<blocks, 256, 0, s>>>(dprob, route_w, route_ids, (const float*)logits, dlogits, t, E, K, mode);
  else moe_router_bwd_kernel<bf16><<<blocks, 256, 0, s>>>(dprob, route_w, route_ids, (const bf16*)logits, dlogits, t, E, K, mode);
  return 0;
}

int moe_dispatch(const void* x, long long ldx, const int* row_src, void* xp, int rows, int d, cudaStream_t s) {
  if (d % 8 || ldx % 8) return -2;
  if (rows) moe_dispatch_kernel<<<rows, 128, 0, s>>>((const bf16*)x, row_src, (bf16*)xp, d, ldx);
  return 0;
}

int moe_combine(const void* base, const void* yp, const float* w, const int* row_of, void* out, int t, int d, int K,
                cudaStream_t s) {
  if (d % 8) return -2;
  if (t) moe_gather_sum_kernel<true><<<t, 128, 0, s>>>((const bf16*)base, (const bf16*)yp, w, row_of, (bf16*)out, d, K, 0);
  return 0;
}

int moe_dispatch_bwd(const void* dxp, const int* row_of, void* out, int t, int d, int K, int accumulate, cudaStream_t s) {
  if (d % 8) return -2;
  if (t) moe_gather_sum_kernel<false><<<t, 128, 0, s>>>(nullptr, (const bf16*)dxp, nullptr, row_of, (bf16*)out, d, K, accumulate);
  return 0;
}

int moe_scale_rows(void* xp, const float* w, const int* row_of, int slots, int d, cudaStream_t s) {
  if (d % 8) return -2;
  if (slots) moe_scale_rows_kernel<<<slots, 128, 0, s>>>((bf16*)xp, w, row_of, d);
  return 0;
}

int moe_rowdot(const void* a, const void* b, const int* row_of, float* out, int slots, int d, cudaStream_t s) {
  if (d % 8) return -2;
  if (slots) moe_rowdot_kernel<<<slots, 128, 0, s>>>((const bf16*)a, (const bf16*)b, row_of, out, d);
  return 0;
}

}  // namespace dfb

// ---------------------------------------------------------------------------- moe_sort: the padded expert-major layout
// A stable counting sort of the t*K routed slots by expert, without a library sort and without a host sync:
//   pass 1  per chunk of kSortChunk consecutive slots: how many go to each expert            (chunk_counts[chunk][e])
//   pass 2  one CTA: per expert, exclusive scan over the chunks; totals -> counts, padded offsets, the expert of every row
//           tile; row_src cleared to -1
//   pass 3  per chunk again: a slot's row = padded offset of its expert + slots of that expert in earlier chunks + slots
//           of that expert EARLIER IN THE CHUNK (counted by comparison: stable, hence deterministic)
namespace dfb {

constexpr int kSortChunk = 1024;
constexpr int kSortMaxE = 1024;

__global__ void moe_sort_count_kernel(const int* __restrict__ ids, int n, int E, int* __restrict__ chunk_counts) {
  extern __shared__ int hist[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int base = blockIdx.x * kSortChunk;
  for (int i = threadIdx.x; i < kSortChunk && base + i < n; i += blockDim.x) {
    const int e = ids[base + i];
    if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) chunk_counts[static_cast<long long>(blockIdx.x) * E + e] = hist[e];
}

__global__ void moe_sort_scan_kernel(int* __restrict__ chunk_counts, int chunks, int E, int tile_rows, int mp, int* __restrict__ counts,
                                     int* __restrict__ offsets_pad, int* __restrict__ tile_expert, int* __restrict__ row_src) {
  __shared__ int s_off[kSortMaxE + 1];
  // per expert: chunk_counts[c][e] becomes the number of that expert's slots in chunks before c
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int c = 0; c < chunks; ++c) {
      const long long at = static_cast<long long>(c) * E + e;
      const int v = chunk_counts[at];
      chunk_counts[at] = run;
      run += v;
    }
    counts[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    for (int e = 0; e < E; ++e) {
      s_off[e] = off;
      offsets_pad[e] = off;
      off += (counts[e] + tile_rows - 1) / tile_rows * tile_rows;
    }
    s_off[E] = off;
    offsets_pad[E] = off;
  }
  __syncthreads();
  const int tiles = mp / tile_rows;
  for (int t = threadIdx.x; t < tiles; t += blockDim.x) {
    const int row = t * tile_rows;
    int e = -1;
    if (row < s_off[E]) {
      int lo = 0, hi = E;                       // the last expert whose padded offset is <= row and that owns rows
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_off[mid] <= row) lo = mid; else hi = mid;
      }
      e = lo;
    }
    tile_expert[t] = e;
  }
  for (int r = threadIdx.x; r < mp; r += blockDim.x) row_src[r] = -1;
}

__global__ void moe_sort_place_kernel(const int* __restrict__ ids, int n, int K, int E, const int* __restrict__ chunk_counts,
                                      const int* __restrict__ offsets_pad, int* __restrict__ row_of, int* __restrict__ row_src) {
  __shared__ int s_ids[kSortChunk];
  const int base = blockIdx.x * kSortChunk;
  const int len = min(kSortChunk, n - base);
  for (int i = threadIdx.x; i < len; i += blockDim.x) s_ids[i] = ids[base + i];
  __syncthreads();
  for (int i = threadIdx.x; i < len; i += blockDim.x) {
    const int e = s_ids[i];
    if (e < 0 || e >= E) { row_of[base + i] = -1; continue; }
    int before = 0;
    for (int j = 0; j < i; ++j) before += (s_ids[j] == e);
    const int row = offsets_pad[e] + chunk_counts[static_cast<long long>(blockIdx.x) * E + e] + before;
    row_of[base + i] = row;
    row_src[row] = (base + i) / K;
  }
}

// scratch: chunks * E ints.  Two experts may share a padded offset only when the first has no rows (then it has no tiles and
// the binary search lands on the later one, which is the owner).
int moe_sort(const int* ids, int t, int K, int E, int tile_rows, int mp, int* row_of, int* row_src, int* offsets_pad, int* tile_expert,
             int* counts, int* scratch, cudaStream_t s) {
  const int n = t * K;
  if (E < 1 || E > kSortMaxE || n <= 0 || tile_rows <= 0 || mp % tile_rows) return -1;
  const int chunks = (n + kSortChunk - 1) / kSortChunk;
  moe_sort_count_kernel<<<chunks, 256, E * sizeof(int), s>>>(ids, n, E, scratch);
  moe_sort_scan_kernel<<<1, 1024, 0, s>>>(scratch, chunks, E, tile_rows, mp, counts, offsets_pad, tile_expert, row_src);
  moe_sort_place_kernel<<<chunks, 256, 0, s>>>(ids, n, K, E, scratch, offsets_pad, row_of, row_src);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace dfb
