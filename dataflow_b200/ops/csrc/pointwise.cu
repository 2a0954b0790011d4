// Memory-bound elementwise kernels: RoPE, SwiGLU (flat and packed), GELU-tanh,
// AdamW (bf16 state and fp32-master variants), SGD / momentum, residual add,
// casts, bias gradients.  All use 16-byte accesses and fp32 math with a single
// rounding to the storage dtype.  Numerics parity: reference
// src/dataflow_training/blocks/ops.py:164-200 (rope), :318-335 (swiglu),
// :406-431 (adamw: moments stored then read back before bias correction).
#include "common.cuh"
#include "ops.h"

namespace dfb {

// ---------------------------------------------------------------------------- RoPE
// x: (tokens, heads, head_dim) with arbitrary row / head strides (in elements); rotates the first
// ``rot_dim`` dims starting at ``col_base`` in place (rotate-half pairing i <-> i + rot_dim/2).
__global__ void rope_kernel(bf16* __restrict__ x, const int* __restrict__ positions, int tokens, int heads,
                            int rot_dim, long long row_stride, int head_stride, int col_base, float log2_theta,
                            float sign) {
  int half = rot_dim >> 1;
  long long total = static_cast<long long>(tokens) * heads * half;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    int i = static_cast<int>(idx % half);
    long long th = idx / half;
    int h = static_cast<int>(th % heads);
    int t = static_cast<int>(th / heads);
    float inv_freq = exp2f(-log2_theta * (2.0f * i / rot_dim));
    float ang = static_cast<float>(positions[t]) * inv_freq;
    float sn, cs;
    sincosf(ang, &sn, &cs);
    sn *= sign;
    bf16* p = x + t * row_stride + static_cast<long long>(h) * head_stride + col_base;
    float a = bf2f(p[i]), b = bf2f(p[i + half]);
    p[i] = f2bf(a * cs - b * sn);
    p[i + half] = f2bf(b * cs + a * sn);
  }
}

// The same rotation with 16-byte accesses: a thread takes 8 consecutive pairs (i, i + rot_dim/2) of HPT heads of one
// token, so the 8 sines / cosines of its column strip are computed once per HPT heads.  Needs 16-byte aligned strips.
template <int HPT>
__global__ void rope_vec_kernel(bf16* __restrict__ x, const int* __restrict__ positions, int tokens, int heads,
                                int rot_dim, long long row_stride, int head_stride, int col_base, float log2_theta,
                                float sign) {
  const int half = rot_dim >> 1, vecs = half >> 3, hgroups = heads / HPT;
  const long long total = static_cast<long long>(tokens) * hgroups * vecs;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int iv = static_cast<int>(idx % vecs);
    const long long th = idx / vecs;
    const int hg = static_cast<int>(th % hgroups);
    const int t = static_cast<int>(th / hgroups);
    bf16* p = x + t * row_stride + static_cast<long long>(hg * HPT) * head_stride + col_base + iv * 8;
    bf16x8 lo[HPT], hi[HPT];
#pragma unroll
    for (int h = 0; h < HPT; ++h) {
      lo[h] = ld8(p + static_cast<long long>(h) * head_stride);
      hi[h] = ld8(p + static_cast<long long>(h) * head_stride + half);
    }
    const float pos = static_cast<float>(positions[t]);
    float sn[8], cs[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      int i = iv * 8 + j;
      float inv_freq = exp2f(-log2_theta * (2.0f * i / rot_dim));
      sincosf(pos * inv_freq, &sn[j], &cs[j]);
      sn[j] *= sign;
    }
#pragma unroll
    for (int h = 0; h < HPT; ++h) {
      float a[8], b[8], oa[8], ob[8];
      unpack8(lo[h], a);
      unpack8(hi[h], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        oa[j] = a[j] * cs[j] - b[j] * sn[j];
        ob[j] = b[j] * cs[j] + a[j] * sn[j];
      }
      st8(p + static_cast<long long>(h) * head_stride, pack8(oa));
      st8(p + static_cast<long long>(h) * head_stride + half, pack8(ob));
    }
  }
}

void rope_inplace(void* x, const int* positions, int tokens, int heads, int rot_dim, long long row_stride,
                  int head_stride, int col_base, float theta, int backward, cudaStream_t s) {
  long long total = static_cast<long long>(tokens) * heads * (rot_dim / 2);
  if (total == 0) return;
  const int half = rot_dim / 2;
  if (half % 8 == 0 && row_stride % 8 == 0 && head_stride % 8 == 0 && col_base % 8 == 0 &&
      (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const int hpt = heads % 4 == 0 ? 4 : 1;
    long long work = static_cast<long long>(tokens) * (heads / hpt) * (half / 8);
    int vblocks = static_cast<int>(std::min<long long>((work + 255) / 256, 148 * 32));
    if (hpt == 4)
      rope_vec_kernel<4><<<vblocks, 256, 0, s>>>((bf16*)x, positions, tokens, heads, rot_dim, row_stride, head_stride, col_base,
                                                 log2f(theta), backward ? -1.f : 1.f);
    else
      rope_vec_kernel<1><<<vblocks, 256, 0, s>>>((bf16*)x, positions, tokens, heads, rot_dim, row_stride, head_stride, col_base,
                                                 log2f(theta), backward ? -1.f : 1.f);
    return;
  }
  int blocks = static_cast<int>(std::min<long long>((total + 255) / 256, 148 * 16));
  rope_kernel<<<blocks, 256, 0, s>>>((bf16*)x, positions, tokens, heads, rot_dim, row_stride, head_stride, col_base,
                                     log2f(theta), backward ? -1.f : 1.f);
}

// ---------------------------------------------------------------------------- SwiGLU
DFB_DEVICE float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// rows x F outputs.  x1 at a + r*lda, x3 at b + r*ldb (packed layout: b = a + F, lda = ldb = 2F).
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, bf16* __restrict__ out,
                                  long long rows, int F, long long lda, long long ldb) {
  int vec_per_row = F >> 3;
  long long total = rows * vec_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    long long r = idx / vec_per_row;
    int v = static_cast<int>(idx % vec_per_row) * 8;
    float f1[8], f3[8];
    unpack8(ld8(a + r * lda + v), f1);
    unpack8(ld8(b + r * ldb + v), f3);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float sl = bf2f(f2bf(f1[i] * sigmoidf_(f1[i])));   // silu rounds to storage before the product
      f1[i] = sl * f3[i];
    }
    st8(out + r * F + v, pack8(f1));
  }
}

// ``s_out`` (optional, rows x F): the forward product silu(x1) * x3 with the forward's rounding, for the caller that needs
// it as a GEMM operand in the same backward (saves re-reading x1 / x3 in a separate forward launch).
__global__ void swiglu_bwd_kernel(const bf16* __restrict__ ds, const bf16* __restrict__ a, const bf16* __restrict__ b,
                                  bf16* __restrict__ da, bf16* __restrict__ db, bf16* __restrict__ s_out, long long rows,
                                  int F, long long lda, long long ldb, long long ldda, long long lddb) {
  int vec_per_row = F >> 3;
  long long total = rows * vec_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    long long r = idx / vec_per_row;
    int v = static_cast<int>(idx % vec_per_row) * 8;
    float f1[8], f3[8], g[8], o1[8], o3[8];
    unpack8(ld8(a + r * lda + v), f1);
    unpack8(ld8(b + r * ldb + v), f3);
    unpack8(ld8(ds + r * F + v), g);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float sg = sigmoidf_(f1[i]);
      float sl = f1[i] * sg;
      o3[i] = g[i] * sl;
      o1[i] = g[i] * f3[i] * (sg + sl * (1.f - sg));
    }
    st8(da + r * ldda + v, pack8(o1));
    st8(db + r * lddb + v, pack8(o3));
    if (s_out) {
#pragma unroll
      for (int i = 0; i < 8; ++i) o1[i] = bf2f(f2bf(f1[i] * sigmoidf_(f1[i]))) * f3[i];
      st8(s_out + r * F + v, pack8(o1));
    }
  }
}

static int ew_blocks(long long n) { return static_cast<int>(std::max<long long>(1, std::min<long long>((n + 255) / 256, 148 * 32))); }

void swiglu_fwd(const void* x1, const void* x3, void* out, long long rows, int F, long long ld1, long long ld3, cudaStream_t s) {
  if (rows == 0) return;
  swiglu_fwd_kernel<<<ew_blocks(rows * (F / 8)), 256, 0, s>>>((const bf16*)x1, (const bf16*)x3, (bf16*)out, rows, F, ld1, ld3);
}

void swiglu_bwd(const void* ds, const void* x1, const void* x3, void* dx1, void* dx3, void* s_out, long long rows, int F,
                long long ld1, long long ld3, long long ldd1, long long ldd3, cudaStream_t s) {
  if (rows == 0) return;
  swiglu_bwd_kernel<<<ew_blocks(rows * (F / 8)), 256, 0, s>>>((const bf16*)ds, (const bf16*)x1, (const bf16*)x3, (bf16*)dx1,
                                                              (bf16*)dx3, (bf16*)s_out, rows, F, ld1, ld3, ldd1, ldd3);
}

// ---------------------------------------------------------------------------- GELU (tanh form)
DFB_DEVICE float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.f + tanhf(u));
}
DFB_DEVICE float gelu_tanh_grad(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  float t = tanhf(u);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k0 * (1.f + 3.f * k1 * x * x);
}

__global__ void gelu_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long n8) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float f[8];
    unpack8(ld8(x + i * 8), f);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = gelu_tanh(f[k]);
    st8(y + i * 8, pack8(f));
  }
}
__global__ void gelu_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, bf16* __restrict__ dx, long long n8) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float f[8], g[8];
    unpack8(ld8(x + i * 8), f);
    unpack8(ld8(dy + i * 8), g);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = g[k] * gelu_tanh_grad(f[k]);
    st8(dx + i * 8, pack8(f));
  }
}
void gelu_fwd(const void* x, void* y, long long n, cudaStream_t s) {
  if (n == 0) return;
  gelu_fwd_kernel<<<ew_blocks(n / 8), 256, 0, s>>>((const bf16*)x, (bf16*)y, n / 8);
}
void gelu_bwd(const void* dy, const void* x, void* dx, long long n, cudaStream_t s) {
  if (n == 0) return;
  gelu_bwd_kernel<<<ew_blocks(n / 8), 256, 0, s>>>((const bf16*)dy, (const bf16*)x, (bf16*)dx, n / 8);
}

// ---------------------------------------------------------------------------- residual add / casts
__global__ void add_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, bf16* __restrict__ out, long long n8) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float f[8], g[8];
    unpack8(ld8(a + i * 8), f);
    unpack8(ld8(b + i * 8), g);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] += g[k];
    st8(out + i * 8, pack8(f));
  }
}
void add_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t s) {
  if (n == 0) return;
  add_kernel<<<ew_blocks(n / 8), 256, 0, s>>>((const bf16*)a, (const bf16*)b, (bf16*)out, n / 8);
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ x, bf16* __restrict__ y, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    y[i] = f2bf(x[i]);
}
__global__ void cast_bf16_f32_kernel(const bf16* __restrict__ x, float* __restrict__ y, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    y[i] = bf2f(x[i]);
}
void cast_f32_to_bf16(const float* x, void* y, long long n, cudaStream_t s) {
  if (n) cast_f32_bf16_kernel<<<ew_blocks(n), 256, 0, s>>>(x, (bf16*)y, n);
}
void cast_bf16_to_f32(const void* x, float* y, long long n, cudaStream_t s) {
  if (n) cast_bf16_f32_kernel<<<ew_blocks(n), 256, 0, s>>>((const bf16*)x, y, n);
}

// column sums of a (rows, cols) bf16 matrix into fp32 partials then bf16/f32 out: bias gradients.
__global__ void colsum_kernel(const bf16* __restrict__ x, float* __restrict__ partial, int rows, int cols) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int r = blockIdx.y; r < rows; r += gridDim.y) s += bf2f(x[static_cast<size_t>(r) * cols + c]);
  partial[static_cast<size_t>(blockIdx.y) * cols + c] = s;
}
__global__ void colsum_reduce_kernel(const float* __restrict__ partial, int parts, int cols, bf16* __restrict__ out, int accumulate) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += partial[static_cast<size_t>(p) * cols + c];
  if (accumulate) s += bf2f(out[c]);
  out[c] = f2bf(s);
}
int colsum_parts(int rows) { return rows < 128 ? (rows > 0 ? rows : 1) : 128; }
void colsum_bf16(const void* x, float* partial, void* out, int accumulate, int rows, int cols, cudaStream_t s) {
  if (rows == 0 || cols == 0) return;
  int parts = colsum_parts(rows);
  dim3 grid(ceil_div(cols, 128), parts);
  colsum_kernel<<<grid, 128, 0, s>>>((const bf16*)x, partial, rows, cols);
  colsum_reduce_kernel<<<ceil_div(cols, 128), 128, 0, s>>>(partial, parts, cols, (bf16*)out, accumulate);
}

DFB_DEVICE float to_f(float x) { return x; }
DFB_DEVICE float to_f(bf16 x) { return bf2f(x); }

// ---------------------------------------------------------------------------- optimizers
// AdamW, all-bf16 state: w, m, v bf16; g bf16 or fp32.
template <typename G>
__global__ void adamw_bf16_kernel(bf16* __restrict__ w, const G* __restrict__ g, bf16* __restrict__ m, bf16* __restrict__ v,
                                  long long n, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                                  float gscale) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float gi = to_f(g[i]) * gscale;
    float mi = b1 * bf2f(m[i]) + (1.f - b1) * gi;
    float vi = b2 * bf2f(v[i]) + (1.f - b2) * gi * gi;
    bf16 ms = f2bf(mi), vs = f2bf(vi);
    m[i] = ms; v[i] = vs;
    float mh = bf2f(ms) / bc1, vh = bf2f(vs) / bc2;      // stored moments are what gets bias-corrected
    float wi = bf2f(w[i]);
    wi -= lr * (mh / (sqrtf(vh) + eps) + wd * wi);
    w[i] = f2bf(wi);
  }
}

// AdamW with fp32 master weights and fp32 moments; writes the bf16 working copy.
template <typename G>
__global__ void adamw_master_kernel(float* __restrict__ master, bf16* __restrict__ w_out, const G* __restrict__ g,
                                    float* __restrict__ m, float* __restrict__ v, long long n, float lr, float b1, float b2,
                                    float eps, float wd, float bc1, float bc2, float gscale) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float gi = to_f(g[i]) * gscale;
    float mi = b1 * m[i] + (1.f - b1) * gi;
    float vi = b2 * v[i] + (1.f - b2) * gi * gi;
    m[i] = mi; v[i] = vi;
    float wi = master[i];
    wi -= lr * ((mi / bc1) / (sqrtf(vi / bc2) + eps) + wd * wi);
    master[i] = wi;
    w_out[i] = f2bf(wi);
  }
}

// fp32 everything (CPU-parity lane for fp32 models running on the GPU).
__global__ void adamw_f32_kernel(float* __restrict__ w, const float* __restrict__ g, float* __restrict__ m,
                                 float* __restrict__ v, long long n, float lr, float b1, float b2, float eps, float wd,
                                 float bc1, float bc2, float gscale) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float gi = g[i] * gscale;
    float mi = b1 * m[i] + (1.f - b1) * gi;
    float vi = b2 * v[i] + (1.f - b2) * gi * gi;
    m[i] = mi; v[i] = vi;
    float wi = w[i];
    wi -= lr * ((mi / bc1) / (sqrtf(vi / bc2) + eps) + wd * wi);
    w[i] = wi;
  }
}

// AdamW on an fp32 master that is stored SPLIT: its high 16 bits are the bf16 working weight itself (kept
// where forward and backward read it) and only its low 16 bits travel with the optimizer state, so the
// state is 6 bytes per parameter (low half + bf16 moments) with an exact fp32 master.  The working
// weight is the master rounded half away from zero, which makes the split exact:
//   master_bits = (w_bits << 16) + (int16) lo,   lo = master_bits & 0xffff.
DFB_DEVICE float split_join(bf16 w, uint16_t lo) {
  uint32_t hi = static_cast<uint32_t>(__bfloat16_as_ushort(w)) << 16;
  return __uint_as_float(hi + static_cast<uint32_t>(static_cast<int32_t>(static_cast<int16_t>(lo))));
}
DFB_DEVICE void split_cut(float x, bf16& w, uint16_t& lo) {
  uint32_t b = __float_as_uint(x);
  w = __ushort_as_bfloat16(static_cast<uint16_t>((b + 0x8000u) >> 16));
  lo = static_cast<uint16_t>(b & 0xffffu);
}
DFB_DEVICE float adamw_split_one(bf16& w, uint16_t& lo, float gi, bf16& m, bf16& v, float lr, float b1, float b2, float eps,
                                 float wd, float bc1, float bc2) {
  float mi = b1 * bf2f(m) + (1.f - b1) * gi;
  float vi = b2 * bf2f(v) + (1.f - b2) * gi * gi;
  m = f2bf(mi); v = f2bf(vi);
  float mh = bf2f(m) / bc1, vh = bf2f(v) / bc2;
  float wi = split_join(w, lo);
  wi -= lr * (mh / (sqrtf(vh) + eps) + wd * wi);
  split_cut(wi, w, lo);
  return wi;
}
// 8 elements per thread through 16-byte accesses (two for fp32 gradients); the tail (n % 8) runs scalar in the
// last block.
template <typename G>
__global__ void adamw_split_kernel(bf16* __restrict__ w, uint16_t* __restrict__ lo, const G* __restrict__ g,
                                   bf16* __restrict__ m, bf16* __restrict__ v, long long n, float lr, float b1, float b2,
                                   float eps, float wd, float bc1, float bc2, float gscale) {
  const long long n8 = n >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    uint4 wq = reinterpret_cast<uint4*>(w)[i], lq = reinterpret_cast<uint4*>(lo)[i];
    uint4 mq = reinterpret_cast<uint4*>(m)[i], vq = reinterpret_cast<uint4*>(v)[i];
    float gf[8];
    if constexpr (sizeof(G) == 4) {
      const float4 a = reinterpret_cast<const float4*>(g)[2 * i], b = reinterpret_cast<const float4*>(g)[2 * i + 1];
      gf[0] = a.x; gf[1] = a.y; gf[2] = a.z; gf[3] = a.w; gf[4] = b.x; gf[5] = b.y; gf[6] = b.z; gf[7] = b.w;
    } else {
      const uint4 gq = reinterpret_cast<const uint4*>(g)[i];
      unpack8(*reinterpret_cast<const bf16x8*>(&gq), gf);
    }
    bf16* wp = reinterpret_cast<bf16*>(&wq); uint16_t* lp = reinterpret_cast<uint16_t*>(&lq);
    bf16* mp = reinterpret_cast<bf16*>(&mq); bf16* vp = reinterpret_cast<bf16*>(&vq);
#pragma unroll
    for (int k = 0; k < 8; ++k) adamw_split_one(wp[k], lp[k], gf[k] * gscale, mp[k], vp[k], lr, b1, b2, eps, wd, bc1, bc2);
    reinterpret_cast<uint4*>(w)[i] = wq; reinterpret_cast<uint4*>(lo)[i] = lq;
    reinterpret_cast<uint4*>(m)[i] = mq; reinterpret_cast<uint4*>(v)[i] = vq;
  }
  if (blockIdx.x == gridDim.x - 1) {
    for (long long i = (n8 << 3) + threadIdx.x; i < n; i += blockDim.x)
      adamw_split_one(w[i], lo[i], to_f(g[i]) * gscale, m[i], v[i], lr, b1, b2, eps, wd, bc1, bc2);
  }
}
// A weight that was never stepped has lo == 0 (master == weight).  All five arrays must be 16-byte aligned
// (fields of packed layouts are 256-byte aligned); returns -2 otherwise.
int adamw_split(void* w, void* lo, const void* g, int g_is_f32, void* m, void* v, long long n, float lr, float b1, float b2,
                float eps, float wd, int step, float gscale, cudaStream_t s) {
  if (n == 0) return 0;
  if ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(lo) | reinterpret_cast<uintptr_t>(g) |
       reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15)
    return -2;
  float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  if (g_is_f32)
    adamw_split_kernel<float><<<ew_blocks((n + 7) / 8), 256, 0, s>>>((bf16*)w, (uint16_t*)lo, (const float*)g, (bf16*)m, (bf16*)v,
                                                                   n, lr, b1, b2, eps, wd, bc1, bc2, gscale);
  else
    adamw_split_kernel<bf16><<<ew_blocks((n + 7) / 8), 256, 0, s>>>((bf16*)w, (uint16_t*)lo, (const bf16*)g, (bf16*)m, (bf16*)v,
                                                                  n, lr, b1, b2, eps, wd, bc1, bc2, gscale);
  return 0;
}

void adamw_bf16(void* w, const void* g, int g_is_f32, void* m, void* v, long long n, float lr, float b1, float b2,
                float eps, float wd, int step, float gscale, cudaStream_t s) {
  if (n == 0) return;
  float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  if (g_is_f32) adamw_bf16_kernel<float><<<ew_blocks(n), 256, 0, s>>>((bf16*)w, (const float*)g, (bf16*)m, (bf16*)v, n, lr, b1, b2, eps, wd, bc1, bc2, gscale);
  else adamw_bf16_kernel<bf16><<<ew_blocks(n), 256, 0, s>>>((bf16*)w, (const bf16*)g, (bf16*)m, (bf16*)v, n, lr, b1, b2, eps, wd, bc1, bc2, gscale);
}

void adamw_master(float* master, void* w_out, const void* g, int g_is_f32, float* m, float* v, long long n, float lr,
                  float b1, float b2, float eps, float wd, int step, float gscale, cudaStream_t s) {
  if (n == 0) return;
  float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  if (g_is_f32) adamw_master_kernel<float><<<ew_blocks(n), 256, 0, s>>>(master, (bf16*)w_out, (const float*)g, m, v, n, lr, b1, b2, eps, wd, bc1, bc2, gscale);
  else adamw_master_kernel<bf16><<<ew_blocks(n), 256, 0, s>>>(master, (bf16*)w_out, (const bf16*)g, m, v, n, lr, b1, b2, eps, wd, bc1, bc2, gscale);
}

void adamw_f32(float* w, const float* g, float* m, float* v, long long n, float lr, float b1, float b2, float eps,
               float wd, int step, float gscale, cudaStream_t s) {
  if (n == 0) return;
  float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  adamw_f32_kernel<<<ew_blocks(n), 256, 0, s>>>(w, g, m, v, n, lr, b1, b2, eps, wd, bc1, bc2, gscale);
}

// SGD (momentum == 0: plain; else m <- mu*m + g, w <- w(1 - lr*wd) - lr*m), bf16 storage.
__global__ void sgd_kernel(bf16* __restrict__ w, const bf16* __restrict__ g, bf16* __restrict__ m, long long n, float lr,
                           float mu, float wd) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float gi = bf2f(g[i]);
    if (m) {
      float mi = mu * bf2f(m[i]) + gi;
      bf16 ms = f2bf(mi);
      m[i] = ms;
      gi = bf2f(ms);
    }
    float wi = bf2f(w[i]);
    w[i] = f2bf(wi * (1.f - lr * wd) - lr * gi);
  }
}
void sgd_bf16(void* w, const void* g, void* m, long long n, float lr, float mu, float wd, cudaStream_t s) {
  if (n) sgd_kernel<<<ew_blocks(n), 256, 0, s>>>((bf16*)w, (const bf16*)g, (bf16*)m, n, lr, mu, wd);
}

}  // namespace dfb
