// RMSNorm and LayerNorm, forward and backward, bf16 storage with fp32 math.
//
// Forward: one CTA per row, 16-byte loads, sum of squares reduced in a fixed
// order, emits the fp32 ``rstd`` (and ``mean`` for LayerNorm) the backward reuses.
// Backward: the normalised tensor is re-derived from x and the saved statistics;
// weight/bias gradients are accumulated per CTA over a strip of rows into fp32
// partials and reduced by a second kernel in a fixed order (deterministic).
// Numerics parity: reference src/dataflow_training/blocks/ops.py:30-144
// (eps inside the rsqrt, fp32 statistics, one rounding to storage).
#include "common.cuh"
#include "ops.h"

namespace dfb {

// ---------------------------------------------------------------------------- forward
template <bool kLayer, bool kHasWeight>
__global__ void __launch_bounds__(256) norm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                        const bf16* __restrict__ b, bf16* __restrict__ y,
                                                        float* __restrict__ rstd_out, float* __restrict__ mean_out,
                                                        int rows, int cols, float eps) {
  __shared__ float scratch[33];
  int row = blockIdx.x;
  if (row >= rows) return;
  const bf16* xr = x + static_cast<size_t>(row) * cols;
  bf16* yr = y + static_cast<size_t>(row) * cols;
  int nvec = cols >> 3;
  float s = 0.f, ss = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    unpack8(ld8(xr + v * 8), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) { s += f[i]; ss += f[i] * f[i]; }
  }
  for (int c = (nvec << 3) + threadIdx.x; c < cols; c += blockDim.x) {
    float f = bf2f(xr[c]);
    s += f; ss += f * f;
  }
  float mean = 0.f;
  if (kLayer) {
    mean = block_sum(s, scratch) / cols;
    // second pass for the variance keeps the subtraction exact
    float vs = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float f[8];
      unpack8(ld8(xr + v * 8), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) { float d = f[i] - mean; vs += d * d; }
    }
    for (int c = (nvec << 3) + threadIdx.x; c < cols; c += blockDim.x) { float d = bf2f(xr[c]) - mean; vs += d * d; }
    ss = vs;
  }
  float var = block_sum(ss, scratch) / cols;
  float rstd = rsqrtf(var + eps);
  if (threadIdx.x == 0) {
    if (rstd_out) rstd_out[row] = rstd;
    if (kLayer && mean_out) mean_out[row] = mean;
  }
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8], g[8], bb[8];
    unpack8(ld8(xr + v * 8), f);
    if (kHasWeight) unpack8(ld8(w + v * 8), g);
    if (kLayer && b) unpack8(ld8(b + v * 8), bb);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float n = (f[i] - mean) * rstd;
      if (kHasWeight) n *= g[i];
      if (kLayer && b) n += bb[i];
      f[i] = n;
    }
    st8(yr + v * 8, pack8(f));
  }
  for (int c = (nvec << 3) + threadIdx.x; c < cols; c += blockDim.x) {
    float n = (bf2f(xr[c]) - mean) * rstd;
    if (kHasWeight) n *= bf2f(w[c]);
    if (kLayer && b) n += bf2f(b[c]);
    yr[c] = f2bf(n);
  }
}

// Re-apply a norm from saved statistics (recompute and backward paths).
template <bool kLayer>
__global__ void __launch_bounds__(256) norm_apply_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                          const bf16* __restrict__ b, const float* __restrict__ rstd,
                                                          const float* __restrict__ mean, bf16* __restrict__ y,
                                                          int rows, int cols) {
  int row = blockIdx.x;
  if (row >= rows) return;
  const bf16* xr = x + static_cast<size_t>(row) * cols;
  bf16* yr = y + static_cast<size_t>(row) * cols;
  float r = rstd[row], m = kLayer ? mean[row] : 0.f;
  int nvec = cols >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8], g[8], bb[8];
    unpack8(ld8(xr + v * 8), f);
    unpack8(ld8(w + v * 8), g);
    if (kLayer && b) unpack8(ld8(b + v * 8), bb);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float n = (f[i] - m) * r * g[i];
      if (kLayer && b) n += bb[i];
      f[i] = n;
    }
    st8(yr + v * 8, pack8(f));
  }
  for (int c = (nvec << 3) + threadIdx.x; c < cols; c += blockDim.x) {
    float n = (bf2f(xr[c]) - m) * r * bf2f(w[c]);
    if (kLayer && b) n += bf2f(b[c]);
    yr[c] = f2bf(n);
  }
}

// ---------------------------------------------------------------------------- backward
// grid.x CTAs, each walks rows blockIdx.x, +gridDim.x, ...  dx is written per row;
// dw/db partial sums live in registers per column strip and land in ``partial``
// (gridDim.x, 2, cols) fp32.  ``add_to_dx``: dx += result (residual-stream gradient).
template <bool kLayer>
__global__ void __launch_bounds__(256) norm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                        const bf16* __restrict__ w, const float* __restrict__ rstd,
                                                        const float* __restrict__ mean, bf16* __restrict__ dx,
                                                        const bf16* __restrict__ dx_add, float* __restrict__ partial,
                                                        int rows, int cols) {
  __shared__ float scratch[33];
  constexpr int kMaxVec = 4;                 // columns per thread = 8 * kMaxVec * passes
  int nvec = cols >> 3;
  // each thread owns vectors v = threadIdx.x + j*blockDim.x
  for (int base = 0; base < nvec; base += blockDim.x * kMaxVec) {
    float dwacc[kMaxVec][8], dbacc[kMaxVec][8];
#pragma unroll
    for (int j = 0; j < kMaxVec; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) { dwacc[j][i] = 0.f; dbacc[j][i] = 0.f; }
    bool last_pass = base + blockDim.x * kMaxVec >= nvec;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
      const bf16* xr = x + static_cast<size_t>(row) * cols;
      const bf16* dyr = dy + static_cast<size_t>(row) * cols;
      float r = rstd[row], m = kLayer ? mean[row] : 0.f;
      if (base == 0) {
        // row statistics c1 = mean(g*xhat), c2 = mean(g) over the whole row (g = w*dy)
        float c1 = 0.f, c2 = 0.f;
        for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
          float fx[8], fd[8], fw[8];
          unpack8(ld8(xr + v * 8), fx);
          unpack8(ld8(dyr + v * 8), fd);
          unpack8(ld8(w + v * 8), fw);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float g = fd[i] * fw[i];
            c1 += g * (fx[i] - m) * r;
            c2 += g;
          }
        }
        c1 = block_sum(c1, scratch) / cols;
        if (kLayer) c2 = block_sum(c2, scratch) / cols; else c2 = 0.f;
        bf16* dxr = dx + static_cast<size_t>(row) * cols;
        const bf16* addr = dx_add ? dx_add + static_cast<size_t>(row) * cols : nullptr;
        for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
          float fx[8], fd[8], fw[8], fa[8];
          unpack8(ld8(xr + v * 8), fx);
          unpack8(ld8(dyr + v * 8), fd);
          unpack8(ld8(w + v * 8), fw);
          if (addr) unpack8(ld8(addr + v * 8), fa);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float xh = (fx[i] - m) * r;
            float o = (fd[i] * fw[i] - xh * c1 - c2) * r;
            if (addr) o += fa[i];
            fx[i] = o;
          }
          st8(dxr + v * 8, pack8(fx));
        }
      }
#pragma unroll
      for (int j = 0; j < kMaxVec; ++j) {
        int v = base + threadIdx.x + j * blockDim.x;
        if (v < nvec) {
          float fx[8], fd[8];
          unpack8(ld8(xr + v * 8), fx);
          unpack8(ld8(dyr + v * 8), fd);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            dwacc[j][i] += fd[i] * (fx[i] - m) * r;
            dbacc[j][i] += fd[i];
          }
        }
      }
    }
    float* pw = partial + static_cast<size_t>(blockIdx.x) * 2 * cols;
    float* pb = pw + cols;
#pragma unroll
    for (int j = 0; j < kMaxVec; ++j) {
      int v = base + threadIdx.x + j * blockDim.x;
      if (v < nvec) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          pw[v * 8 + i] = dwacc[j][i];
          if (kLayer) pb[v * 8 + i] = dbacc[j][i];
        }
      }
    }
    (void)last_pass;
  }
}

// RMSNorm backward for rows that fit the block's registers (cols = 2048 * VPT): every row is read from memory once —
// the next row's x / dy / addend are requested before the current row's reduction, so the loads overlap the block-wide
// sum — and the arithmetic (per-thread order of the row sum, the dx and dw expressions) is the generic kernel's.
template <int VPT>
__global__ void __launch_bounds__(256, VPT <= 2 ? 2 : 1) rmsnorm_bwd_regs_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                                   const bf16* __restrict__ w, const float* __restrict__ rstd,
                                                                   bf16* __restrict__ dx, const bf16* __restrict__ dx_add,
                                                                   float* __restrict__ partial, int rows, int cols) {
  __shared__ float scratch[33];
  const int tid = threadIdx.x;
  bf16x8 wv[VPT];                       // the weight strip stays packed; it is unpacked where it is used
  float dwacc[VPT][8];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    wv[j] = ld8(w + (tid + j * 256) * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) dwacc[j][i] = 0.f;
  }
  bf16x8 nx[VPT], nd[VPT], na[VPT];
  int row = blockIdx.x;
  if (row < rows) {
    size_t off = static_cast<size_t>(row) * cols;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      nx[j] = ld8(x + off + (tid + j * 256) * 8);
      nd[j] = ld8(dy + off + (tid + j * 256) * 8);
      if (dx_add) na[j] = ld8(dx_add + off + (tid + j * 256) * 8);
    }
  }
  for (; row < rows; row += gridDim.x) {
    bf16x8 cx[VPT], cd[VPT], ca[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) { cx[j] = nx[j]; cd[j] = nd[j]; ca[j] = na[j]; }
    float r = rstd[row];
    int nrow = row + gridDim.x;
    if (nrow < rows) {
      size_t off = static_cast<size_t>(nrow) * cols;
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        nx[j] = ld8(x + off + (tid + j * 256) * 8);
        nd[j] = ld8(dy + off + (tid + j * 256) * 8);
        if (dx_add) na[j] = ld8(dx_add + off + (tid + j * 256) * 8);
      }
    }
    float c1 = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      float fx[8], fd[8], fw[8];
      unpack8(cx[j], fx);
      unpack8(cd[j], fd);
      unpack8(wv[j], fw);
#pragma unroll
      for (int i = 0; i < 8; ++i) c1 += fd[i] * fw[i] * fx[i] * r;
    }
    c1 = block_sum(c1, scratch) / cols;
    bf16* dxr = dx + static_cast<size_t>(row) * cols;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      float fx[8], fd[8], fa[8], fw[8], o[8];
      unpack8(cx[j], fx);
      unpack8(cd[j], fd);
      unpack8(wv[j], fw);
      if (dx_add) unpack8(ca[j], fa);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float xh = fx[i] * r;
        o[i] = (fd[i] * fw[i] - xh * c1) * r;
        if (dx_add) o[i] += fa[i];
        dwacc[j][i] += fd[i] * fx[i] * r;
      }
      st8(dxr + (tid + j * 256) * 8, pack8(o));
    }
  }
  float* pw = partial + static_cast<size_t>(blockIdx.x) * 2 * cols;
#pragma unroll
  for (int j = 0; j < VPT; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) pw[(tid + j * 256) * 8 + i] = dwacc[j][i];
}

// Sum the per-CTA partials in index order; optionally accumulate into the existing gradient.
__global__ void norm_bwd_reduce_kernel(const float* __restrict__ partial, int nparts, int cols, bf16* __restrict__ dw,
                                        bf16* __restrict__ db, int accumulate) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float sw = 0.f, sb = 0.f;
  for (int p = 0; p < nparts; ++p) {
    sw += partial[static_cast<size_t>(p) * 2 * cols + c];
    if (db) sb += partial[static_cast<size_t>(p) * 2 * cols + cols + c];
  }
  if (accumulate) { sw += bf2f(dw[c]); if (db) sb += bf2f(db[c]); }
  dw[c] = f2bf(sw);
  if (db) db[c] = f2bf(sb);
}

__global__ void norm_bwd_reduce_f32_kernel(const float* __restrict__ partial, int nparts, int cols,
                                            float* __restrict__ dw, float* __restrict__ db, int accumulate) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float sw = 0.f, sb = 0.f;
  for (int p = 0; p < nparts; ++p) {
    sw += partial[static_cast<size_t>(p) * 2 * cols + c];
    if (db) sb += partial[static_cast<size_t>(p) * 2 * cols + cols + c];
  }
  if (accumulate) { sw += dw[c]; if (db) sb += db[c]; }
  dw[c] = sw;
  if (db) db[c] = sb;
}

// ---------------------------------------------------------------------------- host entry points
void rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int cols, float eps, cudaStream_t s) {
  if (rows == 0) return;
  if (w) norm_fwd_kernel<false, true><<<rows, 256, 0, s>>>((const bf16*)x, (const bf16*)w, nullptr, (bf16*)y, rstd, nullptr, rows, cols, eps);
  else norm_fwd_kernel<false, false><<<rows, 256, 0, s>>>((const bf16*)x, nullptr, nullptr, (bf16*)y, rstd, nullptr, rows, cols, eps);
}

void rmsnorm_apply(const void* x, const void* w, const float* rstd, void* y, int rows, int cols, cudaStream_t s) {
  if (rows == 0) return;
  norm_apply_kernel<false><<<rows, 256, 0, s>>>((const bf16*)x, (const bf16*)w, nullptr, rstd, nullptr, (bf16*)y, rows, cols);
}

void layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int rows, int cols,
                   float eps, cudaStream_t s) {
  if (rows == 0) return;
  norm_fwd_kernel<true, true><<<rows, 256, 0, s>>>((const bf16*)x, (const bf16*)w, (const bf16*)b, (bf16*)y, rstd, mean, rows, cols, eps);
}

void layernorm_apply(const void* x, const void* w, const void* b, const float* mean, const float* rstd, void* y,
                     int rows, int cols, cudaStream_t s) {
  if (rows == 0) return;
  norm_apply_kernel<true><<<rows, 256, 0, s>>>((const bf16*)x, (const bf16*)w, (const bf16*)b, rstd, mean, (bf16*)y, rows, cols);
}

int norm_bwd_parts(int rows) { return rows < 296 ? (rows > 0 ? rows : 1) : 296; }

void rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, const void* dx_add,
                 void* dw, int dw_is_f32, int accumulate, float* partial, int rows, int cols, cudaStream_t s) {
  if (rows == 0) return;
  int parts = norm_bwd_parts(rows);
  // every path below moves 16-byte vectors: callers (the torch binding, the C entry point) refuse operands that are not
  // 16-byte aligned or whose width is not a multiple of 8; ``aligned`` only selects the register-resident variant
  const bool aligned = ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) |
                         reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(dx_add)) & 15) == 0;
#define DFB_RMS_BWD_REGS(V)                                                                                                  \
  rmsnorm_bwd_regs_kernel<V><<<parts, 256, 0, s>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, (bf16*)dx,         \
                                                   (const bf16*)dx_add, partial, rows, cols)
  if (aligned && cols == 2048) DFB_RMS_BWD_REGS(1);
  else if (aligned && cols == 4096) DFB_RMS_BWD_REGS(2);
  else if (aligned && cols == 8192) DFB_RMS_BWD_REGS(4);
  else
    norm_bwd_kernel<false><<<parts, 256, 0, s>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, nullptr, (bf16*)dx,
                                                 (const bf16*)dx_add, partial, rows, cols);
#undef DFB_RMS_BWD_REGS
  if (dw) {
    if (dw_is_f32) norm_bwd_reduce_f32_kernel<<<ceil_div(cols, 256), 256, 0, s>>>(partial, parts, cols, (float*)dw, nullptr, accumulate);
    else norm_bwd_reduce_kernel<<<ceil_div(cols, 256), 256, 0, s>>>(partial, parts, cols, (bf16*)dw, nullptr, accumulate);
  }
}

void layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, void* dx,
                   const void* dx_add, void* dw, void* db, int dw_is_f32, int accumulate, float* partial, int rows,
                   int cols, cudaStream_t s) {
  if (rows == 0) return;
  int parts = norm_bwd_parts(rows);
  norm_bwd_kernel<true><<<parts, 256, 0, s>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, mean, (bf16*)dx,
                                              (const bf16*)dx_add, partial, rows, cols);
  if (dw) {
    if (dw_is_f32) norm_bwd_reduce_f32_kernel<<<ceil_div(cols, 256), 256, 0, s>>>(partial, parts, cols, (float*)dw, (float*)db, accumulate);
    else norm_bwd_reduce_kernel<<<ceil_div(cols, 256), 256, 0, s>>>(partial, parts, cols, (bf16*)dw, (bf16*)db, accumulate);
  }
}

}  // namespace dfb
