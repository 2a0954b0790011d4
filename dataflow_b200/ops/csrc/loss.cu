// Fused cross-entropy forward + backward over a (rows, vocab) bf16 logits chunk.
//
// One CTA per row.  Pass 1: online max / sum-exp in fp32 (one read of the row).
// Pass 2: overwrite the logits in place with dlogits = (softmax - onehot) * scale
// in bf16 and emit the row's negative log-likelihood.  Rows whose target is < 0
// are ignored by mask-multiply (zero loss, zero gradient row), which keeps the
// reduction order fixed.  ``scale`` = 1 / total_rows of the whole round so chunked
// partial losses sum to the round mean.  Numerics parity: reference
// src/dataflow_training/blocks/ops.py:358-394.
#include "common.cuh"
#include "ops.h"

namespace dfb {

__global__ void __launch_bounds__(512) ce_fwd_bwd_kernel(bf16* __restrict__ logits, const int* __restrict__ targets,
                                                          float* __restrict__ nll, int rows, int vocab, long long ld,
                                                          float scale) {
  __shared__ float scratch[33];
  int row = blockIdx.x;
  if (row >= rows) return;
  bf16* lr = logits + static_cast<long long>(row) * ld;
  int tgt = targets[row];
  if (tgt >= vocab) tgt = -1;          // an id outside the vocabulary is ignored like a negative one, never dereferenced
  float keep = tgt >= 0 ? 1.f : 0.f;
  int nvec = vocab >> 3;
  // pass 1: per-thread online (max, sum)
  float mx = -INFINITY, sm = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    unpack8(ld8(lr + v * 8), f);
    float lm = f[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) lm = fmaxf(lm, f[i]);
    if (lm > mx) { sm *= __expf(mx - lm); mx = lm; }
#pragma unroll
    for (int i = 0; i < 8; ++i) sm += __expf(f[i] - mx);
  }
  for (int c = (nvec << 3) + threadIdx.x; c < vocab; c += blockDim.x) {
    float f = bf2f(lr[c]);
    if (f > mx) { sm *= __expf(mx - f); mx = f; }
    sm += __expf(f - mx);
  }
  float gmx = block_max(mx, scratch);
  sm = (mx == -INFINITY) ? 0.f : sm * __expf(mx - gmx);
  float gsum = block_sum(sm, scratch);
  float lse = gmx + logf(gsum);
  if (threadIdx.x == 0) {
    float tl = tgt >= 0 ? bf2f(lr[tgt]) : 0.f;
    nll[row] = keep * (lse - tl) * scale;
  }
  __syncthreads();      // the target logit is read before anyone overwrites it
  float gs = keep * scale;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    unpack8(ld8(lr + v * 8), f);
    int c0 = v * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float p = __expf(f[i] - lse);
      f[i] = (p - ((c0 + i) == tgt ? 1.f : 0.f)) * gs;
    }
    st8(lr + v * 8, pack8(f));
  }
  for (int c = (nvec << 3) + threadIdx.x; c < vocab; c += blockDim.x) {
    float p = __expf(bf2f(lr[c]) - lse);
    lr[c] = f2bf((p - (c == tgt ? 1.f : 0.f)) * gs);
  }
}

// loss_out (+)= sum over rows of nll, single thread block, fixed order
__global__ void ce_reduce_kernel(const float* __restrict__ nll, int rows, float* __restrict__ loss, int accumulate) {
  __shared__ float scratch[33];
  float s = 0.f;
  for (int r = threadIdx.x; r < rows; r += blockDim.x) s += nll[r];
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) loss[0] = (accumulate ? loss[0] : 0.f) + s;
}

void ce_loss_fwd_bwd(void* logits, const int* targets, float* nll_rows, float* loss, int accumulate, int rows, int vocab,
                     long long ld, float scale, cudaStream_t s) {
  if (rows == 0) return;
  ce_fwd_bwd_kernel<<<rows, 512, 0, s>>>((bf16*)logits, targets, nll_rows, rows, vocab, ld, scale);
  if (loss) ce_reduce_kernel<<<1, 1024, 0, s>>>(nll_rows, rows, loss, accumulate);
}

}  // namespace dfb
