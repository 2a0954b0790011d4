// Embedding gather and its deterministic backward.
//
// Backward: tokens are stably sorted on the host-free path by the caller (an
// index permutation ``order`` with ``sorted_tok[p] = tok[order[p]]``); one CTA per
// sorted position that *starts* a run of equal tokens sums that run's dy rows in
// sorted order in fp32 and writes (or accumulates into) that single table row, so
// every row has exactly one writer and a fixed summation order.  Numerics parity:
// reference src/dataflow_training/blocks/ops.py:436-500, kernels/embed.py:51-97.
#include "common.cuh"
#include "ops.h"

namespace dfb {

__global__ void embed_fwd_kernel(const int* __restrict__ tok, const bf16* __restrict__ table, bf16* __restrict__ out,
                                 int tokens, int d, int vocab, const int* __restrict__ positions,
                                 const bf16* __restrict__ pos_table, int pos_rows) {
  int t = blockIdx.x;
  if (t >= tokens) return;
  // ids outside the tables are clamped to their edge rows: a bad id gives a wrong row, never a wild read
  const int id = min(max(tok[t], 0), vocab - 1);
  const bf16* src = table + static_cast<size_t>(id) * d;
  const bf16* ps = pos_table ? pos_table + static_cast<size_t>(min(max(positions[t], 0), pos_rows - 1)) * d : nullptr;
  bf16* dst = out + static_cast<size_t>(t) * d;
  for (int v = threadIdx.x; v < (d >> 3); v += blockDim.x) {
    if (ps) {
      float a[8], b[8];
      unpack8(ld8(src + v * 8), a);
      unpack8(ld8(ps + v * 8), b);
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] += b[i];
      st8(dst + v * 8, pack8(a));
    } else {
      st8(dst + v * 8, ld8(src + v * 8));
    }
  }
}

void embed_fwd(const int* tok, const void* table, void* out, int tokens, int d, int vocab, const int* positions,
               const void* pos_table, int pos_rows, cudaStream_t s) {
  if (tokens == 0 || vocab <= 0) return;
  embed_fwd_kernel<<<tokens, 128, 0, s>>>(tok, (const bf16*)table, (bf16*)out, tokens, d, vocab, positions,
                                          (const bf16*)pos_table, pos_rows);
}

// sorted_key[p] is the table row of sorted position p (token id or position id); order[p] the dy row.
template <typename T>
__global__ void embed_bwd_kernel(const int* __restrict__ sorted_key, const int* __restrict__ order,
                                 const bf16* __restrict__ dy, T* __restrict__ dtable, int n, int d, int table_rows,
                                 int accumulate) {
  int p = blockIdx.x;
  if (p >= n) return;
  int key = sorted_key[p];
  if (key < 0 || key >= table_rows) return;       // ignored ids and ids outside the table write nothing
  if (p > 0 && sorted_key[p - 1] == key) return;       // not the head of its run
  int end = p + 1;
  while (end < n && sorted_key[end] == key) ++end;
  T* dst = dtable + static_cast<size_t>(key) * d;
  for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int q = p; q < end; ++q) {
      float f[8];
      const int src_row = order[q];
      if (src_row < 0 || src_row >= n) continue;
      unpack8(ld8(dy + static_cast<size_t>(src_row) * d + c), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
    if constexpr (sizeof(T) == 2) {
      if (accumulate) {
        float f[8];
        unpack8(ld8(reinterpret_cast<const bf16*>(dst) + c), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
      st8(reinterpret_cast<bf16*>(dst) + c, pack8(acc));
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) dst[c + i] = (accumulate ? dst[c + i] : 0.f) + acc[i];
    }
  }
}

void embed_bwd_sorted(const int* sorted_key, const int* order, const void* dy, void* dtable, int dtable_is_f32, int n,
                      int d, int table_rows, int accumulate, cudaStream_t s) {
  if (n == 0) return;
  if (dtable_is_f32) embed_bwd_kernel<float><<<n, 128, 0, s>>>(sorted_key, order, (const bf16*)dy, (float*)dtable, n, d, table_rows, accumulate);
  else embed_bwd_kernel<bf16><<<n, 128, 0, s>>>(sorted_key, order, (const bf16*)dy, (bf16*)dtable, n, d, table_rows, accumulate);
}

}  // namespace dfb
