// fp8 (e4m3) quantisation for the fp8 GEMM lane: one scale per row (per token for activations, per output channel for
// weights stored (N, K)), scale = amax / 448 so that x ~= q * scale and the scales factor out of the K sum — the GEMM's
// epilogue multiplies by row_scale[m] * col_scale[n] (gemm_tcgen05_2sm.cu, FP8).
#include <cuda_fp8.h>

#include "common.cuh"
#include "ops.h"

namespace dfb {
namespace {

constexpr float kE4M3Max = 448.f;

// one warp per row; two passes over the row (amax, then convert)
__global__ void quant_fp8_rowwise_kernel(const bf16* __restrict__ x, long long ldx, unsigned char* __restrict__ q, long long ldq,
                                         float* __restrict__ scale, long long rows, int K) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const bf16* xr = x + row * ldx;
  float amax = 0.f;
  for (int c = lane * 8; c < K; c += 256) {
    float f[8];
    unpack8(ld8(xr + c), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
  }
  amax = warp_max(amax);
  const float s = amax > 0.f ? amax / kE4M3Max : 1.f;
  const float inv = 1.f / s;
  unsigned char* qr = q + row * ldq;
  for (int c = lane * 8; c < K; c += 256) {
    float f[8];
    unpack8(ld8(xr + c), f);
    unsigned long long packed = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      packed |= static_cast<unsigned long long>(__nv_cvt_float_to_fp8(f[i] * inv, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
    *reinterpret_cast<unsigned long long*>(qr + c) = packed;
  }
  if (lane == 0) scale[row] = s;
}

}  // namespace

int quant_fp8_rowwise(const void* x, long long ldx, void* q, long long ldq, float* scale, long long rows, int K, cudaStream_t s) {
  if ((K & 7) || (ldx & 7) || (ldq & 7)) return -2;
  if (rows) quant_fp8_rowwise_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, s>>>((const bf16*)x, ldx, (unsigned char*)q, ldq, scale, rows, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace dfb
