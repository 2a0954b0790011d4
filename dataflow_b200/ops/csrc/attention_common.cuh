// Helpers shared by the attention kernels: tensor-map encoding for (tokens, heads * 128) bf16 matrices, the exp2 wrapper.
#pragma once
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace dfb {
namespace fa {

DFB_DEVICE float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^x on the FMA pipe for part of the elements (the exponential unit does 16 per clock per SM, a quarter of what the tensor
// pipe needs at head size 128): round x to the nearest integer j through the mantissa trick, 2^(x - j) by a cubic that is
// within 7.5e-5 (relative) on [-0.5, 0.5], and j added into the exponent field.  x is clamped at -126.
DFB_DEVICE float ex2_poly(float x) {
  x = fmaxf(x, -126.f);
  const float t = x + 12582912.f;                 // 1.5 * 2^23: the low mantissa bits now hold round(x)
  const float f = x - (t - 12582912.f);
  float p2 = fmaf(f, 0.0551716648f, 0.2426111251f);
  p2 = fmaf(p2, f, 0.6932609677f);
  p2 = fmaf(p2, f, 0.9999280572f);
  return __int_as_float(__float_as_int(p2) + (__float_as_int(t) << 23));
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess) fn = reinterpret_cast<EncodeFn>(p);
  });
  return fn;
}

// (tokens, heads * 128) bf16 with ``ld`` elements between tokens; boxes of 64 columns x ``box_rows`` tokens, 128-byte swizzle
inline bool make_map(CUtensorMap* m, const void* base, uint64_t cols, uint64_t rows, uint64_t ld, uint32_t box_rows) {
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
}  // namespace dfb
