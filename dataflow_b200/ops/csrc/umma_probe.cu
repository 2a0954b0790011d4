// Issue-to-completion cost of tcgen05.mma by shape and operand source, measured in SM clocks by one CTA: a single thread issues
// ``count`` instructions back to back on dummy operands, commits, and waits for the commit.  A tuning aid for the kernels that
// choose tile shapes (attention, GEMM): it answers "how long does the tensor pipe take for a 128 x N x 16 step when A comes from
// shared or tensor memory and B is K-major or MN-major".  The operands are whatever the shared memory holds (zeros): the
// numerical result is never read.  ``nacc`` > 1 spreads the instructions over that many accumulator tiles in turn: back-to-back
// instructions into ONE accumulator wait for each other, instructions into different accumulators do not.
#include "common.cuh"
#include "ops.h"
#include "ptx.cuh"

namespace dfb {
namespace probe {

constexpr int SMEM_BYTES = 96 * 1024 + 1024 + 128;

// kind: 0 = A shared K-major, B shared K-major; 1 = A shared, B shared MN-major; 2 = A tensor memory, B shared K-major;
//       3 = A tensor memory, B shared MN-major
template <int NACC, bool A_TMEM>
__global__ void __launch_bounds__(128, 1) umma_probe_kernel(int kind, int n, int count, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  for (int i = threadIdx.x; i < 96 * 1024 / 16; i += blockDim.x) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) { ptx::mbar_init(&bar, 1); abort_flag = 0; ptx::mbar_fence_init(); }
  if (threadIdx.x < 32) { ptx::tmem_alloc(&tmem_base_s, 512); ptx::tmem_relinquish(); }
  ptx::fence_proxy_async();
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  if (threadIdx.x == 0) {
    const bool b_mn = kind == 1 || kind == 3;
    const uint32_t idesc = ptx::idesc_bf16_f32(128, n, false, b_mn);
    const uint32_t a_addr = ptx::smem_u32(smem), b_addr = ptx::smem_u32(smem + 32 * 1024);
    const uint64_t adesc = ptx::desc_kmajor_sw128(a_addr);
    const uint64_t bdesc = b_mn ? ptx::desc_mnmajor_sw128(b_addr, 16 * 1024) : ptx::desc_kmajor_sw128(b_addr);
    const uint64_t kstep = b_mn ? ((16 * 128) >> 4) : ((16 * 2) >> 4);
    const long long t0 = clock64();
    // twelve instructions per trip, everything but the trip count known at compile time: the issuing thread spends its time
    // on the instructions themselves, not on address arithmetic
    for (int i = 0; i < count; i += 12) {
#pragma unroll
      for (int u = 0; u < 12; ++u) {
        const uint32_t d = tmem + (u % NACC) * n;      // NACC independent accumulators taken in turn
        const int k = u & 3;
        if (A_TMEM) ptx::umma_bf16_ts(d, tmem + 448 + k * 8, bdesc + k * kstep, idesc, 1);
        else ptx::umma_bf16(d, adesc + k * 2, bdesc + k * kstep, idesc, 1);
      }
    }
    const long long t1 = clock64();
    ptx::umma_commit(&bar);
    const bool ok = ptx::mbar_wait(&bar, 0, &abort_flag);
    const long long t2 = clock64();
    out[0] = t1 - t0;                 // cycles spent issuing
    out[1] = t2 - t0;                 // cycles until the last instruction had completed
    out[2] = ok ? 0 : 1;
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) ptx::tmem_dealloc(tmem, 512);
}

}  // namespace probe

int umma_probe(int kind, int n, int count, int nacc, long long* out, cudaStream_t stream) {
  if (nacc < 1 || nacc * n > 448) return -2;
  if (kind < 0 || kind > 3 || n < 16 || n > 256 || (n % 16) || count < 1 || count > (1 << 16)) return -2;
  if (nacc != 1 && nacc != 2 && nacc != 3 && nacc != 4) return -2;
  count = (count + 11) / 12 * 12;
  auto launch = [&](auto kernel) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, probe::SMEM_BYTES);
    kernel<<<1, 128, probe::SMEM_BYTES, stream>>>(kind, n, count, out);
  };
  const bool t = kind >= 2;
  switch (nacc) {
    case 1: t ? launch(probe::umma_probe_kernel<1, true>) : launch(probe::umma_probe_kernel<1, false>); break;
    case 2: t ? launch(probe::umma_probe_kernel<2, true>) : launch(probe::umma_probe_kernel<2, false>); break;
    case 3: t ? launch(probe::umma_probe_kernel<3, true>) : launch(probe::umma_probe_kernel<3, false>); break;
    default: t ? launch(probe::umma_probe_kernel<4, true>) : launch(probe::umma_probe_kernel<4, false>); break;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace dfb
