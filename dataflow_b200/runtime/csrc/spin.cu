// Busy-wait kernel: holds a stream for a requested number of microseconds by
// watching %globaltimer, so a synthetic task's planned runtime is physically
// true on the GPU.  The loop is bounded by an iteration limit as well as by the
// timer, so it always returns.  Role parity: reference
// src/dataflow/runtime/device/cuda_spin.py:26-36.
#include <cuda_runtime.h>

namespace dfb {

__global__ void spin_ns_kernel(unsigned long long ns, unsigned long long max_iters) {
  unsigned long long t0, t1;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (unsigned long long i = 0; i < max_iters; ++i) {
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    if (t1 - t0 >= ns) break;
    __nanosleep(64);
  }
}

void launch_spin_us(double us, cudaStream_t stream) {
  if (us <= 0) return;
  unsigned long long ns = static_cast<unsigned long long>(us * 1000.0);
  // each iteration sleeps >= 64 ns: this many iterations outlast the request several times over
  unsigned long long max_iters = ns / 16 + 1024;
  spin_ns_kernel<<<1, 32, 0, stream>>>(ns, max_iters);
}

}  // namespace dfb
