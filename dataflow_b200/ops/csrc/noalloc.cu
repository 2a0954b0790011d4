// Allocation-free RMSNorm backward: the scratch the regular entry point takes from its caller is a
// device array inside this translation unit.  See noalloc.h for the contract.
#include "noalloc.h"

#include <atomic>
#include <cstdint>

#include "ops.h"

namespace {

constexpr int kMaxDevices = 64;
constexpr size_t kScratchFloats = DFB_NOALLOC_RMSNORM_SCRATCH_BYTES / sizeof(float);

// Lives in every GPU's memory that loads this library, until the process exits.
static __device__ __align__(256) float g_rmsnorm_scratch[kScratchFloats];

// Host code must not hand `g_rmsnorm_scratch` itself to a kernel: in host code that name is only a
// stand-in.  The device address is looked up once per device and cached here.
// Concurrent first calls may both look the address up; they store the same value.
std::atomic<float*> g_scratch_ptr[kMaxDevices];

int scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -3;
  float* p = g_scratch_ptr[dev].load(std::memory_order_acquire);
  if (!p) {
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rmsnorm_scratch) != cudaSuccess || !p) return -3;
    g_scratch_ptr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return 0;
}

inline bool misaligned(const void* p, uintptr_t mask) { return (reinterpret_cast<uintptr_t>(p) & mask) != 0; }

}  // namespace

extern "C" int dfb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                                        void* dw, int rows, int cols, cudaStream_t stream) {
  if (rows < 0 || cols <= 0 || (cols % 8) != 0 || cols > DFB_NOALLOC_RMSNORM_MAX_COLS) return -1;
  if (!dy || !x || !w || !rstd || !dx || !dw) return -2;
  // the kernels move 16-byte vectors of bf16 and 4-byte statistics: a pointer into the middle of a vector would fault
  if (misaligned(dy, 15) || misaligned(x, 15) || misaligned(w, 15) || misaligned(dx, 15) || misaligned(dw, 15) ||
      misaligned(rstd, 3))
    return -4;
  if (rows == 0) return 0;
  // an error left behind by earlier work on this thread is not this call's: report it without launching
  if (cudaPeekAtLastError() != cudaSuccess) return -3;
  // the regular kernel uses norm_bwd_parts(rows) <= 296 partial rows of 2 * cols floats
  if (static_cast<size_t>(dfb::norm_bwd_parts(rows)) * 2u * static_cast<size_t>(cols) > kScratchFloats) return -1;
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  dfb::rmsnorm_bwd(dy, x, w, rstd, dx, /*dx_add=*/nullptr, dw, /*dw_is_f32=*/0, /*accumulate=*/0, scratch, rows, cols,
                   stream);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" const char* dfb_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case -1: return "size not supported: cols must be a multiple of 8 and at most DFB_NOALLOC_RMSNORM_MAX_COLS (8192)";
    case -2: return "null pointer argument";
    case -3: return "CUDA runtime error: pending from earlier work, or raised by set-up or launch";
    case -4: return "misaligned pointer: dy, x, w, dx, dw must be 16-byte aligned and rstd 4-byte aligned";
    default: return "unknown code";
  }
}
