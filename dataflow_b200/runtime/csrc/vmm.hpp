// The CUDA side of the pool's VMM mode: one reserved virtual address range, physical memory in granule-sized handles
// (2 MiB on this hardware) created on first need up to the pool's budget, mapped where the pool asks and moved — unmap,
// map elsewhere — when the budget is spent.  The driver API is resolved at run time through cudaGetDriverEntryPoint so
// the module loads on a machine without libcuda.  Role parity: reference src/dataflow/runtime/device/vmm.py:77-436.
#pragma once
#include <cuda.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <vector>

#include "backend.hpp"

namespace dfb {

class CudaVmSpace : public VmSpace {
 public:
  // throws EngineError("AllocError") when the driver has no virtual-memory API or refuses the reservation
  CudaVmSpace(int device, size_t va_bytes, size_t phys_bytes);
  ~CudaVmSpace() override;
  void* base() const override { return reinterpret_cast<void*>(base_); }
  int64_t driver_calls = 0;

 protected:
  bool map_page(size_t p) override;
  void unmap_page(size_t p) override;
  void grant(size_t p0, size_t count) override;

 private:
  bool resolve();
  int device_;
  size_t reserved_ = 0;
  CUdeviceptr base_ = 0;
  std::vector<CUmemGenericAllocationHandle> handle_of_;      // per virtual page; 0 = none
  std::vector<CUmemGenericAllocationHandle> parked_;         // created, mapped nowhere
  CUresult (*memAddressReserve_)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*memAddressFree_)(CUdeviceptr, size_t) = nullptr;
  CUresult (*memCreate_)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*memRelease_)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*memMap_)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*memUnmap_)(CUdeviceptr, size_t) = nullptr;
  CUresult (*memSetAccess_)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*memGetGranularity_)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
};

}  // namespace dfb
