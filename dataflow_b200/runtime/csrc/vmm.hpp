// Virtual-memory arena: one reserved VA range backed by 2 MiB-granule physical
// handles that are mapped and unmapped on demand; released handles are parked and
// re-adopted without driver allocation calls.  The driver API is resolved at run
// time through cudaGetDriverEntryPoint so the module loads on a machine without
// libcuda.  Role parity: reference src/dataflow/runtime/device/vmm.py:77-436.
#pragma once
#include <cuda.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <map>
#include <vector>

namespace dfb {

class VmmArena {
 public:
  VmmArena(int device, size_t va_bytes);
  ~VmmArena();
  bool available() const { return ok_; }
  size_t granule() const { return granule_; }
  uint64_t base() const { return static_cast<uint64_t>(base_); }
  // back [offset, offset+bytes) (granule aligned) with physical memory; returns the address
  uint64_t map(size_t offset, size_t bytes);
  void unmap(size_t offset, size_t bytes);      // physical handles are parked for reuse
  size_t mapped_bytes() const { return mapped_.size() * granule_; }
  size_t parked_bytes() const { return parked_.size() * granule_; }
  void trim();                                   // release parked handles to the driver
  int64_t driver_calls() const { return driver_calls_; }

 private:
  bool resolve();
  bool ok_ = false;
  int device_;
  size_t va_bytes_ = 0, granule_ = 2u << 20;
  CUdeviceptr base_ = 0;
  std::map<size_t, CUmemGenericAllocationHandle> mapped_;     // granule index -> handle
  std::vector<CUmemGenericAllocationHandle> parked_;
  int64_t driver_calls_ = 0;
  // driver entry points
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
