#pragma once
#include <algorithm>
#include <deque>
#include <queue>
#include <utility>
#include <vector>

#include "backend.hpp"

namespace dfb {

// Paged range of the host backends: the accounting of the VMM pool mode without a driver.  ``real`` backs the whole range
// with (lazily committed) host memory; otherwise the range is a span of made-up addresses that nothing dereferences.
class HostVmSpace : public VmSpace {
 public:
  HostVmSpace(size_t va_bytes, size_t phys_bytes, bool real, uintptr_t fake_base, size_t page = 2u << 20);
  ~HostVmSpace() override;
  void* base() const override { return base_; }
  int64_t unmaps = 0;

 protected:
  bool map_page(size_t) override { return true; }
  void unmap_page(size_t) override { ++unmaps; }
  void grant(size_t, size_t) override {}

 private:
  void* base_ = nullptr;
  bool real_ = false;
};

// Virtual-time backend: per-stream clocks, a heap of (time, priority, seq) completions.
class FakeBackend : public Backend {
 public:
  const char* name() const override { return "fake"; }
  bool is_virtual() const override { return true; }
  int create_stream(const char*, int) override;
  int record_event(int stream) override;
  void stream_wait_event(int stream, int event) override;
  void release_event(int event) override;
  double event_time_us(int event) override;
  void mark_epoch() override;
  void* alloc(Location, size_t bytes) override;
  void free(Location, void*, size_t) override;
  std::unique_ptr<VmSpace> create_vm_space(size_t va_bytes, size_t phys_bytes) override;
  void memcpy_async(void*, const void*, size_t, int stream, double planned_us) override;
  void memset_async(void*, int, size_t, int) override;
  void busy(int stream, double us) override;
  void notify_after(int event, uint64_t token, int prio) override;
  Completion next_completion(bool) override;
  size_t pending() const override { return heap_.size(); }
  void drain_aborted() override;
  void synchronize() override {}
  double now() const { return now_; }
  double transfer_time_scale = 1.0;   // distort copy durations (valve / jitter tests)
  double compute_time_scale = 1.0;

 private:
  struct Item {
    double t; int prio; uint64_t seq; uint64_t token;
    bool operator<(const Item& o) const {     // std::priority_queue is a max-heap
      if (t != o.t) return t > o.t;
      if (prio != o.prio) return prio > o.prio;
      return seq > o.seq;
    }
  };
  std::vector<double> clocks_;
  std::vector<double> event_time_;
  std::vector<int> free_events_;
  std::priority_queue<Item> heap_;
  double now_ = 0.0;
  uint64_t seq_ = 0;
  uintptr_t next_addr_ = 0x10000000ull;
};

// Real host memory for both tiers, synchronous copies, wall-clock events.
class CpuBackend : public Backend {
 public:
  const char* name() const override { return "cpu"; }
  int create_stream(const char*, int) override;
  int record_event(int stream) override;
  void stream_wait_event(int, int) override {}
  void release_event(int event) override;
  double event_time_us(int event) override;
  void mark_epoch() override;
  void* alloc(Location, size_t bytes) override;
  void free(Location, void* p, size_t) override;
  std::unique_ptr<VmSpace> create_vm_space(size_t va_bytes, size_t phys_bytes) override;
  void memcpy_async(void* dst, const void* src, size_t bytes, int, double) override;
  void memset_async(void* dst, int value, size_t bytes, int) override;
  void busy(int, double us) override;
  void notify_after(int, uint64_t token, int prio) override;
  Completion next_completion(bool) override;
  size_t pending() const override { return done_.size(); }
  void drain_aborted() override { done_.clear(); }
  void synchronize() override {}
  bool spin_busy = false;

 private:
  int n_streams_ = 0;
  double epoch_ = 0.0;
  std::vector<double> event_time_;
  std::vector<int> free_events_;
  std::vector<std::pair<uint64_t, int>> done_;
};

}  // namespace dfb
