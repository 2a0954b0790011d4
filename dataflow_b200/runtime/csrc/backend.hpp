// Device backend interface of the task executor.
//
// A backend owns streams, events, raw allocations, async copies and the
// completion-token queue.  The executor never touches a vendor API directly, so
// the same dispatch loop runs on virtual time (FakeBackend), on host memory
// (CpuBackend) and on CUDA streams (CudaBackend).  Protocol parity: reference
// src/dataflow/runtime/device/base.py:35-163 (priorities, notify_after,
// next_completion, drain_aborted, event_time_us).
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace dfb {

enum Location : int { FAST = 0, BACKING = 1 };

// completion priorities: lower value is handled first at equal times
constexpr int PRIO_H2D_DONE = 0;
constexpr int PRIO_D2H_DONE = 1;
constexpr int PRIO_TASK = 2;

struct Completion {
  bool valid = false;
  uint64_t token = 0;
  int prio = 0;
};

struct EngineError : std::runtime_error {
  std::string kind;
  EngineError(const std::string& k, const std::string& msg) : std::runtime_error(msg), kind(k) {}
};

// A reserved virtual address range backed page by page from a fixed budget of physical pages: the pool's VMM mode.
// Contiguous virtual room is then never what an allocation fails on; only physical pages can run out.  Pages nobody
// holds stay mapped (an allocation that lands on them again costs no driver call) until their physical page is needed
// elsewhere.  The bookkeeping is here; a backend supplies map / unmap / grant.  Role parity: reference
// src/dataflow/runtime/device/vmm.py:77-436 (parked 2 MiB handles behind one reserved range), pool.py:29-341.
class VmSpace {
 public:
  virtual ~VmSpace() = default;
  virtual void* base() const = 0;
  size_t page() const { return page_; }
  size_t va_bytes() const { return ref_.size() * page_; }
  size_t phys_pages() const { return phys_pages_; }
  size_t held_pages() const { return held_; }           // pages some live block touches
  size_t mapped_pages() const { return mapped_count_; }
  int64_t maps = 0, reclaims = 0;                         // pages mapped so far; of those, how many took a page from an idle mapping

  // Back [off, off + bytes): false (and nothing changed) when the physical pages do not suffice.
  bool hold(size_t off, size_t bytes) {
    if (!bytes) return true;
    const size_t p0 = off / page_, p1 = (off + bytes - 1) / page_;
    if (p1 >= ref_.size()) return false;
    size_t need = 0, idle_in = 0;
    for (size_t p = p0; p <= p1; ++p) {
      if (!mapped_[p]) ++need;
      else if (ref_[p] == 0) ++idle_in;
    }
    const size_t spare = phys_pages_ - mapped_count_;                         // physical pages not mapped anywhere
    if (need > spare + (idle_.size() - idle_in)) return false;
    for (size_t p = p0; p <= p1; ++p)
      if (mapped_[p] && ref_[p] == 0) idle_remove(p);                          // taken as they are
    size_t run0 = 0, run = 0;
    for (size_t p = p0; p <= p1; ++p) {
      if (!mapped_[p]) {
        if (mapped_count_ == phys_pages_) {                                     // reclaim: any page nobody holds
          const size_t victim = idle_.back();
          idle_remove(victim);
          unmap_page(victim);
          mapped_[victim] = 0;
          --mapped_count_;
          ++reclaims;
        }
        if (!map_page(p)) {                                                     // the driver refused: undo this call
          if (run) grant(run0, run);
          for (size_t q = p0; q < p; ++q) unref(q);
          for (size_t q = p; q <= p1; ++q)
            if (mapped_[q] && ref_[q] == 0) idle_add(q);
          return false;
        }
        mapped_[p] = 1;
        ++mapped_count_;
        ++maps;
        if (!run) run0 = p;
        ++run;
      } else if (run) {
        grant(run0, run);
        run = 0;
      }
      if (ref_[p]++ == 0) ++held_;
    }
    if (run) grant(run0, run);
    return true;
  }
  void drop(size_t off, size_t bytes) {
    if (!bytes) return;
    const size_t p0 = off / page_, p1 = (off + bytes - 1) / page_;
    for (size_t p = p0; p <= p1 && p < ref_.size(); ++p) unref(p);
  }

 protected:
  void init(size_t page, size_t va_bytes, size_t phys_bytes) {
    page_ = page;
    const size_t n = (va_bytes + page - 1) / page;
    ref_.assign(n, 0);
    mapped_.assign(n, 0);
    idle_pos_.assign(n, SIZE_MAX);
    phys_pages_ = (phys_bytes + page - 1) / page;
  }
  virtual bool map_page(size_t p) = 0;                 // give VA page p a physical page
  virtual void unmap_page(size_t p) = 0;               // take it away (nothing in flight touches the page)
  virtual void grant(size_t p0, size_t count) = 0;     // make freshly mapped pages [p0, p0 + count) accessible

 private:
  void unref(size_t p) {
    if (ref_[p] > 0 && --ref_[p] == 0) { --held_; idle_add(p); }
  }
  void idle_add(size_t p) { idle_pos_[p] = idle_.size(); idle_.push_back(p); }
  void idle_remove(size_t p) {
    const size_t at = idle_pos_[p];
    idle_[at] = idle_.back();
    idle_pos_[idle_[at]] = at;
    idle_.pop_back();
    idle_pos_[p] = SIZE_MAX;
  }
  size_t page_ = 2u << 20, phys_pages_ = 0, mapped_count_ = 0, held_ = 0;
  std::vector<int32_t> ref_;
  std::vector<uint8_t> mapped_;
  std::vector<size_t> idle_, idle_pos_;
};

class Backend {
 public:
  virtual ~Backend() = default;
  virtual const char* name() const = 0;
  virtual bool is_virtual() const { return false; }

  // streams are small integer handles; 0 = compute, 1 = h2d, 2 = d2h are created by the session
  virtual int create_stream(const char* label, int priority) = 0;
  virtual uint64_t stream_handle(int stream) const { return 0; }   // raw vendor handle (cudaStream_t)

  // events
  virtual int record_event(int stream) = 0;            // returns an event handle
  virtual void stream_wait_event(int stream, int event) = 0;
  virtual void release_event(int event) = 0;
  virtual double event_time_us(int event) = 0;          // time since the epoch event; valid once complete
  virtual void mark_epoch() = 0;

  // memory
  virtual void* alloc(Location loc, size_t bytes) = 0;
  virtual void free(Location loc, void* p, size_t bytes) = 0;
  // a paged virtual range in fast memory (nullptr: this backend has none; the pool then stays one allocation)
  virtual std::unique_ptr<VmSpace> create_vm_space(size_t va_bytes, size_t phys_bytes) { return nullptr; }
  virtual void memcpy_async(void* dst, const void* src, size_t bytes, int stream, double planned_us) = 0;
  virtual void memset_async(void* dst, int value, size_t bytes, int stream) = 0;

  // synthetic work: make ``stream`` busy for ``us`` (virtual clock or a spin kernel)
  virtual void busy(int stream, double us) = 0;

  // completion tokens
  virtual void notify_after(int event, uint64_t token, int prio) = 0;
  virtual Completion next_completion(bool block) = 0;   // invalid when nothing is pending
  virtual size_t pending() const = 0;
  virtual void drain_aborted() = 0;                      // wait for everything in flight, drop tokens
  virtual void synchronize() = 0;
};

}  // namespace dfb
