// Task executor: runs one annotated program over a Backend.
//
// One control thread.  Every state change happens in a completion handler, in
// the order the planner's simulator models:
//   task done  : outputs live -> mutations bump versions -> releases (dead-everywhere
//                frees the backing copy too) -> offload enqueue -> prefetch enqueue
//                (deferred while the same object's offload is pending) -> poke lanes
//   h2d done   : fast copy live -> poke lanes
//   d2h done   : fast copy freed, backing copy live, deferred prefetches join the
//                h2d queue -> poke lanes
// When the realised order of completions diverges from the plan (a copy that finishes early takes the room a task's
// outputs were planned into), the pressure-eviction valve keeps the run alive: with nothing in flight and the next task
// still not admissible, the resident object whose next use is farthest is evicted (dropped if its backing copy is current,
// else written back first) and reloaded in front of the task that needs it next; directives that later name the evicted
// object tolerate its absence.  Each eviction is counted (RunStats::pressure_evictions; a healthy run has none).
// Dispatch is strictly paced: task i+1 is launched only after task i's token was
// observed, all its inputs are live in fast memory and the ledger admits its fast
// outputs.  Two FIFO transfer lanes, one transfer in flight each, destination bytes
// charged when the transfer starts.  Behavioural parity: reference
// src/dataflow/runtime/engine.py:508-1329 and transfers.py:46-244.
#pragma once
#include <atomic>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

#include "backend.hpp"
#include "slab.hpp"

namespace dfb {

struct ObjIR {
  std::string id;
  int64_t size = 0;
  bool init_fast = false, init_backing = false;
  int final_loc = -1;      // -1 none, else Location
  int last_ref = -1;       // last task index that reads it or names it in a directive
};
struct OutIR { int obj; int loc; };
struct DirIR { int obj; double runtime_us; };   // runtime_us < 0: derive from bandwidth
struct TaskIR {
  std::string id;
  std::vector<int> inputs, mutates, releases;
  std::vector<OutIR> outputs;
  std::vector<DirIR> offloads, prefetches;
  double runtime_us = 1.0;
  int64_t workspace = 0;
};
struct ProgramIR {
  std::string name;
  std::vector<ObjIR> objs;
  std::vector<TaskIR> tasks;
  int64_t fast_cap = -1, backing_cap = -1;    // -1: unbounded
  int64_t bw_from = 0, bw_to = 0;             // bytes per microsecond
};

struct BufferRef {
  void* ptr = nullptr;
  size_t size = 0;
  size_t slab_off = SlabAllocator::kNone;     // kNone: not from a slab
  bool external = false;                      // caller-owned (store extent); never freed here
  bool overflow = false;                      // vendor allocation outside the slab
};

// Per-location buffer source.  Bounded locations carve from one slab allocation;
// unbounded ones recycle exact-size vendor allocations.
class BufferPool {
 public:
  BufferPool(Backend* be, Location loc) : be_(be), loc_(loc) {}
  ~BufferPool();
  void ensure_slab(size_t capacity);
  // VMM mode (before the first ensure_slab): the slab allocator then manages ``va_factor`` times the capacity of VIRTUAL
  // addresses and the capacity is a budget of physical pages, so fragmentation costs address space, not memory
  void set_vm_mode(bool on, double va_factor = 2.0) { vm_mode_ = on; va_factor_ = va_factor; }
  bool vm_active() const { return vm_ != nullptr; }
  const VmSpace* vm() const { return vm_.get(); }
  // static placement: the buffer at a planned slab offset; an empty ref (ptr == nullptr) when those bytes are taken
  BufferRef get_at(size_t bytes, size_t offset);
  BufferRef get(size_t bytes);
  void put(BufferRef& b);
  void trim();
  size_t slab_capacity() const { return vm_ ? phys_capacity_ : (slab_ ? slab_->capacity() : 0); }
  void* slab_base() const { return base_; }
  // bytes kept behind the managed extent of the NEXT slab allocation (staging that peers must be able to address)
  void set_tail(size_t bytes) { tail_bytes_ = SlabAllocator::round_up(bytes, SlabAllocator::kAlign); }
  size_t slab_tail() const { return base_ && !vm_ ? alloc_bytes_ - slab_->capacity() : 0; }
  int64_t slab_overflows = 0;
  int64_t vendor_allocs = 0;
  // what the slab looked like at the first overflows: (bytes asked, bytes in use, largest free block).  Tells a pool that is
  // too small (in use + asked > capacity) from one that is fragmented (largest free block < asked <= capacity - in use)
  struct Overflow { size_t asked, used, largest_free; };
  std::vector<Overflow> overflow_log;
  // allocator policy of the current and every later slab (see SlabAllocator::set_policy)
  void set_policy(size_t large_div, bool best_fit) { large_div_ = large_div; best_fit_ = best_fit; if (slab_) slab_->set_policy(large_div, best_fit); }
  size_t slab_used() const { return slab_ ? slab_->used() : 0; }
  size_t slab_peak() const { return slab_ ? slab_->peak() : 0; }
  size_t slab_largest_free() const { return slab_ ? slab_->largest_free() : 0; }
 private:
  Backend* be_;
  Location loc_;
  void* base_ = nullptr;
  size_t alloc_bytes_ = 0, tail_bytes_ = 0;
  std::unique_ptr<SlabAllocator> slab_;
  std::unique_ptr<VmSpace> vm_;
  bool vm_mode_ = false;
  double va_factor_ = 2.0;
  size_t phys_capacity_ = 0;
  size_t large_div_ = 48;
  bool best_fit_ = false;
  std::multimap<size_t, void*> free_exact_;
};

// Streams and pools that outlive one execute() so steady-state steps allocate nothing.
class Session {
 public:
  explicit Session(std::shared_ptr<Backend> be);
  ~Session();
  std::shared_ptr<Backend> backend;
  int compute_stream, h2d_stream, d2h_stream;
  BufferPool fast_pool, backing_pool;
  void ensure_pools(int64_t fast_cap, int64_t backing_cap, double headroom, bool fast_vm = false);
  // Fast copies of objects whose final location is "fast", kept out of the pool between execute() calls
  // (ExecOptions::keep_resident).  The next program that starts such an object in fast adopts the bytes
  // in place: parameters stay on the device across steps with no transfer.
  std::unordered_map<std::string, BufferRef> resident;
  void drop_resident();
  void drop_resident(const std::string& id);
};

enum class SlotState : int { ABSENT = 0, RESERVED, LIVE, PENDING_OUTBOUND, OUTBOUND, INBOUND };

struct Slot {
  SlotState state = SlotState::ABSENT;
  BufferRef buf;
  int64_t version = -1;
  int ready_event = -1;       // event after which the bytes are valid for other streams
};

struct ObjState {
  Slot fast, backing;
  int64_t version = 0;
};

struct Interval { std::string name; std::string track; double start, end; };
struct TraceEvent { double t; std::string kind; std::string what; int64_t fast_bytes; };

struct RunStats {
  double makespan_us = 0;
  int64_t peak_fast = 0, peak_backing = 0;
  int64_t slab_overflows = 0, pressure_evictions = 0, placement_escapes = 0, vendor_allocs = 0;
  int64_t h2d_bytes = 0, d2h_bytes = 0, h2d_count = 0, d2h_count = 0;
  double dispatch_us_total = 0;      // host time spent inside launch callbacks
  double wait_us_total = 0;          // host time spent blocked on completions
};

struct AllocRecord { int obj; int64_t size; uint64_t ptr; int kind; };   // kind: 1 allocated, 2 held from the previous run, 0 released

struct FinalBuffer { std::string id; int loc; uint64_t ptr; size_t size; bool external; };

struct RunResult {
  std::string outcome = "SUCCESS";   // SUCCESS | FAILED | CANCELLED
  std::string message, failed_task, error_kind;
  std::vector<Interval> intervals;
  std::vector<TraceEvent> events;
  std::vector<AllocRecord> allocs;
  RunStats stats;
  std::vector<FinalBuffer> finals;
};

struct LaunchArgs {
  int task_index;
  std::vector<uint64_t> input_ptrs, output_ptrs;
  std::vector<size_t> input_sizes, output_sizes;
  uint64_t stream_handle;
};

using LaunchFn = std::function<void(const LaunchArgs&)>;
using RangeFn = std::function<void(const std::string&, bool)>;   // (name, push?) for NVTX

struct InitialBuffer { uint64_t ptr; size_t size; int loc; };

struct ExecOptions {
  bool strict_final_locations = true;
  bool poison_on_free = false;
  bool record_events = false;
  bool keep_finals = true;          // hand final backing buffers to the caller instead of freeing
  double slab_headroom = 0.0;
  bool manage_pools = true;         // size the session's slabs from the program's capacities
  bool keep_resident = false;       // final-fast objects stay in Session::resident for the next execute()
  int dispatch_ahead = 0;           // tasks that may be launched behind an unfinished predecessor (0 = strict pacing)
  bool record_allocs = false;       // log every fast-memory allocation and release (placement recorder)
  // static placement: per object index, the slab offset of its k-th fast allocation in this run (missing = dynamic)
  const std::vector<std::vector<int64_t>>* placement = nullptr;
  std::atomic<bool>* cancel = nullptr;
};

class Engine {
 public:
  Engine(std::shared_ptr<Session> s) : sess_(std::move(s)), be_(sess_->backend.get()) {}
  RunResult execute(const ProgramIR& p, const LaunchFn& launch,
                    const std::unordered_map<std::string, InitialBuffer>& initial,
                    const ExecOptions& opt, const RangeFn& range);

 private:
  struct Xfer { int obj; int dir; int64_t size; double runtime_us; };   // dir 0 = from_slow, 1 = to_slow
  struct Flight { Xfer x; int start_ev, end_ev; std::string name; };

  void run_dispatch(const ProgramIR& p, const LaunchFn& launch,
                    const std::unordered_map<std::string, InitialBuffer>& initial,
                    const ExecOptions& opt, const RangeFn& range, RunResult& out);
  void load_initial(const std::unordered_map<std::string, InitialBuffer>& initial);
  bool try_start(int dir);
  void poke() { try_start(0); try_start(1); }
  void handle(const Completion& c);
  void on_task_done(int idx);
  void on_transfer_done(int dir);
  bool pump_one(bool block);
  void charge(Location loc, int64_t bytes);
  void uncharge(Location loc, int64_t bytes);
  int64_t free_bytes(Location loc) const;
  void free_slot(Slot& s, Location loc);
  BufferRef get_fast(int obj, int64_t size);
  // pressure-eviction valve (see run_dispatch): pick and evict the resident whose next use is farthest; queue reloads
  bool evict_for_pressure(int task, bool need_reload_room);
  bool reload_evicted(int obj);
  int next_use(int obj, int from_task) const;
  double xfer_us(const Xfer& x) const;
  void note(const std::string& kind, const std::string& what);
  [[noreturn]] void deadlock(const std::string& why);
  void cleanup(bool failed);

  std::shared_ptr<Session> sess_;
  Backend* be_;
  const ProgramIR* p_ = nullptr;
  const ExecOptions* opt_ = nullptr;
  RunResult* out_ = nullptr;
  const RangeFn* range_ = nullptr;      // annotation hook of the run in progress (tasks by id, transfers as "xfer:<name>")
  std::vector<ObjState> objs_;
  std::set<int> done_early_;           // completed tasks whose predecessors have not retired yet
  std::vector<int> alloc_count_;       // fast allocations of each object so far in this run (indexes the placement)
  std::vector<char> evicted_;          // objects the valve took out of fast memory although the plan keeps them there
  int64_t used_[2] = {0, 0};
  int64_t workspace_ = 0;
  std::deque<Xfer> queue_[2];
  std::unique_ptr<Flight> flight_[2];
  std::unordered_map<int, std::vector<Xfer>> deferred_;
  std::map<std::pair<int, int>, int> xfer_seq_;
  int task_done_upto_ = -1;
  int running_task_ = -1;
  int task_start_ev_ = -1, task_end_ev_ = -1;
  std::vector<int> events_to_release_;
  struct PendingInterval { std::string name, track; int ev0, ev1; };
  std::vector<PendingInterval> pending_intervals_;
};

ProgramIR make_program_ir();   // helper for bindings

}  // namespace dfb
