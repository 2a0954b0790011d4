#include "engine.hpp"

#include <algorithm>
#include <chrono>
#include <sstream>

namespace dfb {

static inline double host_now_us() {
  using namespace std::chrono;
  return duration<double, std::micro>(steady_clock::now().time_since_epoch()).count();
}

// ----------------------------------------------------------------------------- BufferPool
BufferPool::~BufferPool() {
  trim();
  if (vm_) { vm_.reset(); base_ = nullptr; }
  if (base_) be_->free(loc_, base_, alloc_bytes_);
}

void BufferPool::ensure_slab(size_t capacity) {
  capacity = SlabAllocator::round_up(capacity, SlabAllocator::kAlign);   // the slab's usable extent is aligned
  if (slab_ && slab_capacity() >= capacity) return;
  if (slab_) {
    if (slab_->live_blocks()) return;   // cannot grow under live buffers; overflow handles the rest
    if (vm_) vm_.reset();
    else be_->free(loc_, base_, alloc_bytes_);
    slab_.reset();
    base_ = nullptr;
  }
  if (vm_mode_ && tail_bytes_ == 0) {
    // a tail (staging that peers address through one mapping of the slab) needs the classic single allocation
    auto space = be_->create_vm_space(static_cast<size_t>(capacity * va_factor_), capacity);
    if (space) {
      vm_ = std::move(space);
      base_ = vm_->base();
      phys_capacity_ = capacity;
      alloc_bytes_ = 0;
      vendor_allocs++;
      slab_ = std::make_unique<SlabAllocator>(vm_->va_bytes());
      slab_->set_policy(large_div_, best_fit_);
      return;
    }
  }
  // the tail (set_tail) lies behind the managed extent, in the same allocation: whoever maps the slab for peers
  // gets it too, and the allocator never hands it out
  alloc_bytes_ = capacity + tail_bytes_;
  base_ = be_->alloc(loc_, alloc_bytes_);
  vendor_allocs++;
  slab_ = std::make_unique<SlabAllocator>(capacity);
  slab_->set_policy(large_div_, best_fit_);
}

BufferRef BufferPool::get(size_t bytes) {
  BufferRef b;
  b.size = bytes;
  if (slab_) {
    size_t off = slab_->allocate(bytes);
    if (off != SlabAllocator::kNone && vm_ && !vm_->hold(off, slab_->block_size(off))) {
      slab_->release(off);              // address room but no physical page left
      off = SlabAllocator::kNone;
    }
    if (off != SlabAllocator::kNone) {
      b.ptr = static_cast<char*>(base_) + off;
      b.slab_off = off;
      return b;
    }
    slab_overflows++;
    if (overflow_log.size() < 64) overflow_log.push_back({bytes, slab_->used(), slab_->largest_free()});
  }
  size_t need = SlabAllocator::round_up(bytes ? bytes : 1, SlabAllocator::kAlign);
  auto it = free_exact_.find(need);
  if (it != free_exact_.end()) {
    b.ptr = it->second;
    free_exact_.erase(it);
  } else {
    b.ptr = be_->alloc(loc_, need);
    vendor_allocs++;
  }
  b.overflow = true;
  return b;
}

BufferRef BufferPool::get_at(size_t bytes, size_t offset) {
  BufferRef b;
  if (!slab_ || offset % SlabAllocator::kAlign || !slab_->allocate_at(offset, bytes)) return b;
  if (vm_ && !vm_->hold(offset, slab_->block_size(offset))) { slab_->release(offset); return b; }
  b.size = bytes;
  b.ptr = static_cast<char*>(base_) + offset;
  b.slab_off = offset;
  return b;
}

void BufferPool::put(BufferRef& b) {
  if (!b.ptr || b.external) { b = BufferRef(); return; }
  if (b.slab_off != SlabAllocator::kNone) {
    if (vm_) vm_->drop(b.slab_off, slab_->block_size(b.slab_off));
    slab_->release(b.slab_off);
  } else {
    free_exact_.insert({SlabAllocator::round_up(b.size ? b.size : 1, SlabAllocator::kAlign), b.ptr});
  }
  b = BufferRef();
}

void BufferPool::trim() {
  for (auto& kv : free_exact_) be_->free(loc_, kv.second, kv.first);
  free_exact_.clear();
}

// ----------------------------------------------------------------------------- Session
Session::Session(std::shared_ptr<Backend> be)
    : backend(std::move(be)), fast_pool(backend.get(), FAST), backing_pool(backend.get(), BACKING) {
  compute_stream = backend->create_stream("compute", 0);
  h2d_stream = backend->create_stream("h2d", 0);
  d2h_stream = backend->create_stream("d2h", 0);
}

Session::~Session() { backend->synchronize(); }

void Session::ensure_pools(int64_t fast_cap, int64_t backing_cap, double headroom, bool fast_vm) {
  if (fast_vm) fast_pool.set_vm_mode(true);
  if (fast_cap > 0) fast_pool.ensure_slab(static_cast<size_t>(fast_cap * (1.0 + headroom)) + (1 << 20));
  if (backing_cap > 0) backing_pool.ensure_slab(static_cast<size_t>(backing_cap) + (1 << 20));
}

void Session::drop_resident() {
  for (auto& kv : resident) fast_pool.put(kv.second);
  resident.clear();
}

void Session::drop_resident(const std::string& id) {
  auto it = resident.find(id);
  if (it == resident.end()) return;
  fast_pool.put(it->second);
  resident.erase(it);
}

// ----------------------------------------------------------------------------- Engine helpers
static constexpr uint64_t TOK_TASK = 0, TOK_FROM = 1, TOK_TO = 2;
static inline uint64_t make_token(uint64_t kind, uint64_t idx) { return (kind << 40) | idx; }

void Engine::note(const std::string& kind, const std::string& what) {
  int64_t f = used_[FAST] + workspace_;
  if (f > out_->stats.peak_fast) out_->stats.peak_fast = f;
  if (used_[BACKING] > out_->stats.peak_backing) out_->stats.peak_backing = used_[BACKING];
  if (opt_->record_events) out_->events.push_back({0.0, kind, what, used_[FAST]});
}

void Engine::charge(Location loc, int64_t bytes) {
  int64_t cap = loc == FAST ? p_->fast_cap : p_->backing_cap;
  if (cap >= 0 && used_[loc] + bytes + (loc == FAST ? workspace_ : 0) > cap)
    throw EngineError("LedgerError", "charge of " + std::to_string(bytes) + " bytes on " +
                                         (loc == FAST ? "fast" : "backing") + " was not admitted");
  used_[loc] += bytes;
}

void Engine::uncharge(Location loc, int64_t bytes) { used_[loc] -= bytes; }

int64_t Engine::free_bytes(Location loc) const {
  int64_t cap = loc == FAST ? p_->fast_cap : p_->backing_cap;
  if (cap < 0) return INT64_MAX / 4;
  return cap - used_[loc] - (loc == FAST ? workspace_ : 0);
}

void Engine::free_slot(Slot& s, Location loc) {
  if (s.state == SlotState::ABSENT) return;
  if (loc == FAST && opt_->poison_on_free && s.buf.ptr && !s.buf.external) {
    be_->memset_async(s.buf.ptr, 0xFF, s.buf.size, sess_->compute_stream);
  }
  if (loc == FAST && opt_->record_allocs && s.buf.ptr) out_->allocs.push_back({-1, 0, reinterpret_cast<uint64_t>(s.buf.ptr), 0});
  (loc == FAST ? sess_->fast_pool : sess_->backing_pool).put(s.buf);
  s.state = SlotState::ABSENT;
  s.version = -1;
}

// A fast buffer for object ``obj``: at its planned offset when a static placement names one and those bytes are free
// (otherwise the placement escape valve: the dynamic allocator), logged when the run records allocations.
BufferRef Engine::get_fast(int obj, int64_t size) {
  BufferRef b;
  int k = alloc_count_[obj]++;
  if (opt_->placement && obj < static_cast<int>(opt_->placement->size())) {
    const auto& offs = (*opt_->placement)[obj];
    if (k < static_cast<int>(offs.size()) && offs[k] >= 0) {
      b = sess_->fast_pool.get_at(static_cast<size_t>(size), static_cast<size_t>(offs[k]));
      if (!b.ptr) out_->stats.placement_escapes++;
    }
  }
  if (!b.ptr) b = sess_->fast_pool.get(static_cast<size_t>(size));
  if (opt_->record_allocs) out_->allocs.push_back({obj, size, reinterpret_cast<uint64_t>(b.ptr), 1});
  return b;
}

double Engine::xfer_us(const Xfer& x) const {
  if (x.runtime_us >= 0) return x.runtime_us;
  int64_t bw = x.dir == 0 ? p_->bw_from : p_->bw_to;
  if (bw <= 0) throw EngineError("ExecutionError", "transfer needs a bandwidth or a per-directive runtime");
  return static_cast<double>(std::max<int64_t>((x.size + bw - 1) / bw, 1));
}

void Engine::deadlock(const std::string& why) {
  std::ostringstream os;
  os << "deadlock: " << why << "; fast used " << used_[FAST] << " cap " << p_->fast_cap << "; h2d queue [";
  for (auto& x : queue_[0]) os << p_->objs[x.obj].id << " ";
  os << "] d2h queue [";
  for (auto& x : queue_[1]) os << p_->objs[x.obj].id << " ";
  os << "]";
  throw EngineError("DeadlockError", os.str());
}

// ----------------------------------------------------------------------------- transfers
bool Engine::try_start(int dir) {
  if (flight_[dir] || queue_[dir].empty()) return false;
  Xfer x = queue_[dir].front();
  Location dst = dir == 0 ? FAST : BACKING;
  ObjState& o = objs_[x.obj];
  Slot& d = dst == FAST ? o.fast : o.backing;
  bool exists = d.state != SlotState::ABSENT;
  if (free_bytes(dst) + (exists ? x.size : 0) < x.size) return false;   // blocked head
  queue_[dir].pop_front();
  if (!exists) {
    charge(dst, x.size);
    d.buf = dst == FAST ? get_fast(x.obj, x.size) : sess_->backing_pool.get(x.size);
  }
  d.state = SlotState::INBOUND;
  Slot& s = dir == 0 ? o.backing : o.fast;
  if (dir == 1) s.state = SlotState::OUTBOUND;
  int stream = dir == 0 ? sess_->h2d_stream : sess_->d2h_stream;
  auto fl = std::make_unique<Flight>();
  fl->x = x;
  int n = xfer_seq_[{dir, x.obj}]++;
  fl->name = std::string(dir == 0 ? "from_slow:" : "to_slow:") + p_->objs[x.obj].id;
  if (n) fl->name += "#" + std::to_string(n);
  if (range_) (*range_)("xfer:" + fl->name, true);
  fl->start_ev = be_->record_event(stream);
  be_->memcpy_async(d.buf.ptr, s.buf.ptr, static_cast<size_t>(x.size), stream, xfer_us(x));
  fl->end_ev = be_->record_event(stream);
  if (range_) (*range_)("xfer:" + fl->name, false);
  be_->notify_after(fl->end_ev, make_token(dir == 0 ? TOK_FROM : TOK_TO, 0), dir == 0 ? PRIO_H2D_DONE : PRIO_D2H_DONE);
  pending_intervals_.push_back({fl->name, dir == 0 ? "from_slow" : "to_slow", fl->start_ev, fl->end_ev});
  if (dir == 0) { out_->stats.h2d_bytes += x.size; out_->stats.h2d_count++; }
  else { out_->stats.d2h_bytes += x.size; out_->stats.d2h_count++; }
  flight_[dir] = std::move(fl);
  note("transfer_start", flight_[dir]->name);
  return true;
}

void Engine::on_transfer_done(int dir) {
  auto fl = std::move(flight_[dir]);
  if (!fl) throw EngineError("ExecutionError", "transfer completion without a transfer in flight");
  ObjState& o = objs_[fl->x.obj];
  if (dir == 0) {
    o.fast.state = SlotState::LIVE;
    o.fast.version = o.backing.version;
    evicted_[fl->x.obj] = 0;
  } else {
    o.backing.state = SlotState::LIVE;
    o.backing.version = o.fast.version;
    uncharge(FAST, fl->x.size);
    free_slot(o.fast, FAST);
    auto it = deferred_.find(fl->x.obj);
    if (it != deferred_.end()) {
      for (auto& w : it->second) queue_[0].push_back(w);
      deferred_.erase(it);
    }
  }
  note("transfer_end", fl->name);
  poke();
}

// ----------------------------------------------------------------------------- pressure-eviction valve
int Engine::next_use(int obj, int from_task) const {
  for (int i = from_task; i < static_cast<int>(p_->tasks.size()); ++i) {
    const TaskIR& t = p_->tasks[i];
    for (int in : t.inputs) if (in == obj) return i;
    for (auto& d : t.offloads) if (d.obj == obj) return i;
  }
  return static_cast<int>(p_->tasks.size()) + (p_->objs[obj].final_loc == FAST ? 0 : 1);   // never again: best victim
}

// Called with nothing in flight and task ``task`` not admissible.  Evicts ONE resident that the task does not touch:
// the one whose next use is farthest (Belady).  Returns false when there is nothing to evict.
bool Engine::evict_for_pressure(int task, bool) {
  const TaskIR& t = p_->tasks[task];
  int victim = -1, victim_use = -1;
  for (int o = 0; o < static_cast<int>(objs_.size()); ++o) {
    if (objs_[o].fast.state != SlotState::LIVE || objs_[o].fast.buf.external) continue;
    bool touched = false;
    for (int in : t.inputs) touched |= in == o;
    for (int m : t.mutates) touched |= m == o;
    for (auto& out : t.outputs) touched |= out.obj == o;
    if (touched) continue;
    // it must be possible to bring it back: the backing tier has to admit a copy if there is none yet
    bool has_copy = objs_[o].backing.state == SlotState::LIVE && objs_[o].backing.version == objs_[o].version;
    if (!has_copy && objs_[o].backing.state == SlotState::ABSENT && free_bytes(BACKING) < p_->objs[o].size) continue;
    if (!has_copy && objs_[o].backing.state != SlotState::ABSENT && objs_[o].backing.state != SlotState::LIVE) continue;
    int use = next_use(o, task);
    if (use > victim_use) { victim = o; victim_use = use; }
  }
  if (victim < 0) return false;
  ObjState& o = objs_[victim];
  out_->stats.pressure_evictions++;
  evicted_[victim] = 1;
  bool has_copy = o.backing.state == SlotState::LIVE && o.backing.version == o.version;
  if (has_copy) {
    uncharge(FAST, p_->objs[victim].size);
    free_slot(o.fast, FAST);
    note("evict", p_->objs[victim].id);
  } else {
    o.fast.state = SlotState::PENDING_OUTBOUND;
    queue_[1].push_front({victim, 1, p_->objs[victim].size, -1.0});
    note("evict_writeback", p_->objs[victim].id);
  }
  poke();
  return true;
}

// An input that the valve evicted: queue its reload in front of everything else.  False when it is not such an object.
bool Engine::reload_evicted(int obj) {
  ObjState& o = objs_[obj];
  if (!evicted_[obj] || o.fast.state != SlotState::ABSENT || o.backing.state != SlotState::LIVE) return false;
  for (auto& x : queue_[0]) if (x.obj == obj) return true;
  queue_[0].push_front({obj, 0, p_->objs[obj].size, -1.0});
  note("evict_reload", p_->objs[obj].id);
  poke();
  return true;
}

// ----------------------------------------------------------------------------- task completion
void Engine::on_task_done(int idx) {
  const TaskIR& t = p_->tasks[idx];
  workspace_ -= t.workspace;
  for (auto& out : t.outputs) {
    ObjState& o = objs_[out.obj];
    Slot& s = out.loc == FAST ? o.fast : o.backing;
    s.state = SlotState::LIVE;
    s.version = o.version;
  }
  for (int m : t.mutates) {
    ObjState& o = objs_[m];
    o.version++;
    o.fast.version = o.version;      // backing copy (if any) is now stale
  }
  note("task_end", t.id);
  for (int r : t.releases) {
    ObjState& o = objs_[r];
    if (evicted_[r] && o.fast.state != SlotState::LIVE) {
      // the valve already took it out of fast memory; a reload that has not started yet is dropped, one in flight lands
      // first (the release is then applied by on_transfer_done through ``release_on_arrival``)
      for (auto it = queue_[0].begin(); it != queue_[0].end(); ++it)
        if (it->obj == r) { queue_[0].erase(it); break; }
      if (o.fast.state == SlotState::INBOUND || o.fast.state == SlotState::PENDING_OUTBOUND || o.fast.state == SlotState::OUTBOUND)
        throw EngineError("ExecutionError", "task " + t.id + " releases " + p_->objs[r].id + " while the eviction valve is moving it");
      evicted_[r] = 0;
      if (idx >= p_->objs[r].last_ref && p_->objs[r].final_loc < 0 && o.backing.state == SlotState::LIVE) {
        uncharge(BACKING, p_->objs[r].size);
        free_slot(o.backing, BACKING);
      }
      continue;
    }
    if (o.fast.state != SlotState::LIVE)
      throw EngineError("ExecutionError", "task " + t.id + " releases " + p_->objs[r].id + " which is not live in fast memory");
    uncharge(FAST, p_->objs[r].size);
    free_slot(o.fast, FAST);
    if (idx >= p_->objs[r].last_ref && p_->objs[r].final_loc < 0 && o.backing.state == SlotState::LIVE) {
      uncharge(BACKING, p_->objs[r].size);
      free_slot(o.backing, BACKING);
    }
  }
  for (auto& d : t.offloads) {
    ObjState& o = objs_[d.obj];
    if (evicted_[d.obj] && o.fast.state == SlotState::ABSENT && o.backing.state == SlotState::LIVE && o.backing.version == o.version) {
      evicted_[d.obj] = 0;             // the valve has done this offload already
      for (auto it = queue_[0].begin(); it != queue_[0].end(); ++it)
        if (it->obj == d.obj) { queue_[0].erase(it); break; }
      continue;
    }
    if (o.fast.state != SlotState::LIVE)
      throw EngineError("ExecutionError", "task " + t.id + " offloads " + p_->objs[d.obj].id + " which is not live in fast memory");
    if (o.backing.state != SlotState::ABSENT && o.backing.state != SlotState::LIVE)
      throw EngineError("ExecutionError", "task " + t.id + " offloads " + p_->objs[d.obj].id + " whose backing copy is busy");
    o.fast.state = SlotState::PENDING_OUTBOUND;
    queue_[1].push_back({d.obj, 1, p_->objs[d.obj].size, d.runtime_us});
  }
  for (auto& d : t.prefetches) {
    ObjState& o = objs_[d.obj];
    if (evicted_[d.obj]) {
      // the plan brings it back itself: the valve's own reload (if it queued one) is that prefetch
      evicted_[d.obj] = 0;
      bool queued = false;
      for (auto& x : queue_[0]) queued |= x.obj == d.obj;
      if (queued || o.fast.state == SlotState::INBOUND || o.fast.state == SlotState::LIVE) continue;
    }
    if (o.fast.state == SlotState::LIVE || o.fast.state == SlotState::INBOUND || o.fast.state == SlotState::RESERVED)
      throw EngineError("ExecutionError", "task " + t.id + " prefetches " + p_->objs[d.obj].id + " which already has a fast copy");
    bool going_out = o.fast.state == SlotState::PENDING_OUTBOUND || o.fast.state == SlotState::OUTBOUND ||
                     o.backing.state == SlotState::INBOUND;
    Xfer x{d.obj, 0, p_->objs[d.obj].size, d.runtime_us};
    if (going_out) { deferred_[d.obj].push_back(x); continue; }
    if (o.backing.state != SlotState::LIVE)
      throw EngineError("ExecutionError", "task " + t.id + " prefetches " + p_->objs[d.obj].id + " which has no backing copy");
    queue_[0].push_back(x);
  }
  task_done_upto_ = idx;
  running_task_ = -1;
  poke();
}

void Engine::handle(const Completion& c) {
  uint64_t kind = c.token >> 40;
  if (kind == TOK_TASK) {
    // Tasks retire in chain order.  With dispatch-ahead several tasks are in flight on one stream; a backend that polls
    // may report the completion of a later one first (both events were already done) — it is held until its predecessors
    // have retired, because a task's directives assume everything before it has taken effect.
    int idx = static_cast<int>(c.token & 0xFFFFFFFFFFull);
    done_early_.insert(idx);
    while (!done_early_.empty() && *done_early_.begin() == task_done_upto_ + 1) {
      int next = *done_early_.begin();
      done_early_.erase(done_early_.begin());
      on_task_done(next);
    }
  } else {
    on_transfer_done(kind == TOK_FROM ? 0 : 1);
  }
}

bool Engine::pump_one(bool block) {
  double t0 = host_now_us();
  Completion c = be_->next_completion(block);
  out_->stats.wait_us_total += host_now_us() - t0;
  if (!c.valid) return false;
  handle(c);
  return true;
}

// ----------------------------------------------------------------------------- run
void Engine::load_initial(const std::unordered_map<std::string, InitialBuffer>& initial) {
  bool copied = false;
  for (size_t i = 0; i < p_->objs.size(); ++i) {
    const ObjIR& oi = p_->objs[i];
    ObjState& o = objs_[i];
    if (!oi.init_fast && !oi.init_backing) continue;
    auto it = initial.find(oi.id);
    if (oi.init_backing) {
      charge(BACKING, oi.size);
      if (it != initial.end() && it->second.loc == BACKING) {
        if (static_cast<int64_t>(it->second.size) != oi.size)
          throw EngineError("BindingMismatch", "initial buffer for " + oi.id + " has " + std::to_string(it->second.size) +
                                                   " bytes, program says " + std::to_string(oi.size));
        o.backing.buf.ptr = reinterpret_cast<void*>(it->second.ptr);
        o.backing.buf.size = it->second.size;
        o.backing.buf.external = true;
      } else {
        o.backing.buf = sess_->backing_pool.get(oi.size);
      }
      o.backing.state = SlotState::LIVE;
      o.backing.version = 0;
    }
    if (oi.init_fast) {
      charge(FAST, oi.size);
      auto held = sess_->resident.find(oi.id);
      if (held != sess_->resident.end() && static_cast<int64_t>(held->second.size) == oi.size) {
        o.fast.buf = held->second;               // bytes already on the device from the previous run
        alloc_count_[i]++;
        if (opt_->record_allocs) out_->allocs.push_back({static_cast<int>(i), oi.size, reinterpret_cast<uint64_t>(o.fast.buf.ptr), 2});
        sess_->resident.erase(held);
        o.fast.state = SlotState::LIVE;
        o.fast.version = 0;
        continue;
      }
      o.fast.buf = get_fast(static_cast<int>(i), oi.size);
      o.fast.state = SlotState::LIVE;
      o.fast.version = 0;
      const void* src = nullptr;
      if (oi.init_backing) src = o.backing.buf.ptr;
      else if (it != initial.end()) src = reinterpret_cast<void*>(it->second.ptr);
      if (src && oi.size) {
        be_->memcpy_async(o.fast.buf.ptr, src, static_cast<size_t>(oi.size), sess_->h2d_stream, 0.0);
        copied = true;
      }
    }
  }
  // held copies this program names but does not start in fast are stale for it: back to the pool
  for (size_t i = 0; i < p_->objs.size(); ++i) sess_->drop_resident(p_->objs[i].id);
  if (copied) {
    // preplaced objects are loaded up front; the compute stream must not start before them
    int ev = be_->record_event(sess_->h2d_stream);
    be_->stream_wait_event(sess_->compute_stream, ev);
    events_to_release_.push_back(ev);
  }
  note("initial", "");
}

void Engine::run_dispatch(const ProgramIR& p, const LaunchFn& launch,
                          const std::unordered_map<std::string, InitialBuffer>& initial,
                          const ExecOptions& opt, const RangeFn& range, RunResult& out) {
  p_ = &p; opt_ = &opt; out_ = &out; range_ = range ? &range : nullptr;
  objs_.assign(p.objs.size(), ObjState());
  alloc_count_.assign(p.objs.size(), 0);
  evicted_.assign(p.objs.size(), 0);
  used_[0] = used_[1] = 0; workspace_ = 0;
  queue_[0].clear(); queue_[1].clear(); flight_[0].reset(); flight_[1].reset();
  deferred_.clear(); xfer_seq_.clear(); pending_intervals_.clear(); events_to_release_.clear();
  task_done_upto_ = -1; running_task_ = -1;
  done_early_.clear();
  if (opt.manage_pools) sess_->ensure_pools(p.fast_cap, p.backing_cap, opt.slab_headroom);
  int64_t of0 = sess_->fast_pool.slab_overflows + sess_->backing_pool.slab_overflows;
  int64_t va0 = sess_->fast_pool.vendor_allocs + sess_->backing_pool.vendor_allocs;
  be_->mark_epoch();
  load_initial(initial);

  LaunchArgs args;
  for (int i = 0; i < static_cast<int>(p.tasks.size()); ++i) {
    const TaskIR& t = p.tasks[i];
    if (opt.cancel && opt.cancel->load()) { out.outcome = "CANCELLED"; out.failed_task = t.id; break; }
    // (0) pacing: at most ``dispatch_ahead`` earlier tasks may still be in flight (0 = the previous task must have
    // retired).  Tasks share one stream, so a task launched behind an unfinished predecessor still runs after it;
    // launching ahead only hides the host's dispatch latency behind device work.
    while (task_done_upto_ < i - 1 - opt.dispatch_ahead) {
      if (!pump_one(true)) deadlock("waiting for task " + p.tasks[i - 1].id + " to retire with nothing in flight");
    }
    if (opt.dispatch_ahead > 0) {
      while (pump_one(false)) {}        // retire whatever has completed meanwhile before looking at the ledger
    }
    // (1)+(2) inputs live and the ledger admits outputs + workspace
    int64_t need = t.workspace;
    for (auto& o : t.outputs) if (o.loc == FAST) need += p.objs[o.obj].size;
    for (;;) {
      bool ready = true;
      std::string missing;
      for (int in : t.inputs) {
        SlotState st = objs_[in].fast.state;
        // RESERVED: the output of a task that is still in flight ahead of this one on the same stream
        if (st != SlotState::LIVE && !(opt.dispatch_ahead > 0 && st == SlotState::RESERVED)) {
          ready = false; missing = p.objs[in].id; break;
        }
      }
      bool short_mem = p.fast_cap >= 0 && used_[FAST] + need > p.fast_cap;
      // launched ahead of an unfinished predecessor, a task must not take the room the next queued prefetch is
      // waiting for: reserving early would stall the copy lane, which strict pacing would not have done
      if (!short_mem && p.fast_cap >= 0 && task_done_upto_ < i - 1 && !queue_[0].empty() && !flight_[0])
        short_mem = used_[FAST] + need + queue_[0].front().size > p.fast_cap;
      if (ready && !short_mem) break;
      // an input the valve evicted earlier comes back in front of everything else queued
      bool reloading = false;
      for (int in : t.inputs) reloading |= reload_evicted(in);
      if (!pump_one(true)) {
        // Nothing in flight and the task still cannot start: the realised order has left the plan.  Make room by
        // evicting the resident whose next use is farthest, as often as it takes; give up only when nothing is left.
        if (evict_for_pressure(i, reloading)) continue;
        deadlock("task " + t.id + (missing.empty() ? std::string(" needs ") + std::to_string(need) + " fast bytes"
                                                    : " waits for input " + missing));
      }
    }
    // (3) backing outputs
    int64_t bneed = 0;
    for (auto& o : t.outputs) if (o.loc == BACKING) bneed += p.objs[o.obj].size;
    if (bneed && p.backing_cap >= 0 && used_[BACKING] + bneed > p.backing_cap)
      throw EngineError("CapacityError", "task " + t.id + " cannot allocate its backing outputs");
    // (4) reserve
    args.task_index = i;
    args.input_ptrs.clear(); args.input_sizes.clear(); args.output_ptrs.clear(); args.output_sizes.clear();
    for (int in : t.inputs) {
      args.input_ptrs.push_back(reinterpret_cast<uint64_t>(objs_[in].fast.buf.ptr));
      args.input_sizes.push_back(static_cast<size_t>(p.objs[in].size));
    }
    for (auto& o : t.outputs) {
      ObjState& os = objs_[o.obj];
      Slot& s = o.loc == FAST ? os.fast : os.backing;
      if (s.state != SlotState::ABSENT)
        throw EngineError("ExecutionError", "task " + t.id + " output " + p.objs[o.obj].id + " already exists");
      Location loc = static_cast<Location>(o.loc);
      used_[loc] += p.objs[o.obj].size;   // admitted above (fast) / checked above (backing)
      auto it = initial.find(p.objs[o.obj].id);
      if (loc == BACKING && it != initial.end() && static_cast<int64_t>(it->second.size) == p.objs[o.obj].size) {
        s.buf.ptr = reinterpret_cast<void*>(it->second.ptr);   // caller-provided landing extent
        s.buf.size = it->second.size;
        s.buf.external = true;
      } else {
        s.buf = loc == FAST ? get_fast(o.obj, p.objs[o.obj].size) : sess_->backing_pool.get(p.objs[o.obj].size);
      }
      s.state = SlotState::RESERVED;
      args.output_ptrs.push_back(reinterpret_cast<uint64_t>(s.buf.ptr));
      args.output_sizes.push_back(static_cast<size_t>(p.objs[o.obj].size));
    }
    workspace_ += t.workspace;
    note("task_start", t.id);
    // (5) launch
    args.stream_handle = be_->stream_handle(sess_->compute_stream);
    if (range) range(t.id, true);
    int ev0 = be_->record_event(sess_->compute_stream);
    double h0 = host_now_us();
    if (launch) launch(args);
    else be_->busy(sess_->compute_stream, t.runtime_us);
    out.stats.dispatch_us_total += host_now_us() - h0;
    int ev1 = be_->record_event(sess_->compute_stream);
    if (range) range(t.id, false);
    be_->notify_after(ev1, make_token(TOK_TASK, static_cast<uint64_t>(i)), PRIO_TASK);
    pending_intervals_.push_back({t.id, "compute", ev0, ev1});
    running_task_ = i;
  }
  // drain
  while (be_->pending() > 0 || flight_[0] || flight_[1]) {
    if (!pump_one(true)) break;
  }
  if (out.outcome == "SUCCESS") {
    // what the pressure valve sent away and the program wants on the device at the end comes back now: nothing that reads it
    // ran after the eviction (or it would have been reloaded for that task), so no later task asked for it
    bool reloading = false;
    for (size_t i = 0; i < p.objs.size(); ++i)
      if (p.objs[i].final_loc == FAST && evicted_[i]) reloading |= reload_evicted(static_cast<int>(i));
    while (reloading && (be_->pending() > 0 || flight_[0] || flight_[1])) {
      if (!pump_one(true)) break;
    }
  }
  if (out.outcome == "SUCCESS") {
    if (!queue_[0].empty() || !queue_[1].empty() || !deferred_.empty())
      deadlock("transfers still queued after the last task");
    if (opt.strict_final_locations) {
      for (size_t i = 0; i < p.objs.size(); ++i) {
        int fl = p.objs[i].final_loc;
        if (fl < 0) continue;
        ObjState& o = objs_[i];
        Slot& s = fl == FAST ? o.fast : o.backing;
        if (s.state != SlotState::LIVE || s.version != o.version)
          throw EngineError("FinalLocationError", "object " + p.objs[i].id + " does not end with its latest bytes at " +
                                                      (fl == FAST ? "fast" : "backing"));
      }
    }
  }
  out.stats.slab_overflows = sess_->fast_pool.slab_overflows + sess_->backing_pool.slab_overflows - of0;
  out.stats.vendor_allocs = sess_->fast_pool.vendor_allocs + sess_->backing_pool.vendor_allocs - va0;
}

void Engine::cleanup(bool failed) {
  if (failed) be_->drain_aborted();
  // resolve interval times now that every event has completed
  if (!failed) {
    for (auto& pi : pending_intervals_) {
      double a = be_->event_time_us(pi.ev0), b = be_->event_time_us(pi.ev1);
      out_->intervals.push_back({pi.name, pi.track, a, b});
      if (b > out_->stats.makespan_us) out_->stats.makespan_us = b;
    }
  }
  for (auto& pi : pending_intervals_) { be_->release_event(pi.ev0); be_->release_event(pi.ev1); }
  for (int e : events_to_release_) be_->release_event(e);
  pending_intervals_.clear(); events_to_release_.clear();
  flight_[0].reset(); flight_[1].reset();
  // hand finals to the caller, reclaim everything else
  for (size_t i = 0; i < objs_.size(); ++i) {
    ObjState& o = objs_[i];
    const ObjIR& oi = p_->objs[i];
    if (!failed && opt_->keep_finals && oi.final_loc >= 0) {
      Slot& s = oi.final_loc == FAST ? o.fast : o.backing;
      if (s.state == SlotState::LIVE && !s.buf.external) {
        // engine-owned bytes: valid until the next execute() on this session; the caller copies them out
        out_->finals.push_back({oi.id, oi.final_loc, reinterpret_cast<uint64_t>(s.buf.ptr), s.buf.size, false});
      } else if (s.state == SlotState::LIVE) {
        out_->finals.push_back({oi.id, oi.final_loc, reinterpret_cast<uint64_t>(s.buf.ptr), s.buf.size, true});
      }
    }
    if (!failed && opt_->keep_resident && oi.final_loc == FAST && o.fast.state == SlotState::LIVE && !o.fast.buf.external) {
      sess_->resident[oi.id] = o.fast.buf;
      o.fast.state = SlotState::ABSENT;
    }
    if (o.fast.state != SlotState::ABSENT) { sess_->fast_pool.put(o.fast.buf); o.fast.state = SlotState::ABSENT; }
    if (o.backing.state != SlotState::ABSENT) { sess_->backing_pool.put(o.backing.buf); o.backing.state = SlotState::ABSENT; }
  }
}

RunResult Engine::execute(const ProgramIR& p, const LaunchFn& launch,
                          const std::unordered_map<std::string, InitialBuffer>& initial,
                          const ExecOptions& opt, const RangeFn& range) {
  RunResult out;
  bool failed = false;
  try {
    run_dispatch(p, launch, initial, opt, range, out);
  } catch (const EngineError& e) {
    failed = true;
    out.outcome = "FAILED";
    out.message = e.what();
    out.error_kind = e.kind;
    if (running_task_ >= 0) out.failed_task = p.tasks[running_task_].id;
  } catch (const std::exception& e) {
    failed = true;
    out.outcome = "FAILED";
    out.message = e.what();
    out.error_kind = "Exception";
    if (running_task_ >= 0) out.failed_task = p.tasks[running_task_].id;
  }
  if (out.outcome == "CANCELLED") failed = true;
  cleanup(failed);
  return out;
}

}  // namespace dfb
