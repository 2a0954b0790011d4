// Offset allocator over one contiguous region: exact-fit reuse, then size-segregated
// first fit from both ends, immediate coalescing of neighbours on free.  Used for the fast (device) slab, the pinned
// backing slab and the service store.  Role parity: reference
// src/dataflow/runtime/slab.py:24-113 (best fit, 512-byte alignment, coalescing).
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <set>
#include <utility>

namespace dfb {

class SlabAllocator {
 public:
  static constexpr size_t kAlign = 512;
  static constexpr size_t kNone = static_cast<size_t>(-1);

  // The usable extent is the capacity rounded down to the alignment, so every block edge (carved from
  // either end of a hole) is aligned.
  explicit SlabAllocator(size_t capacity = 0, size_t align = kAlign) : cap_(capacity / align * align), align_(align) {
    if (cap_) insert_free(0, cap_);
  }

  static size_t round_up(size_t n, size_t a) { return (n + a - 1) / a * a; }

  // Requests of at least capacity / ``div`` count as large (lowest-address first fit); smaller ones are carved from the top.
  // ``best_fit``: a large request takes the smallest hole that fits instead of the lowest one.
  void set_policy(size_t div, bool best_fit) { large_div_ = div ? div : 48; best_fit_ = best_fit; }

  // returns an offset or kNone.  Exact-size holes are reused first (training chains allocate a handful of
  // sizes over and over).  Otherwise large requests (>= capacity / 48) take the lowest-address hole that fits
  // and small ones are carved from the END of the highest-address hole that fits, so the two size classes
  // grow towards each other and a small object never splits a hole that a large one will need again.
  size_t allocate(size_t bytes) {
    size_t need = round_up(bytes ? bytes : 1, align_);
    auto exact = by_size_.lower_bound({need, 0});
    if (exact == by_size_.end()) return kNone;
    size_t off, len;
    bool from_end = false;
    if (exact->first == need) {
      off = exact->second; len = exact->first;
    } else if (need >= cap_ / large_div_) {
      off = kNone; len = 0;
      if (best_fit_) {
        off = exact->second; len = exact->first;       // by_size_ is ordered by (length, offset): the smallest hole that fits
      } else {
        for (auto& kv : by_off_) {
          if (kv.second >= need) { off = kv.first; len = kv.second; break; }
        }
      }
      if (off == kNone) return kNone;
    } else {
      off = kNone; len = 0;
      for (auto it = by_off_.rbegin(); it != by_off_.rend(); ++it) {
        if (it->second >= need) { off = it->first; len = it->second; break; }
      }
      if (off == kNone) return kNone;
      from_end = true;
    }
    erase_free(off, len);
    size_t at = off;
    if (len > need) {
      if (from_end) { insert_free(off, len - need); at = off + len - need; }
      else insert_free(off + need, len - need);
    }
    live_[at] = need;
    used_ += need;
    if (used_ > peak_) peak_ = used_;
    return at;
  }

  // place at a fixed offset (static placement); false if any byte is taken
  bool allocate_at(size_t off, size_t bytes) {
    size_t need = round_up(bytes ? bytes : 1, align_);
    auto it = by_off_.upper_bound(off);
    if (it == by_off_.begin()) return false;
    --it;
    size_t foff = it->first, flen = it->second;
    if (off < foff || off + need > foff + flen) return false;
    erase_free(foff, flen);
    if (off > foff) insert_free(foff, off - foff);
    if (foff + flen > off + need) insert_free(off + need, foff + flen - off - need);
    live_[off] = need;
    used_ += need;
    if (used_ > peak_) peak_ = used_;
    return true;
  }

  bool release(size_t off) {
    auto it = live_.find(off);
    if (it == live_.end()) return false;
    size_t len = it->second;
    live_.erase(it);
    used_ -= len;
    // coalesce with the next free block
    auto nx = by_off_.find(off + len);
    if (nx != by_off_.end()) {
      size_t nlen = nx->second;
      erase_free(off + len, nlen);
      len += nlen;
    }
    // and with the previous one
    auto pv = by_off_.lower_bound(off);
    if (pv != by_off_.begin()) {
      --pv;
      if (pv->first + pv->second == off) {
        size_t poff = pv->first, plen = pv->second;
        erase_free(poff, plen);
        off = poff;
        len += plen;
      }
    }
    insert_free(off, len);
    return true;
  }

  size_t capacity() const { return cap_; }
  size_t used() const { return used_; }
  size_t peak() const { return peak_; }
  size_t largest_free() const { return by_size_.empty() ? 0 : by_size_.rbegin()->first; }
  size_t live_blocks() const { return live_.size(); }
  size_t block_size(size_t off) const {
    auto it = live_.find(off);
    return it == live_.end() ? 0 : it->second;
  }

 private:
  void insert_free(size_t off, size_t len) {
    by_off_[off] = len;
    by_size_.insert({len, off});
  }
  void erase_free(size_t off, size_t len) {
    by_off_.erase(off);
    by_size_.erase({len, off});
  }
  size_t cap_, align_;
  size_t large_div_ = 48;
  bool best_fit_ = false;
  size_t used_ = 0, peak_ = 0;
  std::map<size_t, size_t> by_off_;                  // free: offset -> length
  std::set<std::pair<size_t, size_t>> by_size_;      // free: (length, offset)
  std::map<size_t, size_t> live_;                    // allocated: offset -> length
};

}  // namespace dfb
