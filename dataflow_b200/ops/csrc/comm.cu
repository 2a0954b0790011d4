// Fused data-parallel communication kernels over NVLink peer memory (one process per GPU).
//
//   zero_rs_adamw : gradient reduce-scatter fused with the fp32 accumulate / cast and the
//                   partitioned AdamW update.  Every rank owns one flat slice of a layer's
//                   packed weight object.  The owner *pulls* its slice of every rank's local
//                   gradient straight out of that rank's memory (plain peer loads over NVSwitch),
//                   sums the contributions in rank order (deterministic), applies AdamW to its fp32
//                   master / moment slice and writes the bf16 parameter slice — one kernel, no
//                   staging buffers, no library collective.
//                   With an accumulator given instead, the same kernel is the per-round gradient
//                   reduce-scatter of the re-gathering (FSDP) mode: pull, sum in rank order, add into
//                   this rank's fp32 gradient slice; the optimizer then runs locally on the slice.
//   param_gather  : parameter all-gather by peer loads into the full per-layer weight object.
//
// Rendezvous is a small control block per rank in peer-mapped memory: a *mailbox*
// (slot -> byte offset of the published buffer inside the rank's slab, plus a sequence number)
// and an *ack* counter per slot.  A rank publishes a buffer, readers wait for the sequence number,
// read, then bump the owner's ack counter; the owner leaves its kernel only after every reader has
// acked, so the buffer stays valid while peers read it.  Every wait is bounded by %globaltimer;
// on expiry the kernel records {phase, peer} in the error word, skips the rest and returns.
//
// The reference has no such kernels: its ZeRO lane is NCCL reduce-scatter -> Triton AdamW -> NCCL
// all-gather (src/dataflow_training/blocks/adamw/rs.py:34-105).
#include <cstdlib>

#include "common.cuh"
#include "ops.h"

namespace dfb {

constexpr int kMaxWorld = 8;
constexpr int kMaxFields = 16;
// These kernels run on a communication stream WHILE the persistent GEMMs hold every SM (one 192-thread CTA of about 180
// registers per thread and 225 KiB of shared memory per SM).  What an SM has left is about 30 K registers and a few
// hundred bytes of shared memory: a 256-thread CTA of at most 112 registers per thread fits beside the GEMM, a
// 512-thread one does not and would only ever run in the gaps between GEMMs.
constexpr int kCommThreads = 256;
constexpr int kCommRegs = 112;

struct PeerTable {
  unsigned char* slab[kMaxWorld];     // peer-mapped base of each rank's fast slab
  unsigned char* ctrl[kMaxWorld];     // peer-mapped control block of each rank
  int rank, world;
};

// control block layout (bytes): [0, 8*S) mailbox offsets (u64) | [8*S, 12*S) mailbox seq (u32) | [12*S, 16*S) ack (u32)
DFB_DEVICE unsigned long long* mail_off(unsigned char* ctrl, int slots, int slot) {
  return reinterpret_cast<unsigned long long*>(ctrl) + slot;
}
DFB_DEVICE unsigned int* mail_seq(unsigned char* ctrl, int slots, int slot) {
  return reinterpret_cast<unsigned int*>(ctrl + 8ull * slots) + slot;
}
DFB_DEVICE unsigned int* ack_ctr(unsigned char* ctrl, int slots, int slot) {
  return reinterpret_cast<unsigned int*>(ctrl + 12ull * slots) + slot;
}

DFB_DEVICE unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
DFB_DEVICE void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
DFB_DEVICE unsigned long long gtimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Wait until *p >= want (sequence numbers only grow).  false on timeout.
DFB_DEVICE bool wait_ge(const unsigned int* p, unsigned int want, unsigned long long timeout_ns) {
  unsigned long long t0 = gtimer();
  for (;;) {
    if (static_cast<int>(ld_acquire_sys(p) - want) >= 0) return true;
    if (gtimer() - t0 > timeout_ns) return false;
    __nanosleep(200);
  }
}

struct FieldRange { long long begin, end; float wd; };   // element ranges of the flat object that take weight decay

struct RsAdamwParams {
  PeerTable peers;
  int slots, slot;
  unsigned int seq, ack_expect;
  const bf16* grad;             // this rank's full local gradient (flat, n_total elements)
  long long slice_begin;        // first element of this rank's slice in the flat object
  long long slice_len;          // elements in this rank's slice (multiple of 8)
  float* master;                // slice-sized fp32 master weights (may be null: update bf16 in place)
  float* m;
  float* v;
  bf16* shard_out;              // slice-sized bf16 parameter shard
  float* gacc;                  // when set: reduce-scatter + fp32 accumulate only (no optimizer step) into this slice
  int gacc_first;               // 1: overwrite the accumulator (first round of a step), 0: add to it
  FieldRange fields[kMaxFields];
  int n_fields;
  float lr, b1, b2, eps, bc1, bc2, gscale;
  unsigned long long timeout_ns;
  int* err;                     // error word: 0 ok, else (phase << 8 | peer)
  unsigned int* done_ctr;       // local counter for "last CTA" detection (zeroed by the kernel's last CTA)
};

// V 16-byte vectors per thread and iteration from each of at most WMAX ranks: V x world peer loads in flight
template <int V, int WMAX>
__global__ void __maxnreg__(kCommRegs) zero_rs_adamw_kernel(RsAdamwParams p) {
  __shared__ const bf16* src[kMaxWorld];
  __shared__ int failed;
  const int me = p.peers.rank, W = p.peers.world;
  if (threadIdx.x == 0) failed = 0;
  // publish my gradient buffer (one thread of the grid)
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    *mail_off(p.peers.ctrl[me], p.slots, p.slot) =
        static_cast<unsigned long long>(reinterpret_cast<const unsigned char*>(p.grad) - p.peers.slab[me]);
    __threadfence_system();
    st_release_sys(mail_seq(p.peers.ctrl[me], p.slots, p.slot), p.seq);
  }
  __syncthreads();
  // every CTA resolves the peers' published buffers itself (no intra-grid dependency)
  if (threadIdx.x < W) {
    int r = threadIdx.x;
    if (r == me) {
      src[r] = p.grad;
    } else if (wait_ge(mail_seq(p.peers.ctrl[r], p.slots, p.slot), p.seq, p.timeout_ns)) {
      unsigned long long off = *reinterpret_cast<volatile unsigned long long*>(mail_off(p.peers.ctrl[r], p.slots, p.slot));
      src[r] = reinterpret_cast<const bf16*>(p.peers.slab[r] + off);
    } else {
      atomicExch(p.err, (1 << 8) | r);
      failed = 1;
    }
  }
  __syncthreads();
  if (!failed) {
    const long long nvec = p.slice_len >> 3;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long v0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v0 < nvec; v0 += V * stride) {
      // every rank's vectors are requested before the first one is used (a peer load takes microseconds); the sum still
      // runs in rank order: deterministic
      bf16x8 pv[V][WMAX];
#pragma unroll
      for (int u = 0; u < V; ++u) {
        const long long vi = v0 + u * stride;
        if (vi < nvec) {
#pragma unroll
          for (int r = 0; r < WMAX; ++r)
            if (r < W) pv[u][r] = ld8(src[r] + p.slice_begin + (vi << 3));
        }
      }
#pragma unroll
      for (int u = 0; u < V; ++u) {
        const long long vi = v0 + u * stride;
        if (vi >= nvec) continue;
        const long long e0 = vi << 3;                         // element inside the slice
        const long long g0 = p.slice_begin + e0;              // element inside the flat object
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
        for (int r = 0; r < WMAX; ++r) {
          if (r < W) {
            float f[8];
            unpack8(pv[u][r], f);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += f[i];
          }
        }
        if (p.gacc) {
          float4 a = make_float4(acc[0], acc[1], acc[2], acc[3]), b = make_float4(acc[4], acc[5], acc[6], acc[7]);
          if (!p.gacc_first) {
            const float4 c = *reinterpret_cast<const float4*>(p.gacc + e0), d = *reinterpret_cast<const float4*>(p.gacc + e0 + 4);
            a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w; b.x += d.x; b.y += d.y; b.z += d.z; b.w += d.w;
          }
          *reinterpret_cast<float4*>(p.gacc + e0) = a;
          *reinterpret_cast<float4*>(p.gacc + e0 + 4) = b;
          continue;
        }
        float wd = 0.f;
        for (int k = 0; k < p.n_fields; ++k)
          if (g0 >= p.fields[k].begin && g0 < p.fields[k].end) wd = p.fields[k].wd;
        float wv[8];
        if (p.master) {
          float4 a = *reinterpret_cast<const float4*>(p.master + e0), b = *reinterpret_cast<const float4*>(p.master + e0 + 4);
          wv[0] = a.x; wv[1] = a.y; wv[2] = a.z; wv[3] = a.w; wv[4] = b.x; wv[5] = b.y; wv[6] = b.z; wv[7] = b.w;
        } else {
          unpack8(ld8(p.shard_out + e0), wv);
        }
        float mv[8], vv[8];
        {
          float4 a = *reinterpret_cast<const float4*>(p.m + e0), b = *reinterpret_cast<const float4*>(p.m + e0 + 4);
          mv[0] = a.x; mv[1] = a.y; mv[2] = a.z; mv[3] = a.w; mv[4] = b.x; mv[5] = b.y; mv[6] = b.z; mv[7] = b.w;
          float4 c = *reinterpret_cast<const float4*>(p.v + e0), d = *reinterpret_cast<const float4*>(p.v + e0 + 4);
          vv[0] = c.x; vv[1] = c.y; vv[2] = c.z; vv[3] = c.w; vv[4] = d.x; vv[5] = d.y; vv[6] = d.z; vv[7] = d.w;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float g = acc[i] * p.gscale;
          mv[i] = p.b1 * mv[i] + (1.f - p.b1) * g;
          vv[i] = p.b2 * vv[i] + (1.f - p.b2) * g * g;
          wv[i] -= p.lr * ((mv[i] / p.bc1) / (sqrtf(vv[i] / p.bc2) + p.eps) + wd * wv[i]);
        }
        *reinterpret_cast<float4*>(p.m + e0) = make_float4(mv[0], mv[1], mv[2], mv[3]);
        *reinterpret_cast<float4*>(p.m + e0 + 4) = make_float4(mv[4], mv[5], mv[6], mv[7]);
        *reinterpret_cast<float4*>(p.v + e0) = make_float4(vv[0], vv[1], vv[2], vv[3]);
        *reinterpret_cast<float4*>(p.v + e0 + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
        if (p.master) {
          *reinterpret_cast<float4*>(p.master + e0) = make_float4(wv[0], wv[1], wv[2], wv[3]);
          *reinterpret_cast<float4*>(p.master + e0 + 4) = make_float4(wv[4], wv[5], wv[6], wv[7]);
        }
        st8(p.shard_out + e0, pack8(wv));
      }
    }
  }
  // last CTA of the grid: ack every peer (we are done reading them), then hold until every peer acked us
  __threadfence_system();
  __syncthreads();
  __shared__ int is_last;
  if (threadIdx.x == 0) is_last = (atomicAdd(p.done_ctr, 1u) == gridDim.x - 1);
  __syncthreads();
  if (is_last && threadIdx.x == 0) {
    *p.done_ctr = 0;
    for (int r = 0; r < W; ++r)
      if (r != me) atomicAdd_system(ack_ctr(p.peers.ctrl[r], p.slots, p.slot), 1u);
    if (!wait_ge(ack_ctr(p.peers.ctrl[me], p.slots, p.slot), p.ack_expect, p.timeout_ns)) atomicExch(p.err, (2 << 8) | me);
  }
}

struct GatherParams {
  PeerTable peers;
  int slots, slot;
  unsigned int seq, ack_expect;
  const uint4* shard;        // my slice (published to the peers)
  uint4* full;               // destination: the whole object
  long long per_vec;         // 16-byte vectors per slice (slice stride)
  long long total_vec;       // 16-byte vectors in the whole object
  unsigned long long timeout_ns;
  int* err;
  unsigned int* done_ctr;
};

__global__ void __maxnreg__(kCommRegs) param_gather_kernel(GatherParams p) {
  __shared__ const uint4* src[kMaxWorld];
  __shared__ int failed, is_last;
  const int me = p.peers.rank, W = p.peers.world;
  if (threadIdx.x == 0) failed = 0;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    *mail_off(p.peers.ctrl[me], p.slots, p.slot) =
        static_cast<unsigned long long>(reinterpret_cast<const unsigned char*>(p.shard) - p.peers.slab[me]);
    __threadfence_system();
    st_release_sys(mail_seq(p.peers.ctrl[me], p.slots, p.slot), p.seq);
  }
  __syncthreads();
  if (threadIdx.x < W) {
    int r = threadIdx.x;
    if (r == me) {
      src[r] = p.shard;
    } else if (wait_ge(mail_seq(p.peers.ctrl[r], p.slots, p.slot), p.seq, p.timeout_ns)) {
      unsigned long long off = *reinterpret_cast<volatile unsigned long long*>(mail_off(p.peers.ctrl[r], p.slots, p.slot));
      src[r] = reinterpret_cast<const uint4*>(p.peers.slab[r] + off);
    } else {
      atomicExch(p.err, (3 << 8) | r);
      failed = 1;
    }
  }
  __syncthreads();
  if (!failed) {
    // eight vectors in flight per thread (a peer load takes microseconds)
    constexpr int UNR = 8;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long v0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v0 < p.total_vec; v0 += UNR * stride) {
      uint4 x[UNR];
      long long at[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const long long vi = v0 + u * stride;
        at[u] = -1;
        if (vi < p.total_vec) {
          // start with the slice after mine so that the ranks do not all hit the same peer at once
          long long rot = (vi + (static_cast<long long>(me) + 1) * p.per_vec) % p.total_vec;
          int r = static_cast<int>(rot / p.per_vec);
          if (r >= W) r = W - 1;
          at[u] = rot;
          x[u] = src[r][rot - static_cast<long long>(r) * p.per_vec];
        }
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u)
        if (at[u] >= 0) p.full[at[u]] = x[u];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) is_last = (atomicAdd(p.done_ctr, 1u) == gridDim.x - 1);
  __syncthreads();
  if (is_last && threadIdx.x == 0) {
    *p.done_ctr = 0;
    for (int r = 0; r < W; ++r)
      if (r != me) atomicAdd_system(ack_ctr(p.peers.ctrl[r], p.slots, p.slot), 1u);
    if (!wait_ge(ack_ctr(p.peers.ctrl[me], p.slots, p.slot), p.ack_expect, p.timeout_ns)) atomicExch(p.err, (4 << 8) | me);
  }
}

// ---------------------------------------------------------------------------- parameter gather by the copy engines
// The gather is a pure copy, so its bytes can ride the copy engines instead of SM threads (no issue slots, registers or L1
// taken from the GEMM that runs beside it).  What still needs a kernel is the rendezvous, and that is two one-warp
// launches around the copies:
//   open : publish this rank's shard address for the slot, wait (bounded) until every peer has published this sequence
//          number, and CHECK that each peer's shard still lies where the host believes it does (the copies that follow were
//          issued with those addresses; a shard that moved raises the error word, it is never read silently from the wrong place)
//   copies: one cudaMemcpyAsync per rank, peer slab -> this rank's gathered buffer, on the same stream
//   close: tell every peer this rank has finished reading, wait (bounded) for their acknowledgements
struct GatherDmaParams {
  PeerTable peers;
  int slots, slot;
  unsigned int seq, ack_expect;
  unsigned long long my_off;
  unsigned long long expect_off[kMaxWorld];
  unsigned long long timeout_ns;
  int* err;
};

__global__ void gather_open_kernel(GatherDmaParams p) {
  const int me = p.peers.rank, W = p.peers.world;
  if (threadIdx.x == 0) {
    *mail_off(p.peers.ctrl[me], p.slots, p.slot) = p.my_off;
    __threadfence_system();
    st_release_sys(mail_seq(p.peers.ctrl[me], p.slots, p.slot), p.seq);
  }
  __syncwarp();
  const int r = threadIdx.x;
  if (r < W && r != me) {
    if (wait_ge(mail_seq(p.peers.ctrl[r], p.slots, p.slot), p.seq, p.timeout_ns)) {
      const unsigned long long off = *reinterpret_cast<volatile unsigned long long*>(mail_off(p.peers.ctrl[r], p.slots, p.slot));
      if (off != p.expect_off[r]) atomicExch(p.err, (5 << 8) | r);          // the peer's shard is not where the copies will read
    } else {
      atomicExch(p.err, (3 << 8) | r);
    }
  }
}

__global__ void gather_close_kernel(GatherDmaParams p) {
  const int me = p.peers.rank, W = p.peers.world;
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int r = 0; r < W; ++r)
      if (r != me) atomicAdd_system(ack_ctr(p.peers.ctrl[r], p.slots, p.slot), 1u);
    if (!wait_ge(ack_ctr(p.peers.ctrl[me], p.slots, p.slot), p.ack_expect, p.timeout_ns)) atomicExch(p.err, (4 << 8) | me);
  }
}

// ---------------------------------------------------------------------------- host entry points
// CTAs per communication kernel: one per SM unless DATAFLOW_COMM_CTAS names a smaller budget (the kernels are grid-stride
// loops, so any count is correct; fewer CTAs leave more issue slots to the GEMM they run beside).
static int comm_grid(int num_sms) {
  static int budget = [] {
    const char* e = getenv("DATAFLOW_COMM_CTAS");
    return e ? atoi(e) : 0;
  }();
  return budget > 0 && budget < num_sms ? budget : num_sms;
}

static PeerTable make_table(const unsigned long long* slabs, const unsigned long long* ctrls, int rank, int world) {
  PeerTable t{};
  for (int i = 0; i < world && i < kMaxWorld; ++i) {
    t.slab[i] = reinterpret_cast<unsigned char*>(slabs[i]);
    t.ctrl[i] = reinterpret_cast<unsigned char*>(ctrls[i]);
  }
  t.rank = rank;
  t.world = world;
  return t;
}

int zero_rs_adamw(const unsigned long long* slabs, const unsigned long long* ctrls, int rank, int world, int slots, int slot,
                  unsigned int seq, unsigned int ack_expect, const void* grad, long long slice_begin, long long slice_len,
                  float* master, float* m, float* v, void* shard_out, const long long* field_begin,
                  const long long* field_end, const float* field_wd, int n_fields, float lr, float b1, float b2, float eps,
                  int step, float gscale, double timeout_s, int* err, unsigned int* done_ctr, int num_sms, cudaStream_t s,
                  float* gacc, int gacc_first) {
  if (world > kMaxWorld || n_fields > kMaxFields || (slice_len & 7) || (slice_begin & 7)) return -2;
  RsAdamwParams p{};
  p.peers = make_table(slabs, ctrls, rank, world);
  p.slots = slots; p.slot = slot; p.seq = seq; p.ack_expect = ack_expect;
  p.grad = reinterpret_cast<const bf16*>(grad);
  p.slice_begin = slice_begin; p.slice_len = slice_len;
  p.master = master; p.m = m; p.v = v; p.shard_out = reinterpret_cast<bf16*>(shard_out);
  for (int i = 0; i < n_fields; ++i) p.fields[i] = {field_begin[i], field_end[i], field_wd[i]};
  p.n_fields = n_fields;
  p.lr = lr; p.b1 = b1; p.b2 = b2; p.eps = eps;
  p.bc1 = 1.f - powf(b1, (float)step); p.bc2 = 1.f - powf(b2, (float)step);
  p.gscale = gscale;
  p.timeout_ns = static_cast<unsigned long long>(timeout_s * 1e9);
  p.err = err; p.done_ctr = done_ctr;
  p.gacc = gacc; p.gacc_first = gacc_first;
  // peer loads in flight per thread: V vectors x world ranks, about eight either way
  const int grid = comm_grid(num_sms);
  if (world <= 2) zero_rs_adamw_kernel<4, 2><<<grid, kCommThreads, 0, s>>>(p);
  else if (world <= 4) zero_rs_adamw_kernel<2, 4><<<grid, kCommThreads, 0, s>>>(p);
  else zero_rs_adamw_kernel<1, 8><<<grid, kCommThreads, 0, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int param_gather(const unsigned long long* slabs, const unsigned long long* ctrls, int rank, int world, int slots, int slot,
                 unsigned int seq, unsigned int ack_expect, const void* shard, void* full, long long per_bytes,
                 long long total_bytes, double timeout_s, int* err, unsigned int* done_ctr, int num_sms, cudaStream_t s) {
  if (world > kMaxWorld || (per_bytes & 15) || (total_bytes & 15)) return -2;
  GatherParams p{};
  p.peers = make_table(slabs, ctrls, rank, world);
  p.slots = slots; p.slot = slot; p.seq = seq; p.ack_expect = ack_expect;
  p.shard = reinterpret_cast<const uint4*>(shard);
  p.full = reinterpret_cast<uint4*>(full);
  p.per_vec = per_bytes >> 4; p.total_vec = total_bytes >> 4;
  p.timeout_ns = static_cast<unsigned long long>(timeout_s * 1e9);
  p.err = err; p.done_ctr = done_ctr;
  param_gather_kernel<<<comm_grid(num_sms), kCommThreads, 0, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int param_gather_dma(const unsigned long long* slabs, const unsigned long long* ctrls, int rank, int world, int slots, int slot,
                     unsigned int seq, unsigned int ack_expect, const void* shard, const unsigned long long* expect_off, void* full,
                     long long per_bytes, long long total_bytes, double timeout_s, int* err, cudaStream_t s) {
  if (world > kMaxWorld || per_bytes <= 0 || total_bytes <= 0) return -2;
  GatherDmaParams p{};
  p.peers = make_table(slabs, ctrls, rank, world);
  p.slots = slots; p.slot = slot; p.seq = seq; p.ack_expect = ack_expect;
  p.my_off = static_cast<unsigned long long>(reinterpret_cast<const unsigned char*>(shard) - p.peers.slab[rank]);
  for (int r = 0; r < world; ++r) p.expect_off[r] = expect_off[r];
  p.timeout_ns = static_cast<unsigned long long>(timeout_s * 1e9);
  p.err = err;
  gather_open_kernel<<<1, 32, 0, s>>>(p);
  if (cudaGetLastError() != cudaSuccess) return -1;
  for (int i = 0; i < world; ++i) {
    const int r = (rank + 1 + i) % world;                   // start with the next rank so that the ranks do not all read one peer at once
    const long long lo = static_cast<long long>(r) * per_bytes;
    const long long n = lo >= total_bytes ? 0 : (total_bytes - lo < per_bytes ? total_bytes - lo : per_bytes);
    if (n <= 0) continue;
    const void* src = r == rank ? shard : static_cast<const void*>(p.peers.slab[r] + expect_off[r]);
    if (cudaMemcpyAsync(static_cast<unsigned char*>(full) + lo, src, static_cast<size_t>(n), cudaMemcpyDeviceToDevice, s) != cudaSuccess) return -3;
  }
  gather_close_kernel<<<1, 32, 0, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace dfb
