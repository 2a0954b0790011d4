// Expert parallelism over NVLink peer memory: the combine side.
//
// Experts are split over the ranks of a group; every rank keeps its own tokens.  The rows a rank's experts computed
// stay in that rank's memory; the rank that owns a token PULLS them (plain peer loads) and reduces them on the
// fly, so the combine all-to-all and the weighted scatter-add are one kernel with no staging buffer and no atomics:
//     y[t] = base[t] + sum_k w[t, k] * rows_{owner(t, k)}[ row(t, k) ]
// The same kernel, unweighted, is the backward of the dispatch (dx[t] = sum_k dxp[row]); it can also pull one fp32
// per slot (the router-weight gradient <dy, y_row> that the expert's owner computed).
// (The dispatch side is fused into the grouped up-projection: gemm_grouped.cu, GATHER.)
//
// Protocol, per launch ``seq``: a rank publishes "my rows are final" (ready word), waits for the same word of
// every rank it reads from, pulls, then tells every peer it is done (ack counter) and holds the kernel until
// every peer is done with ITS rows — so the stream may overwrite them afterwards.  All waits are bounded by
// ``%globaltimer``; a wait that gives up records (phase << 8 | peer) in the error word and the kernel returns.
// Reference role: src/dataflow_training/model_families/dsv3 expert-parallel all-to-all (NCCL send/recv pairs around
// separate dispatch / combine kernels).
#include "common.cuh"
#include "ops.h"

namespace dfb {
namespace ep {

constexpr int kMaxWorld = 8;
constexpr int kMaxTopK = 16;

DFB_DEVICE unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
DFB_DEVICE unsigned long long gtimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
DFB_DEVICE bool wait_ge(const unsigned int* p, unsigned int want, unsigned long long timeout_ns) {
  unsigned long long t0 = gtimer();
  for (;;) {
    if (static_cast<int>(ld_acquire_sys(p) - want) >= 0) return true;
    if (gtimer() - t0 > timeout_ns) return false;
    __nanosleep(200);
  }
}

struct CombineParams {
  const uint4* rows[kMaxWorld];       // every owner's (C, d) bf16 rows
  const float* scal[kMaxWorld];       // every owner's per-row fp32, or null
  const bf16* base;                   // (T, d) or null
  const float* route_w;               // (T, K) or null (weights 1)
  const int* ids;                     // (T, K) global expert ids
  const int* rows_local;              // (T, K) row at the owner, -1: dropped
  bf16* out;                          // (T, d)
  float* out_s;                       // (T, K) or null
  int T, K, d, e_local, rank, world;
  unsigned int* ready[kMaxWorld];
  unsigned int* acks[kMaxWorld];
  unsigned int seq, ack_expect;
  unsigned long long timeout_ns;
  int* err;
  unsigned int* done_ctr;
};

__global__ void __launch_bounds__(256) ep_combine_kernel(CombineParams p) {
  __shared__ int failed;
  __shared__ int is_last;
  __shared__ int s_row[kMaxTopK], s_owner[kMaxTopK];
  __shared__ float s_w[kMaxTopK];
  const int me = p.rank;
  if (threadIdx.x == 0) failed = 0;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.ready[me]), "r"(p.seq) : "memory");
  }
  __syncthreads();
  if (threadIdx.x < p.world && threadIdx.x != me) {
    if (!wait_ge(p.ready[threadIdx.x], p.seq, p.timeout_ns)) { atomicExch(p.err, (51 << 8) | threadIdx.x); failed = 1; }
  }
  __syncthreads();
  const int vecs = p.d / 8;
  if (!failed) {
    for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
      __syncthreads();
      if (threadIdx.x < p.K) {
        const int i = t * p.K + threadIdx.x;
        const int e = p.ids[i];
        s_row[threadIdx.x] = p.rows_local[i];
        s_owner[threadIdx.x] = e / p.e_local;
        s_w[threadIdx.x] = p.route_w ? p.route_w[i] : 1.f;
        if (p.out_s) {
          const int r = s_row[threadIdx.x];
          p.out_s[i] = r >= 0 ? __ldcg(p.scal[s_owner[threadIdx.x]] + r) : 0.f;
        }
      }
      __syncthreads();
      for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
        float acc[8];
        if (p.base) {
          uint4 b = reinterpret_cast<const uint4*>(p.base)[static_cast<long long>(t) * vecs + v];
          const bf16* bb = reinterpret_cast<const bf16*>(&b);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = __bfloat162float(bb[j]);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        }
        // all K peer loads of this thread in flight before the first use
        for (int k0 = 0; k0 < p.K; k0 += 8) {
          uint4 x[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int k = k0 + u;
            x[u] = make_uint4(0, 0, 0, 0);
            if (k < p.K && s_row[k] >= 0) x[u] = __ldcg(p.rows[s_owner[k]] + static_cast<long long>(s_row[k]) * vecs + v);
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int k = k0 + u;
            if (k < p.K && s_row[k] >= 0) {
              const bf16* xb = reinterpret_cast<const bf16*>(&x[u]);
              const float w = s_w[k];
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[j] = fmaf(w, __bfloat162float(xb[j]), acc[j]);
            }
          }
        }
        uint4 o;
        bf16* ob = reinterpret_cast<bf16*>(&o);
#pragma unroll
        for (int j = 0; j < 8; ++j) ob[j] = __float2bfloat16(acc[j]);
        reinterpret_cast<uint4*>(p.out)[static_cast<long long>(t) * vecs + v] = o;
      }
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = (atomicAdd(p.done_ctr, 1u) == gridDim.x - 1);
  __syncthreads();
  if (is_last && threadIdx.x == 0) {
    *p.done_ctr = 0;
    __threadfence_system();
    for (int r = 0; r < p.world; ++r)
      if (r != me) asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.acks[r]), "r"(1u) : "memory");
    if (!wait_ge(p.acks[me], p.ack_expect, p.timeout_ns)) atomicExch(p.err, (52 << 8) | me);
  }
}

// rows_local[i] = the row slot i of this rank (token i / K, choice i % K) got at the rank that owns its expert
__global__ void ep_pull_rows_kernel(const int* const* tables_dev, const int* ids, int* rows_local, int n, int e_local,
                                    long long my_first_slot) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int owner = ids[i] / e_local;
  rows_local[i] = __ldcg(tables_dev[owner] + my_first_slot + i);
}

}  // namespace ep

int ep_pull_rows(const unsigned long long* tables_dev_array, const int* ids, int* rows_local, int n, int e_local,
                 long long my_first_slot, cudaStream_t stream) {
  if (n <= 0) return 0;
  ep::ep_pull_rows_kernel<<<(n + 255) / 256, 256, 0, stream>>>(reinterpret_cast<const int* const*>(tables_dev_array), ids,
                                                              rows_local, n, e_local, my_first_slot);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int ep_combine(const unsigned long long* rows, const unsigned long long* scal, const void* base, const float* route_w,
               const int* ids, const int* rows_local, void* out, float* out_s, int T, int K, int d, int e_local, int rank,
               int world, const unsigned long long* ready, const unsigned long long* acks, unsigned int seq,
               double timeout_s, int* err, unsigned int* done_ctr, int num_sms, cudaStream_t stream) {
  if (world > ep::kMaxWorld || K > ep::kMaxTopK || (d & 7)) return -2;
  ep::CombineParams p{};
  for (int r = 0; r < world; ++r) {
    p.rows[r] = reinterpret_cast<const uint4*>(rows[r]);
    p.scal[r] = scal ? reinterpret_cast<const float*>(scal[r]) : nullptr;
    p.ready[r] = reinterpret_cast<unsigned int*>(ready[r]);
    p.acks[r] = reinterpret_cast<unsigned int*>(acks[r]);
  }
  p.base = reinterpret_cast<const bf16*>(base); p.route_w = route_w; p.ids = ids; p.rows_local = rows_local;
  p.out = reinterpret_cast<bf16*>(out); p.out_s = scal ? out_s : nullptr;
  p.T = T; p.K = K; p.d = d; p.e_local = e_local; p.rank = rank; p.world = world;
  p.seq = seq; p.ack_expect = static_cast<unsigned int>(world - 1) * seq;
  p.timeout_ns = static_cast<unsigned long long>(timeout_s * 1e9); p.err = err; p.done_ctr = done_ctr;
  int grid = num_sms * 4;
  if (grid > T) grid = T > 0 ? T : 1;
  ep::ep_combine_kernel<<<grid, 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace dfb
