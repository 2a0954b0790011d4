// Plain C++ launch API of the sm_100a kernels: raw pointers, sizes and a stream.
// No allocation happens behind these calls; scratch is passed in by the caller.
// bf16 tensors are passed as void*.
#pragma once
#include <cuda_runtime.h>

namespace dfb {

// ---- norms (norm.cu)
void rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int cols, float eps, cudaStream_t s);
void rmsnorm_apply(const void* x, const void* w, const float* rstd, void* y, int rows, int cols, cudaStream_t s);
void layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int rows, int cols,
                   float eps, cudaStream_t s);
void layernorm_apply(const void* x, const void* w, const void* b, const float* mean, const float* rstd, void* y,
                     int rows, int cols, cudaStream_t s);
int norm_bwd_parts(int rows);   // rows of the (parts, 2, cols) fp32 scratch the backward needs
void rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, const void* dx_add,
                 void* dw, int dw_is_f32, int accumulate, float* partial, int rows, int cols, cudaStream_t s);
void layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, void* dx,
                   const void* dx_add, void* dw, void* db, int dw_is_f32, int accumulate, float* partial, int rows,
                   int cols, cudaStream_t s);

// ---- pointwise (pointwise.cu)
void rope_inplace(void* x, const int* positions, int tokens, int heads, int rot_dim, long long row_stride,
                  int head_stride, int col_base, float theta, int backward, cudaStream_t s);
void swiglu_fwd(const void* x1, const void* x3, void* out, long long rows, int F, long long ld1, long long ld3, cudaStream_t s);
void swiglu_bwd(const void* ds, const void* x1, const void* x3, void* dx1, void* dx3, void* s_out, long long rows, int F,
                long long ld1, long long ld3, long long ldd1, long long ldd3, cudaStream_t s);
void gelu_fwd(const void* x, void* y, long long n, cudaStream_t s);
void gelu_bwd(const void* dy, const void* x, void* dx, long long n, cudaStream_t s);
void add_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t s);
void cast_f32_to_bf16(const float* x, void* y, long long n, cudaStream_t s);
void cast_bf16_to_f32(const void* x, float* y, long long n, cudaStream_t s);
int colsum_parts(int rows);
void colsum_bf16(const void* x, float* partial, void* out, int accumulate, int rows, int cols, cudaStream_t s);
void adamw_bf16(void* w, const void* g, int g_is_f32, void* m, void* v, long long n, float lr, float b1, float b2,
                float eps, float wd, int step, float gscale, cudaStream_t s);
int adamw_split(void* w, void* lo, const void* g, int g_is_f32, void* m, void* v, long long n, float lr, float b1, float b2, float eps,
                float wd, int step, float gscale, cudaStream_t s);
void adamw_master(float* master, void* w_out, const void* g, int g_is_f32, float* m, float* v, long long n, float lr,
                  float b1, float b2, float eps, float wd, int step, float gscale, cudaStream_t s);
void adamw_f32(float* w, const float* g, float* m, float* v, long long n, float lr, float b1, float b2, float eps,
               float wd, int step, float gscale, cudaStream_t s);
void sgd_bf16(void* w, const void* g, void* m, long long n, float lr, float mu, float wd, cudaStream_t s);

// ---- loss (loss.cu)
void ce_loss_fwd_bwd(void* logits, const int* targets, float* nll_rows, float* loss, int accumulate, int rows, int vocab,
                     long long ld, float scale, cudaStream_t s);

// ---- embedding (embed.cu)
void embed_fwd(const int* tok, const void* table, void* out, int tokens, int d, int vocab, const int* positions,
               const void* pos_table, int pos_rows, cudaStream_t s);
void embed_bwd_sorted(const int* sorted_key, const int* order, const void* dy, void* dtable, int dtable_is_f32, int n,
                      int d, int table_rows, int accumulate, cudaStream_t s);

// ---- GEMM (gemm_tcgen05.cu)
int gemm_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn, void* D, long long ldd,
              int d_is_f32, const void* addend, long long ld_add, int add_is_f32, const void* bias, int M, int N, int K,
              int num_sms, cudaStream_t stream);
int gemm_bf16_last_error();
void gemm_bf16_set_mt(int mt);
void gemm_bf16_set_default_path(int path);

// ---- fused data-parallel communication (comm.cu)
int zero_rs_adamw(const unsigned long long* slabs, const unsigned long long* ctrls, int rank, int world, int slots, int slot,
                  unsigned int seq, unsigned int ack_expect, const void* grad, long long slice_begin, long long slice_len,
                  float* master, float* m, float* v, void* shard_out, const long long* field_begin,
                  const long long* field_end, const float* field_wd, int n_fields, float lr, float b1, float b2, float eps,
                  int step, float gscale, double timeout_s, int* err, unsigned int* done_ctr, int num_sms, cudaStream_t s,
                  float* gacc = nullptr, int gacc_first = 0);
int param_gather(const unsigned long long* slabs, const unsigned long long* ctrls, int rank, int world, int slots, int slot,
                 unsigned int seq, unsigned int ack_expect, const void* shard, void* full, long long per_bytes,
                 long long total_bytes, double timeout_s, int* err, unsigned int* done_ctr, int num_sms, cudaStream_t s);
// the same gather with the bytes on the copy engines: two one-warp rendezvous launches around one cudaMemcpyAsync per rank;
// expect_off[r] = where rank r's shard lies in its slab (checked on the device against what r publishes)
int param_gather_dma(const unsigned long long* slabs, const unsigned long long* ctrls, int rank, int world, int slots, int slot,
                     unsigned int seq, unsigned int ack_expect, const void* shard, const unsigned long long* expect_off, void* full,
                     long long per_bytes, long long total_bytes, double timeout_s, int* err, cudaStream_t s);


// Tensor-parallel GEMMs fused with their collective (gemm_tp.cu)
int tp_ag_gemm(const unsigned long long* x_src, long long x_ld, void* gathered, const void* W, long long ldw, int b_mn, void* Y,
               long long ldy, int panel_rows, int N, int K, int rank, int world, unsigned int* flags,
               const unsigned long long* ready, const unsigned long long* acks, unsigned int launch_seq, int chunk_rows,
               double timeout_s, int* err, unsigned int* done_ctr, int num_sms, cudaStream_t stream);
int tp_gemm_rs(const void* X, long long ldx, const void* W, long long ldw, int b_mn, void* D, long long ldd, const void* addend,
               long long ld_add, int panel_rows, int N, int K, int rank, int world, const unsigned long long* stage,
               const unsigned long long* tile_flags, unsigned int launch_seq, double timeout_s, int* err,
               unsigned int* done_ctr, int num_sms, cudaStream_t stream);

// Mixture of experts (moe.cu, gemm_grouped.cu)
int moe_topk_softmax(const void* logits, int logits_f32, float* route_w, int* route_ids, int t, int E, int K, int mode,
                     cudaStream_t s);
int moe_router_bwd(const float* dprob, const float* route_w, const int* route_ids, const void* logits, int logits_f32,
                   float* dlogits, int t, int E, int K, int mode, cudaStream_t s);
// padded expert-major layout of the routed slots (stable counting sort on the device; scratch: ceil(t K / 1024) * E ints)
int moe_sort(const int* ids, int t, int K, int E, int tile_rows, int mp, int* row_of, int* row_src, int* offsets_pad, int* tile_expert,
             int* counts, int* scratch, cudaStream_t s);
int moe_dispatch(const void* x, long long ldx, const int* row_src, void* xp, int rows, int d, cudaStream_t s);
int moe_combine(const void* base, const void* yp, const float* w, const int* row_of, void* out, int t, int d, int K,
                cudaStream_t s);
int moe_dispatch_bwd(const void* dxp, const int* row_of, void* out, int t, int d, int K, int accumulate, cudaStream_t s);
int moe_scale_rows(void* xp, const float* w, const int* row_of, int slots, int d, cudaStream_t s);
int moe_rowdot(const void* a, const void* b, const int* row_of, float* out, int slots, int d, cudaStream_t s);
// tensor-pipe step cost by shape and operand source (umma_probe.cu); out: 3 int64 (issue cycles, total cycles, timed out)
int umma_probe(int kind, int n, int count, int nacc, long long* out, cudaStream_t stream);

// causal varlen flash attention forward on tcgen05 (attention.cu)
int flash_fwd_sm100(const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv, void* out, long long ldo,
                    float* lse, const int* cu_seqlens, int nseg, int max_seqlen, int T, int hq, int hkv, int head_dim, float scale,
                    cudaStream_t stream, long long* trace = nullptr);
// causal varlen flash attention backward on tcgen05 (attention_bwd.cu); ld2: scratch of hq * T float2
int flash_bwd_sm100(const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv, const void* o, long long ldo,
                    const void* dout, long long lddo, const float* lse, void* dq, long long lddq, void* dk, long long lddk, void* dv,
                    long long lddv, void* ld2, const int* cu_seqlens, int nseg, int max_seqlen, int T, int hq, int hkv, int head_dim,
                    float scale, cudaStream_t stream, long long* trace = nullptr);
// sparse-attention indexer (dsa.cu): index scores of query rows [q0, q1) against keys [key_lo, q1) on tcgen05, -inf where a
// query does not see a key; and the k largest entries of every row as ascending key indices (-1 = fewer than k finite entries)
int dsa_index_scores(const void* q, long long ldq, const void* k, long long ldk, const float* wgt, const int* seg_start, float* out,
                     long long ld, int n, int H, int D, int q0, int q1, int key_lo, int* err, cudaStream_t s);
int dsa_topk_rows(const float* scores, long long ld, int rows, int cols, int col_base, int k, int* sel, int sel_ld, cudaStream_t s);
// fp8 lane: row-wise e4m3 quantisation and the dequantising CTA-pair GEMM
int quant_fp8_rowwise(const void* x, long long ldx, void* q, long long ldq, float* scale, long long rows, int K, cudaStream_t s);
int gemm_fp8_2sm(const void* A, long long lda, int a_fmt, const void* B, long long ldb, int b_fmt, void* D, long long ldd, int d_is_f32,
                 const float* row_scale, const float* col_scale, const void* addend, long long ld_add, const void* bias, int M, int N,
                 int K, int num_sms, cudaStream_t stream);
// sequence-mixing helpers of the linear / latent attention families (seqmix.cu)
int l2norm_fwd(const void* x, void* y, float* rstd, long long rows, int D, float eps, cudaStream_t s);
int l2norm_bwd(const void* dy, const void* x, const float* rstd, void* dx, long long rows, int D, cudaStream_t s);
int gated_rmsnorm_fwd(const void* x, const void* g, const void* w, void* y, float* rstd, long long rows, int D, float eps, cudaStream_t s);
int gated_rmsnorm_bwd(const void* dy, const void* x, const void* g, const void* w, const float* rstd, void* dx, void* dg,
                      float* dw_partial, int blocks, long long rows, int D, cudaStream_t s);
int conv_silu_fwd(const void* x, const void* w, const int* seg_start, void* y, long long n, int C, int W, cudaStream_t s);
int conv_silu_bwd(const void* dy, const void* x, const void* w, const int* seg_start, void* dx, float* dw_partial, int row_blocks,
                  int rows_per_block, long long n, int C, int W, cudaStream_t s);
int router_sigmoid_noaux(const void* logits, const float* bias, float* route_w, int* route_ids, int t, int E, int K, int n_group,
                         int topk_group, float scaling, cudaStream_t s);
// expert parallelism: dispatch fused into the grouped up-projection; pull-and-reduce combine (gemm_grouped.cu, moe_ep.cu)
int moe_grouped_mm_gather(const unsigned long long* x_src, void* X, const int* row_src, const void* W, void* Y,
                          const int* tile_expert, int Mp, int N, int K, int E, int w_kn, int tokens_per_rank, int rank,
                          int world, unsigned int* tile_flags, const unsigned long long* ready, const unsigned long long* acks,
                          unsigned int launch_seq, double timeout_s, int* err, unsigned int* done_ctr, int num_sms,
                          cudaStream_t stream);
int ep_pull_rows(const unsigned long long* tables_dev_array, const int* ids, int* rows_local, int n, int e_local,
                 long long my_first_slot, cudaStream_t stream);
int ep_combine(const unsigned long long* rows, const unsigned long long* scal, const void* base, const float* route_w,
               const int* ids, const int* rows_local, void* out, float* out_s, int T, int K, int d, int e_local, int rank,
               int world, const unsigned long long* ready, const unsigned long long* acks, unsigned int seq,
               double timeout_s, int* err, unsigned int* done_ctr, int num_sms, cudaStream_t stream);
int moe_grouped_mm(const void* X, const void* W, void* Y, const int* tile_expert, int Mp, int N, int K, int E, int w_kn,
                   int num_sms, cudaStream_t stream);
int moe_grouped_wgrad(const void* X, const void* dY, void* dW, const int* offsets_pad, int Mp, int Kw, int N, int E,
                      int accumulate, int num_sms, cudaStream_t stream);
}  // namespace dfb
