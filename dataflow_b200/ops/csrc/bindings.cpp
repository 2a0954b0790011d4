// Torch-facing bindings of the kernel launch API: tensors in, raw pointers out,
// on the current CUDA stream.  Shape / dtype / contiguity checks live here so
// the kernels can assume their contracts.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "ops.h"

using at::Tensor;

#define CHECK_CUDA(x) TORCH_CHECK((x).is_cuda(), #x " must be a CUDA tensor")
// every kernel here dereferences its operands on the device: a host tensor is refused, never launched on
#define CHECK_BF16(x) TORCH_CHECK((x).is_cuda() && (x).scalar_type() == at::kBFloat16, #x " must be a bf16 CUDA tensor")
#define CHECK_F32(x) TORCH_CHECK((x).is_cuda() && (x).scalar_type() == at::kFloat, #x " must be an fp32 CUDA tensor")
#define CHECK_I32(x) TORCH_CHECK((x).is_cuda() && (x).scalar_type() == at::kInt, #x " must be an int32 CUDA tensor")
#define CHECK_CONTIG(x) TORCH_CHECK((x).is_contiguous(), #x " must be contiguous")

// One operand check used by every binding below: the kernels dereference raw pointers with 16-byte
// vector accesses, so an operand that is on the host, of another dtype, strided, too short or not
// 16-byte aligned is refused here, before anything is launched.
static void need(const Tensor& t, const char* name, at::ScalarType dt, int64_t numel = -1, bool contiguous = true) {
  TORCH_CHECK(t.defined(), name, " is undefined");
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor (got a host tensor)");
  TORCH_CHECK(t.scalar_type() == dt, name, " must have dtype ", dt, " (got ", t.scalar_type(), ")");
  if (contiguous) TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
  if (numel >= 0) TORCH_CHECK(t.numel() == numel, name, " must have ", numel, " elements (got ", t.numel(), ")");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0, name, " must be 16-byte aligned");
}
static void need_opt(const c10::optional<Tensor>& t, const char* name, at::ScalarType dt, int64_t numel = -1) {
  if (t.has_value()) need(*t, name, dt, numel);
}
// gradient-like operands may be bf16 or fp32
static void need_grad(const Tensor& t, const char* name, int64_t numel) {
  TORCH_CHECK(t.defined() && t.is_cuda() && t.is_contiguous(), name, " must be a contiguous CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kFloat, name, " must be bf16 or fp32");
  TORCH_CHECK(t.numel() == numel, name, " must have ", numel, " elements (got ", t.numel(), ")");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0, name, " must be 16-byte aligned");
}

static cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
static const void* optp(const c10::optional<Tensor>& t) { return t.has_value() ? t->data_ptr() : nullptr; }
static int num_sms() {
  static int n = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return n;
}

// ---------------------------------------------------------------- norms
static void rmsnorm_fwd(const Tensor& x, const c10::optional<Tensor>& w, Tensor& y, c10::optional<Tensor> rstd, double eps) {
  need(x, "x", at::kBFloat16); need(y, "y", at::kBFloat16, x.numel());
  int cols = x.size(-1), rows = x.numel() / std::max(cols, 1);
  TORCH_CHECK(cols % 8 == 0, "rmsnorm_fwd needs cols % 8 == 0");
  need_opt(w, "w", at::kBFloat16, cols); need_opt(rstd, "rstd", at::kFloat, rows);
  dfb::rmsnorm_fwd(x.data_ptr(), optp(w), y.data_ptr(), rstd.has_value() ? rstd->data_ptr<float>() : nullptr, rows, cols,
                   (float)eps, cur_stream());
}
static void rmsnorm_apply(const Tensor& x, const Tensor& w, const Tensor& rstd, Tensor& y) {
  need(x, "x", at::kBFloat16); need(y, "y", at::kBFloat16, x.numel());
  int cols = x.size(-1), rows = x.numel() / std::max(cols, 1);
  TORCH_CHECK(cols % 8 == 0, "rmsnorm_apply needs cols % 8 == 0");
  need(w, "w", at::kBFloat16, cols); need(rstd, "rstd", at::kFloat, rows);
  dfb::rmsnorm_apply(x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), y.data_ptr(), rows, cols, cur_stream());
}
static void rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd, Tensor& dx,
                        const c10::optional<Tensor>& dx_add, c10::optional<Tensor> dw, bool accumulate, Tensor& partial) {
  need(x, "x", at::kBFloat16); need(dy, "dy", at::kBFloat16, x.numel()); need(dx, "dx", at::kBFloat16, x.numel());
  need_opt(dx_add, "dx_add", at::kBFloat16, x.numel());
  int cols = x.size(-1), rows = x.numel() / std::max(cols, 1);
  TORCH_CHECK(cols % 8 == 0, "rmsnorm_bwd needs cols % 8 == 0");
  need(w, "w", at::kBFloat16, cols); need(rstd, "rstd", at::kFloat, rows); need(partial, "partial", at::kFloat);
  if (dw.has_value()) need_grad(*dw, "dw", cols);
  TORCH_CHECK(partial.numel() >= (int64_t)dfb::norm_bwd_parts(rows) * 2 * cols, "rmsnorm_bwd scratch too small");
  dfb::rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(), optp(dx_add),
                   dw.has_value() ? dw->data_ptr() : nullptr, dw.has_value() && dw->scalar_type() == at::kFloat,
                   accumulate, partial.data_ptr<float>(), rows, cols, cur_stream());
}
static void layernorm_fwd(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& b, Tensor& y, Tensor& mean,
                          Tensor& rstd, double eps) {
  need(x, "x", at::kBFloat16); need(y, "y", at::kBFloat16, x.numel());
  int cols = x.size(-1), rows = x.numel() / std::max(cols, 1);
  TORCH_CHECK(cols % 8 == 0, "layernorm_fwd needs cols % 8 == 0");
  need(w, "w", at::kBFloat16, cols); need_opt(b, "b", at::kBFloat16, cols);
  need(mean, "mean", at::kFloat, rows); need(rstd, "rstd", at::kFloat, rows);
  dfb::layernorm_fwd(x.data_ptr(), w.data_ptr(), optp(b), y.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(),
                     rows, cols, (float)eps, cur_stream());
}
static void layernorm_apply(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& b, const Tensor& mean,
                            const Tensor& rstd, Tensor& y) {
  need(x, "x", at::kBFloat16); need(y, "y", at::kBFloat16, x.numel());
  int cols = x.size(-1), rows = x.numel() / std::max(cols, 1);
  TORCH_CHECK(cols % 8 == 0, "layernorm_apply needs cols % 8 == 0");
  need(w, "w", at::kBFloat16, cols); need_opt(b, "b", at::kBFloat16, cols);
  need(mean, "mean", at::kFloat, rows); need(rstd, "rstd", at::kFloat, rows);
  dfb::layernorm_apply(x.data_ptr(), w.data_ptr(), optp(b), mean.data_ptr<float>(), rstd.data_ptr<float>(), y.data_ptr(),
                       rows, cols, cur_stream());
}
static void layernorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& mean, const Tensor& rstd,
                          Tensor& dx, const c10::optional<Tensor>& dx_add, c10::optional<Tensor> dw,
                          c10::optional<Tensor> db, bool accumulate, Tensor& partial) {
  need(x, "x", at::kBFloat16); need(dy, "dy", at::kBFloat16, x.numel()); need(dx, "dx", at::kBFloat16, x.numel());
  need_opt(dx_add, "dx_add", at::kBFloat16, x.numel());
  int cols = x.size(-1), rows = x.numel() / std::max(cols, 1);
  TORCH_CHECK(cols % 8 == 0, "layernorm_bwd needs cols % 8 == 0");
  need(w, "w", at::kBFloat16, cols); need(mean, "mean", at::kFloat, rows); need(rstd, "rstd", at::kFloat, rows);
  need(partial, "partial", at::kFloat);
  if (dw.has_value()) need_grad(*dw, "dw", cols);
  if (db.has_value()) {
    need_grad(*db, "db", cols);
    TORCH_CHECK(dw.has_value() && db->scalar_type() == dw->scalar_type(), "layernorm_bwd: db needs dw of the same dtype");
  }
  TORCH_CHECK(partial.numel() >= (int64_t)dfb::norm_bwd_parts(rows) * 2 * cols, "layernorm_bwd scratch too small");
  dfb::layernorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(),
                     dx.data_ptr(), optp(dx_add), dw.has_value() ? dw->data_ptr() : nullptr,
                     db.has_value() ? db->data_ptr() : nullptr, dw.has_value() && dw->scalar_type() == at::kFloat,
                     accumulate, partial.data_ptr<float>(), rows, cols, cur_stream());
}
static int64_t norm_bwd_scratch_elems(int64_t rows, int64_t cols) { return (int64_t)dfb::norm_bwd_parts((int)rows) * 2 * cols; }

// ---------------------------------------------------------------- pointwise
static void rope_inplace(Tensor& x, const Tensor& positions, int64_t heads, int64_t rot_dim, int64_t row_stride,
                         int64_t head_stride, int64_t col_base, double theta, bool backward) {
  CHECK_CUDA(x); CHECK_BF16(x); CHECK_I32(positions);
  int tokens = positions.numel();
  dfb::rope_inplace(x.data_ptr(), positions.data_ptr<int>(), tokens, (int)heads, (int)rot_dim, row_stride, (int)head_stride,
                    (int)col_base, (float)theta, backward, cur_stream());
}
static void swiglu_fwd(const Tensor& x1, const Tensor& x3, Tensor& out, int64_t rows, int64_t F, int64_t ld1, int64_t ld3) {
  CHECK_BF16(x1); CHECK_BF16(out); TORCH_CHECK(F % 8 == 0 && ld1 % 8 == 0 && ld3 % 8 == 0, "swiglu: dims must be multiples of 8");
  dfb::swiglu_fwd(x1.data_ptr(), x3.data_ptr(), out.data_ptr(), rows, (int)F, ld1, ld3, cur_stream());
}
static void swiglu_bwd(const Tensor& ds, const Tensor& x1, const Tensor& x3, Tensor& dx1, Tensor& dx3, int64_t rows,
                       int64_t F, int64_t ld1, int64_t ld3, int64_t ldd1, int64_t ldd3, c10::optional<Tensor> s_out) {
  TORCH_CHECK(F % 8 == 0, "swiglu: F must be a multiple of 8");
  void* sp = nullptr;
  if (s_out.has_value()) {
    CHECK_BF16(s_out.value());
    TORCH_CHECK(s_out->is_contiguous() && s_out->numel() == rows * F, "swiglu_bwd: s_out is a contiguous (rows, F) bf16 tensor");
    sp = s_out->data_ptr();
  }
  dfb::swiglu_bwd(ds.data_ptr(), x1.data_ptr(), x3.data_ptr(), dx1.data_ptr(), dx3.data_ptr(), sp, rows, (int)F, ld1, ld3, ldd1,
                  ldd3, cur_stream());
}
static void gelu_fwd(const Tensor& x, Tensor& y) {
  need(x, "x", at::kBFloat16); need(y, "y", at::kBFloat16, x.numel());
  TORCH_CHECK(x.numel() % 8 == 0, "gelu_fwd needs numel % 8 == 0");
  dfb::gelu_fwd(x.data_ptr(), y.data_ptr(), x.numel(), cur_stream());
}
static void gelu_bwd(const Tensor& dy, const Tensor& x, Tensor& dx) {
  need(x, "x", at::kBFloat16); need(dy, "dy", at::kBFloat16, x.numel()); need(dx, "dx", at::kBFloat16, x.numel());
  TORCH_CHECK(x.numel() % 8 == 0, "gelu_bwd needs numel % 8 == 0");
  dfb::gelu_bwd(dy.data_ptr(), x.data_ptr(), dx.data_ptr(), x.numel(), cur_stream());
}
static void add_bf16(const Tensor& a, const Tensor& b, Tensor& out) {
  need(a, "a", at::kBFloat16); need(b, "b", at::kBFloat16, a.numel()); need(out, "out", at::kBFloat16, a.numel());
  TORCH_CHECK(a.numel() % 8 == 0, "add_bf16 needs numel % 8 == 0");
  dfb::add_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), cur_stream());
}
static void colsum_bf16(const Tensor& x, Tensor& partial, Tensor& out, bool accumulate) {
  CHECK_BF16(x); CHECK_CONTIG(x); CHECK_F32(partial);
  int cols = x.size(-1), rows = x.numel() / std::max(cols, 1);
  TORCH_CHECK(partial.numel() >= (int64_t)dfb::colsum_parts(rows) * cols, "colsum scratch too small");
  dfb::colsum_bf16(x.data_ptr(), partial.data_ptr<float>(), out.data_ptr(), accumulate, rows, cols, cur_stream());
}
static void adamw_bf16(Tensor& w, const Tensor& g, Tensor& m, Tensor& v, double lr, double b1, double b2, double eps,
                       double wd, int64_t step, double gscale) {
  need(w, "w", at::kBFloat16); need(m, "m", at::kBFloat16, w.numel()); need(v, "v", at::kBFloat16, w.numel());
  need_grad(g, "g", w.numel());
  dfb::adamw_bf16(w.data_ptr(), g.data_ptr(), g.scalar_type() == at::kFloat, m.data_ptr(), v.data_ptr(), w.numel(), lr, b1,
                  b2, eps, wd, (int)step, gscale, cur_stream());
}
static void adamw_master(Tensor& master, Tensor& w_out, const Tensor& g, Tensor& m, Tensor& v, double lr, double b1,
                         double b2, double eps, double wd, int64_t step, double gscale) {
  need(master, "master", at::kFloat); need(w_out, "w_out", at::kBFloat16, master.numel());
  need(m, "m", at::kFloat, master.numel()); need(v, "v", at::kFloat, master.numel()); need_grad(g, "g", master.numel());
  dfb::adamw_master(master.data_ptr<float>(), w_out.data_ptr(), g.data_ptr(), g.scalar_type() == at::kFloat,
                    m.data_ptr<float>(), v.data_ptr<float>(), master.numel(), lr, b1, b2, eps, wd, (int)step, gscale,
                    cur_stream());
}
static void adamw_split(Tensor& w, Tensor& lo, const Tensor& g, Tensor& m, Tensor& v, double lr, double b1, double b2,
                        double eps, double wd, int64_t step, double gscale) {
  TORCH_CHECK(w.scalar_type() == at::kBFloat16 && (g.scalar_type() == at::kBFloat16 || g.scalar_type() == at::kFloat) &&
              m.scalar_type() == at::kBFloat16 && v.scalar_type() == at::kBFloat16 && lo.element_size() == 2,
              "adamw_split: bf16 w/m/v, bf16 or fp32 g, and a 16-bit lo plane");
  TORCH_CHECK(lo.numel() == w.numel() && g.numel() == w.numel() && m.numel() == w.numel() && v.numel() == w.numel(),
              "adamw_split: size mismatch");
  int rc = dfb::adamw_split(w.data_ptr(), lo.data_ptr(), g.data_ptr(), g.scalar_type() == at::kFloat, m.data_ptr(), v.data_ptr(),
                            w.numel(), lr, b1, b2, eps, wd, (int)step, gscale, cur_stream());
  TORCH_CHECK(rc == 0, "adamw_split: arrays must be 16-byte aligned (code ", rc, ")");
}
static void adamw_f32(Tensor& w, const Tensor& g, Tensor& m, Tensor& v, double lr, double b1, double b2, double eps,
                      double wd, int64_t step, double gscale) {
  need(w, "w", at::kFloat); need(g, "g", at::kFloat, w.numel()); need(m, "m", at::kFloat, w.numel());
  need(v, "v", at::kFloat, w.numel());
  dfb::adamw_f32(w.data_ptr<float>(), g.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), w.numel(), lr, b1, b2,
                 eps, wd, (int)step, gscale, cur_stream());
}
static void sgd_bf16(Tensor& w, const Tensor& g, c10::optional<Tensor> m, double lr, double mu, double wd) {
  CHECK_CUDA(w); CHECK_BF16(w); CHECK_BF16(g);
  if (m.has_value()) CHECK_BF16((*m));
  TORCH_CHECK(g.numel() == w.numel() && (!m.has_value() || m->numel() == w.numel()), "sgd_bf16: extents differ");
  dfb::sgd_bf16(w.data_ptr(), g.data_ptr(), m.has_value() ? m->data_ptr() : nullptr, w.numel(), lr, mu, wd, cur_stream());
}

// ---------------------------------------------------------------- loss / embedding
static void ce_loss_fwd_bwd(Tensor& logits, const Tensor& targets, Tensor& nll_rows, c10::optional<Tensor> loss,
                            bool accumulate, double scale) {
  CHECK_CUDA(logits); CHECK_BF16(logits); CHECK_I32(targets); CHECK_F32(nll_rows);
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && logits.stride(0) % 8 == 0, "logits must be (rows, vocab), row stride % 8 == 0");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(logits.data_ptr()) & 15) == 0, "logits must be 16-byte aligned");
  TORCH_CHECK(targets.is_contiguous() && targets.numel() == logits.size(0), "targets: one int32 per logits row");
  TORCH_CHECK(nll_rows.is_contiguous() && nll_rows.numel() >= logits.size(0), "nll_rows: one fp32 per logits row");
  need_opt(loss, "loss", at::kFloat);
  dfb::ce_loss_fwd_bwd(logits.data_ptr(), targets.data_ptr<int>(), nll_rows.data_ptr<float>(),
                       loss.has_value() ? loss->data_ptr<float>() : nullptr, accumulate, logits.size(0), logits.size(1),
                       logits.stride(0), (float)scale, cur_stream());
}
static void embed_fwd(const Tensor& tok, const Tensor& table, Tensor& out, const c10::optional<Tensor>& positions,
                      const c10::optional<Tensor>& pos_table) {
  CHECK_I32(tok); CHECK_CONTIG(tok); need(table, "table", at::kBFloat16);
  TORCH_CHECK(table.dim() == 2, "table must be (vocab, d)");
  int d = table.size(1);
  TORCH_CHECK(d % 8 == 0, "embedding width must be a multiple of 8");
  need(out, "out", at::kBFloat16, tok.numel() * (int64_t)d);
  int pos_rows = 0;
  if (pos_table.has_value()) {
    need(*pos_table, "pos_table", at::kBFloat16);
    TORCH_CHECK(pos_table->dim() == 2 && pos_table->size(1) == d && positions.has_value(), "pos_table must be (positions, d) and come with positions");
    CHECK_I32(*positions);
    TORCH_CHECK(positions->is_contiguous() && positions->numel() == tok.numel(), "positions: one int32 per token");
    pos_rows = pos_table->size(0);
  }
  dfb::embed_fwd(tok.data_ptr<int>(), table.data_ptr(), out.data_ptr(), tok.numel(), d, (int)table.size(0),
                 pos_table.has_value() ? positions->data_ptr<int>() : nullptr, optp(pos_table), pos_rows, cur_stream());
}
static void embed_bwd_sorted(const Tensor& sorted_key, const Tensor& order, const Tensor& dy, Tensor& dtable, bool accumulate) {
  CHECK_I32(sorted_key); CHECK_I32(order); CHECK_CONTIG(sorted_key); CHECK_CONTIG(order); need(dy, "dy", at::kBFloat16);
  int d = dy.size(-1);
  TORCH_CHECK(d % 8 == 0, "embed_bwd_sorted needs a width that is a multiple of 8");
  TORCH_CHECK(order.numel() == sorted_key.numel() && dy.numel() == sorted_key.numel() * (int64_t)d, "embed_bwd_sorted: one dy row per key");
  TORCH_CHECK(dtable.is_cuda() && dtable.is_contiguous() && dtable.dim() == 2 && dtable.size(1) == d &&
              (dtable.scalar_type() == at::kFloat || dtable.scalar_type() == at::kBFloat16) &&
              (reinterpret_cast<uintptr_t>(dtable.data_ptr()) & 15) == 0, "dtable must be a contiguous, 16-byte aligned (vocab, d) bf16 or fp32 CUDA tensor");
  dfb::embed_bwd_sorted(sorted_key.data_ptr<int>(), order.data_ptr<int>(), dy.data_ptr(), dtable.data_ptr(),
                        dtable.scalar_type() == at::kFloat, sorted_key.numel(), d, (int)dtable.size(0), accumulate, cur_stream());
}

// ---------------------------------------------------------------- GEMM
// D(M,N) = op(A) * op(B) (+ addend) (+ bias).  A is (M,K) row-major, or (K,M) row-major when a_mn.
// B is (N,K) row-major, or (K,N) row-major when b_mn.
static void gemm_bf16(const Tensor& A, bool a_mn, const Tensor& B, bool b_mn, Tensor& D,
                      const c10::optional<Tensor>& addend, const c10::optional<Tensor>& bias) {
  CHECK_CUDA(A); CHECK_BF16(A); CHECK_BF16(B);
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && D.dim() == 2, "gemm operands must be 2-D");
  TORCH_CHECK(A.stride(1) == 1 && B.stride(1) == 1 && D.stride(1) == 1, "gemm operands must have unit inner stride");
  int M = a_mn ? A.size(1) : A.size(0), K = a_mn ? A.size(0) : A.size(1);
  int N = b_mn ? B.size(1) : B.size(0), Kb = b_mn ? B.size(0) : B.size(1);
  TORCH_CHECK(K == Kb, "gemm reduction dims differ: ", K, " vs ", Kb);
  TORCH_CHECK(D.size(0) == M && D.size(1) == N, "gemm output shape mismatch");
  bool d32 = D.scalar_type() == at::kFloat;
  TORCH_CHECK(d32 || D.scalar_type() == at::kBFloat16, "gemm output must be bf16 or fp32");
  bool a32 = false;
  long long ld_add = 0;
  if (addend.has_value()) {
    a32 = addend->scalar_type() == at::kFloat;
    TORCH_CHECK(addend->stride(1) == 1 && addend->size(0) == M && addend->size(1) == N, "addend shape mismatch");
    ld_add = addend->stride(0);
  }
  if (bias.has_value()) { CHECK_BF16(*bias); TORCH_CHECK(bias->numel() == N, "bias length mismatch"); }
  int rc = dfb::gemm_bf16(A.data_ptr(), A.stride(0), a_mn, B.data_ptr(), B.stride(0), b_mn, D.data_ptr(), D.stride(0), d32,
                          optp(addend), ld_add, a32, optp(bias), M, N, K, num_sms(), cur_stream());
  TORCH_CHECK(rc == 0, "gemm_bf16 launch failed with code ", rc);
}
static int64_t gemm_last_error() { return dfb::gemm_bf16_last_error(); }

// ---------------------------------------------------------------- fused DP communication
static void zero_rs_adamw(std::vector<int64_t> slabs, std::vector<int64_t> ctrls, int64_t rank, int64_t slots, int64_t slot,
                          int64_t seq, int64_t ack_expect, int64_t grad_ptr, int64_t slice_begin, int64_t slice_len,
                          c10::optional<Tensor> master, Tensor& m, Tensor& v, int64_t shard_ptr,
                          std::vector<int64_t> fbegin, std::vector<int64_t> fend, std::vector<double> fwd, double lr,
                          double b1, double b2, double eps, int64_t step, double gscale, double timeout_s, Tensor& err,
                          Tensor& done_ctr) {
  int world = slabs.size();
  std::vector<unsigned long long> sl(slabs.begin(), slabs.end()), ct(ctrls.begin(), ctrls.end());
  std::vector<long long> fb(fbegin.begin(), fbegin.end()), fe(fend.begin(), fend.end());
  std::vector<float> fw(fwd.begin(), fwd.end());
  CHECK_F32(m); CHECK_F32(v); CHECK_I32(err); CHECK_I32(done_ctr);
  int rc = dfb::zero_rs_adamw(sl.data(), ct.data(), rank, world, slots, slot, (unsigned)seq, (unsigned)ack_expect,
                              reinterpret_cast<const void*>(grad_ptr), slice_begin, slice_len,
                              master.has_value() ? master->data_ptr<float>() : nullptr, m.data_ptr<float>(),
                              v.data_ptr<float>(), reinterpret_cast<void*>(shard_ptr), fb.data(), fe.data(), fw.data(),
                              fb.size(), lr, b1, b2, eps, step, gscale, timeout_s, err.data_ptr<int>(),
                              reinterpret_cast<unsigned int*>(done_ctr.data_ptr<int>()), num_sms(), cur_stream());
  TORCH_CHECK(rc == 0, "zero_rs_adamw launch failed with code ", rc);
}
// Reduce-scatter + fp32 accumulate of one packed gradient object into this rank's slice (no optimizer step).
static void zero_rs_accum(std::vector<int64_t> slabs, std::vector<int64_t> ctrls, int64_t rank, int64_t slots, int64_t slot,
                          int64_t seq, int64_t ack_expect, int64_t grad_ptr, int64_t slice_begin, int64_t slice_len,
                          Tensor& gacc, bool first, double timeout_s, Tensor& err, Tensor& done_ctr) {
  int world = slabs.size();
  std::vector<unsigned long long> sl(slabs.begin(), slabs.end()), ct(ctrls.begin(), ctrls.end());
  CHECK_F32(gacc); CHECK_I32(err); CHECK_I32(done_ctr);
  TORCH_CHECK(gacc.numel() >= slice_len, "zero_rs_accum: accumulator holds ", gacc.numel(), " elements, the slice has ", slice_len);
  int rc = dfb::zero_rs_adamw(sl.data(), ct.data(), rank, world, slots, slot, (unsigned)seq, (unsigned)ack_expect,
                              reinterpret_cast<const void*>(grad_ptr), slice_begin, slice_len, nullptr, nullptr, nullptr,
                              nullptr, nullptr, nullptr, nullptr, 0, 0.f, 0.9f, 0.95f, 1e-8f, 1, 1.f, timeout_s,
                              err.data_ptr<int>(), reinterpret_cast<unsigned int*>(done_ctr.data_ptr<int>()), num_sms(),
                              cur_stream(), gacc.data_ptr<float>(), first ? 1 : 0);
  TORCH_CHECK(rc == 0, "zero_rs_accum launch failed with code ", rc);
}
static void param_gather(std::vector<int64_t> slabs, std::vector<int64_t> ctrls, int64_t rank, int64_t slots, int64_t slot,
                         int64_t seq, int64_t ack_expect, int64_t shard_ptr, int64_t full_ptr, int64_t per_bytes,
                         int64_t total_bytes, double timeout_s, Tensor& err, Tensor& done_ctr) {
  int world = slabs.size();
  std::vector<unsigned long long> sl(slabs.begin(), slabs.end()), ct(ctrls.begin(), ctrls.end());
  int rc = dfb::param_gather(sl.data(), ct.data(), rank, world, slots, slot, (unsigned)seq, (unsigned)ack_expect,
                             reinterpret_cast<const void*>(shard_ptr), reinterpret_cast<void*>(full_ptr), per_bytes,
                             total_bytes, timeout_s, err.data_ptr<int>(),
                             reinterpret_cast<unsigned int*>(done_ctr.data_ptr<int>()), num_sms(), cur_stream());
  TORCH_CHECK(rc == 0, "param_gather launch failed with code ", rc);
}

static void param_gather_dma(std::vector<int64_t> slabs, std::vector<int64_t> ctrls, int64_t rank, int64_t slots, int64_t slot,
                             int64_t seq, int64_t ack_expect, int64_t shard_ptr, std::vector<int64_t> expect_off, int64_t full_ptr,
                             int64_t per_bytes, int64_t total_bytes, double timeout_s, Tensor& err) {
  int world = slabs.size();
  TORCH_CHECK((int)expect_off.size() == world && (int)ctrls.size() == world, "param_gather_dma: one offset and one control block per rank");
  need(err, "err", at::kInt, 1);
  std::vector<unsigned long long> sl(slabs.begin(), slabs.end()), ct(ctrls.begin(), ctrls.end()), eo(expect_off.begin(), expect_off.end());
  int rc = dfb::param_gather_dma(sl.data(), ct.data(), rank, world, slots, slot, (unsigned)seq, (unsigned)ack_expect,
                                 reinterpret_cast<const void*>(shard_ptr), eo.data(), reinterpret_cast<void*>(full_ptr), per_bytes,
                                 total_bytes, timeout_s, err.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "param_gather_dma failed with code ", rc);
}

// ---------------------------------------------------------------- mixture of experts
static int mode_id(const std::string& mode) {
  if (mode == "topk_then_softmax") return 0;
  if (mode == "softmax_then_topk") return 1;
  TORCH_CHECK(false, "unknown routing mode ", mode);
}
static void moe_sort(const Tensor& ids, int64_t E, int64_t tile_rows, Tensor& row_of, Tensor& row_src, Tensor& offsets_pad,
                     Tensor& tile_expert, Tensor& counts, Tensor& scratch) {
  TORCH_CHECK(ids.dim() == 2, "moe_sort: route ids (t, K)");
  const int64_t t = ids.size(0), K = ids.size(1), n = t * K, mp = row_src.numel();
  need(ids, "route_ids", at::kInt, n);
  need(row_of, "row_of", at::kInt, n);
  need(row_src, "row_src", at::kInt);
  need(offsets_pad, "offsets_pad", at::kInt, E + 1);
  need(tile_expert, "tile_expert", at::kInt, mp / tile_rows);
  need(counts, "counts", at::kInt, E);
  need(scratch, "scratch", at::kInt, ((n + 1023) / 1024) * E);
  TORCH_CHECK(mp % tile_rows == 0 && mp >= (n + tile_rows - 1) / tile_rows * tile_rows + E * tile_rows, "moe_sort: row_src too small for the padded layout");
  int rc = dfb::moe_sort(ids.data_ptr<int>(), (int)t, (int)K, (int)E, (int)tile_rows, (int)mp, row_of.data_ptr<int>(), row_src.data_ptr<int>(),
                         offsets_pad.data_ptr<int>(), tile_expert.data_ptr<int>(), counts.data_ptr<int>(), scratch.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "moe_sort: unsupported shape (1 <= E <= 1024), code ", rc);
}
static void moe_topk_softmax(const Tensor& logits, Tensor& route_w, Tensor& route_ids, const std::string& mode) {
  CHECK_F32(route_w); CHECK_I32(route_ids);
  TORCH_CHECK(logits.dim() == 2 && logits.is_contiguous(), "logits must be a contiguous (t, E) matrix");
  int rc = dfb::moe_topk_softmax(logits.data_ptr(), logits.scalar_type() == at::kFloat, route_w.data_ptr<float>(),
                                 route_ids.data_ptr<int>(), logits.size(0), logits.size(1), route_w.size(1), mode_id(mode), cur_stream());
  TORCH_CHECK(rc == 0, "moe_topk_softmax: unsupported shape (E <= 1024, K <= 16), code ", rc);
}
static void moe_router_bwd(const Tensor& dprob, const Tensor& route_w, const Tensor& route_ids, const Tensor& logits,
                           Tensor& dlogits, const std::string& mode) {
  CHECK_F32(dprob); CHECK_F32(route_w); CHECK_I32(route_ids); CHECK_F32(dlogits);
  int rc = dfb::moe_router_bwd(dprob.data_ptr<float>(), route_w.data_ptr<float>(), route_ids.data_ptr<int>(), logits.data_ptr(),
                               logits.scalar_type() == at::kFloat, dlogits.data_ptr<float>(), logits.size(0), logits.size(1),
                               route_w.size(1), mode_id(mode), cur_stream());
  TORCH_CHECK(rc == 0, "moe_router_bwd failed with code ", rc);
}
static void moe_dispatch(const Tensor& x, const Tensor& row_src, Tensor& xp) {
  CHECK_BF16(x); CHECK_BF16(xp); CHECK_I32(row_src);
  int rc = dfb::moe_dispatch(x.data_ptr(), x.stride(0), row_src.data_ptr<int>(), xp.data_ptr(), xp.size(0), xp.size(1), cur_stream());
  TORCH_CHECK(rc == 0, "moe_dispatch: the row width must be a multiple of 8 (code ", rc, ")");
}
static void moe_combine(c10::optional<Tensor> base, const Tensor& yp, const Tensor& route_w, const Tensor& row_of, Tensor& out) {
  CHECK_BF16(yp); CHECK_BF16(out); CHECK_F32(route_w); CHECK_I32(row_of);
  int rc = dfb::moe_combine(base.has_value() ? base->data_ptr() : nullptr, yp.data_ptr(), route_w.data_ptr<float>(),
                            row_of.data_ptr<int>(), out.data_ptr(), out.size(0), out.size(1), row_of.size(1), cur_stream());
  TORCH_CHECK(rc == 0, "moe_combine failed with code ", rc);
}
static void moe_dispatch_bwd(const Tensor& dxp, const Tensor& row_of, Tensor& out, bool accumulate) {
  CHECK_BF16(dxp); CHECK_BF16(out); CHECK_I32(row_of);
  int rc = dfb::moe_dispatch_bwd(dxp.data_ptr(), row_of.data_ptr<int>(), out.data_ptr(), out.size(0), out.size(1), row_of.size(1),
                                 accumulate, cur_stream());
  TORCH_CHECK(rc == 0, "moe_dispatch_bwd failed with code ", rc);
}
static void moe_scale_rows(Tensor& xp, const Tensor& route_w, const Tensor& row_of) {
  CHECK_BF16(xp); CHECK_F32(route_w); CHECK_I32(row_of);
  int rc = dfb::moe_scale_rows(xp.data_ptr(), route_w.data_ptr<float>(), row_of.data_ptr<int>(), row_of.numel(), xp.size(1), cur_stream());
  TORCH_CHECK(rc == 0, "moe_scale_rows failed with code ", rc);
}
static void moe_rowdot(const Tensor& a, const Tensor& b, const Tensor& row_of, Tensor& out) {
  CHECK_BF16(a); CHECK_BF16(b); CHECK_I32(row_of); CHECK_F32(out);
  int rc = dfb::moe_rowdot(a.data_ptr(), b.data_ptr(), row_of.data_ptr<int>(), out.data_ptr<float>(), row_of.numel(), a.size(1), cur_stream());
  TORCH_CHECK(rc == 0, "moe_rowdot failed with code ", rc);
}
static void moe_grouped_mm(const Tensor& x, const Tensor& w, Tensor& y, const Tensor& tile_expert, bool w_kn) {
  CHECK_BF16(x); CHECK_BF16(w); CHECK_BF16(y); CHECK_I32(tile_expert);
  TORCH_CHECK(x.is_contiguous() && w.is_contiguous() && y.is_contiguous(), "moe_grouped_mm: contiguous operands");
  const int64_t K = x.size(1), N = y.size(1);
  TORCH_CHECK(w.dim() == 3 && (w_kn ? (w.size(1) == K && w.size(2) == N) : (w.size(1) == N && w.size(2) == K)), "moe_grouped_mm: weight shape");
  TORCH_CHECK(tile_expert.numel() * 256 >= x.size(0), "moe_grouped_mm: tile_expert too short");
  int rc = dfb::moe_grouped_mm(x.data_ptr(), w.data_ptr(), y.data_ptr(), tile_expert.data_ptr<int>(), x.size(0), N, K, w.size(0), w_kn,
                               num_sms(), cur_stream());
  TORCH_CHECK(rc == 0, "moe_grouped_mm launch failed with code ", rc);
}
static void moe_grouped_wgrad(const Tensor& x, const Tensor& dy, Tensor& dw, const Tensor& offsets_pad, bool accumulate) {
  CHECK_BF16(x); CHECK_BF16(dy); CHECK_BF16(dw); CHECK_I32(offsets_pad);
  TORCH_CHECK(x.is_contiguous() && dy.is_contiguous() && dw.is_contiguous(), "moe_grouped_wgrad: contiguous operands");
  int rc = dfb::moe_grouped_wgrad(x.data_ptr(), dy.data_ptr(), dw.data_ptr(), offsets_pad.data_ptr<int>(), x.size(0), x.size(1),
                                  dy.size(1), dw.size(0), accumulate, num_sms(), cur_stream());
  TORCH_CHECK(rc == 0, "moe_grouped_wgrad launch failed with code ", rc);
}

// ---------------------------------------------------------------- tensor-parallel fused GEMMs
static void tp_ag_gemm(std::vector<int64_t> x_src, int64_t x_ld, int64_t gathered_ptr, const Tensor& w, bool b_mn, Tensor& y,
                       int64_t panel_rows, int64_t rank, Tensor& flags, std::vector<int64_t> ready, std::vector<int64_t> acks,
                       int64_t launch_seq, int64_t chunk_rows, double timeout_s, Tensor& err, Tensor& done_ctr) {
  CHECK_BF16(w); CHECK_BF16(y); CHECK_I32(flags); CHECK_I32(err); CHECK_I32(done_ctr);
  int world = x_src.size();
  const int64_t K = b_mn ? w.size(0) : w.size(1), N = b_mn ? w.size(1) : w.size(0);
  TORCH_CHECK(y.size(0) == panel_rows * world && y.size(1) == N, "tp_ag_gemm: y must be (world * panel_rows, N)");
  std::vector<unsigned long long> xs(x_src.begin(), x_src.end()), rd(ready.begin(), ready.end()), ak(acks.begin(), acks.end());
  int rc = dfb::tp_ag_gemm(xs.data(), x_ld, reinterpret_cast<void*>(gathered_ptr), w.data_ptr(), w.stride(0), b_mn, y.data_ptr(),
                           y.stride(0), panel_rows, N, K, rank, world, reinterpret_cast<unsigned int*>(flags.data_ptr<int>()),
                           rd.data(), ak.data(), (unsigned)launch_seq, chunk_rows, timeout_s, err.data_ptr<int>(),
                           reinterpret_cast<unsigned int*>(done_ctr.data_ptr<int>()), num_sms(), cur_stream());
  TORCH_CHECK(rc == 0, "tp_ag_gemm launch failed with code ", rc);
}
static void tp_gemm_rs(const Tensor& x, const Tensor& w, bool b_mn, Tensor& d, c10::optional<Tensor> addend, int64_t panel_rows,
                       int64_t rank, std::vector<int64_t> stage, std::vector<int64_t> tile_flags, int64_t launch_seq,
                       double timeout_s, Tensor& err, Tensor& done_ctr) {
  CHECK_BF16(x); CHECK_BF16(w); CHECK_BF16(d); CHECK_I32(err); CHECK_I32(done_ctr);
  int world = stage.size();
  const int64_t K = b_mn ? w.size(0) : w.size(1), N = b_mn ? w.size(1) : w.size(0);
  TORCH_CHECK(x.size(0) == panel_rows * world && x.size(1) == K, "tp_gemm_rs: x must be (world * panel_rows, K)");
  TORCH_CHECK(d.size(0) == panel_rows && d.size(1) == N, "tp_gemm_rs: d must be (panel_rows, N)");
  std::vector<unsigned long long> st(stage.begin(), stage.end()), tf(tile_flags.begin(), tile_flags.end());
  int rc = dfb::tp_gemm_rs(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), b_mn, d.data_ptr(), d.stride(0),
                           addend.has_value() ? addend->data_ptr() : nullptr, addend.has_value() ? addend->stride(0) : 0,
                           panel_rows, N, K, rank, world, st.data(), tf.data(), (unsigned)launch_seq, timeout_s,
                           err.data_ptr<int>(), reinterpret_cast<unsigned int*>(done_ctr.data_ptr<int>()), num_sms(), cur_stream());
  TORCH_CHECK(rc == 0, "tp_gemm_rs launch failed with code ", rc);
}

// ---------------------------------------------------------------- attention
static void flash_fwd(const Tensor& q, const Tensor& k, const Tensor& v, Tensor& out, Tensor& lse, const Tensor& cu_seqlens,
                      int64_t max_seqlen, double scale, const c10::optional<Tensor>& trace) {
  if (trace.has_value())
    TORCH_CHECK(trace->is_cuda() && trace->scalar_type() == at::kLong && trace->is_contiguous() && trace->numel() >= 3 * 32 * 8,
                "flash_fwd: trace is a CUDA int64 tensor of at least 768 elements");
  CHECK_BF16(q); CHECK_BF16(k); CHECK_BF16(v); CHECK_BF16(out); CHECK_F32(lse); CHECK_I32(cu_seqlens);
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3 && out.dim() == 3, "flash_fwd: (tokens, heads, dim) tensors");
  const int64_t T = q.size(0), hq = q.size(1), hd = q.size(2), hkv = k.size(1);
  auto rows_ok = [&](const Tensor& t) { return t.stride(2) == 1 && t.stride(1) == hd; };
  TORCH_CHECK(rows_ok(q) && rows_ok(k) && rows_ok(v) && rows_ok(out), "flash_fwd: heads must be contiguous inside a token row");
  TORCH_CHECK(k.size(0) == T && v.size(0) == T && v.size(1) == hkv && out.size(0) == T && out.size(1) == hq && lse.is_contiguous() &&
              lse.size(0) == hq && lse.size(1) == T, "flash_fwd: shapes");
  int rc = dfb::flash_fwd_sm100(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), out.data_ptr(), out.stride(0),
                                lse.data_ptr<float>(), cu_seqlens.data_ptr<int>(), cu_seqlens.numel() - 1, max_seqlen, T, hq, hkv, hd, scale,
                                cur_stream(), trace.has_value() ? reinterpret_cast<long long*>(trace->data_ptr<int64_t>()) : nullptr);
  TORCH_CHECK(rc == 0, "flash_fwd: unsupported shape or alignment (head_dim must be 128; code ", rc, ")");
}

static void flash_bwd(const Tensor& dout, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out, const Tensor& lse,
                      Tensor& dq, Tensor& dk, Tensor& dv, Tensor& scratch, const Tensor& cu_seqlens, int64_t max_seqlen, double scale,
                      const c10::optional<Tensor>& trace) {
  if (trace.has_value())
    TORCH_CHECK(trace->is_cuda() && trace->scalar_type() == at::kLong && trace->is_contiguous() && trace->numel() >= 3 * 32 * 8,
                "flash_bwd: trace is a CUDA int64 tensor of at least 768 elements");
  CHECK_BF16(dout); CHECK_BF16(q); CHECK_BF16(k); CHECK_BF16(v); CHECK_BF16(out); CHECK_BF16(dq); CHECK_BF16(dk); CHECK_BF16(dv);
  CHECK_F32(lse); CHECK_F32(scratch); CHECK_I32(cu_seqlens);
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3, "flash_bwd: (tokens, heads, dim) tensors");
  const int64_t T = q.size(0), hq = q.size(1), hd = q.size(2), hkv = k.size(1);
  auto like = [&](const Tensor& t, int64_t heads) {
    return t.dim() == 3 && t.size(0) == T && t.size(1) == heads && t.size(2) == hd && t.stride(2) == 1 && t.stride(1) == hd;
  };
  TORCH_CHECK(like(q, hq) && like(dout, hq) && like(out, hq) && like(dq, hq) && like(k, hkv) && like(v, hkv) && like(dk, hkv) && like(dv, hkv),
              "flash_bwd: shapes (heads must be contiguous inside a token row)");
  TORCH_CHECK(lse.is_contiguous() && lse.size(0) == hq && lse.size(1) == T, "flash_bwd: lse is (heads, tokens)");
  TORCH_CHECK(scratch.is_contiguous() && scratch.numel() >= 2 * hq * T, "flash_bwd: scratch holds 2 floats per (head, token)");
  TORCH_CHECK(cu_seqlens.is_contiguous() && cu_seqlens.numel() >= 2, "flash_bwd: cu_seqlens");
  int rc = dfb::flash_bwd_sm100(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), out.data_ptr(), out.stride(0),
                                dout.data_ptr(), dout.stride(0), lse.data_ptr<float>(), dq.data_ptr(), dq.stride(0), dk.data_ptr(),
                                dk.stride(0), dv.data_ptr(), dv.stride(0), scratch.data_ptr(), cu_seqlens.data_ptr<int>(),
                                cu_seqlens.numel() - 1, max_seqlen, T, hq, hkv, hd, scale, cur_stream(),
                                trace.has_value() ? reinterpret_cast<long long*>(trace->data_ptr<int64_t>()) : nullptr);
  TORCH_CHECK(rc == 0, "flash_bwd: unsupported shape or alignment (head_dim must be 128; code ", rc, ")");
}

static Tensor umma_probe(int64_t kind, int64_t n, int64_t count, int64_t nacc) {
  Tensor out = at::zeros({3}, at::TensorOptions().dtype(at::kLong).device(at::kCUDA));
  int rc = dfb::umma_probe((int)kind, (int)n, (int)count, (int)nacc, reinterpret_cast<long long*>(out.data_ptr<int64_t>()), cur_stream());
  TORCH_CHECK(rc == 0, "umma_probe: kind 0..3, n a multiple of 16 up to 256, nacc * n <= 448 (code ", rc, ")");
  return out;
}

// ---------------------------------------------------------------- fp8 lane
static bool is_fp8_or_u8(const Tensor& t) {
  return t.scalar_type() == at::kByte || t.scalar_type() == at::kFloat8_e4m3fn || t.scalar_type() == at::kFloat8_e5m2;
}
static void quant_fp8_rowwise(const Tensor& x, Tensor& q, Tensor& scale) {
  CHECK_BF16(x); CHECK_F32(scale);
  TORCH_CHECK(q.is_cuda() && is_fp8_or_u8(q) && x.dim() == 2 && x.stride(1) == 1 && q.stride(1) == 1 && q.sizes() == x.sizes() &&
              scale.numel() == x.size(0), "quant_fp8_rowwise: x (rows, K) bf16, q (rows, K) fp8, scale (rows)");
  int rc = dfb::quant_fp8_rowwise(x.data_ptr(), x.stride(0), q.data_ptr(), q.stride(0), scale.data_ptr<float>(), x.size(0), x.size(1), cur_stream());
  TORCH_CHECK(rc == 0, "quant_fp8_rowwise: K and the row strides must be multiples of 8 (code ", rc, ")");
}
static void gemm_fp8(const Tensor& a, const Tensor& b, Tensor& d, c10::optional<Tensor> row_scale, c10::optional<Tensor> col_scale,
                     c10::optional<Tensor> addend, c10::optional<Tensor> bias) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && d.is_cuda() && is_fp8_or_u8(a) && is_fp8_or_u8(b), "gemm_fp8: fp8 CUDA operands");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && a.size(1) == b.size(1) && d.size(0) == a.size(0) &&
              d.size(1) == b.size(0) && d.stride(1) == 1, "gemm_fp8: a (M, K), b (N, K), d (M, N)");
  const bool f32 = d.scalar_type() == at::kFloat;
  TORCH_CHECK(f32 || d.scalar_type() == at::kBFloat16, "gemm_fp8: d is bf16 or fp32");
  if (row_scale.has_value()) { CHECK_F32((*row_scale)); TORCH_CHECK(row_scale->numel() == a.size(0), "row_scale has M entries"); }
  if (col_scale.has_value()) { CHECK_F32((*col_scale)); TORCH_CHECK(col_scale->numel() == b.size(0), "col_scale has N entries"); }
  if (addend.has_value()) TORCH_CHECK(addend->is_cuda() && addend->scalar_type() == d.scalar_type() && addend->sizes() == d.sizes(), "addend like d");
  if (bias.has_value()) CHECK_BF16((*bias));
  auto fmt = [](const Tensor& t) { return t.scalar_type() == at::kFloat8_e5m2 ? 1 : 0; };
  int rc = dfb::gemm_fp8_2sm(a.data_ptr(), a.stride(0), fmt(a), b.data_ptr(), b.stride(0), fmt(b), d.data_ptr(), d.stride(0), f32,
                             row_scale.has_value() ? row_scale->data_ptr<float>() : nullptr,
                             col_scale.has_value() ? col_scale->data_ptr<float>() : nullptr,
                             addend.has_value() ? addend->data_ptr() : nullptr, addend.has_value() ? addend->stride(0) : 0,
                             bias.has_value() ? bias->data_ptr() : nullptr, a.size(0), b.size(0), a.size(1), num_sms(), cur_stream());
  TORCH_CHECK(rc == 0, "gemm_fp8 failed with code ", rc);
}

// ---------------------------------------------------------------- sparse-attention indexer
// q (n, H, D) bf16, k (n, D) bf16, wgt (n, H) fp32, seg_start (n,) int32; out (q1 - q0, ld) fp32
static void dsa_index_scores(const Tensor& q, const Tensor& k, const Tensor& wgt, const Tensor& seg_start, Tensor& out, int64_t q0,
                             int64_t q1, int64_t key_lo) {
  TORCH_CHECK(q.dim() == 3 && k.dim() == 2 && out.dim() == 2, "dsa_index_scores: q (n, H, D), k (n, D), out (rows, ld)");
  const int64_t n = q.size(0), H = q.size(1), D = q.size(2);
  need(q, "q", at::kBFloat16, n * H * D);
  need(k, "k", at::kBFloat16, n * D);
  need(wgt, "wgt", at::kFloat, n * H);
  need(seg_start, "seg_start", at::kInt, n);
  need(out, "out", at::kFloat);
  TORCH_CHECK(D == 64 || D == 128, "dsa_index_scores: index head dim 64 or 128 (got ", D, ")");
  TORCH_CHECK(0 <= key_lo && key_lo <= q0 && q0 < q1 && q1 <= n, "dsa_index_scores: 0 <= key_lo <= q0 < q1 <= n");
  TORCH_CHECK(out.size(0) >= q1 - q0 && out.size(1) >= q1 - key_lo, "dsa_index_scores: out too small");
  int rc = dfb::dsa_index_scores(q.data_ptr(), H * D, k.data_ptr(), D, wgt.data_ptr<float>(), seg_start.data_ptr<int>(), out.data_ptr<float>(),
                                 out.size(1), (int)n, (int)H, (int)D, (int)q0, (int)q1, (int)key_lo, nullptr, cur_stream());
  TORCH_CHECK(rc == 0, "dsa_index_scores failed with code ", rc);
}
// scores (rows, ld) fp32, the first ``cols`` entries of every row are ranked; sel (rows, >= k) int32
static void dsa_topk_rows(const Tensor& scores, int64_t rows, int64_t cols, int64_t col_base, int64_t k, Tensor& sel) {
  need(scores, "scores", at::kFloat);
  need(sel, "sel", at::kInt);
  TORCH_CHECK(scores.dim() == 2 && sel.dim() == 2, "dsa_topk_rows: 2-D tensors");
  TORCH_CHECK(rows <= scores.size(0) && cols <= scores.size(1) && rows <= sel.size(0) && k <= sel.size(1) && k > 0 && cols > 0,
              "dsa_topk_rows: sizes");
  int rc = dfb::dsa_topk_rows(scores.data_ptr<float>(), scores.size(1), (int)rows, (int)cols, (int)col_base, (int)k, sel.data_ptr<int>(),
                              (int)sel.size(1), cur_stream());
  TORCH_CHECK(rc == 0, "dsa_topk_rows failed with code ", rc);
}

// ---------------------------------------------------------------- sequence-mixing helpers
static void l2norm_fwd(const Tensor& x, Tensor& y, Tensor& rstd, double eps) {
  CHECK_CUDA(x); CHECK_BF16(x); CHECK_BF16(y); CHECK_F32(rstd);
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous(), "l2norm_fwd: contiguous tensors");
  int rc = dfb::l2norm_fwd(x.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), x.numel() / x.size(-1), x.size(-1), eps, cur_stream());
  TORCH_CHECK(rc == 0, "l2norm_fwd failed with code ", rc);
}
static void l2norm_bwd(const Tensor& dy, const Tensor& x, const Tensor& rstd, Tensor& dx) {
  CHECK_CUDA(x); CHECK_BF16(x); CHECK_BF16(dy); CHECK_BF16(dx); CHECK_F32(rstd);
  TORCH_CHECK(x.is_contiguous() && dy.is_contiguous() && dx.is_contiguous(), "l2norm_bwd: contiguous tensors");
  int rc = dfb::l2norm_bwd(dy.data_ptr(), x.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(), x.numel() / x.size(-1), x.size(-1), cur_stream());
  TORCH_CHECK(rc == 0, "l2norm_bwd failed with code ", rc);
}
static void gated_rmsnorm_fwd(const Tensor& x, const Tensor& g, const Tensor& w, Tensor& y, Tensor& rstd, double eps) {
  CHECK_CUDA(x); CHECK_BF16(x); CHECK_BF16(g); CHECK_BF16(w); CHECK_BF16(y); CHECK_F32(rstd);
  TORCH_CHECK(x.is_contiguous() && g.is_contiguous() && y.is_contiguous() && w.numel() == x.size(-1), "gated_rmsnorm_fwd: shapes");
  int rc = dfb::gated_rmsnorm_fwd(x.data_ptr(), g.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), x.numel() / x.size(-1),
                                  x.size(-1), eps, cur_stream());
  TORCH_CHECK(rc == 0, "gated_rmsnorm_fwd failed with code ", rc);
}
static void gated_rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& g, const Tensor& w, const Tensor& rstd, Tensor& dx, Tensor& dg,
                              Tensor& dw_partial) {
  CHECK_CUDA(x); CHECK_BF16(x); CHECK_BF16(g); CHECK_BF16(w); CHECK_BF16(dy); CHECK_BF16(dx); CHECK_BF16(dg); CHECK_F32(rstd); CHECK_F32(dw_partial);
  TORCH_CHECK(x.is_contiguous() && g.is_contiguous() && dy.is_contiguous() && dx.is_contiguous() && dg.is_contiguous() &&
              dw_partial.dim() == 2 && dw_partial.size(1) == x.size(-1), "gated_rmsnorm_bwd: shapes");
  int rc = dfb::gated_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), g.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(), dg.data_ptr(),
                                  dw_partial.data_ptr<float>(), dw_partial.size(0), x.numel() / x.size(-1), x.size(-1), cur_stream());
  TORCH_CHECK(rc == 0, "gated_rmsnorm_bwd failed with code ", rc);
}
static void conv_silu_fwd(const Tensor& x, const Tensor& w, const Tensor& seg_start, Tensor& y) {
  CHECK_CUDA(x); CHECK_BF16(x); CHECK_BF16(w); CHECK_BF16(y); CHECK_I32(seg_start);
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && y.is_contiguous() && w.is_contiguous() && w.size(0) == x.size(1) && seg_start.numel() == x.size(0),
              "conv_silu_fwd: shapes");
  int rc = dfb::conv_silu_fwd(x.data_ptr(), w.data_ptr(), seg_start.data_ptr<int>(), y.data_ptr(), x.size(0), x.size(1), w.size(1), cur_stream());
  TORCH_CHECK(rc == 0, "conv_silu_fwd failed with code ", rc);
}
static void conv_silu_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& seg_start, Tensor& dx, Tensor& dw_partial,
                          int64_t rows_per_block) {
  CHECK_CUDA(x); CHECK_BF16(x); CHECK_BF16(w); CHECK_BF16(dy); CHECK_BF16(dx); CHECK_I32(seg_start); CHECK_F32(dw_partial);
  TORCH_CHECK(x.is_contiguous() && dy.is_contiguous() && dx.is_contiguous() && dw_partial.dim() == 3 && dw_partial.size(1) == x.size(1) &&
              dw_partial.size(2) == w.size(1) && dw_partial.size(0) * rows_per_block >= x.size(0), "conv_silu_bwd: shapes");
  int rc = dfb::conv_silu_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), seg_start.data_ptr<int>(), dx.data_ptr(), dw_partial.data_ptr<float>(),
                              dw_partial.size(0), rows_per_block, x.size(0), x.size(1), w.size(1), cur_stream());
  TORCH_CHECK(rc == 0, "conv_silu_bwd failed with code ", rc);
}
static void router_sigmoid_noaux(const Tensor& logits, const Tensor& bias, Tensor& route_w, Tensor& route_ids, int64_t n_group,
                                 int64_t topk_group, double scaling) {
  CHECK_CUDA(logits); CHECK_BF16(logits); CHECK_F32(bias); CHECK_F32(route_w); CHECK_I32(route_ids);
  TORCH_CHECK(logits.dim() == 2 && logits.is_contiguous() && bias.numel() == logits.size(1) && route_w.size(0) == logits.size(0) &&
              route_ids.sizes() == route_w.sizes(), "router_sigmoid_noaux: shapes");
  int rc = dfb::router_sigmoid_noaux(logits.data_ptr(), bias.data_ptr<float>(), route_w.data_ptr<float>(), route_ids.data_ptr<int>(),
                                     logits.size(0), logits.size(1), route_w.size(1), n_group, topk_group, scaling, cur_stream());
  TORCH_CHECK(rc == 0, "router_sigmoid_noaux failed with code ", rc);
}

// ---------------------------------------------------------------- expert-parallel fused kernels
static void ep_dispatch_mm(std::vector<int64_t> x_src, Tensor& xp, const Tensor& row_src, const Tensor& w, bool transpose_w, Tensor& y,
                           const Tensor& tile_expert, int64_t tokens_per_rank, int64_t rank, Tensor& tile_flags,
                           std::vector<int64_t> ready, std::vector<int64_t> acks, int64_t launch_seq, double timeout_s,
                           Tensor& err, Tensor& done_ctr) {
  CHECK_I32(err);
  CHECK_BF16(xp); CHECK_BF16(w); CHECK_BF16(y); CHECK_I32(row_src); CHECK_I32(tile_expert); CHECK_I32(tile_flags); CHECK_I32(done_ctr);
  const int64_t Mp = xp.size(0), K = xp.size(1), E = w.size(0);
  const int64_t N = transpose_w ? w.size(1) : w.size(2);
  TORCH_CHECK((transpose_w ? w.size(2) : w.size(1)) == K, "ep_dispatch_mm: weight inner extent must match the activations");
  TORCH_CHECK(y.size(0) == Mp && y.size(1) == N && row_src.numel() >= Mp && tile_expert.numel() * 256 >= Mp &&
              tile_flags.numel() * 256 >= Mp, "ep_dispatch_mm: table extents");
  std::vector<unsigned long long> xs(x_src.begin(), x_src.end()), rd(ready.begin(), ready.end()), ak(acks.begin(), acks.end());
  int rc = dfb::moe_grouped_mm_gather(xs.data(), xp.data_ptr(), row_src.data_ptr<int>(), w.data_ptr(), y.data_ptr(),
                                      tile_expert.data_ptr<int>(), Mp, N, K, E, transpose_w ? 0 : 1, tokens_per_rank, rank,
                                      xs.size(), reinterpret_cast<unsigned int*>(tile_flags.data_ptr<int>()), rd.data(), ak.data(),
                                      (unsigned)launch_seq, timeout_s, err.data_ptr<int>(),
                                      reinterpret_cast<unsigned int*>(done_ctr.data_ptr<int>()), num_sms(), cur_stream());
  TORCH_CHECK(rc == 0, "ep_dispatch_mm launch failed with code ", rc);
}
static void ep_pull_rows(const Tensor& tables_dev, const Tensor& ids, Tensor& rows_local, int64_t e_local, int64_t my_first_slot) {
  CHECK_I32(ids); CHECK_I32(rows_local);
  TORCH_CHECK(tables_dev.scalar_type() == at::kLong && tables_dev.is_cuda(), "ep_pull_rows: the pointer table is a device int64 tensor");
  int rc = dfb::ep_pull_rows(reinterpret_cast<const unsigned long long*>(tables_dev.data_ptr<int64_t>()), ids.data_ptr<int>(),
                             rows_local.data_ptr<int>(), ids.numel(), e_local, my_first_slot, cur_stream());
  TORCH_CHECK(rc == 0, "ep_pull_rows launch failed with code ", rc);
}
static void ep_combine(std::vector<int64_t> rows, std::vector<int64_t> scal, c10::optional<Tensor> base, c10::optional<Tensor> route_w,
                       const Tensor& ids, const Tensor& rows_local, Tensor& out, c10::optional<Tensor> out_s, int64_t e_local,
                       int64_t rank, std::vector<int64_t> ready, std::vector<int64_t> acks, int64_t seq, double timeout_s,
                       Tensor& err, Tensor& done_ctr) {
  CHECK_BF16(out); CHECK_I32(ids); CHECK_I32(rows_local); CHECK_I32(err); CHECK_I32(done_ctr);
  const int64_t T = ids.size(0), K = ids.size(1), d = out.size(1);
  std::vector<unsigned long long> rw(rows.begin(), rows.end()), sc(scal.begin(), scal.end()), rd(ready.begin(), ready.end()),
      ak(acks.begin(), acks.end());
  if (route_w.has_value()) CHECK_F32((*route_w));
  if (out_s.has_value()) CHECK_F32((*out_s));
  int rc = dfb::ep_combine(rw.data(), sc.empty() ? nullptr : sc.data(), base.has_value() ? base->data_ptr() : nullptr,
                           route_w.has_value() ? route_w->data_ptr<float>() : nullptr, ids.data_ptr<int>(),
                           rows_local.data_ptr<int>(), out.data_ptr(), out_s.has_value() ? out_s->data_ptr<float>() : nullptr, T, K, d,
                           e_local, rank, rw.size(), rd.data(), ak.data(), (unsigned)seq, timeout_s, err.data_ptr<int>(),
                           reinterpret_cast<unsigned int*>(done_ctr.data_ptr<int>()), num_sms(), cur_stream());
  TORCH_CHECK(rc == 0, "ep_combine launch failed with code ", rc);
}

// ---------------------------------------------------------------- interop
// Zero-copy tensor over engine-owned memory (device or pinned host).
static Tensor tensor_from_ptr(int64_t ptr, std::vector<int64_t> shape, const std::string& dtype, int64_t device) {
  static const std::map<std::string, at::ScalarType> types = {
      {"bf16", at::kBFloat16}, {"fp32", at::kFloat}, {"fp16", at::kHalf}, {"int32", at::kInt}, {"int64", at::kLong},
      {"int16", at::kShort}, {"uint8", at::kByte}, {"int8", at::kChar}, {"fp64", at::kDouble}, {"bool", at::kBool},
      {"fp8_e4m3", at::kFloat8_e4m3fn}, {"fp8_e5m2", at::kFloat8_e5m2}};
  auto it = types.find(dtype);
  TORCH_CHECK(it != types.end(), "unknown dtype ", dtype);
  auto opts = at::TensorOptions().dtype(it->second);
  if (device >= 0) opts = opts.device(at::kCUDA, device);
  return at::from_blob(reinterpret_cast<void*>(ptr), shape, [](void*) {}, opts);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_apply", &rmsnorm_apply);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("layernorm_fwd", &layernorm_fwd);
  m.def("layernorm_apply", &layernorm_apply);
  m.def("layernorm_bwd", &layernorm_bwd);
  m.def("norm_bwd_scratch_elems", &norm_bwd_scratch_elems);
  m.def("rope_inplace", &rope_inplace);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("gelu_fwd", &gelu_fwd);
  m.def("gelu_bwd", &gelu_bwd);
  m.def("add_bf16", &add_bf16);
  m.def("colsum_bf16", &colsum_bf16);
  m.def("colsum_parts", [](int64_t rows) { return (int64_t)dfb::colsum_parts((int)rows); });
  m.def("adamw_bf16", &adamw_bf16);
  m.def("adamw_master", &adamw_master);
  m.def("adamw_f32", &adamw_f32);
  m.def("adamw_split", &adamw_split);
  m.def("sgd_bf16", &sgd_bf16);
  m.def("ce_loss_fwd_bwd", &ce_loss_fwd_bwd);
  m.def("embed_fwd", &embed_fwd);
  m.def("embed_bwd_sorted", &embed_bwd_sorted);
  m.def("gemm_bf16", &gemm_bf16);
  m.def("gemm_last_error", &gemm_last_error);
  m.def("gemm_set_mt", [](int64_t mt) { dfb::gemm_bf16_set_mt((int)mt); });
  m.def("tensor_from_ptr", &tensor_from_ptr);
  m.def("zero_rs_adamw", &zero_rs_adamw);
  m.def("zero_rs_accum", &zero_rs_accum);
  m.def("moe_sort", &moe_sort);
  m.def("moe_topk_softmax", &moe_topk_softmax);
  m.def("moe_router_bwd", &moe_router_bwd);
  m.def("moe_dispatch", &moe_dispatch);
  m.def("moe_combine", &moe_combine);
  m.def("moe_dispatch_bwd", &moe_dispatch_bwd);
  m.def("moe_scale_rows", &moe_scale_rows);
  m.def("moe_rowdot", &moe_rowdot);
  m.def("moe_grouped_mm", &moe_grouped_mm);
  m.def("moe_grouped_wgrad", &moe_grouped_wgrad);
  m.def("flash_fwd", &flash_fwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("out"), py::arg("lse"), py::arg("cu_seqlens"),
        py::arg("max_seqlen"), py::arg("scale"), py::arg("trace") = py::none());
  m.def("umma_probe", &umma_probe);
  m.def("flash_bwd", &flash_bwd, py::arg("dout"), py::arg("q"), py::arg("k"), py::arg("v"), py::arg("out"), py::arg("lse"), py::arg("dq"),
        py::arg("dk"), py::arg("dv"), py::arg("scratch"), py::arg("cu_seqlens"), py::arg("max_seqlen"), py::arg("scale"),
        py::arg("trace") = py::none());
  m.def("quant_fp8_rowwise", &quant_fp8_rowwise);
  m.def("gemm_fp8", &gemm_fp8);
  m.def("dsa_index_scores", &dsa_index_scores);
  m.def("dsa_topk_rows", &dsa_topk_rows);
  m.def("l2norm_fwd", &l2norm_fwd);
  m.def("l2norm_bwd", &l2norm_bwd);
  m.def("gated_rmsnorm_fwd", &gated_rmsnorm_fwd);
  m.def("gated_rmsnorm_bwd", &gated_rmsnorm_bwd);
  m.def("conv_silu_fwd", &conv_silu_fwd);
  m.def("conv_silu_bwd", &conv_silu_bwd);
  m.def("router_sigmoid_noaux", &router_sigmoid_noaux);
  m.def("ep_dispatch_mm", &ep_dispatch_mm);
  m.def("ep_pull_rows", &ep_pull_rows);
  m.def("ep_combine", &ep_combine);
  m.def("tp_ag_gemm", &tp_ag_gemm);
  m.def("tp_gemm_rs", &tp_gemm_rs);
  m.def("param_gather", &param_gather);
  m.def("param_gather_dma", &param_gather_dma);
}
