// torch custom-op bindings (namespace `stb`) for the sm_100a kernels.  All ops write into tensors
// the caller provides and enqueue on the current CUDA stream; none synchronises except
// status_read().  Python wrappers live in shardtrain_b200/ops/.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <ATen/ATen.h>

#include <cstring>
#include <vector>

#include "api.h"

namespace {

using at::Tensor;

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, "shardtrain_b200 kernel launch failed (", what,
              "): ", cudaGetErrorString(e));
}

void need(const Tensor& t, at::ScalarType dt, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == dt, name, " has the wrong dtype");
}

// One status word per process (one process drives one GPU).
Tensor& status_tensor() {
  static Tensor t;
  if (!t.defined())
    t = at::zeros({4}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, at::cuda::current_device()));
  return t;
}
int* status_ptr() { return status_tensor().data_ptr<int>(); }

int64_t status_read() {
  return status_tensor().index({0}).item<int64_t>();
}
void status_reset() { status_tensor().zero_(); }
Tensor status_tensor_op() { return status_tensor(); }

void gemm(const Tensor& a, const Tensor& b, Tensor out, bool a_mn, bool b_mn,
          const c10::optional<Tensor>& bias, const c10::optional<Tensor>& residual,
          bool accumulate, double alpha, int64_t force_bn, int64_t split_k,
          bool staged_store) {
  need(a, at::kBFloat16, "a");
  need(b, at::kBFloat16, "b");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2, "gemm operands must be 2-D");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && out.stride(1) == 1,
              "gemm operands need a contiguous inner dimension");
  const c10::cuda::CUDAGuard guard(a.device());
  stb::GemmCall c{};
  c.M = static_cast<int>(a_mn ? a.size(1) : a.size(0));
  c.K = static_cast<int>(a_mn ? a.size(0) : a.size(1));
  c.N = static_cast<int>(b_mn ? b.size(1) : b.size(0));
  const int64_t kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(kb == c.K, "gemm reduction sizes differ: ", c.K, " vs ", kb);
  TORCH_CHECK(out.size(0) == c.M && out.size(1) == c.N, "gemm output shape mismatch");
  c.a = a.data_ptr();
  c.b = b.data_ptr();
  c.out = out.data_ptr();
  c.lda = a.stride(0);
  c.ldb = b.stride(0);
  c.ldo = out.stride(0);
  c.a_mn = a_mn;
  c.b_mn = b_mn;
  c.out_fp32 = out.scalar_type() == at::kFloat;
  TORCH_CHECK(c.out_fp32 || out.scalar_type() == at::kBFloat16, "gemm out must be fp32 or bf16");
  c.accumulate = accumulate;
  c.alpha = static_cast<float>(alpha);
  c.force_bn = static_cast<int>(force_bn);
  c.split_k = static_cast<int>(split_k);
  c.staged_store = staged_store ? 0 : -1;
  if (bias.has_value()) {
    need(*bias, at::kFloat, "bias");
    TORCH_CHECK(bias->numel() == c.N, "bias length mismatch");
    c.bias = bias->data_ptr<float>();
  }
  if (residual.has_value()) {
    TORCH_CHECK(residual->scalar_type() == out.scalar_type() && residual->stride(0) == c.ldo &&
                    residual->stride(1) == 1,
                "residual must match out's dtype and layout");
    c.residual = residual->data_ptr();
  }
  check(stb::launch_gemm_bf16(c, status_ptr(), cur_stream()), "gemm");
}

// out = A @ B^T (or A @ B with b_mn) where A is gathered along the sequence inside the GEMM:
// `a_dst` is the local [batch * T * seq_local, K] buffer the kernel fills from the T peers'
// [batch * seq_local, K] slices (`peer_ptrs`, contiguous rows) and then reads tile by tile.
void gemm_seq_pull(Tensor a_dst, const Tensor& b, Tensor out, bool b_mn,
                   const c10::optional<Tensor>& bias, c10::ArrayRef<int64_t> peer_ptrs,
                   int64_t batch, int64_t seq_local, int64_t force_bn) {
  need(a_dst, at::kBFloat16, "a_dst");
  need(b, at::kBFloat16, "b");
  TORCH_CHECK(a_dst.dim() == 2 && b.dim() == 2 && out.dim() == 2 && a_dst.stride(1) == 1 &&
                  b.stride(1) == 1 && out.stride(1) == 1, "gemm_seq_pull: 2-D operands expected");
  TORCH_CHECK(peer_ptrs.size() >= 2 && peer_ptrs.size() <= 8, "2..8 sequence owners expected");
  const c10::cuda::CUDAGuard guard(a_dst.device());
  stb::GemmCall c{};
  c.M = static_cast<int>(a_dst.size(0));
  c.K = static_cast<int>(a_dst.size(1));
  c.N = static_cast<int>(b_mn ? b.size(1) : b.size(0));
  TORCH_CHECK((b_mn ? b.size(0) : b.size(1)) == c.K, "gemm reduction sizes differ");
  TORCH_CHECK(out.size(0) == c.M && out.size(1) == c.N, "gemm output shape mismatch");
  c.a = a_dst.data_ptr();
  c.b = b.data_ptr();
  c.out = out.data_ptr();
  c.lda = a_dst.stride(0);
  c.ldb = b.stride(0);
  c.ldo = out.stride(0);
  c.b_mn = b_mn;
  c.out_fp32 = out.scalar_type() == at::kFloat;
  c.alpha = 1.f;
  c.force_bn = static_cast<int>(force_bn);
  if (bias.has_value()) {
    need(*bias, at::kFloat, "bias");
    c.bias = bias->data_ptr<float>();
  }
  c.pull_degree = static_cast<int>(peer_ptrs.size());
  c.pull_batch = static_cast<int>(batch);
  c.pull_seq_local = static_cast<int>(seq_local);
  c.pull_src_ld = c.K;
  for (size_t i = 0; i < peer_ptrs.size(); ++i)
    c.pull_peers[i] = reinterpret_cast<const void*>(peer_ptrs[i]);
  check(stb::launch_gemm_bf16(c, status_ptr(), cur_stream()), "gemm_seq_pull");
}

void rmsnorm_fwd(const Tensor& x, const Tensor& w, Tensor y, Tensor inv, double eps) {
  need(x, at::kFloat, "x");
  need(w, at::kFloat, "w");
  need(inv, at::kFloat, "inv");
  const int cols = static_cast<int>(x.size(-1));
  const int rows = static_cast<int>(x.numel() / cols);
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous() && w.numel() == cols && inv.numel() == rows);
  check(stb::launch_rmsnorm_fwd(x.data_ptr<float>(), w.data_ptr<float>(), y.data_ptr(),
                                inv.data_ptr<float>(), rows, cols, static_cast<float>(eps),
                                y.scalar_type() == at::kFloat, cur_stream()),
        "rmsnorm_fwd");
}

// Row-parallel GEMM whose fp32 result rows are scattered along the sequence into per-owner
// buffers (peer pointers allowed): row b*seq + s -> dest_ptrs[s / seq_local][b*seq_local + s %
// seq_local, :].  `cols` is the row pitch of every destination (= N).
void gemm_scatter(const Tensor& a, const Tensor& b, c10::ArrayRef<int64_t> dest_ptrs, int64_t seq,
                  bool a_mn, bool b_mn, int64_t force_bn) {
  need(a, at::kBFloat16, "a");
  need(b, at::kBFloat16, "b");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1,
              "gemm operands must be 2-D with a contiguous inner dimension");
  TORCH_CHECK(dest_ptrs.size() >= 2 && dest_ptrs.size() <= 8, "2..8 scatter destinations expected");
  const c10::cuda::CUDAGuard guard(a.device());
  stb::GemmCall c{};
  c.M = static_cast<int>(a_mn ? a.size(1) : a.size(0));
  c.K = static_cast<int>(a_mn ? a.size(0) : a.size(1));
  c.N = static_cast<int>(b_mn ? b.size(1) : b.size(0));
  TORCH_CHECK((b_mn ? b.size(0) : b.size(1)) == c.K, "gemm reduction sizes differ");
  c.a = a.data_ptr();
  c.b = b.data_ptr();
  c.lda = a.stride(0);
  c.ldb = b.stride(0);
  c.ldo = c.N;
  c.a_mn = a_mn;
  c.b_mn = b_mn;
  c.out_fp32 = true;
  c.alpha = 1.f;
  c.force_bn = static_cast<int>(force_bn);
  c.scatter_degree = static_cast<int>(dest_ptrs.size());
  c.scatter_seq = static_cast<int>(seq);
  c.scatter_seq_local = static_cast<int>(seq / static_cast<int64_t>(dest_ptrs.size()));
  for (size_t i = 0; i < dest_ptrs.size(); ++i)
    c.scatter_out[i] = reinterpret_cast<float*>(dest_ptrs[i]);
  c.out = c.scatter_out[0];
  check(stb::launch_gemm_bf16(c, status_ptr(), cur_stream()), "gemm_scatter");
}

// gate|up projection with the SwiGLU epilogue: gu [M, 2*inter] and h = silu(gate) * up [M, inter]
void gemm_swiglu(const Tensor& a, const Tensor& w_gu, Tensor gu, Tensor h) {
  need(a, at::kBFloat16, "a");
  need(w_gu, at::kBFloat16, "w_gu");
  need(gu, at::kBFloat16, "gu");
  need(h, at::kBFloat16, "h");
  TORCH_CHECK(a.dim() == 2 && w_gu.dim() == 2 && a.stride(1) == 1 && w_gu.stride(1) == 1 &&
                  gu.is_contiguous() && h.is_contiguous() && w_gu.size(0) % 2 == 0 &&
                  a.size(1) == w_gu.size(1) && gu.size(0) == a.size(0) &&
                  gu.size(1) == w_gu.size(0) && h.size(0) == a.size(0) &&
                  h.size(1) * 2 == w_gu.size(0),
              "gemm_swiglu: shape mismatch");
  const c10::cuda::CUDAGuard guard(a.device());
  stb::GemmCall c{};
  c.M = static_cast<int>(a.size(0));
  c.K = static_cast<int>(a.size(1));
  c.N = static_cast<int>(w_gu.size(0));
  c.a = a.data_ptr();
  c.b = w_gu.data_ptr();
  c.out = gu.data_ptr();
  c.lda = a.stride(0);
  c.ldb = w_gu.stride(0);
  c.ldo = gu.stride(0);
  c.alpha = 1.f;
  c.gated_out = h.data_ptr();
  c.gated_inter = static_cast<int>(h.size(1));
  check(stb::launch_gemm_bf16(c, status_ptr(), cur_stream()), "gemm_swiglu");
}

// Row-parallel GEMM whose fp32 result is stored into every destination (all-reduce push).
void gemm_broadcast(const Tensor& a, const Tensor& b, c10::ArrayRef<int64_t> dest_ptrs, bool b_mn) {
  need(a, at::kBFloat16, "a");
  need(b, at::kBFloat16, "b");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1,
              "gemm operands must be 2-D with a contiguous inner dimension");
  TORCH_CHECK(dest_ptrs.size() >= 2 && dest_ptrs.size() <= 8, "2..8 destinations expected");
  const c10::cuda::CUDAGuard guard(a.device());
  stb::GemmCall c{};
  c.M = static_cast<int>(a.size(0));
  c.K = static_cast<int>(a.size(1));
  c.N = static_cast<int>(b_mn ? b.size(1) : b.size(0));
  TORCH_CHECK((b_mn ? b.size(0) : b.size(1)) == c.K, "gemm reduction sizes differ");
  c.a = a.data_ptr();
  c.b = b.data_ptr();
  c.lda = a.stride(0);
  c.ldb = b.stride(0);
  c.ldo = c.N;
  c.b_mn = b_mn;
  c.out_fp32 = true;
  c.alpha = 1.f;
  c.scatter_degree = static_cast<int>(dest_ptrs.size());
  c.scatter_broadcast = 1;
  for (size_t i = 0; i < dest_ptrs.size(); ++i)
    c.scatter_out[i] = reinterpret_cast<float*>(dest_ptrs[i]);
  c.out = c.scatter_out[0];
  check(stb::launch_gemm_bf16(c, status_ptr(), cur_stream()), "gemm_broadcast");
}

void slot_sum_rmsnorm(const Tensor& slots, const c10::optional<Tensor>& residual, Tensor sum_out,
                      const c10::optional<Tensor>& w, const c10::optional<Tensor>& y,
                      const c10::optional<Tensor>& inv, double eps) {
  need(slots, at::kFloat, "slots");
  need(sum_out, at::kFloat, "sum_out");
  TORCH_CHECK(slots.dim() == 3 && slots.is_contiguous() && sum_out.is_contiguous() &&
                  sum_out.numel() == slots.size(1) * slots.size(2),
              "slots must be [n, rows, cols] and sum_out [rows, cols]");
  const int rows = static_cast<int>(slots.size(1)), cols = static_cast<int>(slots.size(2));
  if (residual.has_value()) {
    need(*residual, at::kFloat, "residual");
    TORCH_CHECK(residual->is_contiguous() && residual->numel() == sum_out.numel());
  }
  if (w.has_value()) {
    need(*w, at::kFloat, "w");
    TORCH_CHECK(y.has_value() && inv.has_value() && y->scalar_type() == at::kBFloat16 &&
                y->is_contiguous() && y->numel() == sum_out.numel() && inv->numel() == rows &&
                w->numel() == cols);
    need(*inv, at::kFloat, "inv");
  }
  check(stb::launch_slot_sum_rmsnorm(
            slots.data_ptr<float>(), static_cast<int>(slots.size(0)), slots.stride(0),
            residual.has_value() ? residual->data_ptr<float>() : nullptr, sum_out.data_ptr<float>(),
            w.has_value() ? w->data_ptr<float>() : nullptr, w.has_value() ? y->data_ptr() : nullptr,
            w.has_value() ? inv->data_ptr<float>() : nullptr, rows, cols, static_cast<float>(eps),
            cur_stream()),
        "slot_sum_rmsnorm");
}

void rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& inv,
                 const c10::optional<Tensor>& dres, Tensor dx, Tensor dw_partial) {
  need(dy, at::kFloat, "dy");
  need(x, at::kFloat, "x");
  need(dx, at::kFloat, "dx");
  need(dw_partial, at::kFloat, "dw_partial");
  const int cols = static_cast<int>(x.size(-1));
  const int rows = static_cast<int>(x.numel() / cols);
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous() && dx.is_contiguous());
  TORCH_CHECK(dw_partial.dim() == 2 && dw_partial.size(1) == cols && dw_partial.is_contiguous());
  check(stb::launch_rmsnorm_bwd(dy.data_ptr<float>(), x.data_ptr<float>(), w.data_ptr<float>(),
                                inv.data_ptr<float>(),
                                dres.has_value() ? dres->data_ptr<float>() : nullptr,
                                dx.data_ptr<float>(), dw_partial.data_ptr<float>(),
                                static_cast<int>(dw_partial.size(0)), rows, cols, cur_stream()),
        "rmsnorm_bwd");
}

void colsum_f32(const Tensor& partial, Tensor out, bool accumulate) {
  need(partial, at::kFloat, "partial");
  need(out, at::kFloat, "out");
  TORCH_CHECK(partial.dim() == 2 && partial.is_contiguous() && out.numel() == partial.size(1));
  check(stb::launch_colsum_f32(partial.data_ptr<float>(), out.data_ptr<float>(),
                               static_cast<int>(partial.size(0)),
                               static_cast<int>(partial.size(1)), accumulate, cur_stream()),
        "colsum_f32");
}

void colsum_bf16(const Tensor& x, Tensor out, bool accumulate, Tensor scratch) {
  need(x, at::kBFloat16, "x");
  need(out, at::kFloat, "out");
  need(scratch, at::kFloat, "scratch");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && scratch.dim() == 2 &&
              scratch.size(1) == x.size(1) && scratch.is_contiguous());
  check(stb::launch_colsum_bf16(x.data_ptr(), x.stride(0), out.data_ptr<float>(),
                                static_cast<int>(x.size(0)), static_cast<int>(x.size(1)),
                                accumulate, scratch.data_ptr<float>(),
                                static_cast<int>(scratch.size(0)), cur_stream()),
        "colsum_bf16");
}

void rope(Tensor qkv, const Tensor& cos, const Tensor& sin, const c10::optional<Tensor>& positions,
          int64_t seq, int64_t hq, int64_t hkv, int64_t d, bool inverse) {
  need(qkv, at::kBFloat16, "qkv");
  need(cos, at::kFloat, "cos");
  need(sin, at::kFloat, "sin");
  TORCH_CHECK(qkv.is_contiguous() && qkv.size(-1) == (hq + 2 * hkv) * d);
  const int rows = static_cast<int>(qkv.numel() / qkv.size(-1));
  const int* pos = nullptr;
  if (positions.has_value()) {
    need(*positions, at::kInt, "positions");
    TORCH_CHECK(positions->numel() == rows);
    pos = positions->data_ptr<int>();
  }
  check(stb::launch_rope(qkv.data_ptr(), cos.data_ptr<float>(), sin.data_ptr<float>(), pos, rows,
                         static_cast<int>(seq), static_cast<int>(hq), static_cast<int>(hkv),
                         static_cast<int>(d), inverse, cur_stream()),
        "rope");
}

void swiglu_fwd(const Tensor& gu, Tensor h) {
  need(gu, at::kBFloat16, "gu");
  need(h, at::kBFloat16, "h");
  TORCH_CHECK(gu.is_contiguous() && h.is_contiguous() && gu.size(-1) == 2 * h.size(-1));
  const int inter = static_cast<int>(h.size(-1));
  check(stb::launch_swiglu_fwd(gu.data_ptr(), h.data_ptr(), static_cast<int>(h.numel() / inter),
                               inter, cur_stream()),
        "swiglu_fwd");
}

void swiglu_bwd(const Tensor& dh, const Tensor& gu, Tensor dgu) {
  need(dh, at::kBFloat16, "dh");
  need(gu, at::kBFloat16, "gu");
  need(dgu, at::kBFloat16, "dgu");
  TORCH_CHECK(dh.is_contiguous() && gu.is_contiguous() && dgu.is_contiguous());
  const int inter = static_cast<int>(dh.size(-1));
  check(stb::launch_swiglu_bwd(dh.data_ptr(), gu.data_ptr(), dgu.data_ptr(),
                               static_cast<int>(dh.numel() / inter), inter, cur_stream()),
        "swiglu_bwd");
}

void ce_fwd(const Tensor& logits, const Tensor& labels, Tensor lse, Tensor loss_rows) {
  need(logits, at::kBFloat16, "logits");
  need(labels, at::kLong, "labels");
  need(lse, at::kFloat, "lse");
  need(loss_rows, at::kFloat, "loss_rows");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && labels.numel() == logits.size(0));
  check(stb::launch_ce_fwd(logits.data_ptr(), logits.stride(0), labels.data_ptr<int64_t>(),
                           lse.data_ptr<float>(), loss_rows.data_ptr<float>(),
                           static_cast<int>(logits.size(0)), static_cast<int>(logits.size(1)),
                           cur_stream()),
        "ce_fwd");
}

void ce_bwd(Tensor logits, const Tensor& labels, const Tensor& lse, const Tensor& scale) {
  need(logits, at::kBFloat16, "logits");
  need(labels, at::kLong, "labels");
  need(scale, at::kFloat, "scale");
  check(stb::launch_ce_bwd(logits.data_ptr(), logits.stride(0), labels.data_ptr<int64_t>(),
                           lse.data_ptr<float>(), scale.data_ptr<float>(),
                           static_cast<int>(logits.size(0)), static_cast<int>(logits.size(1)),
                           cur_stream()),
        "ce_bwd");
}

void sum_f32(const Tensor& x, Tensor out, bool accumulate) {
  need(x, at::kFloat, "x");
  need(out, at::kFloat, "out");
  check(stb::launch_sum_f32(x.data_ptr<float>(), out.data_ptr<float>(),
                            static_cast<int>(x.numel()), accumulate, cur_stream()),
        "sum_f32");
}

void embedding_scatter_add(const Tensor& dx, const Tensor& ids, Tensor dw, int64_t pad_id) {
  need(dx, at::kFloat, "dx");
  need(ids, at::kLong, "ids");
  need(dw, at::kFloat, "dw");
  const int cols = static_cast<int>(dw.size(-1));
  check(stb::launch_embedding_scatter_add(dx.data_ptr<float>(), ids.data_ptr<int64_t>(),
                                          dw.data_ptr<float>(), static_cast<int>(ids.numel()),
                                          cols, dw.numel() / cols, pad_id, cur_stream()),
        "embedding_scatter_add");
}

void cast_bf16(const Tensor& x, Tensor y) {
  need(x, at::kFloat, "x");
  need(y, at::kBFloat16, "y");
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous() && x.numel() == y.numel());
  check(stb::launch_cast_f32_to_bf16(x.data_ptr<float>(), y.data_ptr(), x.numel(), cur_stream()),
        "cast_bf16");
}

void add_f32(const Tensor& a, const Tensor& b, Tensor out) {
  need(a, at::kFloat, "a");
  need(b, at::kFloat, "b");
  need(out, at::kFloat, "out");
  check(stb::launch_add_f32(a.data_ptr<float>(), b.data_ptr<float>(), out.data_ptr<float>(),
                            a.numel(), cur_stream()),
        "add_f32");
}

stb::AdamWArgs adam_args(double lr, double b1, double b2, double eps, double wd, double bc1,
                         double bc2, double gscale) {
  stb::AdamWArgs a;
  a.lr = static_cast<float>(lr);
  a.beta1 = static_cast<float>(b1);
  a.beta2 = static_cast<float>(b2);
  a.eps = static_cast<float>(eps);
  a.weight_decay = static_cast<float>(wd);
  a.bias_correction1 = static_cast<float>(bc1);
  a.bias_correction2 = static_cast<float>(bc2);
  a.grad_scale = static_cast<float>(gscale);
  return a;
}

void adamw(Tensor p, const Tensor& g, Tensor m, Tensor v, double lr, double b1, double b2,
           double eps, double wd, double bc1, double bc2, double gscale) {
  need(p, at::kFloat, "p");
  need(g, at::kFloat, "g");
  need(m, at::kFloat, "m");
  need(v, at::kFloat, "v");
  TORCH_CHECK(p.is_contiguous() && g.is_contiguous() && m.is_contiguous() && v.is_contiguous());
  check(stb::launch_adamw(p.data_ptr<float>(), g.data_ptr<float>(), m.data_ptr<float>(),
                          v.data_ptr<float>(), p.numel(),
                          adam_args(lr, b1, b2, eps, wd, bc1, bc2, gscale), cur_stream()),
        "adamw");
}

void sgd(Tensor p, const Tensor& g, double lr) {
  need(p, at::kFloat, "p");
  need(g, at::kFloat, "g");
  check(stb::launch_sgd(p.data_ptr<float>(), g.data_ptr<float>(), p.numel(),
                        static_cast<float>(lr), cur_stream()),
        "sgd");
}

void unpack_gathered(const Tensor& packed, int64_t slot, const Tensor& table, int64_t largest,
                     Tensor out) {
  need(packed, at::kFloat, "packed");
  need(out, at::kFloat, "out");
  need(table, at::kLong, "table");
  TORCH_CHECK(table.dim() == 2 && table.size(1) == 4 && table.is_contiguous(), "table must be [n, 4]");
  TORCH_CHECK(packed.is_contiguous() && out.is_contiguous() && packed.numel() % slot == 0,
              "packed buffer must be whole rank slots");
  const c10::cuda::CUDAGuard guard(packed.device());
  check(stb::launch_unpack_gathered(packed.data_ptr<float>(), slot, table.data_ptr<int64_t>(),
                                    static_cast<int>(table.size(0)), largest, out.data_ptr<float>(),
                                    at::cuda::getCurrentCUDAStream().stream()),
        "unpack_gathered");
}

void pack_gradients(const Tensor& grad_ptrs, const Tensor& table, int64_t degree, int64_t slot,
                    int64_t used, int64_t largest, Tensor packed) {
  need(grad_ptrs, at::kLong, "grad_ptrs");
  need(table, at::kLong, "table");
  need(packed, at::kFloat, "packed");
  TORCH_CHECK(table.dim() == 2 && table.size(1) == 4 && table.is_contiguous() &&
                  grad_ptrs.numel() == table.size(0),
              "table must be [n, 4] with one gradient pointer per row");
  TORCH_CHECK(packed.is_contiguous() && packed.numel() == degree * slot, "packed has the wrong length");
  const c10::cuda::CUDAGuard guard(packed.device());
  check(stb::launch_pack_gradients(grad_ptrs.data_ptr<int64_t>(), table.data_ptr<int64_t>(),
                                   static_cast<int>(table.size(0)), static_cast<int>(degree), slot,
                                   used, largest, packed.data_ptr<float>(),
                                   at::cuda::getCurrentCUDAStream().stream()),
        "pack_gradients");
}

void grad_check(const Tensor& g, const Tensor& pad_ranges, Tensor flags) {
  need(g, at::kFloat, "g");
  need(pad_ranges, at::kLong, "pad_ranges");
  need(flags, at::kInt, "flags");
  check(stb::launch_grad_check(g.data_ptr<float>(), g.numel(), pad_ranges.data_ptr<int64_t>(),
                               static_cast<int>(pad_ranges.numel() / 2), flags.data_ptr<int>(),
                               cur_stream()),
        "grad_check");
}

// segs: CPU int64 [n, 5] = shard_off, q, numel, full_off, keep_fp32
std::vector<stb::SegmentDesc> read_segs(const Tensor& segs) {
  TORCH_CHECK(!segs.is_cuda() && segs.scalar_type() == at::kLong && segs.dim() == 2 &&
                  segs.size(1) == 5 && segs.is_contiguous(),
              "segment table must be a CPU int64 [n, 5] tensor");
  std::vector<stb::SegmentDesc> out(segs.size(0));
  const int64_t* p = segs.data_ptr<int64_t>();
  for (int64_t i = 0; i < segs.size(0); ++i) {
    out[i].shard_off = p[5 * i];
    out[i].q = p[5 * i + 1];
    out[i].numel = p[5 * i + 2];
    out[i].full_off = p[5 * i + 3];
    // column 4: bit 0 = keep fp32 (gather tables), bit 1 = TP-replicated (reduce tables)
    out[i].keep_fp32 = static_cast<int32_t>(p[5 * i + 4] & 1);
    out[i].pad = static_cast<int32_t>((p[5 * i + 4] >> 1) & 1);
  }
  return out;
}

stb::PeerPtrs peer_ptrs(c10::ArrayRef<int64_t> ptrs) {
  TORCH_CHECK(!ptrs.empty() && ptrs.size() <= stb::kMaxPeers, "1..8 peer pointers expected");
  stb::PeerPtrs pp{};
  for (size_t i = 0; i < ptrs.size(); ++i) pp.p[i] = reinterpret_cast<const float*>(ptrs[i]);
  return pp;
}

// A unit may hold more parameters than one launch's table; split into launches of <= 32.
void gather_params(c10::ArrayRef<int64_t> shard_ptrs, const Tensor& segs, Tensor full_bf16,
                   Tensor full_fp32, c10::ArrayRef<int64_t> shadow_ptrs) {
  need(full_bf16, at::kBFloat16, "full_bf16");
  need(full_fp32, at::kFloat, "full_fp32");
  TORCH_CHECK(shadow_ptrs.empty() || shadow_ptrs.size() == shard_ptrs.size(),
              "one shadow arena per shard arena expected");
  auto table = read_segs(segs);
  const auto pp = peer_ptrs(shard_ptrs);
  std::vector<const void*> shadows(shadow_ptrs.size());
  for (size_t i = 0; i < shadow_ptrs.size(); ++i)
    shadows[i] = reinterpret_cast<const void*>(shadow_ptrs[i]);
  for (size_t i = 0; i < table.size(); i += 32) {
    const int n = static_cast<int>(std::min<size_t>(32, table.size() - i));
    check(stb::launch_gather_params(pp, static_cast<int>(shard_ptrs.size()), table.data() + i, n,
                                    full_bf16.data_ptr(), full_fp32.data_ptr<float>(),
                                    full_bf16.numel(), cur_stream(),
                                    shadows.empty() ? nullptr : shadows.data()),
          "gather_params");
  }
}

int* flags_ptr(const c10::optional<Tensor>& flags) {
  if (!flags.has_value()) return nullptr;
  need(*flags, at::kInt, "flags");
  TORCH_CHECK(flags->numel() >= 2, "flags needs two int32 words");
  return flags->data_ptr<int>();
}

stb::TpAxis tp_axis(c10::ArrayRef<int64_t> full_ptrs, int64_t tp_degree, int64_t tp_rank,
                    double rep_scale) {
  TORCH_CHECK(tp_degree >= 1 && full_ptrs.size() % tp_degree == 0,
              "the pointer table must list fsdp_degree * tp_degree slots");
  stb::TpAxis tp;
  tp.degree = static_cast<int>(tp_degree);
  tp.rank = static_cast<int>(tp_rank);
  tp.replicated_scale = static_cast<float>(rep_scale);
  return tp;
}

void reduce_scatter(c10::ArrayRef<int64_t> full_ptrs, int64_t rank, const Tensor& segs,
                    Tensor grad_shard, double scale, bool accumulate,
                    const c10::optional<Tensor>& flags, int64_t tp_degree, int64_t tp_rank,
                    double rep_scale, int64_t multicast_ptr) {
  auto table = read_segs(segs);
  const auto pp = peer_ptrs(full_ptrs);
  const auto tp = tp_axis(full_ptrs, tp_degree, tp_rank, rep_scale);
  for (size_t i = 0; i < table.size(); i += 32) {
    const int n = static_cast<int>(std::min<size_t>(32, table.size() - i));
    check(stb::launch_reduce_scatter_grads(pp, static_cast<int>(full_ptrs.size() / tp_degree),
                                           static_cast<int>(rank), table.data() + i, n,
                                           grad_shard.data_ptr<float>(), grad_shard.numel(),
                                           static_cast<float>(scale), accumulate, flags_ptr(flags),
                                           cur_stream(), tp, status_ptr(),
                                           reinterpret_cast<const float*>(multicast_ptr)),
          "reduce_scatter");
  }
}

void reduce_scatter_adamw(c10::ArrayRef<int64_t> full_ptrs, int64_t rank, const Tensor& segs,
                          Tensor grad_shard, Tensor p, Tensor m, Tensor v, double scale,
                          bool accumulate, double lr, double b1, double b2, double eps, double wd,
                          double bc1, double bc2, double gscale,
                          const c10::optional<Tensor>& flags, int64_t tp_degree, int64_t tp_rank,
                          double rep_scale, const c10::optional<Tensor>& shadow,
                          int64_t multicast_ptr) {
  auto table = read_segs(segs);
  const auto pp = peer_ptrs(full_ptrs);
  const auto tp = tp_axis(full_ptrs, tp_degree, tp_rank, rep_scale);
  void* shadow_ptr = nullptr;
  if (shadow.has_value()) {
    need(*shadow, at::kBFloat16, "shadow");
    TORCH_CHECK(shadow->numel() == p.numel(), "shadow must mirror the parameter arena");
    shadow_ptr = shadow->data_ptr();
  }
  for (size_t i = 0; i < table.size(); i += 32) {
    const int n = static_cast<int>(std::min<size_t>(32, table.size() - i));
    check(stb::launch_reduce_scatter_adamw(
              pp, static_cast<int>(full_ptrs.size() / tp_degree), static_cast<int>(rank),
              table.data() + i, n, grad_shard.data_ptr<float>(), p.data_ptr<float>(),
              m.data_ptr<float>(), v.data_ptr<float>(), grad_shard.numel(),
              static_cast<float>(scale), accumulate,
              adam_args(lr, b1, b2, eps, wd, bc1, bc2, gscale), flags_ptr(flags), cur_stream(), tp,
              shadow_ptr, status_ptr(), reinterpret_cast<const float*>(multicast_ptr)),
          "reduce_scatter_adamw");
  }
}

// Parameter all-gather fused into the consuming GEMM.  `segs`: CPU int64 [n, 5] rows of the
// unit's gather table (shard_off, q, numel, full_off, flags) for the n <= 4 parameters that form
// the fused weight, in row order.  `arena_ptrs`: one arena base per FSDP rank -- bf16 shadow
// arenas when `wire_fp32` is false, fp32 shard arenas otherwise.  `full` (optional): the unit's
// local bf16 full-parameter buffer; the pulled rows are mirrored into it.
void gemm_allgather(const Tensor& a, Tensor out, const c10::optional<Tensor>& bias,
                    c10::ArrayRef<int64_t> arena_ptrs, bool wire_fp32, const Tensor& segs,
                    const c10::optional<Tensor>& full, const c10::optional<Tensor>& gated_out,
                    int64_t force_bn) {
  need(a, at::kBFloat16, "a");
  need(out, at::kBFloat16, "out");
  TORCH_CHECK(a.dim() == 2 && out.dim() == 2 && a.stride(1) == 1 && out.stride(1) == 1 &&
                  out.size(0) == a.size(0),
              "gemm_allgather: a and out must be 2-D with a contiguous inner dimension");
  TORCH_CHECK(!arena_ptrs.empty() && arena_ptrs.size() <= stb::kMaxPeers, "1..8 arenas expected");
  const auto table = read_segs(segs);
  TORCH_CHECK(!table.empty() && table.size() <= 4, "1..4 weight segments expected");
  const c10::cuda::CUDAGuard guard(a.device());
  stb::AgGemmCall c{};
  c.a = a.data_ptr();
  c.out = out.data_ptr();
  c.M = static_cast<int>(a.size(0));
  c.K = static_cast<int>(a.size(1));
  c.N = static_cast<int>(out.size(1));
  c.lda = a.stride(0);
  c.ldo = out.stride(0);
  c.force_bn = static_cast<int>(force_bn);
  if (bias.has_value()) {
    need(*bias, at::kFloat, "bias");
    TORCH_CHECK(bias->numel() == c.N, "bias length mismatch");
    c.bias = bias->data_ptr<float>();
  }
  c.w.degree = static_cast<int>(arena_ptrs.size());
  for (size_t i = 0; i < arena_ptrs.size(); ++i) {
    if (wire_fp32)
      c.w.shard[i] = reinterpret_cast<const float*>(arena_ptrs[i]);
    else
      c.w.shadow[i] = reinterpret_cast<const __nv_bfloat16*>(arena_ptrs[i]);
  }
  c.w.n_segs = static_cast<int>(table.size());
  for (size_t j = 0; j < table.size(); ++j) {
    TORCH_CHECK(table[j].numel % c.K == 0, "a weight segment is not a whole number of rows");
    c.w.seg[j].shard_off = table[j].shard_off;
    c.w.seg[j].q = table[j].q;
    c.w.seg[j].full_off = table[j].full_off;
    c.w.seg[j].rows = static_cast<int>(table[j].numel / c.K);
  }
  if (full.has_value()) {
    need(*full, at::kBFloat16, "full");
    c.w.full = reinterpret_cast<__nv_bfloat16*>(full->data_ptr());
  }
  if (gated_out.has_value()) {
    need(*gated_out, at::kBFloat16, "gated_out");
    TORCH_CHECK(gated_out->is_contiguous() && gated_out->size(0) == a.size(0) &&
                    gated_out->size(1) * 2 == out.size(1),
                "gemm_allgather: gated_out must be [M, N / 2]");
    c.gated_out = gated_out->data_ptr();
    c.gated_inter = static_cast<int>(gated_out->size(1));
  }
  check(stb::launch_gemm_allgather(c, status_ptr(), cur_stream()), "gemm_allgather");
}

void embedding_gather_sharded(c10::ArrayRef<int64_t> shard_ptrs, int64_t q, const Tensor& ids,
                              Tensor out) {
  need(ids, at::kLong, "ids");
  need(out, at::kFloat, "out");
  const int cols = static_cast<int>(out.size(-1));
  check(stb::launch_embedding_gather_sharded(peer_ptrs(shard_ptrs),
                                             static_cast<int>(shard_ptrs.size()), q,
                                             ids.data_ptr<int64_t>(), out.data_ptr<float>(),
                                             static_cast<int>(ids.numel()), cols, cur_stream()),
        "embedding_gather_sharded");
}

void seq_gather(c10::ArrayRef<int64_t> ptrs, Tensor out, int64_t batch, int64_t seq_local,
                int64_t row_bytes) {
  std::vector<const void*> p(ptrs.size());
  for (size_t i = 0; i < ptrs.size(); ++i) p[i] = reinterpret_cast<const void*>(ptrs[i]);
  check(stb::launch_seq_gather(p.data(), static_cast<int>(ptrs.size()), out.data_ptr(),
                               static_cast<int>(batch), static_cast<int>(seq_local), row_bytes,
                               cur_stream()),
        "seq_gather");
}

void seq_reduce_scatter(c10::ArrayRef<int64_t> ptrs, int64_t rank,
                        const c10::optional<Tensor>& residual, Tensor out, int64_t batch,
                        int64_t seq_local) {
  need(out, at::kFloat, "out");
  std::vector<const float*> p(ptrs.size());
  for (size_t i = 0; i < ptrs.size(); ++i) p[i] = reinterpret_cast<const float*>(ptrs[i]);
  check(stb::launch_seq_reduce_scatter_f32(
            p.data(), static_cast<int>(ptrs.size()), static_cast<int>(rank),
            residual.has_value() ? residual->data_ptr<float>() : nullptr, out.data_ptr<float>(),
            static_cast<int>(batch), static_cast<int>(seq_local),
            static_cast<int>(out.size(-1)), cur_stream()),
        "seq_reduce_scatter");
}

// `wait_us`: time budget of the flag wait in microseconds.
uint64_t budget_ns(int64_t wait_us) {
  TORCH_CHECK(wait_us > 0, "the wait budget must be positive (microseconds)");
  return static_cast<uint64_t>(wait_us) * 1000ull;
}

void peer_barrier(c10::ArrayRef<int64_t> pad_ptrs, int64_t rank, int64_t epoch, int64_t slot,
                  int64_t wait_us) {
  std::vector<uint32_t*> p(pad_ptrs.size());
  for (size_t i = 0; i < pad_ptrs.size(); ++i) p[i] = reinterpret_cast<uint32_t*>(pad_ptrs[i]);
  check(stb::launch_peer_barrier(p.data(), static_cast<int>(pad_ptrs.size()),
                                 static_cast<int>(rank), static_cast<uint32_t>(epoch),
                                 static_cast<int>(slot), status_ptr(),
                                 budget_ns(wait_us), cur_stream()),
        "peer_barrier");
}

void peer_allreduce_small(c10::ArrayRef<int64_t> pad_ptrs, c10::ArrayRef<int64_t> inbox_ptrs,
                          int64_t rank, int64_t epoch, int64_t slot, const Tensor& in, Tensor out,
                          int64_t min_mask, int64_t wait_us) {
  need(in, at::kDouble, "in");
  need(out, at::kDouble, "out");
  TORCH_CHECK(in.is_contiguous() && out.is_contiguous() && in.numel() == out.numel() &&
                  pad_ptrs.size() == inbox_ptrs.size(),
              "peer_allreduce_small: mismatched arguments");
  std::vector<uint32_t*> pads(pad_ptrs.size());
  std::vector<double*> inboxes(inbox_ptrs.size());
  for (size_t i = 0; i < pad_ptrs.size(); ++i) {
    pads[i] = reinterpret_cast<uint32_t*>(pad_ptrs[i]);
    inboxes[i] = reinterpret_cast<double*>(inbox_ptrs[i]);
  }
  check(stb::launch_peer_allreduce_small(
            pads.data(), inboxes.data(), static_cast<int>(pads.size()), static_cast<int>(rank),
            static_cast<uint32_t>(epoch), static_cast<int>(slot), in.data_ptr<double>(),
            out.data_ptr<double>(), static_cast<int>(in.numel()), static_cast<uint32_t>(min_mask),
            status_ptr(), budget_ns(wait_us), cur_stream()),
        "peer_allreduce_small");
}

// ------------------------------------------------------------------ peer memory (CUDA IPC)
int64_t peer_alloc(int64_t nbytes) {
  void* p = nullptr;
  check(cudaMalloc(&p, static_cast<size_t>(nbytes)), "peer_alloc");
  check(cudaMemset(p, 0, static_cast<size_t>(nbytes)), "peer_alloc memset");
  return reinterpret_cast<int64_t>(p);
}
void peer_free(int64_t ptr) { cudaFree(reinterpret_cast<void*>(ptr)); }
void device_synchronize() { check(cudaDeviceSynchronize(), "device_synchronize"); }
int64_t launch_count() { return stb::launches_total(); }
// Let kernels on the current device dereference pointers into `peer_device`'s memory (one
// process driving two GPUs; across processes the CUDA-IPC mappings above do the same).
void enable_peer_access(int64_t peer_device) {
  const cudaError_t e = cudaDeviceEnablePeerAccess(static_cast<int>(peer_device), 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();   // clear the sticky-free error state
    return;
  }
  check(e, "enable_peer_access");
}
Tensor ipc_handle(int64_t ptr) {
  cudaIpcMemHandle_t h;
  check(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(ptr)), "ipc_handle");
  Tensor t = at::empty({static_cast<int64_t>(sizeof(h))}, at::TensorOptions().dtype(at::kByte));
  std::memcpy(t.data_ptr(), &h, sizeof(h));
  return t;
}
int64_t ipc_open(const Tensor& handle) {
  TORCH_CHECK(!handle.is_cuda() && handle.numel() == sizeof(cudaIpcMemHandle_t));
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle.data_ptr(), sizeof(h));
  void* p = nullptr;
  check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "ipc_open");
  return reinterpret_cast<int64_t>(p);
}
void ipc_close(int64_t ptr) { cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)); }
Tensor tensor_from_ptr(int64_t ptr, int64_t numel, int64_t dtype_code) {
  const auto dt = dtype_code == 0 ? at::kFloat
                  : dtype_code == 1 ? at::kBFloat16
                  : dtype_code == 2 ? at::kInt
                                    : at::kByte;
  return at::from_blob(reinterpret_cast<void*>(ptr), {numel},
                          at::TensorOptions().dtype(dt).device(at::kCUDA, at::cuda::current_device()));
}

#ifdef STB_WITH_ATTENTION
// bits[b, w] bit i = (mask[b, 32 w + i] != 0); `bits` is int32 [B, pitch], pitch a multiple of 4
// with at least four words per 128-key block.
void pack_key_mask(const Tensor& mask, Tensor bits) {
  need(mask, at::kByte, "mask");
  need(bits, at::kInt, "bits");
  TORCH_CHECK(mask.dim() == 2 && bits.dim() == 2 && mask.is_contiguous() && bits.is_contiguous() &&
                  mask.size(0) == bits.size(0), "pack_key_mask: [B, S] uint8 -> [B, pitch] int32");
  check(stb::launch_pack_key_mask(mask.data_ptr<uint8_t>(),
                                  reinterpret_cast<uint32_t*>(bits.data_ptr<int>()),
                                  static_cast<int>(mask.size(0)), static_cast<int>(mask.size(1)),
                                  static_cast<int>(bits.size(1)), cur_stream()),
        "pack_key_mask");
}

// `mask`: uint8 [B, S] key mask, or its packed int32 form (pack_key_mask)
void set_mask(const c10::optional<Tensor>& mask, const uint8_t** bytes, const uint32_t** bits,
              int* pitch) {
  *bytes = nullptr;
  *bits = nullptr;
  *pitch = 0;
  if (!mask.has_value()) return;
  if (mask->scalar_type() == at::kInt) {
    TORCH_CHECK(mask->dim() == 2 && mask->is_contiguous(), "packed key mask must be [B, words]");
    *bits = reinterpret_cast<const uint32_t*>(mask->data_ptr<int>());
    *pitch = static_cast<int>(mask->size(1));
  } else {
    *bytes = mask->data_ptr<uint8_t>();
  }
}

void attention_fwd(const Tensor& qkv, Tensor out, Tensor lse, const c10::optional<Tensor>& mask,
                   int64_t batch, int64_t seq, int64_t hq, int64_t hkv, double scale) {
  need(qkv, at::kBFloat16, "qkv");
  need(out, at::kBFloat16, "out");
  need(lse, at::kFloat, "lse");
  stb::AttnCall c{};
  c.qkv = qkv.data_ptr();
  c.out = out.data_ptr();
  c.lse = lse.data_ptr<float>();
  set_mask(mask, &c.key_mask, &c.key_bits, &c.key_bits_pitch);
  c.batch = static_cast<int>(batch);
  c.seq = static_cast<int>(seq);
  c.hq = static_cast<int>(hq);
  c.hkv = static_cast<int>(hkv);
  c.scale = static_cast<float>(scale);
  check(stb::launch_attention_fwd(c, status_ptr(), cur_stream()), "attention_fwd");
}

void attention_bwd(const Tensor& qkv, const Tensor& out, const Tensor& dout, const Tensor& lse,
                   Tensor delta, Tensor dqkv, Tensor dkv_accum, const c10::optional<Tensor>& mask,
                   int64_t batch, int64_t seq, int64_t hq, int64_t hkv, double scale) {
  stb::AttnBwdCall c{};
  c.qkv = qkv.data_ptr();
  c.out = out.data_ptr();
  c.dout = dout.data_ptr();
  c.lse = lse.data_ptr<float>();
  c.delta = delta.data_ptr<float>();
  c.dqkv = dqkv.data_ptr();
  const int parts = stb::attention_bwd_parts(static_cast<int>(batch), static_cast<int>(seq),
                                             static_cast<int>(hq), static_cast<int>(hkv));
  const int64_t need = static_cast<int64_t>(parts) * batch * seq * 2 * hkv * 128;
  // a scratch too small for the split (callers may pass any placeholder) keeps the unsplit path
  const bool split = parts > 1 && dkv_accum.defined() && dkv_accum.scalar_type() == at::kFloat &&
                     dkv_accum.numel() >= need;
  c.dkv_accum = split ? dkv_accum.data_ptr<float>() : nullptr;
  c.dkv_accum_floats = split ? dkv_accum.numel() : 0;
  set_mask(mask, &c.key_mask, &c.key_bits, &c.key_bits_pitch);
  c.batch = static_cast<int>(batch);
  c.seq = static_cast<int>(seq);
  c.hq = static_cast<int>(hq);
  c.hkv = static_cast<int>(hkv);
  c.scale = static_cast<float>(scale);
  check(stb::launch_attention_bwd(c, status_ptr(), cur_stream()), "attention_bwd");
}
#endif

}  // namespace

TORCH_LIBRARY(stb, m) {
  m.def("status_read", &status_read);
  m.def("status_reset", &status_reset);
  m.def("status_tensor", &status_tensor_op);
  m.def("gemm(Tensor a, Tensor b, Tensor out, bool a_mn, bool b_mn, Tensor? bias, Tensor? residual, "
        "bool accumulate, float alpha, int force_bn, int split_k=0, bool staged_store=True) -> ()",
        &gemm);
  m.def("gemm_scatter", &gemm_scatter);
  m.def("gemm_seq_pull", &gemm_seq_pull);
  m.def("gemm_swiglu", &gemm_swiglu);
  m.def("gemm_broadcast", &gemm_broadcast);
  m.def("slot_sum_rmsnorm", &slot_sum_rmsnorm);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("colsum_f32", &colsum_f32);
  m.def("colsum_bf16", &colsum_bf16);
  m.def("rope", &rope);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("ce_fwd", &ce_fwd);
  m.def("ce_bwd", &ce_bwd);
  m.def("sum_f32", &sum_f32);
  m.def("embedding_scatter_add", &embedding_scatter_add);
  m.def("cast_bf16", &cast_bf16);
  m.def("add_f32", &add_f32);
  m.def("adamw", &adamw);
  m.def("sgd", &sgd);
  m.def("grad_check", &grad_check);
  m.def("gather_params(int[] shard_ptrs, Tensor segs, Tensor full_bf16, Tensor full_fp32, "
        "int[] shadow_ptrs=[]) -> ()",
        &gather_params);
  m.def("reduce_scatter(int[] full_ptrs, int rank, Tensor segs, Tensor grad_shard, float scale, "
        "bool accumulate, Tensor? flags, int tp_degree=1, int tp_rank=0, float rep_scale=1.0, "
        "int multicast_ptr=0) -> ()",
        &reduce_scatter);
  m.def("reduce_scatter_adamw(int[] full_ptrs, int rank, Tensor segs, Tensor grad_shard, Tensor p, "
        "Tensor m, Tensor v, float scale, bool accumulate, float lr, float b1, float b2, float eps, "
        "float wd, float bc1, float bc2, float gscale, Tensor? flags, int tp_degree=1, "
        "int tp_rank=0, float rep_scale=1.0, Tensor? shadow=None, int multicast_ptr=0) -> ()",
        &reduce_scatter_adamw);
  m.def("gemm_allgather(Tensor a, Tensor out, Tensor? bias, int[] arena_ptrs, bool wire_fp32, "
        "Tensor segs, Tensor? full, Tensor? gated_out, int force_bn=0) -> ()",
        &gemm_allgather);
  m.def("embedding_gather_sharded", &embedding_gather_sharded);
  m.def("seq_gather", &seq_gather);
  m.def("seq_reduce_scatter", &seq_reduce_scatter);
  m.def("peer_barrier", &peer_barrier);
  m.def("peer_allreduce_small", &peer_allreduce_small);
  m.def("peer_alloc", &peer_alloc);
  m.def("peer_free", &peer_free);
  m.def("device_synchronize", &device_synchronize);
  m.def("launch_count", &launch_count);
  m.def("unpack_gathered", &unpack_gathered);
  m.def("pack_gradients", &pack_gradients);
  m.def("enable_peer_access", &enable_peer_access);
  m.def("ipc_handle", &ipc_handle);
  m.def("ipc_open", &ipc_open);
  m.def("ipc_close", &ipc_close);
  m.def("tensor_from_ptr", &tensor_from_ptr);
#ifdef STB_WITH_ATTENTION
  m.def("pack_key_mask", &pack_key_mask);
  m.def("attention_fwd", &attention_fwd);
  m.def("attention_bwd", &attention_bwd);
#endif
}
