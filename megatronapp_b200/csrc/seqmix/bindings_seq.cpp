// PyTorch bindings of the sequence-mixing kernels (pybind11 module megatronapp_b200._C_seq).
#include <torch/extension.h>
#include <algorithm>
#include <atomic>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "seqmix_api.h"

using torch::Tensor;

namespace {

std::atomic<int64_t> g_launches{0};
inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline void count(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

bool act_is_bf16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kFloat, name, " must be bf16 or fp32, got ", t.scalar_type());
  return t.scalar_type() == at::kBFloat16;
}
void check_f32(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous(), name, " must be a contiguous fp32 CUDA tensor");
}
void check_i32(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous(), name, " must be a contiguous int32 CUDA tensor");
}
void check_rows(const Tensor& t, const char* name) {   // [T, ...] with contiguous trailing dims and a free row stride
  TORCH_CHECK(t.dim() == 3 && t.stride(2) == 1 && t.stride(1) == t.size(2), name, " must be [T, heads, dim] with contiguous heads");
}
void check_last_error(const char* what) {
  cudaError_t e = cudaGetLastError();
  TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e));
}

void add_rms_norm(Tensor x, c10::optional<Tensor> delta, const Tensor& w, Tensor y, double eps, double w_off) {
  check_f32(x, "x");
  const bool bf16 = act_is_bf16(y, "y");
  TORCH_CHECK(x.dim() == 2 && y.is_contiguous() && y.sizes() == x.sizes(), "x / y must be [rows, cols]");
  TORCH_CHECK(w.scalar_type() == y.scalar_type() && w.is_contiguous() && w.numel() == x.size(1), "weight must match y's dtype and cols");
  TORCH_CHECK(x.size(1) * sizeof(float) <= 48 * 1024, "row too wide");
  const void* d = nullptr;
  if (delta.has_value() && delta->defined()) {
    TORCH_CHECK(delta->scalar_type() == y.scalar_type() && delta->is_contiguous() && delta->sizes() == x.sizes(),
                "delta must be contiguous, shaped like x, in y's dtype");
    d = delta->data_ptr();
  }
  c10::cuda::CUDAGuard g(x.device());
  b200seq::add_rms_norm(x.data_ptr<float>(), d, w.data_ptr(), y.data_ptr(), static_cast<int>(x.size(0)), static_cast<int>(x.size(1)),
                        static_cast<float>(eps), static_cast<float>(w_off), bf16, cur_stream());
  count(); check_last_error("add_rms_norm");
}

void gated_head_rms_norm(const Tensor& o, c10::optional<Tensor> w_opt, c10::optional<Tensor> gate, Tensor y, double eps, bool silu) {
  check_f32(o, "o");
  TORCH_CHECK(o.dim() == 3, "o must be [T, H, dv]");
  const bool bf16 = act_is_bf16(y, "y");
  const int T = static_cast<int>(o.size(0)), H = static_cast<int>(o.size(1)), dv = static_cast<int>(o.size(2));
  TORCH_CHECK(y.is_contiguous() && y.numel() == o.numel(), "y must be [T, H * dv]");
  const void* wp = nullptr;
  bool per_head = false;
  if (w_opt.has_value() && w_opt->defined()) {
    const Tensor& w = *w_opt;
    TORCH_CHECK(w.is_cuda() && w.scalar_type() == y.scalar_type() && w.is_contiguous() && (w.numel() == dv || w.numel() == H * dv), "bad weight");
    wp = w.data_ptr(); per_head = w.numel() != dv || H == 1;
  }
  const void* gp = nullptr;
  int64_t ldg = 0;
  if (gate.has_value() && gate->defined()) {
    TORCH_CHECK(gate->is_cuda() && gate->scalar_type() == y.scalar_type() && gate->dim() == 2 && gate->stride(1) == 1 && gate->size(0) == T &&
                gate->size(1) == static_cast<int64_t>(H) * dv, "gate must be [T, H * dv] with unit inner stride");
    gp = gate->data_ptr(); ldg = gate->stride(0);
  }
  c10::cuda::CUDAGuard g(o.device());
  b200seq::gated_head_rms_norm(o.data_ptr<float>(), wp, gp, ldg, y.data_ptr(), T, H, dv, per_head, eps, silu, bf16, cur_stream());
  count(); check_last_error("gated_head_rms_norm");
}

void causal_conv(const Tensor& x, const Tensor& w, c10::optional<Tensor> bias, const Tensor& cu, const Tensor& rows,
                 const Tensor& tok_seq, Tensor window, Tensor y, int64_t max_len, bool silu, bool residual) {
  const bool bf16 = act_is_bf16(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1, "x must be [T, C] with unit inner stride");
  const int T = static_cast<int>(x.size(0)), C = static_cast<int>(x.size(1)), taps = static_cast<int>(w.size(1));
  TORCH_CHECK(w.scalar_type() == x.scalar_type() && w.is_contiguous() && w.size(0) == C, "bad conv weight");
  TORCH_CHECK(y.scalar_type() == x.scalar_type() && y.is_contiguous() && y.sizes() == x.sizes(), "bad y");
  TORCH_CHECK(window.scalar_type() == x.scalar_type() && window.is_contiguous() && window.dim() == 3 && window.size(1) == taps - 1 &&
              window.size(2) == C, "window must be [rows, taps - 1, C]");
  check_i32(cu, "cu"); check_i32(rows, "rows"); check_i32(tok_seq, "tok_seq");
  TORCH_CHECK(tok_seq.numel() == T && cu.numel() == rows.numel() + 1, "bad packed-batch tensors");
  const void* bp = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->scalar_type() == x.scalar_type() && bias->is_contiguous() && bias->numel() == C, "bad conv bias");
    bp = bias->data_ptr();
  }
  c10::cuda::CUDAGuard g(x.device());
  b200seq::causal_conv_silu(x.data_ptr(), x.stride(0), w.data_ptr(), bp, cu.data_ptr<int>(), rows.data_ptr<int>(), tok_seq.data_ptr<int>(),
                            window.data_ptr(), y.data_ptr(), T, static_cast<int>(rows.numel()), C, taps, static_cast<int>(max_len), silu, residual, bf16,
                            cur_stream());
  count(2); check_last_error("causal_conv_silu");
}

void delta_rule_scan(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& log_decay, const Tensor& beta, const Tensor& cu,
                     const Tensor& rows, Tensor state, Tensor out, double unit_eps, double q_scale, int64_t max_len) {
  const bool bf16 = act_is_bf16(q, "q");
  TORCH_CHECK(k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type(), "q / k / v dtypes differ");
  check_rows(q, "q"); check_rows(k, "k"); check_rows(v, "v");
  check_f32(log_decay, "log_decay"); check_f32(beta, "beta"); check_f32(state, "state"); check_f32(out, "out");
  check_i32(cu, "cu"); check_i32(rows, "rows");
  b200seq::DeltaArgs p{};
  p.q = q.data_ptr(); p.k = k.data_ptr(); p.v = v.data_ptr();
  p.ldq = q.stride(0); p.ldk = k.stride(0); p.ldv = v.stride(0);
  p.H = static_cast<int>(v.size(1)); p.KH = static_cast<int>(q.size(1)); p.d = static_cast<int>(q.size(2)); p.dv = static_cast<int>(v.size(2));
  TORCH_CHECK(p.H % p.KH == 0 && k.size(1) == p.KH && k.size(2) == p.d, "bad head layout");
  p.decay_per_head = log_decay.numel() == q.size(0) * p.H && (log_decay.dim() == 2 || p.d == 1) ? 1 : 0;
  TORCH_CHECK((p.decay_per_head || log_decay.numel() == q.size(0) * p.H * p.d) && beta.numel() == q.size(0) * p.H, "bad decay / beta shape");
  TORCH_CHECK(state.dim() == 4 && state.size(1) == p.H && state.size(2) == p.d && state.size(3) == p.dv, "bad state shape");
  TORCH_CHECK(out.numel() == q.size(0) * p.H * p.dv, "bad out shape");
  p.log_decay = log_decay.data_ptr<float>(); p.beta = beta.data_ptr<float>();
  p.cu = cu.data_ptr<int>(); p.rows = rows.data_ptr<int>();
  p.state = state.data_ptr<float>(); p.out = out.data_ptr<float>();
  p.unit_eps = static_cast<float>(unit_eps); p.q_scale = static_cast<float>(q_scale);
  p.max_len = max_len > 0 ? static_cast<int>(max_len) : (1 << 30);
  c10::cuda::CUDAGuard g(q.device());
  TORCH_CHECK(b200seq::delta_rule_scan(p, static_cast<int>(rows.numel()), bf16, cur_stream()), "delta_rule_scan: key dim ", p.d,
              " above the largest kernel instance (256)");
  count(); check_last_error("delta_rule_scan");
}

void mlstm_scan(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& log_i, const Tensor& log_f, const Tensor& cu,
                const Tensor& rows, Tensor state, Tensor norm_state, Tensor max_state, Tensor out, double q_scale, double denom_eps,
                int64_t max_len) {
  const bool bf16 = act_is_bf16(q, "q");
  TORCH_CHECK(k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type(), "q / k / v dtypes differ");
  check_rows(q, "q"); check_rows(k, "k"); check_rows(v, "v");
  check_f32(log_i, "log_i"); check_f32(log_f, "log_f"); check_f32(state, "state"); check_f32(norm_state, "norm_state");
  check_f32(max_state, "max_state"); check_f32(out, "out");
  check_i32(cu, "cu"); check_i32(rows, "rows");
  b200seq::MlstmArgs p{};
  p.q = q.data_ptr(); p.k = k.data_ptr(); p.v = v.data_ptr();
  p.ldq = q.stride(0); p.ldk = k.stride(0); p.ldv = v.stride(0);
  p.H = static_cast<int>(v.size(1)); p.d = static_cast<int>(q.size(2)); p.dv = static_cast<int>(v.size(2));
  TORCH_CHECK(q.size(1) == p.H && k.size(1) == p.H && k.size(2) == p.d, "bad head layout");
  TORCH_CHECK(log_i.numel() == q.size(0) * p.H && log_f.numel() == q.size(0) * p.H, "bad gate shape");
  TORCH_CHECK(state.dim() == 4 && state.size(1) == p.H && state.size(2) == p.d && state.size(3) == p.dv, "bad state shape");
  TORCH_CHECK(norm_state.numel() == state.size(0) * p.H * p.d && max_state.numel() == state.size(0) * p.H, "bad n / m shape");
  TORCH_CHECK(out.numel() == q.size(0) * p.H * p.dv, "bad out shape");
  p.log_i = log_i.data_ptr<float>(); p.log_f = log_f.data_ptr<float>();
  p.cu = cu.data_ptr<int>(); p.rows = rows.data_ptr<int>();
  p.state = state.data_ptr<float>(); p.norm_state = norm_state.data_ptr<float>(); p.max_state = max_state.data_ptr<float>();
  p.out = out.data_ptr<float>();
  p.q_scale = static_cast<float>(q_scale); p.denom_eps = static_cast<float>(denom_eps);
  p.max_len = max_len > 0 ? static_cast<int>(max_len) : (1 << 30);
  c10::cuda::CUDAGuard g(q.device());
  TORCH_CHECK(b200seq::mlstm_scan(p, static_cast<int>(rows.numel()), bf16, cur_stream()), "mlstm_scan: key dim ", p.d,
              " above the largest kernel instance (256)");
  count(); check_last_error("mlstm_scan");
}

void latent_attention_paged(const Tensor& q, const Tensor& cache, const Tensor& block_table, const Tensor& tok_req, const Tensor& tok_len,
                            Tensor out, int64_t block_size, double scale, int64_t max_len) {
  const bool bf16 = act_is_bf16(q, "q_lat");
  TORCH_CHECK(q.dim() == 3 && q.is_contiguous(), "q_lat must be contiguous [T, H, r]");
  TORCH_CHECK(cache.scalar_type() == q.scalar_type() && cache.dim() == 2 && cache.is_contiguous() && cache.size(1) == q.size(2),
              "cache must be [slots, r] in q_lat's dtype");
  check_i32(block_table, "block_table"); check_i32(tok_req, "tok_req"); check_i32(tok_len, "tok_len"); check_f32(out, "out");
  TORCH_CHECK(block_table.dim() == 2 && tok_req.numel() == q.size(0) && tok_len.numel() == q.size(0) && out.numel() == q.numel(),
              "bad shapes");
  b200seq::LatentAttnArgs p{};
  p.q = q.data_ptr(); p.cache = cache.data_ptr();
  p.block_table = block_table.data_ptr<int>(); p.tok_req = tok_req.data_ptr<int>(); p.tok_len = tok_len.data_ptr<int>();
  p.out = out.data_ptr<float>();
  p.H = static_cast<int>(q.size(1)); p.r = static_cast<int>(q.size(2)); p.block_size = static_cast<int>(block_size);
  p.max_blocks = static_cast<int>(block_table.size(1)); p.scale = static_cast<float>(scale);
  c10::cuda::CUDAGuard g(q.device());
  p.n_splits = b200seq::latent_attention_splits(p.H, p.r, static_cast<int>(q.size(0)), static_cast<int>(max_len));
  const int64_t vec = 16 / static_cast<int64_t>(cache.element_size());
  p.vec_ok = (p.r % vec == 0 && reinterpret_cast<uintptr_t>(cache.data_ptr()) % 16 == 0) ? 1 : 0;
  Tensor ws;
  if (p.n_splits > 1) {
    ws = torch::empty({q.size(0), q.size(1), p.n_splits, q.size(2) + 2}, out.options());
    p.ws = ws.data_ptr<float>();
  }
  TORCH_CHECK(b200seq::latent_attention_paged(p, static_cast<int>(q.size(0)), bf16, cur_stream()), "latent_attention_paged: rank ", p.r,
              " above the largest kernel instance (1024)");
  count(p.n_splits > 1 ? 2 : 1); check_last_error("latent_attention_paged");
}

void group_limited_router(const Tensor& logits, Tensor probs, Tensor rmap, int64_t topk, int64_t groups, int64_t keep, bool renorm) {
  check_f32(logits, "logits"); check_f32(probs, "probs");
  TORCH_CHECK(logits.dim() == 2 && probs.sizes() == logits.sizes() && rmap.sizes() == logits.sizes() && rmap.scalar_type() == at::kBool &&
              rmap.is_contiguous(), "bad shapes");
  c10::cuda::CUDAGuard g(logits.device());
  TORCH_CHECK(b200seq::group_limited_router(logits.data_ptr<float>(), probs.data_ptr<float>(), rmap.data_ptr<bool>(),
                                            static_cast<int>(logits.size(0)), static_cast<int>(logits.size(1)), static_cast<int>(topk),
                                            static_cast<int>(groups), static_cast<int>(keep), renorm, cur_stream()),
              "group_limited_router: unsupported sizes (experts ", logits.size(1), ", groups ", groups, ", top ", topk, ")");
  count(); check_last_error("group_limited_router");
}


// ---- side-by-side mixer, minGRU, clamped gated activation ------------------------------------------------------------------
const void* opt_ptr(const c10::optional<Tensor>& t) { return (t.has_value() && t->defined()) ? t->data_ptr() : nullptr; }
void check_act2(const Tensor& t, const Tensor& like, const char* name) {   // [T, C], unit inner stride, free row stride
  TORCH_CHECK(t.is_cuda() && t.dim() == 2 && t.stride(1) == 1 && t.scalar_type() == like.scalar_type(), name,
              " must be a [T, C] CUDA tensor with unit inner stride in the activation dtype");
}

void norm_add(Tensor x, const Tensor& a, c10::optional<Tensor> b, c10::optional<Tensor> wa, c10::optional<Tensor> wb,
              c10::optional<Tensor> w, Tensor y, double eps, double w_off, c10::optional<Tensor> extra, c10::optional<Tensor> next_w) {
  check_f32(x, "x");
  const bool bf16 = act_is_bf16(y, "y");
  TORCH_CHECK(x.dim() == 2 && y.is_contiguous() && y.sizes() == x.sizes(), "x / y must be [rows, cols]");
  TORCH_CHECK(a.is_cuda() && a.scalar_type() == y.scalar_type() && a.is_contiguous() && a.sizes() == x.sizes(), "a must be contiguous, shaped like x");
  TORCH_CHECK(x.size(1) * sizeof(float) <= 48 * 1024, "row too wide");
  auto vec = [&](const c10::optional<Tensor>& t, const char* name) -> const void* {
    if (!t.has_value() || !t->defined()) return nullptr;
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == y.scalar_type() && t->is_contiguous() && t->numel() == x.size(1), name,
                " must be a contiguous [cols] tensor in y's dtype");
    return t->data_ptr();
  };
  const bool two = b.has_value() && b->defined();
  if (two) {
    TORCH_CHECK(b->is_cuda() && b->scalar_type() == y.scalar_type() && b->is_contiguous() && b->sizes() == x.sizes(), "b must be shaped like a");
    TORCH_CHECK(vec(wa, "weight_a") != nullptr && vec(wb, "weight_b") != nullptr, "two branches need their norm weights");
  }
  const void* ex = nullptr;
  if (extra.has_value() && extra->defined()) {
    TORCH_CHECK(extra->is_cuda() && extra->scalar_type() == y.scalar_type() && extra->is_contiguous() && extra->sizes() == x.sizes(),
                "extra must be contiguous, shaped like x, in y's dtype");
    ex = extra->data_ptr();
  }
  c10::cuda::CUDAGuard g(x.device());
  b200seq::norm_add(x.data_ptr<float>(), a.data_ptr(), two ? b->data_ptr() : nullptr, two ? vec(wa, "weight_a") : nullptr,
                    two ? vec(wb, "weight_b") : nullptr, vec(w, "weight"), y.data_ptr(), static_cast<int>(x.size(0)),
                    static_cast<int>(x.size(1)), static_cast<float>(eps), static_cast<float>(w_off), ex, vec(next_w, "next_weight"), bf16,
                    cur_stream());
  count(); check_last_error("norm_add");
}

void retention_scan(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& decay, c10::optional<Tensor> positions,
                    c10::optional<Tensor> inv_freq, const Tensor& cu, const Tensor& rows, Tensor state, Tensor out, double k_scale,
                    int64_t max_len) {
  const bool bf16 = act_is_bf16(q, "q");
  TORCH_CHECK(k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type(), "q / k / v dtypes differ");
  check_rows(q, "q"); check_rows(k, "k"); check_rows(v, "v");
  check_f32(decay, "decay"); check_f32(state, "state"); check_f32(out, "out");
  check_i32(cu, "cu"); check_i32(rows, "rows");
  b200seq::RetentionArgs p{};
  p.q = q.data_ptr(); p.k = k.data_ptr(); p.v = v.data_ptr();
  p.ldq = q.stride(0); p.ldk = k.stride(0); p.ldv = v.stride(0);
  p.H = static_cast<int>(v.size(1)); p.d = static_cast<int>(q.size(2)); p.dv = static_cast<int>(v.size(2));
  TORCH_CHECK(q.size(1) == p.H && k.size(1) == p.H && k.size(2) == p.d && v.size(0) == q.size(0) && k.size(0) == q.size(0), "bad head layout");
  TORCH_CHECK(decay.numel() == p.H, "decay must be [H]");
  TORCH_CHECK(state.dim() == 4 && state.size(1) == p.H && state.size(2) == p.d && state.size(3) == p.dv, "bad state shape");
  TORCH_CHECK(out.numel() == q.size(0) * p.H * p.dv, "bad out shape");
  if (inv_freq.has_value() && inv_freq->defined() && inv_freq->numel() > 0) {
    check_f32(*inv_freq, "inv_freq");
    p.n_rot = static_cast<int>(inv_freq->numel());
    TORCH_CHECK(2 * p.n_rot <= p.d, "more rotated dimensions than the head has");
    TORCH_CHECK(positions.has_value() && positions->is_cuda() && positions->scalar_type() == at::kLong && positions->is_contiguous() &&
                positions->numel() == q.size(0), "positions must be a contiguous int64 [T]");
    p.inv_freq = inv_freq->data_ptr<float>(); p.positions = positions->data_ptr<int64_t>();
  }
  p.decay = decay.data_ptr<float>();
  p.cu = cu.data_ptr<int>(); p.rows = rows.data_ptr<int>();
  p.state = state.data_ptr<float>(); p.out = out.data_ptr<float>();
  p.k_scale = static_cast<float>(k_scale);
  p.max_len = max_len > 0 ? static_cast<int>(max_len) : (1 << 30);
  c10::cuda::CUDAGuard g(q.device());
  TORCH_CHECK(b200seq::retention_scan(p, static_cast<int>(rows.numel()), bf16, cur_stream()), "retention_scan: key dim ", p.d,
              " above the largest kernel instance (256)");
  count(); check_last_error("retention_scan");
}

void poly_norm(const Tensor& z, const Tensor& coef, Tensor y, double eps) {
  const bool bf16 = act_is_bf16(z, "z");
  check_act2(z, z, "z"); check_f32(coef, "coef");
  TORCH_CHECK(coef.numel() == 4, "coef must hold four numbers");
  TORCH_CHECK(y.scalar_type() == z.scalar_type() && y.is_contiguous() && y.sizes() == z.sizes(), "bad y");
  c10::cuda::CUDAGuard g(z.device());
  TORCH_CHECK(b200seq::poly_norm(z.data_ptr(), z.stride(0), coef.data_ptr<float>(), y.data_ptr(), z.size(0), static_cast<int>(z.size(1)),
                                 static_cast<float>(eps), bf16, cur_stream()), "poly_norm: row too wide");
  count(); check_last_error("poly_norm");
}

void decay_gates(const Tensor& a, const Tensor& b, const Tensor& A_log, const Tensor& dt_bias, Tensor log_decay, Tensor beta) {
  const bool bf16 = act_is_bf16(a, "a");
  check_act2(a, a, "a"); check_act2(b, a, "b");
  check_f32(log_decay, "log_decay"); check_f32(beta, "beta");
  const int64_t rows = a.size(0);
  const int C = static_cast<int>(a.size(1)), H = static_cast<int>(b.size(1));
  TORCH_CHECK(b.size(0) == rows && H > 0 && C % H == 0, "a must be [T, C] and b [T, H] with C a multiple of H");
  TORCH_CHECK(A_log.is_cuda() && A_log.scalar_type() == a.scalar_type() && A_log.is_contiguous() && A_log.numel() == H &&
              dt_bias.is_cuda() && dt_bias.scalar_type() == a.scalar_type() && dt_bias.is_contiguous() && dt_bias.numel() == C, "bad A_log / dt_bias");
  TORCH_CHECK(log_decay.numel() == rows * C && beta.numel() == rows * H, "bad output shapes");
  c10::cuda::CUDAGuard g(a.device());
  b200seq::decay_gates(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), A_log.data_ptr(), dt_bias.data_ptr(), log_decay.data_ptr<float>(),
                       beta.data_ptr<float>(), rows, C, H, bf16, cur_stream());
  count(); check_last_error("decay_gates");
}

void gelu_mul(const Tensor& gt, const Tensor& e, Tensor y) {
  const bool bf16 = act_is_bf16(gt, "g");
  check_act2(gt, gt, "g"); check_act2(e, gt, "e");
  TORCH_CHECK(e.sizes() == gt.sizes() && y.scalar_type() == gt.scalar_type() && y.is_contiguous() && y.sizes() == gt.sizes(), "bad e / y");
  c10::cuda::CUDAGuard g(gt.device());
  b200seq::gelu_mul(gt.data_ptr(), gt.stride(0), e.data_ptr(), e.stride(0), y.data_ptr(), gt.size(0), static_cast<int>(gt.size(1)), bf16,
                    cur_stream());
  count(); check_last_error("gelu_mul");
}

void norm_rope(const Tensor& q, const Tensor& k, const Tensor& wq, const Tensor& wk, const Tensor& positions, const Tensor& inv_freq,
               Tensor q_out, Tensor k_out, int64_t head_dim, int64_t rot, double eps) {
  const bool bf16 = act_is_bf16(q, "q");
  check_act2(q, q, "q"); check_act2(k, q, "k");
  check_f32(inv_freq, "inv_freq");
  TORCH_CHECK(positions.is_cuda() && positions.scalar_type() == at::kLong && positions.is_contiguous() && positions.numel() == q.size(0),
              "positions must be a contiguous int64 [T]");
  TORCH_CHECK(rot % 2 == 0 && rot <= head_dim && inv_freq.numel() * 2 == rot, "rot must be even, at most head_dim, with rot / 2 frequencies");
  TORCH_CHECK(q.size(1) % head_dim == 0 && k.size(1) % head_dim == 0 && k.size(0) == q.size(0), "bad q / k shape");
  TORCH_CHECK(wq.scalar_type() == q.scalar_type() && wk.scalar_type() == q.scalar_type() && wq.is_contiguous() && wk.is_contiguous() &&
              wq.numel() == q.size(1) && wk.numel() == k.size(1), "bad norm weights");
  TORCH_CHECK(q_out.scalar_type() == q.scalar_type() && k_out.scalar_type() == q.scalar_type() && q_out.is_contiguous() &&
              k_out.is_contiguous() && q_out.numel() == q.numel() && k_out.numel() == k.numel(), "bad outputs");
  TORCH_CHECK((std::max(q.size(1), k.size(1)) + 1 + rot) * sizeof(float) <= 48 * 1024, "projection too wide");
  b200seq::NormRopeArgs p{};
  p.q = q.data_ptr(); p.k = k.data_ptr(); p.ldq = q.stride(0); p.ldk = k.stride(0);
  p.wq = wq.data_ptr(); p.wk = wk.data_ptr(); p.positions = positions.data_ptr<int64_t>(); p.inv_freq = inv_freq.data_ptr<float>();
  p.q_out = q_out.data_ptr(); p.k_out = k_out.data_ptr();
  p.q_ch = static_cast<int>(q.size(1)); p.k_ch = static_cast<int>(k.size(1)); p.head_dim = static_cast<int>(head_dim);
  p.rot = static_cast<int>(rot); p.eps = static_cast<float>(eps);
  c10::cuda::CUDAGuard g(q.device());
  b200seq::norm_rope(p, static_cast<int>(q.size(0)), bf16, cur_stream());
  count(); check_last_error("norm_rope");
}

void mixed_attention_paged(const Tensor& q, const Tensor& kcache, const Tensor& vcache, const Tensor& block_table, const Tensor& tok_req,
                           const Tensor& tok_len, c10::optional<Tensor> talk, c10::optional<Tensor> gate, Tensor out, int64_t block_size,
                           double scale, int64_t max_len, bool force_generic) {
  const bool bf16 = act_is_bf16(q, "q");
  check_rows(q, "q");
  TORCH_CHECK(kcache.scalar_type() == q.scalar_type() && vcache.scalar_type() == q.scalar_type() && kcache.dim() == 3 && vcache.dim() == 3 &&
              kcache.is_contiguous() && vcache.is_contiguous() && kcache.size(2) == q.size(2) && vcache.size(1) == kcache.size(1),
              "caches must be contiguous [slots, G, d] / [slots, G, dv] in q's dtype");
  check_i32(block_table, "block_table"); check_i32(tok_req, "tok_req"); check_i32(tok_len, "tok_len");
  b200seq::MixAttnArgs p{};
  p.H = static_cast<int>(q.size(1)); p.G = static_cast<int>(kcache.size(1)); p.d = static_cast<int>(q.size(2));
  p.dv = static_cast<int>(vcache.size(2));
  TORCH_CHECK(block_table.dim() == 2 && tok_req.numel() == q.size(0) && tok_len.numel() == q.size(0), "bad packed-batch tensors");
  TORCH_CHECK(out.scalar_type() == q.scalar_type() && out.is_contiguous() && out.numel() == q.size(0) * p.H * p.dv, "bad out");
  p.q = q.data_ptr(); p.ldq = q.stride(0); p.kcache = kcache.data_ptr(); p.vcache = vcache.data_ptr();
  p.block_table = block_table.data_ptr<int>(); p.tok_req = tok_req.data_ptr<int>(); p.tok_len = tok_len.data_ptr<int>();
  if (talk.has_value() && talk->defined()) {
    check_f32(*talk, "talk");
    TORCH_CHECK(talk->numel() == static_cast<int64_t>(p.H) * p.H, "talk must be [H, H]");
    p.talk = talk->data_ptr<float>();
  }
  if (gate.has_value() && gate->defined()) {
    check_act2(*gate, q, "gate");
    TORCH_CHECK(gate->size(0) == q.size(0) && gate->size(1) == p.H * p.dv, "gate must be [T, H * dv]");
    p.gate = gate->data_ptr(); p.ldg = gate->stride(0);
  }
  p.out = out.data_ptr();
  p.block_size = static_cast<int>(block_size); p.max_blocks = static_cast<int>(block_table.size(1)); p.scale = static_cast<float>(scale);
  c10::cuda::CUDAGuard g(q.device());
  p.n_splits = b200seq::mixed_attention_splits(static_cast<int>(q.size(0)), static_cast<int>(max_len));
  p.query_block = static_cast<int>(q.size(0) / std::max<int64_t>(1, block_table.size(0)));
  p.force_generic = force_generic ? 1 : 0;
  Tensor ws1, ws2;
  if (p.n_splits > 1) {
    auto o32 = q.options().dtype(at::kFloat);
    ws1 = torch::empty({q.size(0), p.n_splits, p.H, 2}, o32);
    ws2 = torch::empty({q.size(0), p.n_splits, static_cast<int64_t>(p.H) * p.dv}, o32);
    p.ws_stats = ws1.data_ptr<float>(); p.ws_acc = ws2.data_ptr<float>();
  }
  TORCH_CHECK(b200seq::mixed_attention_paged(p, static_cast<int>(q.size(0)), bf16, cur_stream()),
              "mixed_attention_paged: no kernel instance for heads ", p.H, " / ", p.G, ", dims ", p.d, " / ", p.dv);
  count(p.n_splits > 1 ? 3 : 1); check_last_error("mixed_attention_paged");
}

void gen_delta_scan(const Tensor& r, const Tensor& k, const Tensor& v, const Tensor& w_pre, const Tensor& a_pre, c10::optional<Tensor> w_bias,
                    const Tensor& cu, const Tensor& rows, Tensor state, Tensor out, double decay_scale, double unit_eps,
                    int64_t max_len) {
  const bool bf16 = act_is_bf16(r, "r");
  check_rows(r, "r"); check_rows(k, "k"); check_rows(v, "v");
  check_act2(w_pre, r, "w_pre"); check_act2(a_pre, r, "a_pre");
  TORCH_CHECK(k.scalar_type() == r.scalar_type() && v.scalar_type() == r.scalar_type(), "r / k / v dtypes differ");
  check_f32(state, "state"); check_f32(out, "out"); check_i32(cu, "cu"); check_i32(rows, "rows");
  b200seq::GenDeltaArgs p{};
  p.H = static_cast<int>(r.size(1)); p.d = static_cast<int>(r.size(2)); p.dv = static_cast<int>(v.size(2));
  TORCH_CHECK(k.size(1) == p.H && k.size(2) == p.d && v.size(1) == p.H, "bad head layout");
  TORCH_CHECK(w_pre.size(0) == r.size(0) && a_pre.size(0) == r.size(0) && w_pre.size(1) == p.H * p.d && a_pre.size(1) == p.H * p.d,
              "decay / removal pre-activations must be [T, H * d]");
  TORCH_CHECK(state.dim() == 4 && state.size(1) == p.H && state.size(2) == p.d && state.size(3) == p.dv, "bad state shape");
  TORCH_CHECK(out.numel() == r.size(0) * p.H * p.dv, "bad out shape");
  if (w_bias.has_value() && w_bias->defined()) {
    TORCH_CHECK(w_bias->scalar_type() == r.scalar_type() && w_bias->is_contiguous() && w_bias->numel() == p.H * p.d, "bad decay bias");
    p.w_bias = w_bias->data_ptr();
  }
  p.r = r.data_ptr(); p.k = k.data_ptr(); p.v = v.data_ptr(); p.w_pre = w_pre.data_ptr(); p.a_pre = a_pre.data_ptr();
  p.ldr = r.stride(0); p.ldk = k.stride(0); p.ldv = v.stride(0); p.ldw = w_pre.stride(0); p.lda = a_pre.stride(0);
  p.cu = cu.data_ptr<int>(); p.rows = rows.data_ptr<int>(); p.state = state.data_ptr<float>(); p.out = out.data_ptr<float>();
  p.decay_scale = static_cast<float>(decay_scale); p.unit_eps = static_cast<float>(unit_eps);
  p.max_len = max_len > 0 ? static_cast<int>(max_len) : (1 << 30);
  c10::cuda::CUDAGuard g(r.device());
  TORCH_CHECK(b200seq::gen_delta_scan(p, static_cast<int>(rows.numel()), bf16, cur_stream()), "gen_delta_scan: key dim ", p.d,
              " above the largest kernel instance (256)");
  count(); check_last_error("gen_delta_scan");
}

void mingru_scan(const Tensor& z_pre, const Tensor& u_pre, const Tensor& g_pre, const Tensor& cu, const Tensor& rows, Tensor state, Tensor y,
                 int64_t max_len) {
  const bool bf16 = act_is_bf16(z_pre, "z_pre");
  check_act2(z_pre, z_pre, "z_pre"); check_act2(u_pre, z_pre, "u_pre"); check_act2(g_pre, z_pre, "g_pre");
  check_f32(state, "state"); check_i32(cu, "cu"); check_i32(rows, "rows");
  b200seq::MinGruArgs p{};
  p.C = static_cast<int>(z_pre.size(1));
  TORCH_CHECK(u_pre.sizes() == z_pre.sizes() && g_pre.sizes() == z_pre.sizes() && state.dim() == 2 && state.size(1) == p.C, "bad shapes");
  TORCH_CHECK(y.scalar_type() == z_pre.scalar_type() && y.is_contiguous() && y.sizes() == z_pre.sizes(), "bad y");
  p.z_pre = z_pre.data_ptr(); p.u_pre = u_pre.data_ptr(); p.g_pre = g_pre.data_ptr();
  p.ldz = z_pre.stride(0); p.ldu = u_pre.stride(0); p.ldg = g_pre.stride(0);
  p.cu = cu.data_ptr<int>(); p.rows = rows.data_ptr<int>(); p.state = state.data_ptr<float>(); p.y = y.data_ptr();
  c10::cuda::CUDAGuard g(z_pre.device());
  const int R = static_cast<int>(rows.numel());
  p.max_runs = b200seq::mingru_runs(static_cast<int>(max_len));
  Tensor ws;
  if (p.max_runs > 1) {
    ws = torch::empty({R, p.max_runs, p.C, 2}, state.options());
    p.ws = ws.data_ptr<float>();
  }
  b200seq::mingru_scan(p, R, bf16, cur_stream());
  count(p.max_runs > 1 ? 3 : 1); check_last_error("mingru_scan");
}

void clamped_glu(const Tensor& x, Tensor y, double limit, double alpha, double shift) {
  const bool bf16 = act_is_bf16(x, "x");
  check_act2(x, x, "x");
  TORCH_CHECK(x.size(1) % 2 == 0 && y.scalar_type() == x.scalar_type() && y.is_contiguous() && y.dim() == 2 && y.size(0) == x.size(0) &&
              y.size(1) * 2 == x.size(1), "x must be [T, 2 F], y [T, F]");
  c10::cuda::CUDAGuard g(x.device());
  b200seq::clamped_glu(x.data_ptr(), x.stride(0), y.data_ptr(), x.size(0), static_cast<int>(y.size(1)), static_cast<float>(limit),
                       static_cast<float>(alpha), static_cast<float>(shift), bf16, cur_stream());
  count(); check_last_error("clamped_glu");
}



void stream_mix_norm(Tensor x, c10::optional<Tensor> a, c10::optional<Tensor> b, c10::optional<Tensor> bias_a, c10::optional<Tensor> ls,
                     double scale_a, double scale_b, c10::optional<Tensor> mix, c10::optional<Tensor> outc, c10::optional<Tensor> inp,
                     c10::optional<Tensor> w, c10::optional<Tensor> beta, c10::optional<Tensor> h, double eps, bool center) {
  check_f32(x, "x");
  TORCH_CHECK(x.dim() == 3, "x must be [T, S, W]");
  b200seq::StreamNormArgs p{};
  p.x = x.data_ptr<float>(); p.S = static_cast<int>(x.size(1)); p.W = static_cast<int>(x.size(2));
  const int64_t T = x.size(0);
  bool bf16 = false, have_dtype = false;
  auto act = [&](const Tensor& t, const char* name) {
    const bool is = act_is_bf16(t, name);
    TORCH_CHECK(!have_dtype || is == bf16, name, ": activation dtypes differ");
    bf16 = is; have_dtype = true;
  };
  auto vec = [&](const c10::optional<Tensor>& t, const char* name) -> const void* {
    if (!(t.has_value() && t->defined())) return nullptr;
    act(*t, name);
    TORCH_CHECK(t->is_contiguous() && t->numel() == p.W, name, " must hold W values");
    return t->data_ptr();
  };
  auto rows2 = [&](const c10::optional<Tensor>& t, const char* name, int64_t& ld) -> const void* {
    if (!(t.has_value() && t->defined())) return nullptr;
    act(*t, name);
    TORCH_CHECK(t->dim() == 2 && t->size(0) == T && t->size(1) == p.W && t->stride(1) == 1, name, " must be [T, W] with unit inner stride");
    ld = t->stride(0);
    return t->data_ptr();
  };
  p.a = rows2(a, "a", p.lda); p.b = rows2(b, "b", p.ldb);
  p.bias_a = vec(bias_a, "bias_a"); p.ls = vec(ls, "ls");
  p.scale_a = static_cast<float>(scale_a); p.scale_b = static_cast<float>(scale_b);
  if (p.a != nullptr) {
    TORCH_CHECK(mix.has_value() && outc.has_value(), "an update needs mix and out coefficients");
    check_f32(*mix, "mix"); check_f32(*outc, "outc");
    TORCH_CHECK(mix->numel() == p.S * p.S && outc->numel() == p.S, "mix must be [S, S], outc [S]");
    p.mix = mix->data_ptr<float>(); p.outc = outc->data_ptr<float>();
  }
  if (inp.has_value() && inp->defined()) {
    check_f32(*inp, "inp");
    TORCH_CHECK(inp->numel() == p.S && w.has_value() && h.has_value(), "inp must be [S]; the norm needs w and h");
    p.inp = inp->data_ptr<float>();
    p.w = vec(w, "w"); p.beta = vec(beta, "beta");
    act(*h, "h");
    TORCH_CHECK(h->is_contiguous() && h->numel() == T * p.W, "h must be contiguous [T, W]");
    p.h = h->data_ptr();
  }
  p.eps = static_cast<float>(eps); p.center = center ? 1 : 0;
  c10::cuda::CUDAGuard g(x.device());
  TORCH_CHECK(b200seq::stream_mix_norm(p, static_cast<int>(T), bf16, cur_stream()), "stream_mix_norm: ", p.S, " streams of width ", p.W,
              " have no kernel instance");
  count(); check_last_error("stream_mix_norm");
}

void add_sinusoid(Tensor x, const Tensor& positions, const Tensor& freq) {
  check_f32(x, "x"); check_f32(freq, "freq");
  TORCH_CHECK(x.dim() == 2 && x.size(1) % 2 == 0 && freq.numel() == x.size(1) / 2, "x must be [T, W] with even W and W / 2 frequencies");
  TORCH_CHECK(positions.is_cuda() && positions.scalar_type() == at::kLong && positions.is_contiguous() && positions.numel() == x.size(0),
              "positions must be a contiguous int64 CUDA tensor [T]");
  c10::cuda::CUDAGuard g(x.device());
  b200seq::add_sinusoid(x.data_ptr<float>(), positions.data_ptr<int64_t>(), freq.data_ptr<float>(), static_cast<int>(x.size(0)),
                        static_cast<int>(x.size(1)), cur_stream());
  count(); check_last_error("add_sinusoid");
}

void head_rms_norm(const Tensor& x, const Tensor& w, Tensor y, double eps) {
  const bool bf16 = act_is_bf16(x, "x");
  check_rows(x, "x");
  TORCH_CHECK(w.scalar_type() == x.scalar_type() && w.is_contiguous() && w.numel() == x.size(2), "weight must hold one value per channel of a head");
  TORCH_CHECK(y.scalar_type() == x.scalar_type() && y.is_contiguous() && y.numel() == x.numel(), "bad y");
  c10::cuda::CUDAGuard g(x.device());
  b200seq::head_rms_norm(x.data_ptr(), x.stride(0), w.data_ptr(), y.data_ptr(), static_cast<int>(x.size(0)), static_cast<int>(x.size(1)),
                         static_cast<int>(x.size(2)), static_cast<float>(eps), bf16, cur_stream());
  count(); check_last_error("head_rms_norm");
}

void window_attention_paged(const Tensor& q, const Tensor& kcache, const Tensor& vcache, const Tensor& block_table, const Tensor& tok_req,
                            const Tensor& tok_len, c10::optional<Tensor> slopes, c10::optional<Tensor> gate, Tensor out, int64_t block_size,
                            double scale, int64_t window, bool sink, double out_scale, int64_t max_len, c10::optional<Tensor> dist_bias) {
  const bool bf16 = act_is_bf16(q, "q");
  check_rows(q, "q");
  TORCH_CHECK(kcache.scalar_type() == q.scalar_type() && vcache.scalar_type() == q.scalar_type() && kcache.dim() == 3 && vcache.dim() == 3 &&
              kcache.is_contiguous() && vcache.is_contiguous() && kcache.size(2) == q.size(2) && vcache.size(1) == kcache.size(1),
              "caches must be contiguous [slots, G, d] / [slots, G, dv] in q's dtype");
  check_i32(block_table, "block_table"); check_i32(tok_req, "tok_req"); check_i32(tok_len, "tok_len");
  b200seq::WindowAttnArgs p{};
  p.n_tok = static_cast<int>(q.size(0));
  p.H = static_cast<int>(q.size(1)); p.G = static_cast<int>(kcache.size(1)); p.d = static_cast<int>(q.size(2));
  p.dv = static_cast<int>(vcache.size(2));
  TORCH_CHECK(block_table.dim() == 2 && tok_req.numel() == q.size(0) && tok_len.numel() == q.size(0), "bad packed-batch tensors");
  TORCH_CHECK(out.scalar_type() == q.scalar_type() && out.is_contiguous() && out.numel() == q.size(0) * p.H * p.dv, "bad out");
  p.q = q.data_ptr(); p.ldq = q.stride(0); p.kcache = kcache.data_ptr(); p.vcache = vcache.data_ptr();
  p.block_table = block_table.data_ptr<int>(); p.tok_req = tok_req.data_ptr<int>(); p.tok_len = tok_len.data_ptr<int>();
  if (slopes.has_value() && slopes->defined()) {
    check_f32(*slopes, "slopes");
    TORCH_CHECK(slopes->numel() == p.H, "slopes must be [H]");
    p.slopes = slopes->data_ptr<float>();
  }
  if (dist_bias.has_value() && dist_bias->defined()) {
    check_f32(*dist_bias, "dist_bias");
    TORCH_CHECK(dist_bias->dim() == 2 && dist_bias->size(0) >= 1 && dist_bias->size(1) == p.H, "dist_bias must be [L, H]");
    p.dist_bias = dist_bias->data_ptr<float>(); p.n_bias = static_cast<int>(dist_bias->size(0));
  }
  if (gate.has_value() && gate->defined()) {
    check_act2(*gate, q, "gate");
    TORCH_CHECK(gate->size(0) == q.size(0) && gate->size(1) == p.H, "gate must be [T, H]");
    p.gate = gate->data_ptr(); p.ldg = gate->stride(0);
  }
  p.out = out.data_ptr();
  p.block_size = static_cast<int>(block_size); p.max_blocks = static_cast<int>(block_table.size(1));
  p.scale = static_cast<float>(scale); p.out_scale = static_cast<float>(out_scale);
  p.window = static_cast<int>(window); p.sink = sink ? 1 : 0;
  c10::cuda::CUDAGuard g(q.device());
  p.n_splits = 1;
  Tensor ws;
  if (block_table.size(0) == q.size(0) && q.size(0) > 0) {   // one token per sequence: a decoding batch
    p.decode = 1;
    const int64_t longest = max_len > 0 ? max_len : block_table.size(1) * block_size;      // unknown: what the tables can hold
    const int keys = static_cast<int>(window > 0 ? std::min<int64_t>(window, longest) : longest);
    p.n_splits = b200seq::window_attention_splits(p.H, p.G, p.n_tok, keys);
    if (p.n_splits > 1) {
      ws = torch::empty({q.size(0), p.H, p.n_splits, p.dv + 2}, q.options().dtype(at::kFloat));
      p.ws = ws.data_ptr<float>();
    }
  }
  TORCH_CHECK(b200seq::window_attention_paged(p, bf16, cur_stream()), "window_attention_paged: no kernel instance for heads ", p.H, " / ",
              p.G, ", dims ", p.d, " / ", p.dv);
  count(p.n_splits > 1 ? 2 : 1); check_last_error("window_attention_paged");
}

void selective_scan(const Tensor& x, c10::optional<Tensor> z, const Tensor& B, const Tensor& Cm, const Tensor& dt_pre,
                    c10::optional<Tensor> dt_bias, const Tensor& A_log, const Tensor& D, const Tensor& cu, const Tensor& rows, Tensor state,
                    Tensor y, double out_scale) {
  const bool bf16 = act_is_bf16(x, "x");
  check_act2(x, x, "x"); check_act2(B, x, "B"); check_act2(Cm, x, "C"); check_act2(y, x, "y");
  check_f32(state, "state"); check_i32(cu, "cu"); check_i32(rows, "rows");
  b200seq::SelScanArgs p{};
  p.C = static_cast<int>(x.size(1)); p.N = static_cast<int>(B.size(1));
  const int64_t T = x.size(0);
  TORCH_CHECK(B.size(0) == T && Cm.size(0) == T && Cm.size(1) == p.N && y.size(0) == T && y.size(1) == p.C, "bad B / C / y shapes");
  TORCH_CHECK(dt_pre.is_cuda() && dt_pre.scalar_type() == at::kFloat && dt_pre.dim() == 2 && dt_pre.stride(1) == 1 && dt_pre.size(0) == T &&
              dt_pre.size(1) == p.C, "dt_pre must be fp32 [T, C]");
  TORCH_CHECK(state.dim() == 3 && state.size(1) == p.C && state.size(2) == p.N, "state must be [rows, C, N]");
  TORCH_CHECK(A_log.scalar_type() == x.scalar_type() && A_log.is_contiguous() && A_log.numel() == static_cast<int64_t>(p.C) * p.N &&
              D.scalar_type() == x.scalar_type() && D.is_contiguous() && D.numel() == p.C, "bad A_log / D");
  if (z.has_value() && z->defined()) { check_act2(*z, x, "z"); TORCH_CHECK(z->size(0) == T && z->size(1) == p.C, "bad z"); p.z = z->data_ptr(); p.ldz = z->stride(0); }
  if (dt_bias.has_value() && dt_bias->defined()) {
    TORCH_CHECK(dt_bias->scalar_type() == x.scalar_type() && dt_bias->is_contiguous() && dt_bias->numel() == p.C, "bad dt_bias");
    p.dt_bias = dt_bias->data_ptr();
  }
  p.x = x.data_ptr(); p.B = B.data_ptr(); p.Cm = Cm.data_ptr(); p.y = y.data_ptr(); p.dt_pre = dt_pre.data_ptr<float>();
  p.ldx = x.stride(0); p.ldb = B.stride(0); p.ldc = Cm.stride(0); p.ldy = y.stride(0); p.lddt = dt_pre.stride(0);
  p.A_log = A_log.data_ptr(); p.D = D.data_ptr();
  p.cu = cu.data_ptr<int>(); p.rows = rows.data_ptr<int>(); p.state = state.data_ptr<float>();
  p.out_scale = static_cast<float>(out_scale);
  c10::cuda::CUDAGuard g(x.device());
  TORCH_CHECK(b200seq::selective_scan(p, static_cast<int>(rows.numel()), bf16, cur_stream()), "selective_scan: ", p.N,
              " states per channel exceed the largest kernel instance (128)");
  count(); check_last_error("selective_scan");
}
}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("add_rms_norm", &add_rms_norm);
  m.def("retention_scan", &retention_scan);
  m.def("poly_norm", &poly_norm);
  m.def("gelu_mul", &gelu_mul);
  m.def("decay_gates", &decay_gates);
  m.def("gated_head_rms_norm", &gated_head_rms_norm);
  m.def("causal_conv", &causal_conv);
  m.def("stream_mix_norm", &stream_mix_norm);
  m.def("add_sinusoid", &add_sinusoid);
  m.def("head_rms_norm", &head_rms_norm);
  m.def("window_attention_paged", &window_attention_paged);
  m.def("selective_scan", &selective_scan);
  m.def("delta_rule_scan", &delta_rule_scan);
  m.def("mlstm_scan", &mlstm_scan);
  m.def("latent_attention_paged", &latent_attention_paged);
  m.def("group_limited_router", &group_limited_router);
  m.def("norm_add", &norm_add);
  m.def("norm_rope", &norm_rope);
  m.def("mixed_attention_paged", &mixed_attention_paged);
  m.def("gen_delta_scan", &gen_delta_scan);
  m.def("mingru_scan", &mingru_scan);
  m.def("clamped_glu", &clamped_glu);
  m.def("launch_count", []() { return g_launches.load(); });
  m.def("reset_launch_count", []() { g_launches.store(0); });
}
