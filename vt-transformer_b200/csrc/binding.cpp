// Python bindings of the kernels: tensors in, checks of device, dtype, shape and layout,
// then the plain-pointer launchers of kernels.h on the current stream.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "kernels.h"

namespace {

using torch::Tensor;

int dtype_code(const Tensor& t, const char* name) {
    if (t.scalar_type() == torch::kFloat32) return vtb::kF32;
    if (t.scalar_type() == torch::kBFloat16) return vtb::kBF16;
    TORCH_CHECK(false, name, ": dtype must be float32 or bfloat16, found ", t.scalar_type());
}

void check_cuda(const Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda(), name, ": must be a CUDA tensor (there is no CPU path)");
    TORCH_CHECK(t.is_contiguous(), name, ": must be contiguous");
}

void check_i32(const Tensor& t, const char* name) {
    check_cuda(t, name);
    TORCH_CHECK(t.scalar_type() == torch::kInt32, name, ": must be int32");
}

void check_f32(const Tensor& t, const char* name) {
    check_cuda(t, name);
    TORCH_CHECK(t.scalar_type() == torch::kFloat32, name, ": must be float32");
}

void check_launch(cudaError_t e, const char* what) {
    TORCH_CHECK(e == cudaSuccess, what, ": launch failed: ", cudaGetErrorString(e));
}

cudaStream_t stream_of(const Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

int* status_ptr(const c10::optional<Tensor>& status) {
    if (!status.has_value()) return nullptr;
    check_i32(*status, "status");
    TORCH_CHECK(status->numel() >= 2, "status: needs two ints");
    return status->data_ptr<int>();
}

void embedding(const Tensor& table, const Tensor& ids, Tensor& out, c10::optional<Tensor> status, double scale) {
    check_cuda(table, "table"); check_i32(ids, "ids"); check_f32(out, "out");
    TORCH_CHECK(table.dim() == 2 && out.dim() == 2, "embedding: table and out must be 2-d");
    const int hidden = table.size(1);
    TORCH_CHECK(hidden % 8 == 0, "embedding: hidden size ", hidden, " must be a multiple of 8");
    TORCH_CHECK(out.size(1) == hidden && out.size(0) == ids.numel(), "embedding: out must be [tokens, hidden]");
    c10::cuda::CUDAGuard guard(table.device());
    check_launch(vtb::launch_embedding(dtype_code(table, "table"), table.data_ptr(), ids.data_ptr<int>(),
                                       out.data_ptr<float>(), ids.numel(), hidden, table.size(0), (float)scale,
                                       status_ptr(status), stream_of(table)), "embedding");
}

void logits_scale_cap(Tensor& logits, double scale, double cap) {
    check_f32(logits, "logits");
    TORCH_CHECK(logits.is_contiguous(), "logits_scale_cap: logits must be contiguous");
    TORCH_CHECK(cap >= 0.0, "logits_scale_cap: the cap must not be negative");
    c10::cuda::CUDAGuard guard(logits.device());
    check_launch(vtb::launch_logits_scale_cap(logits.data_ptr<float>(), logits.numel(), (float)scale, (float)cap,
                                              stream_of(logits)), "logits_scale_cap");
}

void norm_rows(bool center, Tensor& x, c10::optional<Tensor> delta, const Tensor& weight, double eps, c10::optional<Tensor> out_opt,
               c10::optional<Tensor> rows, c10::optional<Tensor> status, c10::optional<Tensor> post_weight, double post_eps,
               double post_mult, int64_t groups = 1, double x_scale = 1.0, bool write_normed = false) {
    check_f32(x, "x"); check_f32(weight, "weight");
    TORCH_CHECK(x.dim() == 2, "rmsnorm: x must be 2-d");
    const int hidden = x.size(1);
    TORCH_CHECK(hidden % 8 == 0, "rmsnorm: hidden size ", hidden, " must be a multiple of 8");
    TORCH_CHECK(groups >= 1 && hidden % groups == 0, "rmsnorm: ", groups, " groups must cut the hidden size ", hidden, " into equal parts");
    TORCH_CHECK((hidden / groups) % 8 == 0 || (!center && !post_weight.has_value()), "rmsnorm: groups of a size that is no multiple of 8 "
                "take no delta that is normed first");
    TORCH_CHECK(!center || (groups == 1 && x_scale == 1.0 && !write_normed), "layernorm: no groups, scale of the stream or normed stream");
    TORCH_CHECK(out_opt.has_value() || (write_normed && delta.has_value() && delta->dim() == 2),
                "rmsnorm: without out the stream takes the normed row, and a delta tensor gives the dtype");
    // without out (the normed row goes to the stream alone) the delta names the compute dtype
    const Tensor& out = out_opt.has_value() ? *out_opt : *delta;
    check_cuda(out, "out");
    TORCH_CHECK(out.dim() == 2, "rmsnorm: out must be 2-d");
    TORCH_CHECK(weight.numel() == hidden && out.size(1) == hidden, "rmsnorm: weight and out must match hidden size");
    TORCH_CHECK(!write_normed || !rows.has_value(), "rmsnorm: the normed row goes back to the stream for all rows or none");
    const int code = dtype_code(out, "out");
    const void* dp = nullptr;
    const float* pp = nullptr;
    int n_parts = 0;
    if (delta.has_value() && delta->dim() == 3) {
        // the unadded shares of a matrix product: [shares, tokens, hidden] in 32-bit
        check_f32(*delta, "delta");
        TORCH_CHECK(delta->size(1) == x.size(0) && delta->size(2) == hidden && delta->size(0) >= 1,
                    "rmsnorm: shares of a delta must be [shares, tokens, hidden]");
        pp = delta->data_ptr<float>();
        n_parts = delta->size(0);
    } else if (delta.has_value()) {
        check_cuda(*delta, "delta");
        TORCH_CHECK(delta->scalar_type() == out.scalar_type(), "rmsnorm: delta and out must have one dtype");
        TORCH_CHECK(delta->sizes() == x.sizes(), "rmsnorm: delta must have the shape of x");
        dp = delta->data_ptr();
    }
    const int* rp = nullptr;
    int n_rows = x.size(0);
    if (rows.has_value()) {
        check_i32(*rows, "rows");
        rp = rows->data_ptr<int>();
        n_rows = rows->numel();
    }
    TORCH_CHECK(out.size(0) == n_rows, "rmsnorm: out must have one row for each normed row");
    TORCH_CHECK(out_opt.has_value() || (dp != nullptr), "rmsnorm: without out the delta must be a tensor");
    const float* pw = nullptr;
    if (post_weight.has_value()) {
        // the delta is normed (root mean square, this weight, post_mult) before it is added
        check_f32(*post_weight, "post_weight");
        TORCH_CHECK(post_weight->numel() == hidden, "rmsnorm: the weight of the delta's norm must match hidden size");
        TORCH_CHECK(dp != nullptr || pp != nullptr, "rmsnorm: a norm of the delta without a delta");
        pw = post_weight->data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(x.device());
    void* op = out_opt.has_value() ? out.data_ptr() : nullptr;
    if (center)
        check_launch(vtb::launch_layernorm(code, x.data_ptr<float>(), dp, pp, n_parts, weight.data_ptr<float>(), (float)eps, op, rp, n_rows,
                                           x.size(0), hidden, status_ptr(status), pw, (float)post_eps, (float)post_mult, stream_of(x)),
                     "layernorm");
    else
        check_launch(vtb::launch_rmsnorm(code, x.data_ptr<float>(), dp, pp, n_parts, weight.data_ptr<float>(), (float)eps, op, rp, n_rows,
                                         x.size(0), hidden, status_ptr(status), pw, (float)post_eps, (float)post_mult, stream_of(x),
                                         (int)groups, (float)x_scale, write_normed ? 1 : 0), "rmsnorm");
}

void rmsnorm(Tensor& x, c10::optional<Tensor> delta, const Tensor& weight, double eps, c10::optional<Tensor> out,
             c10::optional<Tensor> rows, c10::optional<Tensor> status, c10::optional<Tensor> post_weight, double post_eps,
             double post_mult, int64_t groups, double x_scale, bool write_normed) {
    norm_rows(false, x, delta, weight, eps, out, rows, status, post_weight, post_eps, post_mult, groups, x_scale, write_normed);
}

void layernorm(Tensor& x, c10::optional<Tensor> delta, const Tensor& weight, double eps, Tensor& out,
               c10::optional<Tensor> rows, c10::optional<Tensor> status, c10::optional<Tensor> post_weight, double post_eps,
               double post_mult) {
    norm_rows(true, x, delta, weight, eps, out, rows, status, post_weight, post_eps, post_mult);
}

void polynorm(const Tensor& z, const Tensor& coef, double eps, Tensor& out, int64_t n_mean) {
    check_cuda(z, "z"); check_cuda(out, "out"); check_f32(coef, "coefficients");
    TORCH_CHECK(z.dim() == 2 && out.sizes() == z.sizes() && out.scalar_type() == z.scalar_type(), "polynorm: out must be like z [tokens, inter]");
    TORCH_CHECK(coef.numel() == 4, "polynorm: four coefficients");
    TORCH_CHECK(z.size(1) % 8 == 0, "polynorm: inner size ", z.size(1), " must be a multiple of 8");
    if (n_mean <= 0) n_mean = z.size(1);
    TORCH_CHECK(n_mean <= z.size(1), "polynorm: more columns to average than the row has");
    c10::cuda::CUDAGuard guard(z.device());
    check_launch(vtb::launch_polynorm(dtype_code(z, "z"), z.data_ptr(), coef.data_ptr<float>(), (float)eps, out.data_ptr(), z.size(0),
                                      z.size(1), n_mean, stream_of(z)), "polynorm");
}

// columns [col, col + n) of a row-major [tokens, stride] tensor
void check_cols(const Tensor& y, int64_t col, int64_t n, const char* what) {
    TORCH_CHECK(col >= 0 && n >= 0 && col + n <= y.size(1), what, ": columns [", col, ", ", col + n, ") lie outside the ", y.size(1), " of y");
}

void head_norm_gate(const Tensor& o, const Tensor& y, int64_t gate_col, const Tensor& weight, bool weight_per_channel, double eps,
                    int64_t act, Tensor& out, int64_t out_col, double out_scale, int64_t heads, int64_t v_dim,
                    c10::optional<Tensor> token_seq) {
    check_f32(o, "o"); check_cuda(y, "y"); check_cuda(out, "out"); check_f32(weight, "weight");
    TORCH_CHECK(o.dim() == 2 && y.dim() == 2 && out.dim() == 2 && o.size(1) == heads * v_dim && y.size(0) == o.size(0) && out.size(0) == o.size(0),
                "head_norm_gate: o [tokens, heads * v_dim], y and out with as many rows");
    TORCH_CHECK(y.scalar_type() == out.scalar_type(), "head_norm_gate: y and out must have one dtype");
    TORCH_CHECK(weight.numel() == (weight_per_channel ? heads * v_dim : v_dim), "head_norm_gate: the weight's size");
    TORCH_CHECK(act == 0 || act == 1, "head_norm_gate: act 0 (silu) or 1 (sigmoid)");
    check_cols(y, gate_col, heads * v_dim, "head_norm_gate (gate)"); check_cols(out, out_col, heads * v_dim, "head_norm_gate (out)");
    const int* ts = nullptr;
    if (token_seq.has_value()) { check_i32(*token_seq, "token_seq"); TORCH_CHECK(token_seq->numel() == o.size(0), "head_norm_gate: one sequence index a token"); ts = token_seq->data_ptr<int>(); }
    c10::cuda::CUDAGuard guard(o.device());
    check_launch(vtb::launch_head_norm_gate(dtype_code(y, "y"), o.data_ptr<float>(), y.data_ptr(), y.size(1), gate_col, weight.data_ptr<float>(),
                                            weight_per_channel, (float)eps, act, out.data_ptr(), out.size(1), out_col, (float)out_scale, ts,
                                            o.size(0), heads, v_dim, stream_of(o)), "head_norm_gate");
}

void scale_into(const Tensor& src, Tensor& dst, int64_t dst_col, double scale) {
    check_cuda(src, "src"); check_cuda(dst, "dst");
    TORCH_CHECK(src.dim() == 2 && dst.dim() == 2 && src.size(0) == dst.size(0) && src.scalar_type() == dst.scalar_type(),
                "scale_into: src [tokens, n] and dst [tokens, stride] of one dtype");
    check_cols(dst, dst_col, src.size(1), "scale_into");
    c10::cuda::CUDAGuard guard(src.device());
    check_launch(vtb::launch_scale_into(dtype_code(src, "src"), src.data_ptr(), dst.data_ptr(), src.size(0), src.size(1), dst.size(1),
                                        dst_col, (float)scale, stream_of(src)), "scale_into");
}

void gate_into(const Tensor& src, const Tensor& y, int64_t gate_col, int64_t mode, Tensor& dst, int64_t dst_col, double scale, int64_t heads,
               int64_t v_dim) {
    check_cuda(src, "src"); check_cuda(y, "y"); check_cuda(dst, "dst");
    TORCH_CHECK(src.dim() == 2 && dst.dim() == 2 && y.dim() == 2 && src.size(0) == dst.size(0) && y.size(0) == src.size(0) &&
                src.scalar_type() == dst.scalar_type() && y.scalar_type() == src.scalar_type() && src.size(1) == heads * v_dim,
                "gate_into: src [tokens, heads * v_dim], y and dst with as many rows, of one dtype");
    TORCH_CHECK(mode >= 0 && mode <= 2, "gate_into: mode 0, 1 or 2");
    check_cols(dst, dst_col, src.size(1), "gate_into");
    if (mode != 0) check_cols(y, gate_col, mode == 1 ? heads : heads * v_dim, "gate_into (gate)");
    c10::cuda::CUDAGuard guard(src.device());
    check_launch(vtb::launch_gate_into(dtype_code(src, "src"), src.data_ptr(), y.data_ptr(), y.size(1), gate_col, mode, dst.data_ptr(), src.size(0),
                                       heads, v_dim, dst.size(1), dst_col, (float)scale, stream_of(src)), "gate_into");
}

void check_scan(const Tensor& y, const Tensor& state, const Tensor& cu_q, const Tensor& rows, const Tensor& o, int64_t heads, int64_t dim,
                int64_t v_dim, const char* who) {
    check_cuda(y, "y"); check_f32(state, "state"); check_i32(cu_q, "cu_q"); check_i32(rows, "rows"); check_f32(o, "o");
    TORCH_CHECK(y.dim() == 2 && o.dim() == 2 && o.size(0) == y.size(0) && o.size(1) == heads * v_dim, who, ": o must be [tokens, heads * v_dim]");
    TORCH_CHECK(state.dim() == 4 && state.size(1) == heads && state.size(2) == dim && state.size(3) == v_dim, who,
                ": state must be [rows, heads, dim, v_dim]");
    TORCH_CHECK(cu_q.numel() == rows.numel() + 1, who, ": cu_q has one entry more than rows");
}

void gla_scan(const Tensor& y, int64_t q_col, int64_t k_col, int64_t v_col, int64_t low_col, const Tensor& a2, const Tensor& a2_bias,
              double inv_tau, double q_scale, Tensor& state, const Tensor& cu_q, const Tensor& rows, Tensor& o, int64_t heads,
              int64_t dim, int64_t v_dim, c10::optional<Tensor> status, int64_t most_threads) {
    check_scan(y, state, cu_q, rows, o, heads, dim, v_dim, "gla_scan");
    check_f32(a2, "a2"); check_f32(a2_bias, "a2_bias");
    TORCH_CHECK(a2.dim() == 2 && a2.size(0) == heads * dim && a2_bias.numel() == heads * dim, "gla_scan: a2 [heads * dim, rank] and its bias");
    const int rank = a2.size(1);
    check_cols(y, q_col, heads * dim, "gla_scan (q)"); check_cols(y, k_col, heads * dim, "gla_scan (k)");
    check_cols(y, v_col, heads * v_dim, "gla_scan (v)"); check_cols(y, low_col, rank, "gla_scan (gate)");
    c10::cuda::CUDAGuard guard(y.device());
    check_launch(vtb::launch_gla_scan(dtype_code(y, "y"), y.data_ptr(), y.size(1), q_col, k_col, v_col, low_col, rank, a2.data_ptr<float>(),
                                      a2_bias.data_ptr<float>(), (float)inv_tau, (float)q_scale, state.data_ptr<float>(), state.size(0),
                                      cu_q.data_ptr<int>(), rows.data_ptr<int>(), rows.numel(), o.data_ptr<float>(), heads, dim, v_dim,
                                      (int)most_threads, status_ptr(status), stream_of(y)), "gla_scan");
}

void delta_scan(const Tensor& y, int64_t r_col, int64_t k_col, int64_t v_col, int64_t a_col, int64_t low_col, const Tensor& w2,
                const Tensor& w0, const Tensor& a_bias, double decay_rate, double key_eps, Tensor& state, const Tensor& cu_q,
                const Tensor& rows, Tensor& o, int64_t heads, int64_t dim, c10::optional<Tensor> status, int64_t most_threads) {
    check_scan(y, state, cu_q, rows, o, heads, dim, dim, "delta_scan");
    check_f32(w2, "w2"); check_f32(w0, "w0"); check_f32(a_bias, "a_bias");
    TORCH_CHECK(w2.dim() == 2 && w2.size(0) == heads * dim && w0.numel() == heads * dim && a_bias.numel() == heads * dim,
                "delta_scan: w2 [heads * dim, rank], w0 and a_bias [heads * dim]");
    const int rank = w2.size(1);
    for (int64_t col : {r_col, k_col, v_col, a_col}) check_cols(y, col, heads * dim, "delta_scan");
    check_cols(y, low_col, rank, "delta_scan (decay)");
    c10::cuda::CUDAGuard guard(y.device());
    check_launch(vtb::launch_delta_scan(dtype_code(y, "y"), y.data_ptr(), y.size(1), r_col, k_col, v_col, a_col, low_col, rank,
                                        w2.data_ptr<float>(), w0.data_ptr<float>(), a_bias.data_ptr<float>(), (float)decay_rate,
                                        (float)key_eps, state.data_ptr<float>(), state.size(0), cu_q.data_ptr<int>(), rows.data_ptr<int>(),
                                        rows.numel(), o.data_ptr<float>(), heads, dim, (int)most_threads, status_ptr(status), stream_of(y)), "delta_scan");
}

void check_gated(const Tensor& y, const Tensor& state, const Tensor& cu_q, const Tensor& rows, const Tensor& o, int64_t heads,
                 int64_t v_dim, const char* who) {
    check_cuda(y, "y"); check_f32(state, "state"); check_i32(cu_q, "cu_q"); check_i32(rows, "rows"); check_f32(o, "o");
    TORCH_CHECK(y.dim() == 2 && o.dim() == 2 && o.size(0) == y.size(0) && o.size(1) == heads * v_dim, who, ": o must be [tokens, heads * v_dim]");
    TORCH_CHECK(cu_q.numel() == rows.numel() + 1, who, ": cu_q has one entry more than rows");
}

void gated_delta_scan(const Tensor& y, int64_t q_col, int64_t k_col, int64_t v_col, int64_t b_col, int64_t a_col, const Tensor& conv_q,
                      const Tensor& conv_k, const Tensor& conv_v, const Tensor& a_log, const Tensor& dt_bias, double key_eps, double q_scale,
                      Tensor& state, c10::optional<Tensor> tail, const Tensor& cu_q, const Tensor& rows, Tensor& o, int64_t heads,
                      int64_t kv_heads, int64_t dim, int64_t v_dim, c10::optional<Tensor> status, int64_t most_threads) {
    check_gated(y, state, cu_q, rows, o, heads, v_dim, "gated_delta_scan");
    TORCH_CHECK(state.dim() == 4 && state.size(1) == heads && state.size(2) == dim && state.size(3) == v_dim,
                "gated_delta_scan: state must be [rows, heads, dim, v_dim]");
    TORCH_CHECK(kv_heads >= 1 && heads % kv_heads == 0, "gated_delta_scan: heads a multiple of kv_heads");
    check_f32(conv_q, "conv_q"); check_f32(conv_k, "conv_k"); check_f32(conv_v, "conv_v"); check_f32(a_log, "a_log"); check_f32(dt_bias, "dt_bias");
    const int64_t nq = kv_heads * dim, nv = heads * v_dim;
    TORCH_CHECK(conv_q.dim() == 2 && conv_k.dim() == 2 && conv_v.dim() == 2 && conv_q.size(0) == nq && conv_k.size(0) == nq && conv_v.size(0) == nv,
                "gated_delta_scan: the convolutions' weights are [channels, taps]");
    const int64_t taps = conv_q.size(1);
    TORCH_CHECK(taps >= 1 && taps <= 16 && conv_k.size(1) == taps && conv_v.size(1) == taps, "gated_delta_scan: 1 to 16 taps, the same for q, k and v");
    TORCH_CHECK(a_log.numel() == heads && dt_bias.numel() == heads, "gated_delta_scan: a_log and dt_bias [heads]");
    const float* tp = nullptr;
    if (taps > 1) {
        TORCH_CHECK(tail.has_value(), "gated_delta_scan: more than one tap needs the kept inputs");
        check_f32(*tail, "tail");
        TORCH_CHECK(tail->dim() == 3 && tail->size(0) == state.size(0) && tail->size(1) == taps - 1 && tail->size(2) == 2 * nq + nv,
                    "gated_delta_scan: tail must be [rows, taps - 1, channels of q, k and v]");
        tp = tail->data_ptr<float>();
    }
    check_cols(y, q_col, nq, "gated_delta_scan (q)"); check_cols(y, k_col, nq, "gated_delta_scan (k)"); check_cols(y, v_col, nv, "gated_delta_scan (v)");
    check_cols(y, b_col, heads, "gated_delta_scan (beta)"); check_cols(y, a_col, heads, "gated_delta_scan (decay)");
    TORCH_CHECK(dim <= 512, "gated_delta_scan: head sizes up to 512");
    c10::cuda::CUDAGuard guard(y.device());
    check_launch(vtb::launch_gated_delta_scan(dtype_code(y, "y"), y.data_ptr(), y.size(1), q_col, k_col, v_col, b_col, a_col,
                                              conv_q.data_ptr<float>(), conv_k.data_ptr<float>(), conv_v.data_ptr<float>(), taps,
                                              a_log.data_ptr<float>(), dt_bias.data_ptr<float>(), (float)key_eps, (float)q_scale,
                                              state.data_ptr<float>(), state.size(0), tp, cu_q.data_ptr<int>(), rows.data_ptr<int>(),
                                              rows.numel(), o.data_ptr<float>(), heads, kv_heads, dim, v_dim, (int)most_threads,
                                              status_ptr(status), stream_of(y)), "gated_delta_scan");
}

void conv_tail_update(const Tensor& y, std::vector<int64_t> cols, std::vector<int64_t> widths, Tensor& tail, const Tensor& cu_q,
                      const Tensor& rows, c10::optional<Tensor> status) {
    check_cuda(y, "y"); check_f32(tail, "tail"); check_i32(cu_q, "cu_q"); check_i32(rows, "rows");
    TORCH_CHECK(y.dim() == 2 && tail.dim() == 3 && cols.size() == widths.size() && cols.size() >= 1 && cols.size() <= 4,
                "conv_tail_update: y [tokens, .], tail [rows, kept, channels], one to four groups of columns");
    int c[4] = {0, 0, 0, 0}, w[4] = {0, 0, 0, 0};
    int64_t total = 0;
    for (size_t i = 0; i < cols.size(); ++i) {
        check_cols(y, cols[i], widths[i], "conv_tail_update");
        c[i] = (int)cols[i]; w[i] = (int)widths[i]; total += widths[i];
    }
    TORCH_CHECK(total == tail.size(2) && tail.size(1) >= 1 && tail.size(1) <= 15, "conv_tail_update: the groups' widths add up to tail's channels; 1 to 15 kept inputs");
    TORCH_CHECK(cu_q.numel() == rows.numel() + 1, "conv_tail_update: cu_q has one entry more than rows");
    c10::cuda::CUDAGuard guard(y.device());
    check_launch(vtb::launch_conv_tail_update(dtype_code(y, "y"), y.data_ptr(), y.size(1), c[0], w[0], c[1], w[1], c[2], w[2], c[3], w[3],
                                              tail.data_ptr<float>(), tail.size(0), tail.size(1), tail.size(2), cu_q.data_ptr<int>(),
                                              rows.data_ptr<int>(), rows.numel(), status_ptr(status), stream_of(y)), "conv_tail_update");
}

void memory_scan(const Tensor& y, int64_t q_col, int64_t k_col, int64_t v_col, int64_t i_col, int64_t f_col, const Tensor& i_bias,
                 const Tensor& f_bias, double gate_cap, double q_scale, double den_eps, Tensor& state, const Tensor& cu_q, const Tensor& rows,
                 Tensor& o, int64_t heads, int64_t dim, int64_t v_dim, c10::optional<Tensor> status, int64_t most_threads) {
    check_gated(y, state, cu_q, rows, o, heads, v_dim, "memory_scan");
    TORCH_CHECK(state.dim() == 4 && state.size(1) == heads && state.size(2) == dim + 1 && state.size(3) == v_dim + 1,
                "memory_scan: state must be [rows, heads, dim + 1, v_dim + 1]");
    check_f32(i_bias, "i_bias"); check_f32(f_bias, "f_bias");
    TORCH_CHECK(i_bias.numel() == heads && f_bias.numel() == heads && gate_cap > 0.0, "memory_scan: the gates' biases [heads]; a positive cap");
    check_cols(y, q_col, heads * dim, "memory_scan (q)"); check_cols(y, k_col, heads * dim, "memory_scan (k)");
    check_cols(y, v_col, heads * v_dim, "memory_scan (v)"); check_cols(y, i_col, heads, "memory_scan (i)"); check_cols(y, f_col, heads, "memory_scan (f)");
    TORCH_CHECK(dim <= 512, "memory_scan: head sizes up to 512");
    c10::cuda::CUDAGuard guard(y.device());
    Tensor snap = torch::empty({rows.numel(), heads, dim + 1}, state.options());
    check_launch(vtb::launch_memory_scan(dtype_code(y, "y"), y.data_ptr(), y.size(1), q_col, k_col, v_col, i_col, f_col, i_bias.data_ptr<float>(),
                                         f_bias.data_ptr<float>(), (float)gate_cap, (float)q_scale, (float)den_eps, state.data_ptr<float>(),
                                         state.size(0), cu_q.data_ptr<int>(), rows.data_ptr<int>(), rows.numel(), o.data_ptr<float>(), heads,
                                         dim, v_dim, (int)most_threads, status_ptr(status), stream_of(y), snap.data_ptr<float>()), "memory_scan");
}

void normed_sum(std::vector<Tensor> parts, std::vector<Tensor> weights, double eps, std::vector<double> scales, Tensor& out) {
    check_f32(out, "out");
    const size_t n = parts.size();
    TORCH_CHECK(n >= 1 && n <= 4 && weights.size() == n && scales.size() == n && out.dim() == 2, "normed_sum: one to four parts, a weight and a scale each");
    const float* pp[4] = {nullptr, nullptr, nullptr, nullptr};
    const float* wp[4] = {nullptr, nullptr, nullptr, nullptr};
    float sc[4] = {0.f, 0.f, 0.f, 0.f};
    for (size_t i = 0; i < n; ++i) {
        check_f32(parts[i], "part"); check_f32(weights[i], "weight");
        TORCH_CHECK(parts[i].sizes() == out.sizes() && weights[i].numel() == out.size(1), "normed_sum: parts [tokens, width] like out, weights [width]");
        pp[i] = parts[i].data_ptr<float>(); wp[i] = weights[i].data_ptr<float>(); sc[i] = (float)scales[i];
    }
    c10::cuda::CUDAGuard guard(out.device());
    check_launch(vtb::launch_normed_sum((int)n, pp[0], pp[1], pp[2], pp[3], wp[0], wp[1], wp[2], wp[3], sc[0], sc[1], sc[2], sc[3], (float)eps,
                                        out.data_ptr<float>(), out.size(0), out.size(1), stream_of(out)), "normed_sum");
}

void add_rows(Tensor& x, const Tensor& other) {
    check_f32(x, "x"); check_f32(other, "other");
    TORCH_CHECK(x.sizes() == other.sizes(), "add_rows: two tensors of one shape");
    c10::cuda::CUDAGuard guard(x.device());
    check_launch(vtb::launch_add_rows(x.data_ptr<float>(), other.data_ptr<float>(), x.numel(), stream_of(x)), "add_rows");
}

void check_pages(const Tensor& k_cache, const Tensor& v_cache, const Tensor& ref, int kv_heads, int dim, int v_dim, int v_heads = -1) {
    check_cuda(k_cache, "k_cache"); check_cuda(v_cache, "v_cache");
    if (v_heads < 0) v_heads = kv_heads;
    TORCH_CHECK(k_cache.dim() == 4 && v_cache.dim() == 4 && k_cache.size(0) == v_cache.size(0) && k_cache.size(2) == v_cache.size(2),
                "cache: k [pages, kv_heads, page_size, dim] and v [pages, kv_heads, page_size, v_dim]");
    TORCH_CHECK(k_cache.size(1) == kv_heads && v_cache.size(1) == v_heads && k_cache.size(3) == dim && v_cache.size(3) == v_dim,
                "cache: kv_heads, dim or v_dim differ");
    TORCH_CHECK(k_cache.scalar_type() == ref.scalar_type() && v_cache.scalar_type() == ref.scalar_type(),
                "cache: dtype differs from the activations'");
}

void attention_prepare(Tensor& y, int64_t q_col, int64_t k_col, int64_t v_col, const Tensor& positions, const Tensor& token_seq,
                       c10::optional<Tensor> frequencies, double norm_eps, Tensor& k_cache, Tensor& v_cache, const Tensor& block_table,
                       int64_t heads, int64_t kv_heads, int64_t dim, int64_t v_dim, bool store, c10::optional<Tensor> status,
                       int64_t v_heads, c10::optional<Tensor> q_weight, c10::optional<Tensor> k_weight, bool norm_first,
                       bool whole_projection, double rot_mult, double q_temp_coef, int64_t q_temp_every) {
    check_cuda(y, "y"); check_i32(positions, "positions"); check_i32(token_seq, "token_seq"); check_i32(block_table, "block_table");
    TORCH_CHECK(y.dim() == 2 && positions.numel() == y.size(0) && token_seq.numel() == y.size(0), "attention_prepare: one position and sequence a token");
    TORCH_CHECK(block_table.dim() == 2, "attention_prepare: block_table must be [sequences, stride]");
    if (v_heads < 0) v_heads = kv_heads;
    check_cols(y, q_col, heads * dim, "attention_prepare (q)"); check_cols(y, k_col, kv_heads * dim, "attention_prepare (k)");
    check_cols(y, v_col, v_heads * v_dim, "attention_prepare (v)");
    check_pages(k_cache, v_cache, y, kv_heads, dim, v_dim, v_heads);
    const float* qw = nullptr;
    const float* kw = nullptr;
    TORCH_CHECK(!whole_projection || norm_first, "attention_prepare: the norm over the whole projection comes before the rotation");
    TORCH_CHECK(q_temp_every >= 1, "attention_prepare: q_temp_every must be at least 1");
    const int64_t qn = whole_projection ? heads * dim : dim, kn = whole_projection ? kv_heads * dim : dim;
    if (q_weight.has_value()) { check_f32(*q_weight, "q_weight"); TORCH_CHECK(q_weight->numel() == qn, "attention_prepare: q_weight [dim], or [heads * dim] over the whole projection"); qw = q_weight->data_ptr<float>(); }
    if (k_weight.has_value()) { check_f32(*k_weight, "k_weight"); TORCH_CHECK(k_weight->numel() == kn, "attention_prepare: k_weight [dim], or [kv_heads * dim] over the whole projection"); kw = k_weight->data_ptr<float>(); }
    const float* fp = nullptr;
    int half = 0;
    if (frequencies.has_value()) {
        check_f32(*frequencies, "frequencies");
        fp = frequencies->data_ptr<float>();
        half = frequencies->numel();
        TORCH_CHECK(2 * half <= dim, "attention_prepare: the rotation covers more than the head");
    }
    TORCH_CHECK(dim <= 256, "attention_prepare: head sizes up to 256");
    c10::cuda::CUDAGuard guard(y.device());
    check_launch(vtb::launch_attention_prepare(dtype_code(y, "y"), y.data_ptr(), y.size(1), q_col, k_col, v_col, positions.data_ptr<int>(),
                                               token_seq.data_ptr<int>(), fp, half, (float)norm_eps, k_cache.data_ptr(), v_cache.data_ptr(),
                                               block_table.data_ptr<int>(), block_table.size(1), block_table.size(0), k_cache.size(0),
                                               y.size(0), heads, kv_heads, dim, v_dim, k_cache.size(2), store ? 1 : 0, status_ptr(status),
                                               v_heads, qw, kw, norm_first ? 1 : 0, stream_of(y), whole_projection ? 1 : 0, (float)rot_mult,
                                               (float)q_temp_coef, (int)q_temp_every), "attention_prepare");
}

void attention_general(const Tensor& y, int64_t q_col, Tensor& out, int64_t out_col, double out_scale, const Tensor& k_cache,
                       const Tensor& v_cache, const Tensor& positions, const Tensor& token_seq, const Tensor& block_table, int64_t heads,
                       int64_t kv_heads, int64_t dim, int64_t v_dim, int64_t window, int64_t chunk, double scale, c10::optional<Tensor> status,
                       int64_t keep_first, int64_t maps, double lam, double sub_eps, c10::optional<Tensor> sinks, bool values_in_keys,
                       double softcap, int64_t gate_mode, int64_t gate_col) {
    check_cuda(y, "y"); check_cuda(out, "out"); check_i32(positions, "positions"); check_i32(token_seq, "token_seq");
    TORCH_CHECK(gate_mode >= 0 && gate_mode <= 2 && softcap >= 0.0, "attention_general: gate_mode 0, 1 or 2; softcap not negative");
    TORCH_CHECK((gate_mode == 0 && softcap == 0.0) || maps == 1, "attention_general: a gate or capped scores take one map");
    if (gate_mode != 0) check_cols(y, gate_col, gate_mode == 1 ? heads : heads * v_dim, "attention_general (gate)");
    TORCH_CHECK(maps == 1 || maps == 2, "attention_general: one map of queries and keys a head, or two");
    const float* sp = nullptr;
    if (sinks.has_value()) {
        check_f32(*sinks, "sinks");
        TORCH_CHECK(sinks->numel() == heads && maps == 1, "attention_general: one sink a head, with one map");
        sp = sinks->data_ptr<float>();
    }
    check_i32(block_table, "block_table");
    TORCH_CHECK(y.dim() == 2 && out.dim() == 2 && out.size(0) == y.size(0) && out.scalar_type() == y.scalar_type(),
                "attention_general: y and out [tokens, .] of one dtype");
    TORCH_CHECK(positions.numel() == y.size(0) && token_seq.numel() == y.size(0), "attention_general: one position and sequence a token");
    TORCH_CHECK(block_table.dim() == 2 && heads % kv_heads == 0, "attention_general: block_table [sequences, stride]; heads a multiple of kv_heads");
    check_cols(y, q_col, heads * maps * dim, "attention_general (q)"); check_cols(out, out_col, heads * v_dim, "attention_general (out)");
    if (values_in_keys) {
        // a value is the first v_dim numbers of its key's row: one tensor of pages serves as both
        TORCH_CHECK(maps == 1 && v_dim <= dim && v_cache.data_ptr() == k_cache.data_ptr(), "attention_general: values inside the keys' rows "
                    "take one map, v_dim <= dim and the keys' pages as the values' pages");
        check_pages(k_cache, k_cache, y, kv_heads, dim, dim, kv_heads);
    } else {
        check_pages(k_cache, v_cache, y, kv_heads * maps, dim, v_dim, kv_heads);
    }
    TORCH_CHECK(dim <= 2048 && v_dim <= (maps == 2 ? 256 : 1024), "attention_general: keys up to 2048 numbers, values up to 1024 (256 with two maps)");
    c10::cuda::CUDAGuard guard(y.device());
    check_launch(vtb::launch_attention_general(dtype_code(y, "y"), y.data_ptr(), y.size(1), q_col, out.data_ptr(), out.size(1), out_col,
                                               (float)out_scale, k_cache.data_ptr(), v_cache.data_ptr(), positions.data_ptr<int>(),
                                               token_seq.data_ptr<int>(), block_table.data_ptr<int>(), block_table.size(1),
                                               block_table.size(0), k_cache.size(0), y.size(0), heads, kv_heads, dim, v_dim, k_cache.size(2),
                                               window, chunk, (float)scale, status_ptr(status), keep_first, maps, (float)lam,
                                               (float)sub_eps, stream_of(y), sp, values_in_keys ? (int)dim : 0, (float)softcap, (int)gate_mode,
                                               (int)gate_col), "attention_general");
}

void attention_diff(const Tensor& y, int64_t q_col, Tensor& out, int64_t out_col, double out_scale, const Tensor& k_cache,
                    const Tensor& v_cache, const Tensor& cu_q, const Tensor& q_start, const Tensor& block_table,
                    c10::optional<Tensor> tiles, int64_t heads, int64_t kv_heads, int64_t dim, int64_t v_dim, int64_t window,
                    int64_t keep_first, double scale, double lam, double sub_eps, c10::optional<Tensor> status) {
    check_cuda(y, "y"); check_cuda(out, "out"); check_i32(cu_q, "cu_q"); check_i32(q_start, "q_start"); check_i32(block_table, "block_table");
    TORCH_CHECK(y.scalar_type() == torch::kBFloat16 && out.scalar_type() == torch::kBFloat16, "attention_diff: bfloat16 only");
    TORCH_CHECK(y.dim() == 2 && out.dim() == 2 && out.size(0) == y.size(0), "attention_diff: y and out [tokens, .]");
    TORCH_CHECK(block_table.dim() == 2 && cu_q.numel() == q_start.numel() + 1 && block_table.size(0) >= q_start.numel(),
                "attention_diff: cu_q [sequences + 1], q_start [sequences], block_table [sequences, stride]");
    TORCH_CHECK(vtb::attention_diff_supports(dim, v_dim, heads, kv_heads), "attention_diff: sizes that the kernel does not take");
    TORCH_CHECK(q_col % 8 == 0 && out_col % 8 == 0 && y.size(1) % 8 == 0 && out.size(1) % 8 == 0,
                "attention_diff: columns and rows must start on 16-byte boundaries");
    check_cols(y, q_col, heads * 2 * dim, "attention_diff (q)"); check_cols(out, out_col, heads * v_dim, "attention_diff (out)");
    check_pages(k_cache, v_cache, y, kv_heads * 2, dim, v_dim, kv_heads);
    TORCH_CHECK(k_cache.size(2) % 16 == 0, "attention_diff: pages of a multiple of 16 tokens");
    const int group = heads / kv_heads;
    const int per_tile = vtb::attention_diff_tile_rows() / group;
    const int* tp = nullptr;
    int n_tiles = q_start.numel();
    if (tiles.has_value()) {
        check_i32(*tiles, "tiles");
        TORCH_CHECK(tiles->dim() == 2 && tiles->size(1) == 2, "attention_diff: tiles [n, 2]");
        tp = tiles->data_ptr<int>();
        n_tiles = tiles->size(0);
    } else {
        TORCH_CHECK(y.size(0) >= n_tiles, "attention_diff: a step of single tokens has a token for each sequence");
    }
    c10::cuda::CUDAGuard guard(y.device());
    check_launch(vtb::launch_attention_diff(y.data_ptr(), y.size(1), q_col, out.data_ptr(), out.size(1), out_col, (float)out_scale,
                                            k_cache.data_ptr(), v_cache.data_ptr(), cu_q.data_ptr<int>(), q_start.data_ptr<int>(),
                                            block_table.data_ptr<int>(), block_table.size(1), tp, n_tiles, per_tile, k_cache.size(0),
                                            heads, kv_heads, dim, v_dim, k_cache.size(2), window, keep_first, (float)scale, (float)lam,
                                            (float)sub_eps, status_ptr(status), stream_of(y)), "attention_diff");
}

void attention_latent(const Tensor& q, int64_t q_col, Tensor& out, int64_t out_col, const Tensor& pages, const Tensor& cu_q,
                      const Tensor& q_start, const Tensor& block_table, c10::optional<Tensor> tiles, int64_t heads, int64_t key,
                      int64_t v_dim, double scale, c10::optional<Tensor> sinks, c10::optional<Tensor> part) {
    check_cuda(q, "q"); check_cuda(out, "out"); check_cuda(pages, "pages");
    check_i32(cu_q, "cu_q"); check_i32(q_start, "q_start"); check_i32(block_table, "block_table");
    TORCH_CHECK(q.scalar_type() == torch::kBFloat16 && out.scalar_type() == torch::kBFloat16 && pages.scalar_type() == torch::kBFloat16,
                "attention_latent: bfloat16 only");
    TORCH_CHECK(q.dim() == 2 && out.dim() == 2 && out.size(0) == q.size(0) && q.is_contiguous() && out.is_contiguous(),
                "attention_latent: q and out [tokens, .]");
    TORCH_CHECK(block_table.dim() == 2 && cu_q.numel() == q_start.numel() + 1 && block_table.size(0) >= q_start.numel(),
                "attention_latent: cu_q [sequences + 1], q_start [sequences], block_table [sequences, stride]");
    TORCH_CHECK(vtb::attention_latent_supports(key, v_dim), "attention_latent: sizes that the kernel does not take");
    TORCH_CHECK(pages.dim() == 4 && pages.size(1) == 1 && pages.size(3) == key && pages.is_contiguous(),
                "attention_latent: pages [pages, 1, page_size, key]");
    TORCH_CHECK(q_col % 8 == 0 && out_col % 2 == 0 && q.size(1) % 8 == 0 && out.size(1) % 2 == 0,
                "attention_latent: queries must start on 16-byte boundaries");
    check_cols(q, q_col, heads * key, "attention_latent (q)"); check_cols(out, out_col, heads * v_dim, "attention_latent (out)");
    const float* sp = nullptr;
    if (sinks.has_value()) {
        check_f32(*sinks, "sinks");
        TORCH_CHECK(sinks->numel() == heads, "attention_latent: one sink a head");
        sp = sinks->data_ptr<float>();
    }
    const int* tp = nullptr;
    int n_tiles = q_start.numel();
    if (tiles.has_value()) {
        check_i32(*tiles, "tiles");
        TORCH_CHECK(tiles->dim() == 2 && tiles->size(1) == 2, "attention_latent: tiles [n, 2]");
        tp = tiles->data_ptr<int>();
        n_tiles = tiles->size(0);
    } else {
        TORCH_CHECK(q.size(0) >= n_tiles, "attention_latent: a step of single tokens has a token for each sequence");
    }
    float* pp = nullptr;
    int n_splits = 1;
    if (part.has_value()) {
        check_f32(*part, "part");
        TORCH_CHECK(!tiles.has_value() && part->dim() == 4 && part->size(0) >= 1 && part->size(0) <= 16 && part->size(1) == q.size(0) &&
                    part->size(2) == heads && part->size(3) == v_dim + 2 && part->is_contiguous(),
                    "attention_latent: part [runs <= 16, tokens, heads, v_dim + 2], with a step of single tokens");
        pp = part->data_ptr<float>();
        n_splits = part->size(0);
    }
    c10::cuda::CUDAGuard guard(q.device());
    check_launch(vtb::launch_attention_latent(q.data_ptr(), q.size(1), q_col, out.data_ptr(), out.size(1), out_col, pages.data_ptr(),
                                              cu_q.data_ptr<int>(), q_start.data_ptr<int>(), block_table.data_ptr<int>(),
                                              block_table.size(1), tp, n_tiles, pages.size(0), heads, key, v_dim, pages.size(2),
                                              (float)scale, sp, n_splits, pp, q.size(0), stream_of(q)), "attention_latent");
}

void retention_scan(const Tensor& y, int64_t q_col, int64_t k_col, int64_t v_col, const Tensor& decay, double k_scale,
                    c10::optional<Tensor> frequencies, const Tensor& positions, Tensor& state, const Tensor& cu_q, const Tensor& rows,
                    Tensor& o, int64_t heads, int64_t dim, int64_t v_dim, c10::optional<Tensor> status, int64_t most_threads,
                    c10::optional<Tensor> ends, int64_t act) {
    check_scan(y, state, cu_q, rows, o, heads, dim, v_dim, "retention_scan");
    float* ep = nullptr;
    int end_rows = 0;
    if (ends.has_value()) {
        check_f32(*ends, "ends");
        TORCH_CHECK(ends->dim() == 4 && ends->size(1) == heads && ends->size(2) == dim && ends->size(3) == v_dim, "retention_scan: ends [n, heads, dim, v_dim]");
        ep = ends->data_ptr<float>();
        end_rows = ends->size(0);
    }
    check_f32(decay, "decay"); check_i32(positions, "positions");
    TORCH_CHECK(decay.numel() == heads, "retention_scan: one decay for each head");
    TORCH_CHECK(positions.numel() == y.size(0), "retention_scan: one position a token");
    check_cols(y, q_col, heads * dim, "retention_scan (q)"); check_cols(y, k_col, heads * dim, "retention_scan (k)");
    check_cols(y, v_col, heads * v_dim, "retention_scan (v)");
    const float* fp = nullptr;
    int half = 0;
    if (frequencies.has_value()) {
        check_f32(*frequencies, "frequencies");
        fp = frequencies->data_ptr<float>();
        half = frequencies->numel();
        TORCH_CHECK(2 * half <= dim, "retention_scan: the rotation covers more than the head");
    }
    c10::cuda::CUDAGuard guard(y.device());
    check_launch(vtb::launch_retention_scan(dtype_code(y, "y"), y.data_ptr(), y.size(1), q_col, k_col, v_col, decay.data_ptr<float>(),
                                            (float)k_scale, fp, half, positions.data_ptr<int>(), state.data_ptr<float>(), state.size(0),
                                            cu_q.data_ptr<int>(), rows.data_ptr<int>(), rows.numel(), o.data_ptr<float>(), heads, dim,
                                            v_dim, (int)most_threads, status_ptr(status), ep, end_rows, stream_of(y), (int)act), "retention_scan");
}

void retention_carry(Tensor& state, const Tensor& ends, Tensor& starts, const Tensor& seq_row, const Tensor& seq_first,
                     const Tensor& seq_count, const Tensor& seg_len, const Tensor& decay, c10::optional<Tensor> status) {
    check_f32(state, "state"); check_f32(ends, "ends"); check_f32(starts, "starts"); check_f32(decay, "decay");
    check_i32(seq_row, "seq_row"); check_i32(seq_first, "seq_first"); check_i32(seq_count, "seq_count"); check_i32(seg_len, "seg_len");
    TORCH_CHECK(state.dim() == 4 && ends.dim() == 4 && starts.sizes() == ends.sizes() && ends.size(1) == state.size(1) &&
                ends.size(2) == state.size(2) && ends.size(3) == state.size(3) && decay.numel() == state.size(1),
                "retention_carry: state [rows, heads, dim, v_dim], ends and starts [n, heads, dim, v_dim], decay [heads]");
    TORCH_CHECK(seq_first.numel() == seq_row.numel() && seq_count.numel() == seq_row.numel() && seg_len.numel() == ends.size(0),
                "retention_carry: one row, first and count a split sequence; one length a later segment");
    c10::cuda::CUDAGuard guard(state.device());
    check_launch(vtb::launch_retention_carry(state.data_ptr<float>(), state.size(0), ends.data_ptr<float>(), starts.data_ptr<float>(),
                                             seq_row.data_ptr<int>(), seq_first.data_ptr<int>(), seq_count.data_ptr<int>(),
                                             seg_len.data_ptr<int>(), seq_row.numel(), decay.data_ptr<float>(), state.size(1), state.size(2),
                                             state.size(3), status_ptr(status), stream_of(state)), "retention_carry");
}

void retention_fix(const Tensor& y, int64_t q_col, const Tensor& positions, c10::optional<Tensor> frequencies, const Tensor& starts,
                   const Tensor& tiles, const Tensor& decay, Tensor& o, int64_t act) {
    check_cuda(y, "y"); check_i32(positions, "positions"); check_f32(starts, "starts"); check_i32(tiles, "tiles"); check_f32(decay, "decay");
    check_f32(o, "o");
    TORCH_CHECK(starts.dim() == 4 && tiles.dim() == 2 && tiles.size(1) == 4, "retention_fix: starts [n, heads, dim, v_dim], tiles [m, 4]");
    const int heads = starts.size(1), dim = starts.size(2), v_dim = starts.size(3);
    TORCH_CHECK(y.dim() == 2 && o.dim() == 2 && o.size(0) == y.size(0) && o.size(1) == heads * v_dim && decay.numel() == heads &&
                positions.numel() == y.size(0), "retention_fix: o [tokens, heads * v_dim], one position a token, one decay a head");
    check_cols(y, q_col, heads * dim, "retention_fix (q)");
    const float* fp = nullptr;
    int half = 0;
    if (frequencies.has_value()) {
        check_f32(*frequencies, "frequencies");
        fp = frequencies->data_ptr<float>();
        half = frequencies->numel();
        TORCH_CHECK(2 * half <= dim, "retention_fix: the rotation covers more than the head");
    }
    c10::cuda::CUDAGuard guard(y.device());
    check_launch(vtb::launch_retention_fix(dtype_code(y, "y"), y.data_ptr(), y.size(1), q_col, positions.data_ptr<int>(), fp, half,
                                           starts.data_ptr<float>(), tiles.data_ptr<int>(), tiles.size(0), decay.data_ptr<float>(),
                                           o.data_ptr<float>(), heads, dim, v_dim, stream_of(y), (int)act), "retention_fix");
}

// the router's logits as a tensor [tokens, experts], or the token's input x [tokens, width] and the router's matrix
// [experts, width] (float32) from which the kernel forms them
struct RouterInput {
    const float* logits = nullptr;
    const void* x = nullptr;
    const float* router = nullptr;
    int width = 0, tokens = 0, experts = 0, x_dtype = vtb::kF32;
};

RouterInput router_input(const c10::optional<Tensor>& logits, const c10::optional<Tensor>& x, const c10::optional<Tensor>& router, const char* who) {
    RouterInput r;
    if (logits.has_value()) {
        check_f32(*logits, "logits");
        TORCH_CHECK(logits->dim() == 2, who, ": logits [tokens, experts]");
        r.logits = logits->data_ptr<float>(); r.tokens = logits->size(0); r.experts = logits->size(1);
        return r;
    }
    TORCH_CHECK(x.has_value() && router.has_value(), who, ": logits, or the input rows and the router's matrix");
    check_cuda(*x, "x"); check_f32(*router, "router");
    TORCH_CHECK(x->dim() == 2 && router->dim() == 2 && router->size(1) == x->size(1) && x->size(1) % 8 == 0, who,
                ": x [tokens, width], router [experts, width], width a multiple of 8");
    r.x = x->data_ptr(); r.router = router->data_ptr<float>(); r.width = x->size(1); r.tokens = x->size(0); r.experts = router->size(0);
    r.x_dtype = dtype_code(*x, "x");
    return r;
}

void route_topk(c10::optional<Tensor> logits, int64_t top, Tensor& ids, Tensor& weights, c10::optional<Tensor> x, c10::optional<Tensor> router,
                int64_t mode, double scale) {
    check_i32(ids, "ids"); check_f32(weights, "weights");
    const RouterInput r = router_input(logits, x, router, "route_topk");
    TORCH_CHECK(ids.dim() == 2 && ids.size(0) == r.tokens && ids.size(1) == top && weights.sizes() == ids.sizes(),
                "route_topk: ids and weights [tokens, top]");
    TORCH_CHECK(r.experts <= 1024 && top >= 1 && top <= r.experts, "route_topk: 1 <= top <= experts <= 1024");
    c10::cuda::CUDAGuard guard(ids.device());
    check_launch(vtb::launch_route_topk(r.x_dtype, r.logits, r.x, r.router, r.width, r.tokens, r.experts, top, ids.data_ptr<int>(),
                                        weights.data_ptr<float>(), stream_of(ids), (int)mode, (float)scale), "route_topk");
}

void expert_lists(const Tensor& ids, Tensor& lists, Tensor& counts) {
    check_i32(ids, "ids"); check_i32(lists, "lists"); check_i32(counts, "counts");
    TORCH_CHECK(lists.dim() == 2 && counts.numel() == lists.size(0) && lists.size(1) >= ids.size(0),
                "expert_lists: lists [experts, at least tokens], counts [experts]");
    c10::cuda::CUDAGuard guard(ids.device());
    check_launch(vtb::launch_expert_lists(ids.data_ptr<int>(), ids.numel(), lists.size(0), lists.size(1), lists.data_ptr<int>(),
                                          counts.data_ptr<int>(), stream_of(ids)), "expert_lists");
}

void gather_picks(const Tensor& x, const Tensor& lists, const Tensor& counts, int64_t top, Tensor& sorted, Tensor& where) {
    check_cuda(x, "x"); check_cuda(sorted, "sorted"); check_i32(lists, "lists"); check_i32(counts, "counts"); check_i32(where, "where");
    TORCH_CHECK(x.dim() == 2 && sorted.dim() == 2 && sorted.size(1) == x.size(1) && sorted.size(0) == x.size(0) * top &&
                where.numel() == sorted.size(0) && x.scalar_type() == sorted.scalar_type() && x.size(1) % 8 == 0,
                "gather_picks: x [tokens, width], sorted [tokens * top, width], where [tokens * top]");
    c10::cuda::CUDAGuard guard(x.device());
    check_launch(vtb::launch_gather_picks(dtype_code(x, "x"), x.data_ptr(), x.size(1), lists.data_ptr<int>(), lists.size(1),
                                          counts.data_ptr<int>(), lists.size(0), top, sorted.size(0), sorted.data_ptr(),
                                          where.data_ptr<int>(), stream_of(x)), "gather_picks");
}

void combine_picks(const Tensor& y, const Tensor& where, const Tensor& weights, c10::optional<Tensor> shared_y, Tensor& out) {
    check_cuda(y, "y"); check_cuda(out, "out"); check_i32(where, "where"); check_f32(weights, "weights");
    TORCH_CHECK(weights.dim() == 2 && out.dim() == 2 && y.dim() == 2 && out.size(0) == weights.size(0) && y.size(1) == out.size(1) &&
                y.size(0) == where.numel() && where.numel() == weights.numel() && y.scalar_type() == out.scalar_type() && out.size(1) % 8 == 0,
                "combine_picks: y [tokens * top, width], where [tokens * top], weights [tokens, top], out [tokens, width]");
    const void* sp = nullptr;
    if (shared_y.has_value()) {
        check_cuda(*shared_y, "shared_y");
        TORCH_CHECK(shared_y->sizes() == out.sizes() && shared_y->scalar_type() == out.scalar_type(), "combine_picks: shared_y like out");
        sp = shared_y->data_ptr();
    }
    c10::cuda::CUDAGuard guard(y.device());
    check_launch(vtb::launch_combine_picks(dtype_code(y, "y"), y.data_ptr(), y.size(1), where.data_ptr<int>(), weights.data_ptr<float>(),
                                           weights.size(1), out.size(0), sp, out.data_ptr(), stream_of(y)), "combine_picks");
}

void route_experts(c10::optional<Tensor> logits, int64_t top, Tensor& act, int64_t inter, c10::optional<Tensor> x, c10::optional<Tensor> router,
                   int64_t mode, double scale) {
    check_cuda(act, "act");
    const RouterInput r = router_input(logits, x, router, "route_experts");
    TORCH_CHECK(act.dim() == 2 && act.size(0) == r.tokens, "route_experts: act [tokens, .]");
    TORCH_CHECK(r.x == nullptr || r.x_dtype == dtype_code(act, "act"), "route_experts: x and act of one dtype");
    TORCH_CHECK(r.experts >= 1 && r.experts <= 1024 && top >= 1 && top <= r.experts, "route_experts: 1 <= top <= experts <= 1024");
    TORCH_CHECK(inter >= 0 && r.experts * inter <= act.size(1), "route_experts: experts * inter columns lie outside act");
    c10::cuda::CUDAGuard guard(act.device());
    check_launch(vtb::launch_route_experts(dtype_code(act, "act"), r.logits, r.x, r.router, r.width, r.tokens, r.experts, top, act.data_ptr(),
                                           act.size(1), inter, stream_of(act), (int)mode, (float)scale), "route_experts");
}



// ---- layers with a latent for each token (latent.cu)

void token_shift(const Tensor& x, const Tensor& mu, Tensor& state, const Tensor& cu_q, const Tensor& rows, const Tensor& token_seq,
                 Tensor& out, c10::optional<Tensor> status) {
    check_f32(x, "x"); check_f32(mu, "mu"); check_f32(state, "state"); check_i32(cu_q, "cu_q"); check_i32(rows, "rows");
    check_i32(token_seq, "token_seq"); check_cuda(out, "out");
    TORCH_CHECK(x.dim() == 2 && out.dim() == 2 && out.sizes() == x.sizes(), "token_shift: x and out [tokens, width]");
    const int width = x.size(1);
    TORCH_CHECK(mu.numel() == width && state.dim() == 2 && state.size(1) == width, "token_shift: mu [width], state [rows, width]");
    TORCH_CHECK(cu_q.numel() == rows.numel() + 1 && token_seq.numel() == x.size(0), "token_shift: cu_q [sequences + 1], a sequence a token");
    c10::cuda::CUDAGuard guard(x.device());
    check_launch(vtb::launch_token_shift(dtype_code(out, "out"), x.data_ptr<float>(), mu.data_ptr<float>(), state.data_ptr<float>(),
                                         state.size(0), cu_q.data_ptr<int>(), rows.data_ptr<int>(), token_seq.data_ptr<int>(), rows.numel(),
                                         out.data_ptr(), x.size(0), width, status_ptr(status), stream_of(x)), "token_shift");
}

// (frequencies, half) of an optional tensor of rotation frequencies
const float* frequencies_of(const c10::optional<Tensor>& frequencies, int& half) {
    half = 0;
    if (!frequencies.has_value()) return nullptr;
    check_f32(*frequencies, "frequencies");
    half = frequencies->numel();
    return frequencies->data_ptr<float>();
}

void latent_prepare(const Tensor& y, int64_t q_col, int64_t q_rank, int64_t kv_col, int64_t kv_rank, int64_t rot_dim, const Tensor& q_weight,
                    const Tensor& k_weight, double eps, c10::optional<Tensor> frequencies, double mult, const Tensor& positions,
                    const Tensor& token_seq, const Tensor& block_table, Tensor& cq, Tensor& pages, bool store, c10::optional<Tensor> status) {
    check_cuda(y, "y"); check_f32(q_weight, "q_weight"); check_f32(k_weight, "k_weight"); check_i32(positions, "positions");
    check_i32(token_seq, "token_seq"); check_i32(block_table, "block_table"); check_cuda(cq, "cq"); check_cuda(pages, "pages");
    TORCH_CHECK(y.dim() == 2 && cq.dim() == 2 && cq.size(0) == y.size(0) && cq.size(1) >= q_rank && cq.scalar_type() == y.scalar_type() &&
                pages.scalar_type() == y.scalar_type(), "latent_prepare: y and cq [tokens, .] and the pages of one dtype");
    check_cols(y, q_col, q_rank, "latent_prepare (queries' latent)"); check_cols(y, kv_col, kv_rank + rot_dim, "latent_prepare (keys' latent)");
    TORCH_CHECK(pages.dim() == 4 && pages.size(1) == 1 && pages.size(3) == kv_rank + rot_dim, "latent_prepare: pages [pages, 1, page_size, kv_rank + rot_dim]");
    TORCH_CHECK(q_weight.numel() == q_rank && k_weight.numel() == kv_rank, "latent_prepare: a weight for each latent");
    TORCH_CHECK(positions.numel() == y.size(0) && token_seq.numel() == y.size(0) && block_table.dim() == 2, "latent_prepare: a position and "
                "a sequence a token, block_table [sequences, stride]");
    int half = 0;
    const float* fp = frequencies_of(frequencies, half);
    TORCH_CHECK(2 * half <= rot_dim, "latent_prepare: the rotation covers more than the rotated part");
    c10::cuda::CUDAGuard guard(y.device());
    check_launch(vtb::launch_latent_prepare(dtype_code(y, "y"), y.data_ptr(), y.size(1), q_col, q_rank, kv_col, kv_rank, rot_dim,
                                            q_weight.data_ptr<float>(), k_weight.data_ptr<float>(), (float)eps, fp, half, (float)mult,
                                            positions.data_ptr<int>(), token_seq.data_ptr<int>(), block_table.data_ptr<int>(),
                                            block_table.size(1), block_table.size(0), pages.size(0), pages.size(2), cq.data_ptr(), cq.size(1),
                                            pages.data_ptr(), store ? 1 : 0, y.size(0), status_ptr(status), stream_of(y)), "latent_prepare");
}

void head_matmul(const Tensor& x, int64_t x_col, int64_t x_head, const Tensor& m, Tensor& out, int64_t out_col, int64_t out_head, int64_t mode,
                 int64_t tail, c10::optional<Tensor> frequencies, double mult, c10::optional<Tensor> positions,
                 c10::optional<Tensor> token_seq, c10::optional<Tensor> gate, int64_t gate_col) {
    check_cuda(x, "x"); check_cuda(m, "m"); check_cuda(out, "out");
    TORCH_CHECK(x.dim() == 2 && out.dim() == 2 && m.dim() == 3 && out.size(0) == x.size(0) && out.scalar_type() == x.scalar_type(),
                "head_matmul: x and out [tokens, .] of one dtype, m [heads, inner, outer]");
    TORCH_CHECK(mode >= 0 && mode <= 2 && tail >= 0, "head_matmul: mode 0, 1 (a rotated tail) or 2 (a gate)");
    const int heads = m.size(0), inner = m.size(1), outer = m.size(2);
    TORCH_CHECK(inner <= 1536, "head_matmul: inner sizes up to 1536");
    TORCH_CHECK(x_head >= inner + (mode == 1 ? tail : 0) && out_head >= outer + (mode == 1 ? tail : 0), "head_matmul: a head's inputs and "
                "outputs overlap the next head's");
    check_cols(x, x_col, (heads - 1) * x_head + inner + (mode == 1 ? tail : 0), "head_matmul (x)");
    check_cols(out, out_col, (heads - 1) * out_head + outer + (mode == 1 ? tail : 0), "head_matmul (out)");
    int half = 0;
    const float* fp = frequencies_of(frequencies, half);
    const int* pp = nullptr;
    const int* tp = nullptr;
    if (mode == 1) {
        TORCH_CHECK(positions.has_value() && token_seq.has_value(), "head_matmul: a rotated tail needs positions and sequences");
        check_i32(*positions, "positions"); check_i32(*token_seq, "token_seq");
        TORCH_CHECK(positions->numel() == x.size(0) && token_seq->numel() == x.size(0) && 2 * half <= tail, "head_matmul: a position a token; "
                    "the rotation within the tail");
        pp = positions->data_ptr<int>();
        tp = token_seq->data_ptr<int>();
    }
    const void* gp = nullptr;
    int gate_stride = 0;
    if (gate.has_value()) {
        check_cuda(*gate, "gate");
        TORCH_CHECK(mode == 2 && gate->dim() == 2 && gate->size(0) == x.size(0) && gate->scalar_type() == x.scalar_type(),
                    "head_matmul: a gate [tokens, .] of x's dtype, with mode 2");
        check_cols(*gate, gate_col, heads * outer, "head_matmul (gate)");
        gp = gate->data_ptr();
        gate_stride = gate->size(1);
    }
    c10::cuda::CUDAGuard guard(x.device());
    check_launch(vtb::launch_head_matmul(dtype_code(x, "x"), dtype_code(m, "m"), x.data_ptr(), x.size(1), x_col, x_head, m.data_ptr(), heads,
                                         inner, outer, out.data_ptr(), out.size(1), out_col, out_head, x.size(0), mode, tail, fp, half,
                                         (float)mult, pp, tp, gp, gate_stride, gate_col, stream_of(x)), "head_matmul");
}

void xielu(const Tensor& z, Tensor& out, double ap, double an) {
    check_cuda(z, "z"); check_cuda(out, "out");
    TORCH_CHECK(out.sizes() == z.sizes() && out.scalar_type() == z.scalar_type(), "xielu: z and out of one shape and dtype");
    c10::cuda::CUDAGuard guard(z.device());
    check_launch(vtb::launch_xielu(dtype_code(z, "z"), z.data_ptr(), out.data_ptr(), z.numel(), (float)ap, (float)an, stream_of(z)), "xielu");
}

void gate_clamp(const Tensor& gu, Tensor& out, int64_t interleave, double alpha, double limit, int64_t split, double limit2) {
    check_cuda(gu, "gu"); check_cuda(out, "out");
    TORCH_CHECK(gu.dim() == 2 && out.dim() == 2 && gu.size(0) == out.size(0) && gu.size(1) == 2 * out.size(1) && out.size(1) % 8 == 0 &&
                gu.scalar_type() == out.scalar_type(), "gate_clamp: gu [tokens, 2 n], out [tokens, n] of one dtype, n a multiple of 8");
    TORCH_CHECK((interleave == 0 || interleave == 8) && split % 8 == 0, "gate_clamp: interleave 0 or 8; the second limit starts at a multiple of 8");
    c10::cuda::CUDAGuard guard(gu.device());
    check_launch(vtb::launch_gate_clamp(dtype_code(gu, "gu"), gu.data_ptr(), out.data_ptr(), gu.size(0), out.size(1), interleave, (float)alpha,
                                        (float)limit, (int)split, (float)limit2, stream_of(gu)), "gate_clamp");
}

void scale_into(const Tensor& src, Tensor& dst, int64_t dst_col, double scale);

void silu_mul(const Tensor& gu, Tensor& out, int64_t interleave) {
    check_cuda(gu, "gu"); check_cuda(out, "out");
    TORCH_CHECK(gu.dim() == 2 && out.dim() == 2 && gu.size(1) == 2 * out.size(1) && gu.size(0) == out.size(0),
                "silu_mul: gu must be [tokens, 2 * inter] and out [tokens, inter]");
    TORCH_CHECK(gu.scalar_type() == out.scalar_type(), "silu_mul: one dtype");
    TORCH_CHECK(out.size(1) % 8 == 0, "silu_mul: intermediate size ", out.size(1), " must be a multiple of 8");
    c10::cuda::CUDAGuard guard(gu.device());
    TORCH_CHECK(interleave == 0 || interleave == 8, "silu_mul: interleave must be 0 or 8");
    check_launch(vtb::launch_silu_mul(dtype_code(gu, "gu"), gu.data_ptr(), out.data_ptr(), gu.size(0), out.size(1),
                                      interleave, stream_of(gu)), "silu_mul");
}

void check_cache(const Tensor& k_cache, const Tensor& v_cache, const Tensor& ref, int kv_heads, int head_dim) {
    check_cuda(k_cache, "k_cache"); check_cuda(v_cache, "v_cache");
    TORCH_CHECK(k_cache.dim() == 4 && k_cache.sizes() == v_cache.sizes(),
                "cache: k and v must be [pages, kv_heads, page_size, head_dim]");
    TORCH_CHECK(k_cache.size(1) == kv_heads && k_cache.size(3) == head_dim, "cache: kv_heads or head_dim differ");
    TORCH_CHECK(k_cache.scalar_type() == ref.scalar_type() && v_cache.scalar_type() == ref.scalar_type(),
                "cache: dtype differs from the activations'");
}

void rope_store(Tensor& qkv, const Tensor& positions, c10::optional<Tensor> cos_sin, Tensor& k_cache, Tensor& v_cache,
                const Tensor& token_seq, const Tensor& block_table, int64_t heads, int64_t kv_heads, int64_t head_dim,
                bool store, c10::optional<Tensor> status) {
    check_cuda(qkv, "qkv"); check_i32(positions, "positions"); check_i32(token_seq, "token_seq");
    check_i32(block_table, "block_table");
    TORCH_CHECK(qkv.dim() == 2 && qkv.size(1) == (heads + 2 * kv_heads) * head_dim,
                "rope_store: qkv must be [tokens, (heads + 2 kv_heads) * head_dim]");
    TORCH_CHECK(head_dim % 2 == 0, "rope_store: head_dim must be even");
    const int n = qkv.size(0);
    TORCH_CHECK(positions.numel() == n && token_seq.numel() == n, "rope_store: one position and sequence a token");
    TORCH_CHECK(block_table.dim() == 2, "rope_store: block_table must be [sequences, stride]");
    check_cache(k_cache, v_cache, qkv, kv_heads, head_dim);
    const float2* cs = nullptr;
    int max_pos = 0;
    if (cos_sin.has_value()) {
        check_f32(*cos_sin, "cos_sin");
        TORCH_CHECK(cos_sin->dim() == 3 && cos_sin->size(1) == head_dim / 2 && cos_sin->size(2) == 2,
                    "rope_store: cos_sin must be [positions, head_dim / 2, 2]");
        cs = reinterpret_cast<const float2*>(cos_sin->data_ptr<float>());
        max_pos = cos_sin->size(0);
    }
    c10::cuda::CUDAGuard guard(qkv.device());
    check_launch(vtb::launch_rope_store(dtype_code(qkv, "qkv"), qkv.data_ptr(), positions.data_ptr<int>(), cs, max_pos,
                                        k_cache.data_ptr(), v_cache.data_ptr(), token_seq.data_ptr<int>(),
                                        block_table.data_ptr<int>(), block_table.size(1), block_table.size(0),
                                        k_cache.size(0), n, heads, kv_heads, head_dim, k_cache.size(2),
                                        cs != nullptr, store, status_ptr(status), stream_of(qkv)), "rope_store");
}

void gemm_simt(const Tensor& a, const Tensor& w, c10::optional<Tensor> bias, Tensor& c) {
    check_cuda(a, "a"); check_cuda(w, "w"); check_cuda(c, "c");
    TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && c.dim() == 2, "gemm_simt: 2-d tensors");
    TORCH_CHECK(a.scalar_type() == w.scalar_type(), "gemm_simt: a and w must have one dtype");
    const int in_code = dtype_code(a, "a"), out_code = dtype_code(c, "c");
    TORCH_CHECK(out_code == vtb::kF32 || out_code == in_code, "gemm_simt: out must be float32 or the dtype of a");
    const int m = a.size(0), k = a.size(1), n = w.size(0);
    TORCH_CHECK(w.size(1) == k && c.size(0) == m && c.size(1) == n, "gemm_simt: shapes [m,k] x [n,k] -> [m,n]");
    TORCH_CHECK(k % 8 == 0, "gemm_simt: inner size ", k, " must be a multiple of 8");
    const float* bp = nullptr;
    if (bias.has_value()) {
        check_f32(*bias, "bias");
        TORCH_CHECK(bias->numel() == n, "gemm_simt: bias must have one entry for each output column");
        bp = bias->data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(a.device());
    check_launch(vtb::launch_gemm_simt(in_code, out_code, a.data_ptr(), w.data_ptr(), bp, c.data_ptr(), m, n, k,
                                       stream_of(a)), "gemm_simt");
}

void gemm_skinny(const Tensor& x, const Tensor& w, c10::optional<Tensor> bias, Tensor& out) {
    check_cuda(x, "x"); check_cuda(w, "w"); check_cuda(out, "out");
    TORCH_CHECK(x.scalar_type() == torch::kBFloat16 && w.scalar_type() == torch::kBFloat16,
                "gemm_skinny: x and w must be bfloat16");
    TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && out.dim() == 2, "gemm_skinny: 2-d tensors");
    const int m = x.size(0), k = x.size(1), n = w.size(0);
    TORCH_CHECK(w.size(1) == k && out.size(0) == m && out.size(1) == n, "gemm_skinny: shapes [m,k] x [n,k] -> [m,n]");
    TORCH_CHECK(m <= 64, "gemm_skinny: at most 64 rows, found ", m);
    TORCH_CHECK(k % 8 == 0, "gemm_skinny: inner size ", k, " must be a multiple of 8");
    const float* bp = nullptr;
    if (bias.has_value()) {
        check_f32(*bias, "bias");
        TORCH_CHECK(bias->numel() == n, "gemm_skinny: bias must have one entry for each output column");
        bp = bias->data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(x.device());
    check_launch(vtb::launch_gemm_skinny(dtype_code(out, "out"), x.data_ptr(), w.data_ptr(), bp, out.data_ptr(), m, n, k,
                                         stream_of(x)), "gemm_skinny");
}

// The hint of a product that runs next (kernels.h: NextProduct), from the arguments that carry it.
vtb::NextProduct next_product(const Tensor& like, const c10::optional<Tensor>& next_w, int64_t next_epilogue, int64_t next_bytes,
                              const char* who) {
    vtb::NextProduct next = {nullptr, 0, 0, 0, 0};
    if (next_w.has_value() && next_bytes > 0) {
        TORCH_CHECK(next_w->is_cuda() && next_w->scalar_type() == torch::kBFloat16 && next_w->dim() == 2 && next_w->is_contiguous() &&
                        next_w->device() == like.device() && next_epilogue >= 0 && next_epilogue <= 2,
                    who, ": next_w must be a contiguous bfloat16 matrix on the same device, next_epilogue 0, 1 or 2");
        next = {next_w->data_ptr(), (int)next_w->size(0), (int)next_w->size(1), (int)next_epilogue, (long long)next_bytes};
    }
    return next;
}

void gemm_tc(const Tensor& x, const Tensor& w, c10::optional<Tensor> bias, Tensor& out, c10::optional<Tensor> status,
             c10::optional<Tensor> scratch, c10::optional<Tensor> counters, int64_t epilogue, c10::optional<Tensor> next_w,
             int64_t next_epilogue, int64_t next_bytes) {
    check_cuda(x, "x"); check_cuda(w, "w"); check_cuda(out, "out");
    TORCH_CHECK(x.scalar_type() == torch::kBFloat16 && w.scalar_type() == torch::kBFloat16, "gemm_tc: x and w must be bfloat16");
    TORCH_CHECK(x.dim() == 2 && w.dim() == 2, "gemm_tc: x and w must be 2-d");
    const int m = x.size(0), k = x.size(1), n = w.size(0);
    TORCH_CHECK(epilogue >= 0 && epilogue <= 2, "gemm_tc: epilogue must be 0 (bias), 1 (silu(gate) * up) or 2 (unadded shares)");
    if (epilogue == 2) {
        TORCH_CHECK(w.size(1) == k && out.dim() == 3 && out.scalar_type() == torch::kFloat32 && out.is_contiguous() &&
                        out.size(0) == vtb::gemm_tc_shares(m, n, k) && out.size(1) == m && out.size(2) == n,
                    "gemm_tc: the shares of k go to a float32 out [gemm_tc_shares(m, n, k), m, n]");
    } else {
        TORCH_CHECK(w.size(1) == k && out.dim() == 2 && out.size(0) == m && out.size(1) == (epilogue == 1 ? n / 2 : n),
                    "gemm_tc: shapes [m,k] x [n,k] -> [m,n] (or [m,n/2] with the silu epilogue)");
    }
    TORCH_CHECK(epilogue != 1 || (n % 16 == 0 && !bias.has_value() && out.scalar_type() == torch::kBFloat16),
                "gemm_tc: the silu epilogue takes n % 16 == 0, no bias and a bfloat16 out");
    TORCH_CHECK(k % 8 == 0, "gemm_tc: inner size ", k, " must be a multiple of 8 (TMA rows start on 16-byte boundaries)");
    TORCH_CHECK(((uintptr_t)x.data_ptr() & 15) == 0 && ((uintptr_t)w.data_ptr() & 15) == 0,
                "gemm_tc: x and w must start on 16-byte boundaries");
    const float* bp = nullptr;
    if (bias.has_value()) {
        check_f32(*bias, "bias");
        TORCH_CHECK(bias->numel() == n, "gemm_tc: bias must have one entry for each output column");
        bp = bias->data_ptr<float>();
    }
    float* sp = nullptr;
    int* cp = nullptr;
    long long sn = 0;
    int cn = 0;
    if (scratch.has_value() && counters.has_value()) {
        check_f32(*scratch, "scratch"); check_i32(*counters, "counters");
        sp = scratch->data_ptr<float>();
        sn = scratch->numel();
        cp = counters->data_ptr<int>();
        cn = counters->numel();
    }
    const vtb::NextProduct next = next_product(x, next_w, next_epilogue, next_bytes, "gemm_tc");
    c10::cuda::CUDAGuard guard(x.device());
    check_launch(vtb::launch_gemm_tc(dtype_code(out, "out"), x.data_ptr(), w.data_ptr(), bp, out.data_ptr(), m, n, k,
                                     (int)epilogue, sp, sn, cp, cn, status_ptr(status), stream_of(x),
                                     next.w != nullptr ? &next : nullptr), "gemm_tc");
}

void gemm_tc_pair(const Tensor& x, const Tensor& w, c10::optional<Tensor> bias, Tensor& out, int64_t epilogue, int64_t bn,
                  c10::optional<Tensor> status, c10::optional<Tensor> scratch, c10::optional<Tensor> counters) {
    check_cuda(x, "x"); check_cuda(w, "w"); check_cuda(out, "out");
    TORCH_CHECK(x.scalar_type() == torch::kBFloat16 && w.scalar_type() == torch::kBFloat16 && out.scalar_type() == torch::kBFloat16,
                "gemm_tc_pair: x, w and out must be bfloat16");
    TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && out.dim() == 2, "gemm_tc_pair: x, w and out must be 2-d");
    const int m = x.size(0), k = x.size(1), n = w.size(0);
    TORCH_CHECK(epilogue == 0 || epilogue == 1, "gemm_tc_pair: epilogue must be 0 (bias) or 1 (silu(gate) * up)");
    TORCH_CHECK(bn == 0 || bn == 256 || bn == 224 || bn == 192, "gemm_tc_pair: tiles of 256, 224 or 192 rows of w (0: chosen by the sizes)");
    TORCH_CHECK(w.size(1) == k && out.size(0) == m && out.size(1) == (epilogue == 1 ? n / 2 : n),
                "gemm_tc_pair: shapes [m,k] x [n,k] -> [m,n] (or [m,n/2] with the silu epilogue)");
    TORCH_CHECK(epilogue != 1 || (n % 16 == 0 && !bias.has_value()), "gemm_tc_pair: the silu epilogue takes n % 16 == 0 and no bias");
    TORCH_CHECK(k % 8 == 0, "gemm_tc_pair: inner size ", k, " must be a multiple of 8 (TMA rows start on 16-byte boundaries)");
    TORCH_CHECK(((uintptr_t)x.data_ptr() & 15) == 0 && ((uintptr_t)w.data_ptr() & 15) == 0,
                "gemm_tc_pair: x and w must start on 16-byte boundaries");
    const float* bp = nullptr;
    if (bias.has_value()) {
        check_f32(*bias, "bias");
        TORCH_CHECK(bias->numel() == n, "gemm_tc_pair: bias must have one entry for each output column");
        bp = bias->data_ptr<float>();
    }
    // scratch and counters (zeroed once; the kernel leaves them zero): with them, k is cut over pairs where the tiles are few
    float* sp = nullptr;
    int* cp = nullptr;
    long long scratch_floats = 0;
    int n_counters = 0;
    if (scratch.has_value() && counters.has_value()) {
        check_f32(*scratch, "scratch");
        check_cuda(*counters, "counters");
        TORCH_CHECK(counters->scalar_type() == torch::kInt32 && counters->is_contiguous(), "gemm_tc_pair: counters must be contiguous int32");
        sp = scratch->data_ptr<float>();
        scratch_floats = scratch->numel();
        cp = counters->data_ptr<int>();
        n_counters = (int)counters->numel();
    }
    c10::cuda::CUDAGuard guard(x.device());
    check_launch(vtb::launch_gemm_tc_pair(x.data_ptr(), w.data_ptr(), bp, out.data_ptr(), m, n, k, (int)epilogue, (int)bn, sp,
                                          scratch_floats, cp, n_counters, status_ptr(status), stream_of(x)), "gemm_tc_pair");
}

bool attention_mma_supports(int64_t head_dim, int64_t heads, int64_t kv_heads, int64_t warps) {
    return vtb::attention_mma_supports(head_dim, heads, kv_heads, warps);
}

void attention_mma(const Tensor& qkv, Tensor& out, const Tensor& k_cache, const Tensor& v_cache, const Tensor& cu_q,
                   const Tensor& q_start, const Tensor& block_table, c10::optional<Tensor> tiles, int64_t heads,
                   int64_t kv_heads, int64_t head_dim, int64_t window, double scale, int64_t warps, int64_t n_splits,
                   c10::optional<Tensor> part_o, c10::optional<Tensor> part_ml, c10::optional<Tensor> status, int64_t chunk,
                   c10::optional<Tensor> sinks, double softcap) {
    check_cuda(qkv, "qkv"); check_cuda(out, "out"); check_i32(cu_q, "cu_q"); check_i32(q_start, "q_start");
    check_i32(block_table, "block_table");
    TORCH_CHECK(qkv.scalar_type() == torch::kBFloat16 && out.scalar_type() == torch::kBFloat16,
                "attention_mma: bfloat16 only");
    const float* sp = nullptr;
    if (sinks.has_value()) {
        check_f32(*sinks, "sinks");
        TORCH_CHECK(sinks->numel() == heads, "attention_mma: one sink a head");
        sp = sinks->data_ptr<float>();
    }
    TORCH_CHECK(softcap >= 0.0, "attention_mma: softcap not negative");
    TORCH_CHECK(qkv.dim() == 2 && qkv.size(1) >= heads * head_dim, "attention_mma: qkv must hold the queries first");
    TORCH_CHECK(out.dim() == 2 && out.size(0) == qkv.size(0) && out.size(1) == heads * head_dim,
                "attention_mma: out must be [tokens, heads * head_dim]");
    TORCH_CHECK(heads % kv_heads == 0, "attention_mma: heads must be a multiple of kv_heads");
    TORCH_CHECK(vtb::attention_mma_supports(head_dim, heads, kv_heads, warps),
                "attention_mma: head_dim ", head_dim, " with ", heads / kv_heads, " heads in a group and ", warps,
                " warps is not supported (head_dim a multiple of 16 up to 128, group <= 16 * warps)");
    check_cache(k_cache, v_cache, qkv, kv_heads, head_dim);
    TORCH_CHECK(k_cache.size(2) % 16 == 0, "attention_mma: page size must be a multiple of 16");
    const int n_seqs = cu_q.numel() - 1;
    TORCH_CHECK(q_start.numel() == n_seqs && block_table.dim() == 2 && block_table.size(0) == n_seqs,
                "attention_mma: one q_start and one block-table row for each sequence");
    const int* tp = nullptr;
    int n_tiles = n_seqs;
    if (tiles.has_value()) {
        check_i32(*tiles, "tiles");
        TORCH_CHECK(tiles->dim() == 2 && tiles->size(1) == 2, "attention_mma: tiles must be [n, 2]");
        tp = tiles->data_ptr<int>();
        n_tiles = tiles->size(0);
    }
    float *po = nullptr, *pm = nullptr;
    const int n_tokens = qkv.size(0);
    if (n_splits > 1) {
        TORCH_CHECK(part_o.has_value() && part_ml.has_value(), "attention_mma: splits need scratch tensors");
        check_f32(*part_o, "part_o"); check_f32(*part_ml, "part_ml");
        TORCH_CHECK(part_o->numel() >= n_splits * n_tokens * heads * head_dim &&
                        part_ml->numel() >= n_splits * n_tokens * heads * 2, "attention_mma: scratch too small");
        po = part_o->data_ptr<float>();
        pm = part_ml->data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(qkv.device());
    check_launch(vtb::launch_attention_mma(qkv.data_ptr(), qkv.size(1), out.data_ptr(), k_cache.data_ptr(),
                                           v_cache.data_ptr(), cu_q.data_ptr<int>(), q_start.data_ptr<int>(),
                                           block_table.data_ptr<int>(), block_table.size(1), tp, n_tiles,
                                           k_cache.size(0), n_tokens, heads, kv_heads, head_dim, k_cache.size(2), window,
                                           (float)scale, warps, n_splits, po, pm, status_ptr(status), stream_of(qkv), (int)chunk, sp,
                                           (float)softcap),
                 "attention_mma");
}

bool attention_tc_supports(int64_t head_dim, int64_t heads, int64_t kv_heads) {
    return vtb::attention_tc_supports(head_dim, heads, kv_heads);
}

void attention_tc(const Tensor& qkv, Tensor& out, const Tensor& k_cache, const Tensor& v_cache, const Tensor& cu_q,
                  const Tensor& q_start, const Tensor& block_table, const Tensor& tiles, int64_t heads, int64_t kv_heads,
                  int64_t head_dim, int64_t window, double scale, c10::optional<Tensor> status, int64_t chunk, c10::optional<Tensor> sinks) {
    check_cuda(qkv, "qkv"); check_cuda(out, "out"); check_i32(cu_q, "cu_q"); check_i32(q_start, "q_start");
    check_i32(block_table, "block_table"); check_i32(tiles, "tiles");
    TORCH_CHECK(qkv.scalar_type() == torch::kBFloat16 && out.scalar_type() == torch::kBFloat16,
                "attention_tc: bfloat16 only");
    TORCH_CHECK(qkv.dim() == 2 && qkv.size(1) >= heads * head_dim && qkv.size(1) % 8 == 0 && qkv.is_contiguous(),
                "attention_tc: qkv must hold the queries first, rows a multiple of 16 bytes");
    TORCH_CHECK(out.dim() == 2 && out.size(0) == qkv.size(0) && out.size(1) == heads * head_dim && out.is_contiguous(),
                "attention_tc: out must be [tokens, heads * head_dim]");
    TORCH_CHECK(heads % kv_heads == 0 && vtb::attention_tc_supports(head_dim, heads, kv_heads),
                "attention_tc: head_dim ", head_dim, " with ", heads / std::max<int64_t>(kv_heads, 1),
                " heads in a group is not supported (head_dim 128, group <= 128)");
    check_cache(k_cache, v_cache, qkv, kv_heads, head_dim);
    TORCH_CHECK(k_cache.size(2) % 16 == 0, "attention_tc: page size must be a multiple of 16");
    TORCH_CHECK(k_cache.is_contiguous() && v_cache.is_contiguous() &&
                    reinterpret_cast<uintptr_t>(k_cache.data_ptr()) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(v_cache.data_ptr()) % 16 == 0,
                "attention_tc: the caches must be dense and 16-byte aligned");
    const int n_seqs = cu_q.numel() - 1;
    TORCH_CHECK(q_start.numel() == n_seqs && block_table.dim() == 2 && block_table.size(0) == n_seqs,
                "attention_tc: one q_start and one block-table row for each sequence");
    TORCH_CHECK(tiles.dim() == 2 && tiles.size(1) == 2, "attention_tc: tiles must be [n, 2]");
    const float* sinks_tc = nullptr;
    if (sinks.has_value()) {
        check_f32(*sinks, "sinks");
        TORCH_CHECK(sinks->numel() == heads, "attention_tc: one sink a head");
        sinks_tc = sinks->data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(qkv.device());
    check_launch(vtb::launch_attention_tc(qkv.data_ptr(), qkv.size(1), out.data_ptr(), k_cache.data_ptr(),
                                          v_cache.data_ptr(), cu_q.data_ptr<int>(), q_start.data_ptr<int>(),
                                          block_table.data_ptr<int>(), block_table.size(1), tiles.data_ptr<int>(),
                                          tiles.size(0), k_cache.size(0), heads, kv_heads, head_dim, k_cache.size(2),
                                          window, (float)scale, status_ptr(status), stream_of(qkv), (int)chunk, sinks_tc),
                 "attention_tc");
}

void attention_decode(const Tensor& qkv, Tensor& out, const Tensor& k_cache, const Tensor& v_cache, const Tensor& cu_q,
                      const Tensor& q_start, const Tensor& block_table, int64_t heads, int64_t kv_heads, int64_t head_dim,
                      int64_t window, double scale, int64_t n_splits, c10::optional<Tensor> part_o,
                      c10::optional<Tensor> part_ml, c10::optional<Tensor> counters, bool fuse_rope,
                      c10::optional<Tensor> cos_sin, bool store_kv, c10::optional<Tensor> status,
                      c10::optional<Tensor> qkv_shares, bool long_runs, int64_t run_blocks, int64_t chunk) {
    check_cuda(qkv, "qkv"); check_cuda(out, "out"); check_i32(cu_q, "cu_q"); check_i32(q_start, "q_start");
    check_i32(block_table, "block_table");
    TORCH_CHECK(qkv.scalar_type() == torch::kBFloat16 && out.scalar_type() == torch::kBFloat16,
                "attention_decode: bfloat16 only");
    TORCH_CHECK(qkv.dim() == 2 && qkv.size(1) >= heads * head_dim, "attention_decode: qkv must hold the queries first");
    TORCH_CHECK(out.dim() == 2 && out.size(0) == qkv.size(0) && out.size(1) == heads * head_dim,
                "attention_decode: out must be [tokens, heads * head_dim]");
    TORCH_CHECK(heads % kv_heads == 0 && vtb::attention_mma_supports(head_dim, heads, kv_heads, 1),
                "attention_decode: head_dim ", head_dim, " with ", heads / std::max<int64_t>(kv_heads, 1),
                " heads in a group is not supported (head_dim a multiple of 16 up to 128, group <= 16)");
    check_cache(k_cache, v_cache, qkv, kv_heads, head_dim);
    TORCH_CHECK(k_cache.size(2) % 16 == 0, "attention_decode: page size must be a multiple of 16");
    const int n_seqs = cu_q.numel() - 1, n_tokens = qkv.size(0);
    TORCH_CHECK(q_start.numel() == n_seqs && block_table.dim() == 2 && block_table.size(0) == n_seqs,
                "attention_decode: one q_start and one block-table row for each sequence");
    float *po = nullptr, *pm = nullptr;
    int* pc = nullptr;
    if (n_splits > 8 || part_o.has_value()) {
        TORCH_CHECK(part_o.has_value() && part_ml.has_value() && counters.has_value(),
                    "attention_decode: more than 8 runs need scratch tensors and counters");
        check_f32(*part_o, "part_o"); check_f32(*part_ml, "part_ml"); check_i32(*counters, "counters");
        TORCH_CHECK(part_o->numel() >= n_splits * n_tokens * heads * head_dim &&
                        part_ml->numel() >= n_splits * n_tokens * heads * 2 && counters->numel() >= n_seqs * kv_heads,
                    "attention_decode: scratch too small");
        po = part_o->data_ptr<float>();
        pm = part_ml->data_ptr<float>();
        pc = counters->data_ptr<int>();
    }
    const float2* cs = nullptr;
    int max_pos = 0;
    if (cos_sin.has_value()) {
        check_f32(*cos_sin, "cos_sin");
        TORCH_CHECK(cos_sin->dim() == 3 && cos_sin->size(1) == head_dim / 2 && cos_sin->size(2) == 2,
                    "attention_decode: cos_sin must be [positions, head_dim / 2, 2]");
        cs = reinterpret_cast<const float2*>(cos_sin->data_ptr<float>());
        max_pos = cos_sin->size(0);
    }
    if (fuse_rope) {
        TORCH_CHECK(n_tokens == n_seqs, "attention_decode: the fused rotation takes one token a sequence");
        TORCH_CHECK(qkv.size(1) == (heads + 2 * kv_heads) * head_dim, "attention_decode: qkv must hold q, k and v");
    }
    const float* shp = nullptr;
    int n_shares = 0;
    if (qkv_shares.has_value()) {
        check_f32(*qkv_shares, "qkv_shares");
        TORCH_CHECK(fuse_rope && qkv_shares->dim() == 3 && qkv_shares->size(1) == n_tokens && qkv_shares->size(2) == qkv.size(1) &&
                        qkv_shares->is_contiguous() && qkv_shares->size(0) >= 1 && qkv.size(1) % 2 == 0,
                    "attention_decode: shares of qkv must be [shares, tokens, width of qkv] float, with the fused rotation");
        shp = qkv_shares->data_ptr<float>();
        n_shares = qkv_shares->size(0);
    }
    c10::cuda::CUDAGuard guard(qkv.device());
    check_launch(vtb::launch_attention_decode(qkv.data_ptr(), qkv.size(1), out.data_ptr(), k_cache.data_ptr(),
                                              v_cache.data_ptr(), cu_q.data_ptr<int>(), q_start.data_ptr<int>(),
                                              block_table.data_ptr<int>(), block_table.size(1), n_seqs, k_cache.size(0),
                                              n_tokens, heads, kv_heads, head_dim, k_cache.size(2), window, (float)scale,
                                              n_splits, po, pm, pc, fuse_rope ? 1 : 0, cs, max_pos, store_kv ? 1 : 0,
                                              shp, n_shares, long_runs ? 1 : 0, (int)run_blocks, status_ptr(status),
                                              stream_of(qkv), (int)chunk), "attention_decode");
}

void attention_simt(const Tensor& qkv, Tensor& out, const Tensor& k_cache, const Tensor& v_cache,
                    const Tensor& positions, const Tensor& token_seq, const Tensor& block_table, int64_t heads,
                    int64_t kv_heads, int64_t head_dim, int64_t window, double scale, c10::optional<Tensor> status) {
    check_cuda(qkv, "qkv"); check_cuda(out, "out"); check_i32(positions, "positions");
    check_i32(token_seq, "token_seq"); check_i32(block_table, "block_table");
    TORCH_CHECK(qkv.dim() == 2 && qkv.size(1) >= heads * head_dim, "attention: qkv must hold the queries first");
    TORCH_CHECK(out.dim() == 2 && out.size(0) == qkv.size(0) && out.size(1) == heads * head_dim,
                "attention: out must be [tokens, heads * head_dim]");
    TORCH_CHECK(out.scalar_type() == qkv.scalar_type(), "attention: one dtype");
    TORCH_CHECK(head_dim <= 256, "attention: head_dim ", head_dim, " is above 256");
    TORCH_CHECK(heads % kv_heads == 0, "attention: heads must be a multiple of kv_heads");
    check_cache(k_cache, v_cache, qkv, kv_heads, head_dim);
    const int n = qkv.size(0);
    TORCH_CHECK(positions.numel() == n && token_seq.numel() == n, "attention: one position and sequence a token");
    c10::cuda::CUDAGuard guard(qkv.device());
    check_launch(vtb::launch_attention_simt(dtype_code(qkv, "qkv"), qkv.data_ptr(), qkv.size(1), out.data_ptr(),
                                            k_cache.data_ptr(), v_cache.data_ptr(), positions.data_ptr<int>(),
                                            token_seq.data_ptr<int>(), block_table.data_ptr<int>(),
                                            block_table.size(1), block_table.size(0), k_cache.size(0), n, heads,
                                            kv_heads, head_dim, k_cache.size(2), window, (float)scale,
                                            status_ptr(status), stream_of(qkv)), "attention_simt");
}

void argmax(const Tensor& logits, Tensor& out) {
    check_f32(logits, "logits"); check_i32(out, "out");
    TORCH_CHECK(logits.dim() == 2 && out.numel() == logits.size(0), "argmax: logits [rows, vocab], out [rows]");
    c10::cuda::CUDAGuard guard(logits.device());
    check_launch(vtb::launch_argmax(logits.data_ptr<float>(), out.data_ptr<int>(), logits.size(0), logits.size(1),
                                    stream_of(logits)), "argmax");
}

void sample(const Tensor& logits, const Tensor& temperature, const Tensor& top_k, const Tensor& top_p, const Tensor& u,
            Tensor& out) {
    check_f32(logits, "logits"); check_f32(temperature, "temperature"); check_i32(top_k, "top_k");
    check_f32(top_p, "top_p"); check_f32(u, "u"); check_i32(out, "out");
    const int rows = logits.size(0);
    TORCH_CHECK(logits.dim() == 2 && temperature.numel() == rows && top_k.numel() == rows && top_p.numel() == rows &&
                    u.numel() == rows && out.numel() == rows,
                "sample: one parameter of each kind for each row of logits");
    c10::cuda::CUDAGuard guard(logits.device());
    check_launch(vtb::launch_sample(logits.data_ptr<float>(), temperature.data_ptr<float>(), top_k.data_ptr<int>(),
                                    top_p.data_ptr<float>(), u.data_ptr<float>(), out.data_ptr<int>(), rows,
                                    logits.size(1), stream_of(logits)), "sample");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    namespace py = pybind11;
    m.def("embedding", &embedding, py::arg("table"), py::arg("ids"), py::arg("out"), py::arg("status") = py::none(),
          py::arg("scale") = 1.0);
    m.def("logits_scale_cap", &logits_scale_cap, py::arg("logits"), py::arg("scale"), py::arg("cap"));
    m.def("rmsnorm", &rmsnorm, py::arg("x"), py::arg("delta"), py::arg("weight"), py::arg("eps"), py::arg("out"),
          py::arg("rows") = py::none(), py::arg("status") = py::none(), py::arg("post_weight") = py::none(),
          py::arg("post_eps") = 0.0, py::arg("post_mult") = 1.0, py::arg("groups") = 1, py::arg("x_scale") = 1.0,
          py::arg("write_normed") = false);
    m.def("layernorm", &layernorm, py::arg("x"), py::arg("delta"), py::arg("weight"), py::arg("eps"), py::arg("out"),
          py::arg("rows") = py::none(), py::arg("status") = py::none(), py::arg("post_weight") = py::none(),
          py::arg("post_eps") = 0.0, py::arg("post_mult") = 1.0);
    m.def("polynorm", &polynorm, py::arg("z"), py::arg("coefficients"), py::arg("eps"), py::arg("out"), py::arg("n_mean") = 0);
    m.def("scale_into", &scale_into);
    m.def("head_norm_gate", &head_norm_gate, py::arg("o"), py::arg("y"), py::arg("gate_col"), py::arg("weight"),
          py::arg("weight_per_channel"), py::arg("eps"), py::arg("act"), py::arg("out"), py::arg("out_col"), py::arg("out_scale"),
          py::arg("heads"), py::arg("v_dim"), py::arg("token_seq") = py::none());
    m.def("gla_scan", &gla_scan, py::arg("y"), py::arg("q_col"), py::arg("k_col"), py::arg("v_col"), py::arg("low_col"), py::arg("a2"),
          py::arg("a2_bias"), py::arg("inv_tau"), py::arg("q_scale"), py::arg("state"), py::arg("cu_q"), py::arg("rows"), py::arg("o"),
          py::arg("heads"), py::arg("dim"), py::arg("v_dim"), py::arg("status") = py::none(), py::arg("most_threads") = 0);
    m.def("delta_scan", &delta_scan, py::arg("y"), py::arg("r_col"), py::arg("k_col"), py::arg("v_col"), py::arg("a_col"), py::arg("low_col"),
          py::arg("w2"), py::arg("w0"), py::arg("a_bias"), py::arg("decay_rate"), py::arg("key_eps"), py::arg("state"), py::arg("cu_q"),
          py::arg("rows"), py::arg("o"), py::arg("heads"), py::arg("dim"), py::arg("status") = py::none(), py::arg("most_threads") = 0);
    m.def("attention_prepare", &attention_prepare, py::arg("y"), py::arg("q_col"), py::arg("k_col"), py::arg("v_col"), py::arg("positions"),
          py::arg("token_seq"), py::arg("frequencies"), py::arg("norm_eps"), py::arg("k_cache"), py::arg("v_cache"), py::arg("block_table"),
          py::arg("heads"), py::arg("kv_heads"), py::arg("dim"), py::arg("v_dim"), py::arg("store"), py::arg("status") = py::none(),
          py::arg("v_heads") = -1, py::arg("q_weight") = py::none(), py::arg("k_weight") = py::none(), py::arg("norm_first") = false,
          py::arg("whole_projection") = false, py::arg("rot_mult") = 1.0, py::arg("q_temp_coef") = 0.0, py::arg("q_temp_every") = 1);
    m.def("attention_general", &attention_general, py::arg("y"), py::arg("q_col"), py::arg("out"), py::arg("out_col"), py::arg("out_scale"),
          py::arg("k_cache"), py::arg("v_cache"), py::arg("positions"), py::arg("token_seq"), py::arg("block_table"), py::arg("heads"),
          py::arg("kv_heads"), py::arg("dim"), py::arg("v_dim"), py::arg("window"), py::arg("chunk"), py::arg("scale"),
          py::arg("status") = py::none(), py::arg("keep_first") = 0, py::arg("maps") = 1, py::arg("lam") = 0.0, py::arg("sub_eps") = 0.0,
          py::arg("sinks") = py::none(), py::arg("values_in_keys") = false, py::arg("softcap") = 0.0, py::arg("gate_mode") = 0,
          py::arg("gate_col") = 0);
    m.def("gate_into", &gate_into);
    m.def("gated_delta_scan", &gated_delta_scan);
    m.def("conv_tail_update", &conv_tail_update);
    m.def("memory_scan", &memory_scan);
    m.def("normed_sum", &normed_sum);
    m.def("add_rows", &add_rows);
    m.def("attention_diff", &attention_diff);
    m.def("attention_diff_supports", &vtb::attention_diff_supports);
    m.def("attention_diff_tile_rows", &vtb::attention_diff_tile_rows);
    m.def("attention_latent", &attention_latent);
    m.def("attention_latent_supports", &vtb::attention_latent_supports);
    m.def("attention_latent_tile_rows", &vtb::attention_latent_tile_rows);
    m.def("retention_scan", &retention_scan, py::arg("y"), py::arg("q_col"), py::arg("k_col"), py::arg("v_col"), py::arg("decay"),
          py::arg("k_scale"), py::arg("frequencies"), py::arg("positions"), py::arg("state"), py::arg("cu_q"), py::arg("rows"), py::arg("o"),
          py::arg("heads"), py::arg("dim"), py::arg("v_dim"), py::arg("status") = py::none(), py::arg("most_threads") = 0,
          py::arg("ends") = py::none(), py::arg("act") = 0);
    m.def("retention_carry", &retention_carry);
    m.def("retention_fix", &retention_fix, py::arg("y"), py::arg("q_col"), py::arg("positions"), py::arg("frequencies"), py::arg("starts"),
          py::arg("tiles"), py::arg("decay"), py::arg("o"), py::arg("act") = 0);
    m.def("route_experts", &route_experts, py::arg("logits"), py::arg("top"), py::arg("act"), py::arg("inter"), py::arg("x") = py::none(),
          py::arg("router") = py::none(), py::arg("mode") = 0, py::arg("scale") = 1.0);
    m.def("route_topk", &route_topk, py::arg("logits"), py::arg("top"), py::arg("ids"), py::arg("weights"), py::arg("x") = py::none(),
          py::arg("router") = py::none(), py::arg("mode") = 0, py::arg("scale") = 1.0);
    m.def("token_shift", &token_shift, py::arg("x"), py::arg("mu"), py::arg("state"), py::arg("cu_q"), py::arg("rows"), py::arg("token_seq"),
          py::arg("out"), py::arg("status") = py::none());
    m.def("latent_prepare", &latent_prepare, py::arg("y"), py::arg("q_col"), py::arg("q_rank"), py::arg("kv_col"), py::arg("kv_rank"),
          py::arg("rot_dim"), py::arg("q_weight"), py::arg("k_weight"), py::arg("eps"), py::arg("frequencies"), py::arg("mult"),
          py::arg("positions"), py::arg("token_seq"), py::arg("block_table"), py::arg("cq"), py::arg("pages"), py::arg("store") = true,
          py::arg("status") = py::none());
    m.def("head_matmul", &head_matmul, py::arg("x"), py::arg("x_col"), py::arg("x_head"), py::arg("m"), py::arg("out"), py::arg("out_col"),
          py::arg("out_head"), py::arg("mode") = 0, py::arg("tail") = 0, py::arg("frequencies") = py::none(), py::arg("mult") = 1.0,
          py::arg("positions") = py::none(), py::arg("token_seq") = py::none(), py::arg("gate") = py::none(), py::arg("gate_col") = 0);
    m.def("xielu", &xielu, py::arg("z"), py::arg("out"), py::arg("ap"), py::arg("an"));
    m.def("gate_clamp", &gate_clamp, py::arg("gu"), py::arg("out"), py::arg("interleave"), py::arg("alpha"), py::arg("limit"),
          py::arg("split"), py::arg("limit2"));
    m.def("expert_lists", &expert_lists);
    m.def("gather_picks", &gather_picks);
    m.def("combine_picks", &combine_picks);
    m.def("silu_mul", &silu_mul, py::arg("gu"), py::arg("out"), py::arg("interleave") = 0);
    m.def("rope_store", &rope_store, py::arg("qkv"), py::arg("positions"), py::arg("cos_sin"), py::arg("k_cache"),
          py::arg("v_cache"), py::arg("token_seq"), py::arg("block_table"), py::arg("heads"), py::arg("kv_heads"),
          py::arg("head_dim"), py::arg("store"), py::arg("status") = py::none());
    m.def("gemm_simt", &gemm_simt, py::arg("a"), py::arg("w"), py::arg("bias"), py::arg("c"));
    m.def("attention_simt", &attention_simt, py::arg("qkv"), py::arg("out"), py::arg("k_cache"), py::arg("v_cache"),
          py::arg("positions"), py::arg("token_seq"), py::arg("block_table"), py::arg("heads"), py::arg("kv_heads"),
          py::arg("head_dim"), py::arg("window"), py::arg("scale"), py::arg("status") = py::none());
    m.def("gemm_skinny", &gemm_skinny, py::arg("x"), py::arg("w"), py::arg("bias"), py::arg("out"));
    m.def("gemm_tc", &gemm_tc, py::arg("x"), py::arg("w"), py::arg("bias"), py::arg("out"), py::arg("status") = py::none(),
          py::arg("scratch") = py::none(), py::arg("counters") = py::none(), py::arg("epilogue") = 0,
          py::arg("next_w") = py::none(), py::arg("next_epilogue") = 0, py::arg("next_bytes") = 0);
    m.def("gemm_tc_pair", &gemm_tc_pair, py::arg("x"), py::arg("w"), py::arg("bias"), py::arg("out"), py::arg("epilogue") = 0,
          py::arg("bn") = 256, py::arg("status") = py::none(), py::arg("scratch") = py::none(), py::arg("counters") = py::none());
    m.def("gemm_tc_shares", [](int64_t m, int64_t n, int64_t k) { return (int64_t)vtb::gemm_tc_shares(m, n, k); });
    m.def("attention_mma_supports", &attention_mma_supports);
    m.def("attention_mma", &attention_mma, py::arg("qkv"), py::arg("out"), py::arg("k_cache"), py::arg("v_cache"),
          py::arg("cu_q"), py::arg("q_start"), py::arg("block_table"), py::arg("tiles"), py::arg("heads"),
          py::arg("kv_heads"), py::arg("head_dim"), py::arg("window"), py::arg("scale"), py::arg("warps"),
          py::arg("n_splits"), py::arg("part_o") = py::none(), py::arg("part_ml") = py::none(),
          py::arg("status") = py::none(), py::arg("chunk") = 0, py::arg("sinks") = py::none(), py::arg("softcap") = 0.0);
    m.def("attention_tc_supports", &attention_tc_supports);
    m.def("attention_tc", &attention_tc, py::arg("qkv"), py::arg("out"), py::arg("k_cache"), py::arg("v_cache"),
          py::arg("cu_q"), py::arg("q_start"), py::arg("block_table"), py::arg("tiles"), py::arg("heads"),
          py::arg("kv_heads"), py::arg("head_dim"), py::arg("window"), py::arg("scale"), py::arg("status") = py::none(),
          py::arg("chunk") = 0, py::arg("sinks") = py::none());
    m.def("attention_decode", &attention_decode, py::arg("qkv"), py::arg("out"), py::arg("k_cache"), py::arg("v_cache"),
          py::arg("cu_q"), py::arg("q_start"), py::arg("block_table"), py::arg("heads"), py::arg("kv_heads"),
          py::arg("head_dim"), py::arg("window"), py::arg("scale"), py::arg("n_splits"), py::arg("part_o") = py::none(),
          py::arg("part_ml") = py::none(), py::arg("counters") = py::none(), py::arg("fuse_rope") = false,
          py::arg("cos_sin") = py::none(), py::arg("store_kv") = false, py::arg("status") = py::none(),
          py::arg("qkv_shares") = py::none(), py::arg("long_runs") = false, py::arg("run_blocks") = 0,
          py::arg("chunk") = 0);
    m.def("argmax", &argmax, py::arg("logits"), py::arg("out"));
    m.def("sample", &sample, py::arg("logits"), py::arg("temperature"), py::arg("top_k"), py::arg("top_p"),
          py::arg("u"), py::arg("out"));
}
