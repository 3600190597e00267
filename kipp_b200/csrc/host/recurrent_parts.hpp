// Mixers that carry a matrix state per request instead of a key/value cache, a mixer made of
// several mixers side by side, and the feed-forward with a PolyNorm activation.
//
//   retention     linear attention with one fixed decay per head, no softmax and no denominator
//   delta_rule    the generalized delta rule: decay and removal rate per head, key channel and token
//   gated_memory  the matrix memory of the xLSTM: exponential input and forget gates per head and
//                 token, held stable by a running maximum, with a normalizer vector beside the matrix
//   wkv           time mixing with a decay per head, key channel and token and a bonus for the current
//                 token; every projection reads its own mix of the token's input and the one before
//   parallel      the sum of several mixers that read the same input
//   polynorm_mlp  W_down act(W_up h), act = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3
//
// Every constant (sizes, decays, scales, gates, eps) and every tensor name is a parameter of the
// plan, so another model can use these parts with other values.  The state is float32
// [heads, key dim, value dim] per request slot, zeroed by the engine at admission and advanced
// by exactly the tokens a step brings (kernels in recurrent.cu).
#pragma once
#include "parts.hpp"

namespace kipp {

inline float* upload_floats(Binder& b, const std::vector<float>& v, const std::string& what) {
    float* d = static_cast<float*>(b.allocate(std::max<size_t>(1, v.size()) * sizeof(float), what));
    if (!v.empty())
        cuda_check(cudaMemcpy(d, v.data(), v.size() * sizeof(float), cudaMemcpyHostToDevice), what.c_str());
    return d;
}
inline float* load_f32(Binder& b, const std::string& name, int64_t n) {
    float* d = static_cast<float*>(b.allocate((size_t)n * sizeof(float), name));
    b.load(name, d, F32, n, 1, n);
    return d;
}
inline int gate_code(const std::string& g) {
    if (g == "none") return 0;
    if (g == "silu") return 1;
    if (g == "sigmoid") return 2;
    fail(KIPP_E_CONFIG, "gate must be none, silu or sigmoid, not '" + g + "'");
}

// ---------------------------------------------------------------------------------------------
// Retention.  q = W_q h, k = W_k h [heads, dim], v = W_v h [heads, value_dim], no biases; q and k
// rotated by the position encoding; k scaled by key_scale (default dim^-1/2) after the rotation;
// per head S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t; each head's o divided by its root
// mean square (eps inside the root, no weight); heads concatenated, times gate(W_g h), times
// output_scale, through W_o into the residual stream.
class RetentionMixer : public Mixer {
public:
    RetentionMixer(const Json& j, const BuildContext& ctx) {
        hidden_ = (int)j.get("hidden_size").as_int();
        heads_ = (int)j.get("num_heads").as_int();
        dim_ = (int)j.get("head_dim").as_int();
        v_dim_ = (int)j.get_int("value_dim", dim_);
        eps_ = (float)j.get("eps").as_double();
        out_scale_ = (float)j.get_double("output_scale", 1.0);
        key_scale_ = (float)j.get_double("key_scale", 1.0 / std::sqrt((double)dim_));
        gate_ = gate_code(j.get_string("gate", "silu"));
        for (auto& d : j.get("decay").items()) decay_.push_back((float)d.as_double());
        position_ = make_position(j.get("position"), ctx);
        names_ = tensor_names(j, {{"q", "q"}, {"k", "k"}, {"v", "v"}, {"g", "g"}, {"o", "o"}});
        if (hidden_ <= 0 || heads_ <= 0 || dim_ <= 0 || v_dim_ <= 0) fail(KIPP_E_CONFIG, "retention: sizes must be positive");
        if ((int)decay_.size() != heads_) fail(KIPP_E_CONFIG, "retention: one decay per head is needed");
        if (position_->rotary_dim() > dim_ || position_->rotary_dim() % 2)
            fail(KIPP_E_CONFIG, "retention: rotary_dim must be even and at most head_dim");
        qk_ = heads_ * dim_;
        vv_ = heads_ * v_dim_;
        cols_ = 2 * qk_ + (gate_ ? 2 : 1) * vv_;
    }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        auto add = [&](const char* role, std::vector<int64_t> shape) {
            TensorSpec s;
            s.name = p + names_.at(role);
            s.shape = std::move(shape);
            out.push_back(s);
        };
        add("q", {qk_, hidden_});
        add("k", {qk_, hidden_});
        add("v", {vv_, hidden_});
        if (gate_) add("g", {vv_, hidden_});
        add("o", {hidden_, vv_});
        position_->tensor_specs(p, out);
    }
    std::optional<StateSpec> state_spec() const override { return StateSpec{{heads_, dim_, v_dim_}, F32}; }
    void bind(Binder& b, const std::string& p) override {
        dtype_ = b.compute_dtype();
        const size_t es = dtype_size(dtype_);
        // one matrix for q, k, v and the gate so that one product makes them all
        w_in_ = b.allocate((size_t)cols_ * hidden_ * es, p + "qkvg");
        char* base = static_cast<char*>(w_in_);
        b.load(p + names_.at("q"), base, dtype_, hidden_, qk_, hidden_);
        b.load(p + names_.at("k"), base + (size_t)qk_ * hidden_ * es, dtype_, hidden_, qk_, hidden_);
        b.load(p + names_.at("v"), base + (size_t)2 * qk_ * hidden_ * es, dtype_, hidden_, vv_, hidden_);
        if (gate_) b.load(p + names_.at("g"), base + (size_t)(2 * qk_ + vv_) * hidden_ * es, dtype_, hidden_, vv_, hidden_);
        w_o_ = b.allocate((size_t)hidden_ * vv_ * es, p + names_.at("o"));
        b.load(p + names_.at("o"), w_o_, dtype_, vv_, hidden_, vv_);
        decay_dev_ = upload_floats(b, decay_, "retention decays");
        position_->bind(b, p);
        if (!Ops::recurrent_scan_ok(dim_, v_dim_, false))
            fail(KIPP_E_UNSUPPORTED, format("retention: the scan kernel does not take heads of %d x %d", dim_, v_dim_));
    }
    size_t weight_bytes() const override { return ((size_t)cols_ + vv_) * hidden_ * dtype_size(dtype_); }
    bool folds_rms() const override { return Ops::gemm_scale_ok(dtype_, w_in_, hidden_, w_in_, hidden_); }
    void forward(StepContext& ctx, const LayerRun& run, int mixer_slot, const void* h, float* residual) override {
        const int T = ctx.tokens();
        const size_t es = ctx.element();
        Ops& ops = *ctx.ops;
        const StepMeta& m = *ctx.meta;
        NormFold fold_in, fold_out;
        void* proj = ctx.workspace->buffer("retention_proj", (size_t)T * cols_ * es);
        ops.gemm(proj, ctx.dtype, cols_, h, hidden_, w_in_, hidden_, dtype_, T, cols_, hidden_, EPI_STORE,
                 fold_input(ctx, fold_in));
        const float* cos_sin = step_rope_table(ctx, *position_, false);
        float* state = static_cast<float*>(ctx.state_view(run, mixer_slot, nullptr));
        void* gated = ctx.workspace->buffer("retention_out", (size_t)T * vv_ * es);
        ops.retention_scan(gated, vv_, proj, cols_, ctx.dtype, 0, qk_, 2 * qk_, 2 * qk_ + vv_, state, decay_dev_, cos_sin,
                           position_->rotary_dim(), m.q_start, m.slots, m.shape.entries, T, heads_, dim_, v_dim_,
                           key_scale_, eps_, out_scale_, gate_);
        const NormFold* emit = fold_emit(ctx, fold_out, hidden_);
        ops.gemm(residual, F32, hidden_, gated, vv_, w_o_, vv_, dtype_, T, hidden_, vv_, EPI_ADD, emit);
        fold_emitted(ctx, emit, hidden_);
    }

private:
    int hidden_ = 0, heads_ = 0, dim_ = 0, v_dim_ = 0, qk_ = 0, vv_ = 0, cols_ = 0, gate_ = 1, dtype_ = BF16;
    float eps_ = 0.f, out_scale_ = 1.f, key_scale_ = 1.f;
    std::vector<float> decay_;
    std::unique_ptr<PositionEncoding> position_;
    std::map<std::string, std::string> names_;
    void *w_in_ = nullptr, *w_o_ = nullptr;
    float* decay_dev_ = nullptr;
};

// ---------------------------------------------------------------------------------------------
// Generalized delta rule.  r = W_r h, k = W_k h, v = W_v h, all [heads, dim].  Per head and key
// channel: decay w = exp(-exp(-1/2) sigmoid(W_w2 tanh(W_w1 h) + w0)), removal rate a =
// sigmoid(W_a h + a_bias).  With the unit key u = k / sqrt(sum k^2 + 1e-6) of each head:
// S_t = diag(w) S_{t-1} - (a * u)(u^T S_{t-1}) + k v^T (both terms read the old state), o_t =
// S_t^T r.  Each head's o divided by its root mean square (eps inside the root), heads
// concatenated, times the weight `norm`, times gate(W_g h), times output_scale, through W_o.
class DeltaRuleMixer : public Mixer {
public:
    DeltaRuleMixer(const Json& j, const BuildContext&) {
        hidden_ = (int)j.get("hidden_size").as_int();
        heads_ = (int)j.get("num_heads").as_int();
        dim_ = (int)j.get("head_dim").as_int();
        rank_ = (int)j.get_int("decay_rank", 0);      // 0: the width of the bottleneck is read from its tensor
        eps_ = (float)j.get("eps").as_double();
        out_scale_ = (float)j.get_double("output_scale", 1.0);
        gate_ = gate_code(j.get_string("gate", "sigmoid"));
        names_ = tensor_names(j, {{"r", "r"}, {"k", "k"}, {"v", "v"}, {"g", "g"}, {"a", "a"}, {"a_bias", "a.b"},
                                  {"w1", "w1"}, {"w2", "w2"}, {"w_bias", "w0"}, {"norm", "norm"}, {"o", "o"}});
        if (hidden_ <= 0 || heads_ <= 0 || dim_ <= 0 || rank_ < 0) fail(KIPP_E_CONFIG, "delta_rule: sizes must be positive");
        hd_ = heads_ * dim_;
        set_rank(rank_);
    }
    // the low-rank bottleneck sits last in the fused projection; rows padded to 16 bytes
    void set_rank(int rank) {
        rank_ = rank;
        cols_ = (gate_ ? 5 : 4) * hd_ + rank_;
        ld_ = (cols_ + 7) / 8 * 8;
        rank_ld_ = (rank_ + 7) / 8 * 8;
    }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        auto add = [&](const char* role, std::vector<int64_t> shape, const char* init = "normal") {
            TensorSpec s;
            s.name = p + names_.at(role);
            s.shape = std::move(shape);
            s.init = init;
            out.push_back(s);
        };
        add("r", {hd_, hidden_});
        add("k", {hd_, hidden_});
        add("v", {hd_, hidden_});
        if (gate_) add("g", {hd_, hidden_});
        add("a", {hd_, hidden_});
        add("a_bias", {hd_});
        add("w1", {rank_ > 0 ? rank_ : -1, hidden_});
        add("w2", {hd_, rank_ > 0 ? rank_ : -1});
        add("w_bias", {hd_});
        add("norm", {hd_}, "near_one");
        add("o", {hidden_, hd_});
    }
    std::optional<StateSpec> state_spec() const override { return StateSpec{{heads_, dim_, dim_}, F32}; }
    void bind(Binder& b, const std::string& p) override {
        dtype_ = b.compute_dtype();
        const size_t es = dtype_size(dtype_);
        if (rank_ == 0) {
            const std::vector<int64_t> s1 = b.stored_shape(p + names_.at("w1")), s2 = b.stored_shape(p + names_.at("w2"));
            if (s1.size() != 2 || s2.size() != 2 || s1[0] <= 0 || s1[0] != s2[1])
                fail(KIPP_E_WEIGHTS, "delta_rule: " + p + names_.at("w1") + " and " + p + names_.at("w2") +
                                         " do not agree on the width of the bottleneck");
            set_rank((int)s1[0]);
        }
        // one matrix for r, k, v, the gate, the removal rate and the decay's bottleneck
        w_in_ = b.allocate((size_t)cols_ * hidden_ * es, p + "rkvgaw");
        char* base = static_cast<char*>(w_in_);
        int row = 0;
        auto put = [&](const char* role, int rows) {
            b.load(p + names_.at(role), base + (size_t)row * hidden_ * es, dtype_, hidden_, rows, hidden_);
            row += rows;
        };
        put("r", hd_);
        put("k", hd_);
        put("v", hd_);
        if (gate_) put("g", hd_);
        put("a", hd_);
        put("w1", rank_);
        // the bottleneck's rows of W_w2 are padded to a multiple of 8 elements (zeros beyond the rank)
        w2_ = b.allocate((size_t)hd_ * rank_ld_ * es, p + names_.at("w2"));
        cuda_check(cudaMemset(w2_, 0, (size_t)hd_ * rank_ld_ * es), "clearing a padded weight");
        b.load(p + names_.at("w2"), w2_, dtype_, rank_ld_, hd_, rank_);
        w_o_ = b.allocate((size_t)hidden_ * hd_ * es, p + names_.at("o"));
        b.load(p + names_.at("o"), w_o_, dtype_, hd_, hidden_, hd_);
        a_bias_ = load_f32(b, p + names_.at("a_bias"), hd_);
        w_bias_ = load_f32(b, p + names_.at("w_bias"), hd_);
        norm_ = load_f32(b, p + names_.at("norm"), hd_);
        if (!Ops::recurrent_scan_ok(dim_, dim_, true))
            fail(KIPP_E_UNSUPPORTED, format("delta_rule: the scan kernel does not take heads of %d x %d", dim_, dim_));
    }
    size_t weight_bytes() const override {
        return ((size_t)cols_ * hidden_ + (size_t)hd_ * rank_ + (size_t)hidden_ * hd_) * dtype_size(dtype_) + (size_t)3 * hd_ * 4;
    }
    bool folds_rms() const override { return Ops::gemm_scale_ok(dtype_, w_in_, hidden_, w_in_, hidden_); }
    void forward(StepContext& ctx, const LayerRun& run, int mixer_slot, const void* h, float* residual) override {
        const int T = ctx.tokens();
        const size_t es = ctx.element();
        Ops& ops = *ctx.ops;
        const StepMeta& m = *ctx.meta;
        NormFold fold_in, fold_out;
        void* proj = ctx.workspace->buffer("delta_proj", (size_t)T * ld_ * es);
        ops.gemm(proj, ctx.dtype, ld_, h, hidden_, w_in_, hidden_, dtype_, T, cols_, hidden_, EPI_STORE,
                 fold_input(ctx, fold_in));
        const int g_off = 3 * hd_, a_off = (gate_ ? 4 : 3) * hd_, w1_off = a_off + hd_;
        // the decay: tanh of the bottleneck, then its second product; the bias and the squashing
        // are the scan kernel's, in float32
        void* low = ctx.workspace->buffer("delta_low_rank", (size_t)T * rank_ld_ * es);
        if (rank_ld_ != rank_) cuda_check(cudaMemsetAsync(low, 0, (size_t)T * rank_ld_ * es, ctx.stream), "clearing the bottleneck");
        ops.tanh_rows(low, rank_ld_, static_cast<const char*>(proj) + (size_t)w1_off * es, ld_, ctx.dtype, T, rank_);
        void* w_raw = ctx.workspace->buffer("delta_decay", (size_t)T * hd_ * es);
        ops.gemm(w_raw, ctx.dtype, hd_, low, rank_ld_, w2_, rank_ld_, dtype_, T, hd_, rank_ld_, EPI_STORE);
        float* state = static_cast<float*>(ctx.state_view(run, mixer_slot, nullptr));
        void* gated = ctx.workspace->buffer("delta_out", (size_t)T * hd_ * es);
        ops.delta_rule_scan(gated, hd_, proj, ld_, ctx.dtype, 0, hd_, 2 * hd_, g_off, a_off, w_raw, hd_, a_bias_, w_bias_,
                            norm_, state, m.q_start, m.slots, m.shape.entries, T, heads_, dim_, eps_, out_scale_, gate_);
        const NormFold* emit = fold_emit(ctx, fold_out, hidden_);
        ops.gemm(residual, F32, hidden_, gated, hd_, w_o_, hd_, dtype_, T, hidden_, hd_, EPI_ADD, emit);
        fold_emitted(ctx, emit, hidden_);
    }

private:
    int hidden_ = 0, heads_ = 0, dim_ = 0, rank_ = 0, rank_ld_ = 0, hd_ = 0, cols_ = 0, ld_ = 0, gate_ = 2, dtype_ = BF16;
    float eps_ = 0.f, out_scale_ = 1.f;
    std::map<std::string, std::string> names_;
    void *w_in_ = nullptr, *w2_ = nullptr, *w_o_ = nullptr;
    float *a_bias_ = nullptr, *w_bias_ = nullptr, *norm_ = nullptr;
};

// ---------------------------------------------------------------------------------------------
// Gated matrix memory.  q = W_q h * query_scale (default dim^-1/2), k = W_k h [heads, dim],
// v = W_v h [heads, value_dim]; per head a log input gate i = cap tanh((W_i h + b_i) / cap) and a
// log forget gate f = logsigmoid(cap tanh((W_f h + b_f) / cap)).  With a running maximum m (0 at
// the start): m_t = max(f_t + m_{t-1}, i_t), S_t = e^(f_t + m_{t-1} - m_t) S_{t-1} + e^(i_t - m_t) k_t v_t^T,
// n_t the same with k_t alone, o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6).  Each head's o
// divided by its root mean square (eps inside the root), heads concatenated, times the weight
// `norm`, times gate(W_g h), times output_scale, through W_o.  S, n and m are float32 per request.
class GatedMemoryMixer : public Mixer {
public:
    GatedMemoryMixer(const Json& j, const BuildContext&) {
        hidden_ = (int)j.get("hidden_size").as_int();
        heads_ = (int)j.get("num_heads").as_int();
        dim_ = (int)j.get("head_dim").as_int();
        v_dim_ = (int)j.get_int("value_dim", dim_);
        cap_ = (float)j.get("gate_cap").as_double();
        eps_ = (float)j.get("eps").as_double();
        out_scale_ = (float)j.get_double("output_scale", 1.0);
        q_scale_ = (float)j.get_double("query_scale", 1.0 / std::sqrt((double)dim_));
        gate_ = gate_code(j.get_string("gate", "sigmoid"));
        names_ = tensor_names(j, {{"q", "q"}, {"k", "k"}, {"v", "v"}, {"g", "g"}, {"i", "i"}, {"i_bias", "i.b"},
                                  {"f", "f"}, {"f_bias", "f.b"}, {"norm", "norm"}, {"o", "o"}});
        if (hidden_ <= 0 || heads_ <= 0 || dim_ <= 0 || v_dim_ <= 0) fail(KIPP_E_CONFIG, "gated_memory: sizes must be positive");
        if (!(cap_ > 0)) fail(KIPP_E_CONFIG, "gated_memory: gate_cap must be positive");
        qk_ = heads_ * dim_;
        vv_ = heads_ * v_dim_;
        g_off_ = 2 * qk_ + vv_;
        i_off_ = g_off_ + (gate_ ? vv_ : 0);
        cols_ = i_off_ + 2 * heads_;
        ld_ = (cols_ + 7) / 8 * 8;
    }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        auto add = [&](const char* role, std::vector<int64_t> shape, const char* init = "normal") {
            TensorSpec s;
            s.name = p + names_.at(role);
            s.shape = std::move(shape);
            s.init = init;
            out.push_back(s);
        };
        add("q", {qk_, hidden_});
        add("k", {qk_, hidden_});
        add("v", {vv_, hidden_});
        if (gate_) add("g", {vv_, hidden_});
        add("i", {heads_, hidden_});
        add("i_bias", {heads_});
        add("f", {heads_, hidden_});
        add("f_bias", {heads_});
        add("norm", {vv_}, "near_one");
        add("o", {hidden_, vv_});
    }
    std::optional<StateSpec> state_spec() const override {
        return StateSpec{{Ops::gated_memory_state_floats(heads_, dim_, v_dim_)}, F32};
    }
    void bind(Binder& b, const std::string& p) override {
        dtype_ = b.compute_dtype();
        const size_t es = dtype_size(dtype_);
        // one matrix for q, k, v, the output gate and the two gates of the memory
        w_in_ = b.allocate((size_t)cols_ * hidden_ * es, p + "qkvgif");
        char* base = static_cast<char*>(w_in_);
        int row = 0;
        auto put = [&](const char* role, int rows) {
            b.load(p + names_.at(role), base + (size_t)row * hidden_ * es, dtype_, hidden_, rows, hidden_);
            row += rows;
        };
        put("q", qk_);
        put("k", qk_);
        put("v", vv_);
        if (gate_) put("g", vv_);
        put("i", heads_);
        put("f", heads_);
        w_o_ = b.allocate((size_t)hidden_ * vv_ * es, p + names_.at("o"));
        b.load(p + names_.at("o"), w_o_, dtype_, vv_, hidden_, vv_);
        i_bias_ = load_f32(b, p + names_.at("i_bias"), heads_);
        f_bias_ = load_f32(b, p + names_.at("f_bias"), heads_);
        norm_ = load_f32(b, p + names_.at("norm"), vv_);
        if (!Ops::gated_memory_ok(dim_, v_dim_))
            fail(KIPP_E_UNSUPPORTED, format("gated_memory: the scan kernel does not take heads of %d x %d", dim_, v_dim_));
    }
    size_t weight_bytes() const override {
        return ((size_t)cols_ + vv_) * hidden_ * dtype_size(dtype_) + ((size_t)2 * heads_ + vv_) * 4;
    }
    bool folds_rms() const override { return Ops::gemm_scale_ok(dtype_, w_in_, hidden_, w_in_, hidden_); }
    void forward(StepContext& ctx, const LayerRun& run, int mixer_slot, const void* h, float* residual) override {
        const int T = ctx.tokens();
        const size_t es = ctx.element();
        Ops& ops = *ctx.ops;
        const StepMeta& m = *ctx.meta;
        NormFold fold_in, fold_out;
        void* proj = ctx.workspace->buffer("memory_proj", (size_t)T * ld_ * es);
        ops.gemm(proj, ctx.dtype, ld_, h, hidden_, w_in_, hidden_, dtype_, T, cols_, hidden_, EPI_STORE,
                 fold_input(ctx, fold_in));
        float* state = static_cast<float*>(ctx.state_view(run, mixer_slot, nullptr));
        void* gated = ctx.workspace->buffer("memory_out", (size_t)T * vv_ * es);
        ops.gated_memory_scan(gated, vv_, proj, ld_, ctx.dtype, 0, qk_, 2 * qk_, g_off_, i_off_, i_off_ + heads_, i_bias_,
                              f_bias_, norm_, state, m.q_start, m.slots, m.shape.entries, T, heads_, dim_, v_dim_, cap_,
                              q_scale_, eps_, out_scale_, gate_);
        const NormFold* emit = fold_emit(ctx, fold_out, hidden_);
        ops.gemm(residual, F32, hidden_, gated, vv_, w_o_, vv_, dtype_, T, hidden_, vv_, EPI_ADD, emit);
        fold_emitted(ctx, emit, hidden_);
    }

private:
    int hidden_ = 0, heads_ = 0, dim_ = 0, v_dim_ = 0, qk_ = 0, vv_ = 0, cols_ = 0, ld_ = 0, g_off_ = 0, i_off_ = 0;
    int gate_ = 2, dtype_ = BF16;
    float cap_ = 0.f, eps_ = 0.f, out_scale_ = 1.f, q_scale_ = 1.f;
    std::map<std::string, std::string> names_;
    void *w_in_ = nullptr, *w_o_ = nullptr;
    float *i_bias_ = nullptr, *f_bias_ = nullptr, *norm_ = nullptr;
};

// ---------------------------------------------------------------------------------------------
// Several mixers side by side: each reads the same input and adds its (scaled) output to the
// residual stream; each has its own cache or state (mixer slot = its index).  The scale of a
// branch is that mixer's own output_scale.
class ParallelMixer : public Mixer {
public:
    ParallelMixer(const Json& j, const BuildContext& ctx) {
        for (auto& b : j.get("branches").items()) {
            prefixes_.push_back(b.get_string("prefix", ""));
            branches_.push_back(Registry::get().make_as<Mixer>(b.get("part"), ctx, "a mixer"));
        }
        if (branches_.empty()) fail(KIPP_E_CONFIG, "parallel: at least one branch is needed");
        if (branches_.size() > 16) fail(KIPP_E_CONFIG, "parallel: at most 16 branches");
    }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        for (size_t i = 0; i < branches_.size(); ++i) branches_[i]->tensor_specs(p + prefixes_[i], out);
    }
    void bind(Binder& b, const std::string& p) override {
        for (size_t i = 0; i < branches_.size(); ++i) branches_[i]->bind(b, p + prefixes_[i]);
    }
    size_t weight_bytes() const override {
        size_t n = 0;
        for (auto& m : branches_) n += m->weight_bytes();
        return n;
    }
    bool graph_safe() const override {
        for (auto& m : branches_)
            if (!m->graph_safe()) return false;
        return true;
    }
    bool folds_rms() const override {
        for (auto& m : branches_)
            if (!m->folds_rms()) return false;
        return true;
    }
    std::vector<Mixer*> parts() override {
        std::vector<Mixer*> v;
        for (auto& m : branches_) v.push_back(m.get());
        return v;
    }
    void forward(StepContext& ctx, const LayerRun& run, int mixer_slot, const void* h, float* residual) override {
        // only the last residual add may leave the next norm's deferred form: the stream is
        // complete only then
        const RmsNormSpec* emit_for = ctx.emit_for;
        for (size_t i = 0; i < branches_.size(); ++i) {
            ctx.emit_for = i + 1 == branches_.size() ? emit_for : nullptr;
            branches_[i]->forward(ctx, run, mixer_slot + (int)i, h, residual);
        }
    }

private:
    std::vector<std::string> prefixes_;
    std::vector<std::unique_ptr<Mixer>> branches_;
};

// ---------------------------------------------------------------------------------------------
// x += W_down act(W_up n), act = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3 with powers taken element
// by element and N the division of a token's vector by its root mean square (eps inside the
// root).  The four numbers are the tensor `act`.
class PolyNormFeedForward : public FeedForward {
public:
    explicit PolyNormFeedForward(const Json& j) {
        hidden_ = (int)j.get("hidden_size").as_int();
        inter_ = (int)j.get("intermediate_size").as_int();
        eps_ = (float)j.get("eps").as_double();
        names_ = tensor_names(j, {{"up", "up"}, {"down", "down"}, {"act", "act"}});
        if (hidden_ <= 0 || inter_ <= 0) fail(KIPP_E_CONFIG, "polynorm_mlp: sizes must be positive");
    }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        auto add = [&](const char* role, std::vector<int64_t> shape, const char* init = "normal") {
            TensorSpec s;
            s.name = p + names_.at(role);
            s.shape = std::move(shape);
            s.init = init;
            out.push_back(s);
        };
        add("up", {inter_, hidden_});
        add("down", {hidden_, inter_});
        add("act", {4}, "near_one");
    }
    void bind(Binder& b, const std::string& p) override {
        dtype_ = b.compute_dtype();
        const size_t es = dtype_size(dtype_);
        w_up_ = b.allocate((size_t)inter_ * hidden_ * es, p + names_.at("up"));
        b.load(p + names_.at("up"), w_up_, dtype_, hidden_, inter_, hidden_);
        w_down_ = b.allocate((size_t)hidden_ * inter_ * es, p + names_.at("down"));
        b.load(p + names_.at("down"), w_down_, dtype_, inter_, hidden_, inter_);
        coef_ = load_f32(b, p + names_.at("act"), 4);
    }
    size_t weight_bytes() const override { return (size_t)2 * inter_ * hidden_ * dtype_size(dtype_) + 16; }
    bool folds_rms() const override { return Ops::gemm_scale_ok(dtype_, w_up_, hidden_, w_up_, hidden_); }
    void forward(StepContext& ctx, const void* h, float* residual) override {
        const int T = ctx.tokens();
        NormFold in, out;
        void* z = ctx.workspace->buffer("ffn_up", (size_t)T * inter_ * ctx.element());
        ctx.ops->gemm(z, ctx.dtype, inter_, h, hidden_, w_up_, hidden_, dtype_, T, inter_, hidden_, EPI_STORE,
                      fold_input(ctx, in));
        void* act = ctx.workspace->buffer("ffn_act", (size_t)T * inter_ * ctx.element());
        ctx.ops->polynorm(act, inter_, z, inter_, ctx.dtype, coef_, T, inter_, eps_);
        const NormFold* emit = fold_emit(ctx, out, hidden_);
        ctx.ops->gemm(residual, F32, hidden_, act, inter_, w_down_, inter_, dtype_, T, hidden_, inter_, EPI_ADD, emit);
        fold_emitted(ctx, emit, hidden_);
    }

private:
    int hidden_ = 0, inter_ = 0, dtype_ = BF16;
    float eps_ = 0.f;
    std::map<std::string, std::string> names_;
    void *w_up_ = nullptr, *w_down_ = nullptr;
    float* coef_ = nullptr;
};

// ---------------------------------------------------------------------------------------------
// Time mixing with a decay that depends on the token (the wkv recurrence).  With h' the input row of
// the token before (zeros before the first token of a sequence), each of r, k, v, g, w reads its own
// mix h + (h' - h) * mu_s.  r, k, v = W_r, W_k, W_v of their mixes [heads, dim]; the gate is
// gate(W_g mix_g); the decay w = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0)) per head and key channel, bias,
// both exponentials and the state in float32.  Per head o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t, then
// S_t = diag(w_t) S_{t-1} + k_t v_t^T.  Each head's o divided by its root mean square (eps inside the
// root), heads concatenated, times the weight `norm`, times the gate, times output_scale, through W_o.
// Per request slot the state is S [heads, dim, dim] followed by h' [hidden], float32.
class WkvMixer : public Mixer {
public:
    WkvMixer(const Json& j, const BuildContext&) {
        hidden_ = (int)j.get("hidden_size").as_int();
        heads_ = (int)j.get("num_heads").as_int();
        dim_ = (int)j.get("head_dim").as_int();
        rank_ = (int)j.get_int("decay_rank", 0);      // 0: the width of the bottleneck is read from its tensor
        eps_ = (float)j.get("eps").as_double();
        out_scale_ = (float)j.get_double("output_scale", 1.0);
        gate_ = gate_code(j.get_string("gate", "silu"));
        names_ = tensor_names(j, {{"r", "r"}, {"k", "k"}, {"v", "v"}, {"g", "g"}, {"w1", "w1"}, {"w2", "w2"},
                                  {"w_bias", "w0"}, {"bonus", "u"}, {"norm", "norm"}, {"o", "o"}, {"mu_r", "mu.r"},
                                  {"mu_k", "mu.k"}, {"mu_v", "mu.v"}, {"mu_g", "mu.g"}, {"mu_w", "mu.w"}});
        if (hidden_ <= 0 || heads_ <= 0 || dim_ <= 0 || rank_ < 0) fail(KIPP_E_CONFIG, "wkv: sizes must be positive");
        hd_ = heads_ * dim_;
        hd_ld_ = (hd_ + 7) / 8 * 8;                    // r, k, v and g each start on a 16-byte boundary of the row
        n_proj_ = gate_ ? 4 : 3;
        set_rank(rank_);
    }
    void set_rank(int rank) {
        rank_ = rank;
        rank_ld_ = (rank_ + 7) / 8 * 8;
    }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        auto add = [&](const char* role, std::vector<int64_t> shape, const char* init = "normal") {
            TensorSpec s;
            s.name = p + names_.at(role);
            s.shape = std::move(shape);
            s.init = init;
            out.push_back(s);
        };
        for (const char* mu : {"mu_r", "mu_k", "mu_v", "mu_g", "mu_w"})
            if (gate_ || std::string(mu) != "mu_g") add(mu, {hidden_});
        add("r", {hd_, hidden_});
        add("k", {hd_, hidden_});
        add("v", {hd_, hidden_});
        if (gate_) add("g", {hd_, hidden_});
        add("w1", {rank_ > 0 ? rank_ : -1, hidden_});
        add("w2", {hd_, rank_ > 0 ? rank_ : -1});
        add("w_bias", {hd_});
        add("bonus", {heads_, dim_});
        add("norm", {hd_}, "near_one");
        add("o", {hidden_, hd_});
    }
    long long state_floats() const { return (long long)heads_ * dim_ * dim_ + hidden_; }
    std::optional<StateSpec> state_spec() const override { return StateSpec{{state_floats()}, F32}; }
    void bind(Binder& b, const std::string& p) override {
        dtype_ = b.compute_dtype();
        const size_t es = dtype_size(dtype_);
        if (rank_ == 0) {
            const std::vector<int64_t> s1 = b.stored_shape(p + names_.at("w1")), s2 = b.stored_shape(p + names_.at("w2"));
            if (s1.size() != 2 || s2.size() != 2 || s1[0] <= 0 || s1[0] != s2[1])
                fail(KIPP_E_WEIGHTS, "wkv: " + p + names_.at("w1") + " and " + p + names_.at("w2") +
                                         " do not agree on the width of the bottleneck");
            set_rank((int)s1[0]);
        }
        // every projection reads a mix of its own, so each is a product of its own
        const char* roles[4] = {"r", "k", "v", "g"};
        for (int i = 0; i < n_proj_; ++i) {
            w_in_[i] = b.allocate((size_t)hd_ * hidden_ * es, p + names_.at(roles[i]));
            b.load(p + names_.at(roles[i]), w_in_[i], dtype_, hidden_, hd_, hidden_);
        }
        w1_ = b.allocate((size_t)rank_ * hidden_ * es, p + names_.at("w1"));
        b.load(p + names_.at("w1"), w1_, dtype_, hidden_, rank_, hidden_);
        // rows of W_w2 and W_o padded to a multiple of 8 elements (zeros beyond)
        w2_ = b.allocate((size_t)hd_ * rank_ld_ * es, p + names_.at("w2"));
        cuda_check(cudaMemset(w2_, 0, (size_t)hd_ * rank_ld_ * es), "clearing a padded weight");
        b.load(p + names_.at("w2"), w2_, dtype_, rank_ld_, hd_, rank_);
        w_o_ = b.allocate((size_t)hidden_ * hd_ld_ * es, p + names_.at("o"));
        cuda_check(cudaMemset(w_o_, 0, (size_t)hidden_ * hd_ld_ * es), "clearing a padded weight");
        b.load(p + names_.at("o"), w_o_, dtype_, hd_ld_, hidden_, hd_);
        // the mixing vectors in the order of the mixes: r, k, v, (g,) w
        n_mix_ = n_proj_ + 1;
        mu_ = static_cast<float*>(b.allocate((size_t)n_mix_ * hidden_ * sizeof(float), p + "mu"));
        const char* mus[5] = {"mu_r", "mu_k", "mu_v", "mu_g", "mu_w"};
        int row = 0;
        for (int i = 0; i < 5; ++i) {
            if (!gate_ && i == 3) continue;
            b.load(p + names_.at(mus[i]), mu_ + (size_t)row * hidden_, F32, hidden_, 1, hidden_);
            ++row;
        }
        w_bias_ = load_f32(b, p + names_.at("w_bias"), hd_);
        bonus_ = load_f32(b, p + names_.at("bonus"), hd_);
        norm_ = load_f32(b, p + names_.at("norm"), hd_);
        if (!Ops::wkv_ok(dim_)) fail(KIPP_E_UNSUPPORTED, format("wkv: the scan kernel does not take heads of %d x %d", dim_, dim_));
    }
    size_t weight_bytes() const override {
        return ((size_t)n_proj_ * hd_ * hidden_ + (size_t)rank_ * hidden_ + (size_t)hd_ * rank_ + (size_t)hidden_ * hd_) *
                   dtype_size(dtype_) + ((size_t)3 * hd_ + (size_t)n_mix_ * hidden_) * 4;
    }
    void forward(StepContext& ctx, const LayerRun& run, int mixer_slot, const void* h, float* residual) override {
        const int T = ctx.tokens();
        const size_t es = ctx.element();
        Ops& ops = *ctx.ops;
        const StepMeta& m = *ctx.meta;
        float* state = static_cast<float*>(ctx.state_view(run, mixer_slot, nullptr));
        const long long stride = state_floats();
        float* prev = state + (size_t)heads_ * dim_ * dim_;          // h' of slot 0; the slots are `stride` apart
        // the mixes, one [T, hidden] after another, then the row the next step's first token will want
        char* mixes = static_cast<char*>(ctx.workspace->buffer("wkv_mixes", (size_t)n_mix_ * T * hidden_ * es));
        const size_t mix_bytes = (size_t)T * hidden_ * es;
        ops.token_shift_mix(mixes, (long long)T * hidden_, h, mu_, prev, stride, m.q_start, m.entry_of_token, m.slots,
                            ctx.dtype, T, hidden_, n_mix_);
        ops.token_shift_keep(prev, stride, h, m.q_start, m.slots, ctx.dtype, m.shape.entries, hidden_);
        const int ld = n_proj_ * hd_ld_;
        char* proj = static_cast<char*>(ctx.workspace->buffer("wkv_proj", (size_t)T * ld * es));
        for (int i = 0; i < n_proj_; ++i)
            ops.gemm(proj + (size_t)i * hd_ld_ * es, ctx.dtype, ld, mixes + (size_t)i * mix_bytes, hidden_, w_in_[i], hidden_,
                     dtype_, T, hd_, hidden_, EPI_STORE);
        // the decay: the bottleneck with its tanh, then its second product; bias and both exponentials
        // are the scan kernel's, in float32
        void* low = ctx.workspace->buffer("wkv_low_rank", (size_t)T * rank_ld_ * es);
        if (rank_ld_ != rank_) cuda_check(cudaMemsetAsync(low, 0, (size_t)T * rank_ld_ * es, ctx.stream), "clearing the bottleneck");
        void* low_raw = ctx.workspace->buffer("wkv_low_rank_raw", (size_t)T * rank_ld_ * es);
        ops.gemm(low_raw, ctx.dtype, rank_ld_, mixes + (size_t)n_proj_ * mix_bytes, hidden_, w1_, hidden_, dtype_, T, rank_,
                 hidden_, EPI_STORE);
        ops.tanh_rows(low, rank_ld_, low_raw, rank_ld_, ctx.dtype, T, rank_);
        void* w_raw = ctx.workspace->buffer("wkv_decay", (size_t)T * hd_ld_ * es);
        ops.gemm(w_raw, ctx.dtype, hd_ld_, low, rank_ld_, w2_, rank_ld_, dtype_, T, hd_, rank_ld_, EPI_STORE);
        void* gated = ctx.workspace->buffer("wkv_out", (size_t)T * hd_ld_ * es);
        if (hd_ld_ != hd_) cuda_check(cudaMemsetAsync(gated, 0, (size_t)T * hd_ld_ * es, ctx.stream), "clearing the padding");
        ops.wkv_scan(gated, hd_ld_, proj, ld, ctx.dtype, 0, hd_ld_, 2 * hd_ld_, 3 * hd_ld_, w_raw, hd_ld_, w_bias_, bonus_,
                     norm_, state, stride, m.q_start, m.slots, m.shape.entries, T, heads_, dim_, eps_, out_scale_, gate_);
        ops.gemm(residual, F32, hidden_, gated, hd_ld_, w_o_, hd_ld_, dtype_, T, hidden_, hd_ld_, EPI_ADD);
    }

private:
    int hidden_ = 0, heads_ = 0, dim_ = 0, rank_ = 0, rank_ld_ = 0, hd_ = 0, hd_ld_ = 0, n_proj_ = 4, n_mix_ = 5, gate_ = 1,
        dtype_ = BF16;
    float eps_ = 0.f, out_scale_ = 1.f;
    std::map<std::string, std::string> names_;
    void* w_in_[4] = {nullptr, nullptr, nullptr, nullptr};
    void *w1_ = nullptr, *w2_ = nullptr, *w_o_ = nullptr;
    float *mu_ = nullptr, *w_bias_ = nullptr, *bonus_ = nullptr, *norm_ = nullptr;
};

// The selective state space layer in its matrix-state form (recurrent.cu, kind 4).  One product makes
// [z: inner | x: inner | B: groups * state | C: groups * state | dt: heads] with inner = heads * v_dim;
// x, B and C pass a causal convolution per channel (taps from the tensor's shape or `conv`) with bias
// and silu; dt = softplus(dt + dt_bias); per head (head h uses group h / (heads / groups)):
// S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T (S is state x v_dim), y_t = S_t^T C_t + D_h x_t;
// y silu(z), divided by the root mean square in norm_groups equal parts of the row, times a weight; then
// the output projection.  Per request slot: S in float32 and the last taps - 1 inputs of every convolved
// channel.  Everything behind the projection is float32.
class StateSpaceMixer : public Mixer {
public:
    StateSpaceMixer(const Json& j, const BuildContext&) {
        hidden_ = (int)j.get("hidden_size").as_int();
        heads_ = (int)j.get("num_heads").as_int();
        v_dim_ = (int)j.get("value_dim").as_int();
        state_ = (int)j.get("state_dim").as_int();
        groups_ = (int)j.get_int("groups", 1);
        taps_ = (int)j.get("conv").as_int();
        norm_groups_ = (int)j.get_int("norm_groups", 1);
        eps_ = (float)j.get("eps").as_double();
        names_ = tensor_names(j, {{"in", "in"}, {"conv", "conv"}, {"conv_bias", "conv.b"}, {"dt_bias", "dt_bias"},
                                  {"a_log", "A_log"}, {"d", "D"}, {"norm", "norm"}, {"o", "o"}});
        if (hidden_ <= 0 || heads_ <= 0 || v_dim_ <= 0 || state_ <= 0 || groups_ <= 0 || taps_ <= 0 || norm_groups_ <= 0)
            fail(KIPP_E_CONFIG, "state_space: sizes must be positive");
        if (heads_ % groups_) fail(KIPP_E_CONFIG, "state_space: num_heads must be a multiple of groups");
        inner_ = heads_ * v_dim_;
        if (inner_ % norm_groups_) fail(KIPP_E_CONFIG, "state_space: norm_groups must divide num_heads * value_dim");
        channels_ = inner_ + 2 * groups_ * state_;
        proj_cols_ = inner_ + channels_ + heads_;
        proj_ld_ = (proj_cols_ + 7) / 8 * 8;
        inner_ld_ = (inner_ + 7) / 8 * 8;
    }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        auto add = [&](const char* role, std::vector<int64_t> shape, const char* init = "normal") {
            TensorSpec s;
            s.name = p + names_.at(role);
            s.shape = std::move(shape);
            s.init = init;
            out.push_back(s);
        };
        add("in", {proj_cols_, hidden_});
        add("conv", {channels_, taps_});
        add("conv_bias", {channels_});
        add("dt_bias", {heads_});
        add("a_log", {heads_});
        add("d", {heads_});
        add("norm", {inner_}, "near_one");
        add("o", {hidden_, inner_});
    }
    long long state_floats() const { return (long long)heads_ * state_ * v_dim_ + (long long)(taps_ - 1) * channels_; }
    std::optional<StateSpec> state_spec() const override { return StateSpec{{state_floats()}, F32}; }
    void bind(Binder& b, const std::string& p) override {
        dtype_ = b.compute_dtype();
        const size_t es = dtype_size(dtype_);
        w_in_ = b.allocate((size_t)proj_cols_ * hidden_ * es, p + names_.at("in"));
        b.load(p + names_.at("in"), w_in_, dtype_, hidden_, proj_cols_, hidden_);
        w_o_ = b.allocate((size_t)hidden_ * inner_ld_ * es, p + names_.at("o"));
        cuda_check(cudaMemset(w_o_, 0, (size_t)hidden_ * inner_ld_ * es), "clearing a padded weight");
        b.load(p + names_.at("o"), w_o_, dtype_, inner_ld_, hidden_, inner_);
        conv_ = load_f32(b, p + names_.at("conv"), (int64_t)channels_ * taps_);
        conv_b_ = load_f32(b, p + names_.at("conv_bias"), channels_);
        dt_bias_ = load_f32(b, p + names_.at("dt_bias"), heads_);
        a_log_ = load_f32(b, p + names_.at("a_log"), heads_);
        d_ = load_f32(b, p + names_.at("d"), heads_);
        norm_ = load_f32(b, p + names_.at("norm"), inner_);
        if (!Ops::ssd_ok(state_, v_dim_))
            fail(KIPP_E_UNSUPPORTED, format("state_space: the scan kernel does not take a state of %d x %d", state_, v_dim_));
        if (taps_ > Ops::ssd_max_taps())
            fail(KIPP_E_UNSUPPORTED, format("state_space: at most %d taps", Ops::ssd_max_taps()));
        if (Ops::ssd_state_floats(heads_, groups_, state_, v_dim_, taps_) != state_floats())
            fail(KIPP_E_STATE, "state_space: the kernel library lays the slot out otherwise");
    }
    size_t weight_bytes() const override {
        return ((size_t)proj_cols_ * hidden_ + (size_t)hidden_ * inner_) * dtype_size(dtype_) +
               ((size_t)channels_ * (taps_ + 1) + 3 * (size_t)heads_ + inner_) * 4;
    }
    bool folds_rms() const override { return Ops::gemm_scale_ok(dtype_, w_in_, hidden_, w_in_, hidden_); }
    void forward(StepContext& ctx, const LayerRun& run, int mixer_slot, const void* h, float* residual) override {
        const int T = ctx.tokens();
        const size_t es = ctx.element();
        Ops& ops = *ctx.ops;
        const StepMeta& m = *ctx.meta;
        NormFold fold_in, fold_out;
        float* state = static_cast<float*>(ctx.state_view(run, mixer_slot, nullptr));
        void* proj = ctx.workspace->buffer("state_space_proj", (size_t)T * proj_ld_ * es);
        ops.gemm(proj, ctx.dtype, proj_ld_, h, hidden_, w_in_, hidden_, dtype_, T, proj_cols_, hidden_, EPI_STORE,
                 fold_input(ctx, fold_in));
        void* gated = ctx.workspace->buffer("state_space_out", (size_t)T * inner_ld_ * es);
        if (inner_ld_ != inner_) cuda_check(cudaMemsetAsync(gated, 0, (size_t)T * inner_ld_ * es, ctx.stream), "clearing the padding");
        ops.ssd_scan(gated, inner_ld_, proj, proj_ld_, ctx.dtype, 0, inner_, inner_ + channels_, conv_, conv_b_, taps_, dt_bias_,
                     a_log_, d_, norm_, norm_groups_, state, state_floats(), m.q_start, m.entry_of_token, m.slots,
                     m.shape.entries, T, heads_, groups_, state_, v_dim_, eps_);
        const NormFold* emit = fold_emit(ctx, fold_out, hidden_);
        ops.gemm(residual, F32, hidden_, gated, inner_ld_, w_o_, inner_ld_, dtype_, T, hidden_, inner_ld_, EPI_ADD, emit);
        fold_emitted(ctx, emit, hidden_);
    }

private:
    int hidden_ = 0, heads_ = 0, v_dim_ = 0, state_ = 0, groups_ = 1, taps_ = 1, norm_groups_ = 1, inner_ = 0, channels_ = 0,
        proj_cols_ = 0, proj_ld_ = 0, inner_ld_ = 0, dtype_ = BF16;
    float eps_ = 0.f;
    std::map<std::string, std::string> names_;
    void *w_in_ = nullptr, *w_o_ = nullptr;
    float *conv_ = nullptr, *conv_b_ = nullptr, *dt_bias_ = nullptr, *a_log_ = nullptr, *d_ = nullptr, *norm_ = nullptr;
};

inline void register_recurrent_parts(Registry& r) {
    r.add_part_kind("state_space", [](const Json& j, const BuildContext& ctx) -> std::unique_ptr<Part> {
        return std::make_unique<StateSpaceMixer>(j, ctx);
    });
    r.add_part_kind("wkv", [](const Json& j, const BuildContext& ctx) -> std::unique_ptr<Part> {
        return std::make_unique<WkvMixer>(j, ctx);
    });
    r.add_part_kind("retention", [](const Json& j, const BuildContext& ctx) -> std::unique_ptr<Part> {
        return std::make_unique<RetentionMixer>(j, ctx);
    });
    r.add_part_kind("delta_rule", [](const Json& j, const BuildContext& ctx) -> std::unique_ptr<Part> {
        return std::make_unique<DeltaRuleMixer>(j, ctx);
    });
    r.add_part_kind("gated_memory", [](const Json& j, const BuildContext& ctx) -> std::unique_ptr<Part> {
        return std::make_unique<GatedMemoryMixer>(j, ctx);
    });
    r.add_part_kind("parallel", [](const Json& j, const BuildContext& ctx) -> std::unique_ptr<Part> {
        return std::make_unique<ParallelMixer>(j, ctx);
    });
    r.add_part_kind("polynorm_mlp", [](const Json& j, const BuildContext&) -> std::unique_ptr<Part> {
        return std::make_unique<PolyNormFeedForward>(j);
    });
}

}  // namespace kipp
