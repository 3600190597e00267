// The parts the library brings: token embedding, RMSNorm and layer norm, rotary position
// encodings (plain, or with long wavelengths stretched), causal grouped-query attention over the
// paged cache, the SwiGLU and the plain dense feed-forward, the output head, the pre-norm block and
// the block whose sublayers share one norm, and the wrapper behind parts whose forward pass the
// caller supplies.  Each
// is registered under a kind name; a plan builds them from JSON objects of sizes and constants.
#pragma once
#include "model.hpp"

namespace kipp {

// ---------------------------------------------------------------------------------------------
// x_t = float(E[id_t, :]) with no scale (src/kipp.c:2940-2942).
class TokenEmbedding : public EmbeddingStage {
public:
    TokenEmbedding(int vocab, int hidden, std::string weight_name = "weight")
        : vocab_(vocab), hidden_(hidden), name_(std::move(weight_name)) {
        if (vocab <= 0 || hidden <= 0) fail(KIPP_E_CONFIG, "token_embedding: sizes must be positive");
    }
    void tensor_specs(const std::string& prefix, std::vector<TensorSpec>& out) const override {
        TensorSpec s;
        s.name = prefix + name_;
        s.shape = {vocab_, hidden_};
        out.push_back(s);
    }
    void bind(Binder& b, const std::string& prefix) override {
        dtype_ = b.compute_dtype();
        weight_ = b.shared(prefix + name_, dtype_, vocab_, hidden_);
    }
    void forward(StepContext& ctx, float* x) override {
        ctx.ops->embed_gather(x, weight_, dtype_, ctx.meta->token_ids, ctx.tokens(), hidden_, vocab_);
    }

private:
    int vocab_, hidden_, dtype_ = BF16;
    std::string name_;
    void* weight_ = nullptr;
};

// A second table addressed by a hash of the token pair, added to the stream: x_t += B[row_t, :] with
// row_t = (id_{t-1} * mul_prev + id_t * mul_cur) mod buckets and, for the first token of a sequence,
// the table's extra last row (B has buckets + 1 rows).  The token before a step's first token is
// per-request state of the stage (one int32 per slot), written after every step.
class HashedPairEmbedding : public EmbeddingStage {
public:
    HashedPairEmbedding(int vocab, int hidden, long long buckets, long long mul_prev, long long mul_cur,
                        std::string weight_name)
        : vocab_(vocab), hidden_(hidden), buckets_(buckets), mul_prev_(mul_prev), mul_cur_(mul_cur),
          name_(std::move(weight_name)) {
        if (vocab <= 0 || hidden <= 0 || buckets <= 0) fail(KIPP_E_CONFIG, "hashed_pair_embedding: sizes must be positive");
        if (mul_prev < 0 || mul_cur < 0) fail(KIPP_E_CONFIG, "hashed_pair_embedding: the multipliers must not be negative");
        // (previous * mul_prev + current * mul_cur) is formed in 64 bits
        if ((double)vocab * ((double)mul_prev + (double)mul_cur) > 9.0e18)
            fail(KIPP_E_CONFIG, "hashed_pair_embedding: the multipliers are too large for this vocabulary");
    }
    void tensor_specs(const std::string& prefix, std::vector<TensorSpec>& out) const override {
        TensorSpec s;
        s.name = prefix + name_;
        s.shape = {buckets_ + 1, hidden_};
        out.push_back(s);
    }
    std::optional<StateSpec> state_spec() const override { return StateSpec{{1}, I32}; }
    void bind(Binder& b, const std::string& prefix) override {
        dtype_ = b.compute_dtype();
        weight_ = b.shared(prefix + name_, dtype_, buckets_ + 1, hidden_);
    }
    void forward(StepContext& ctx, float* x) override {
        const StepMeta& m = *ctx.meta;
        int* last = static_cast<int*>(ctx.stage_state(this, nullptr));
        ctx.ops->hashed_pair_add(x, weight_, dtype_, m.token_ids, m.positions, m.entry_of_token, m.q_start, m.slots, last,
                                 1, ctx.tokens(), hidden_, vocab_, buckets_, mul_prev_, mul_cur_);
        ctx.ops->keep_last_token(last, 1, m.token_ids, m.q_start, m.slots, m.shape.entries);
    }

private:
    int vocab_, hidden_;
    long long buckets_, mul_prev_, mul_cur_;
    int dtype_ = BF16;
    std::string name_;
    void* weight_ = nullptr;
};

// logits = W n for the wanted rows only; W is the tensor `tied_to` when the checkpoint has no
// head of its own (src/kipp.c:951-956, 3013-3018).
class OutputHead : public Head {
public:
    OutputHead(int vocab, int hidden, std::string tied_to, std::string weight_name = "weight", double logit_scale = 1.0,
               double logit_softcap = 0.0)
        : vocab_(vocab), hidden_(hidden), tied_to_(std::move(tied_to)), name_(std::move(weight_name)),
          scale_((float)logit_scale), softcap_((float)logit_softcap) {
        if (vocab <= 0 || hidden <= 0) fail(KIPP_E_CONFIG, "output_head: sizes must be positive");
        if (logit_softcap < 0) fail(KIPP_E_CONFIG, "output_head: logit_softcap must not be negative");
    }
    void tensor_specs(const std::string& prefix, std::vector<TensorSpec>& out) const override {
        TensorSpec s;
        s.name = prefix + name_;
        s.shape = {vocab_, hidden_};
        if (!tied_to_.empty()) {
            s.optional = true;
            s.alias_of = tied_to_;
            s.ignore_if_present = true;
        }
        out.push_back(s);
    }
    void bind(Binder& b, const std::string& prefix) override {
        dtype_ = b.compute_dtype();
        weight_ = b.shared(tied_to_.empty() ? prefix + name_ : tied_to_, dtype_, vocab_, hidden_);
    }
    size_t weight_bytes() const override { return (size_t)vocab_ * hidden_ * dtype_size(dtype_); }
    int vocab_size() const override { return vocab_; }
    void forward(StepContext& ctx, const void* h, int n_rows, float* logits) override {
        ctx.ops->gemm(logits, F32, vocab_, h, hidden_, weight_, hidden_, dtype_, n_rows, vocab_, hidden_, EPI_STORE);
        if (scale_ != 1.0f) ctx.ops->scale_f32(logits, (long long)n_rows * vocab_, scale_);     // logit_scale, in float32
        // logit_softcap c > 0: logits <- c tanh(logits / c), in float32
        if (softcap_ > 0.f) ctx.ops->softcap_f32(logits, (long long)n_rows * vocab_, softcap_);
    }

private:
    int vocab_, hidden_, dtype_ = BF16;
    std::string tied_to_, name_;
    float scale_ = 1.f, softcap_ = 0.f;
    void* weight_ = nullptr;
};

// y = x * rsqrt(mean(x^2) + eps) * w, computed in float32 (src/kipp.c:2221-2231).
class RMSNorm : public Norm {
public:
    RMSNorm(int size, double eps, std::string weight_name) : size_(size), eps_((float)eps), name_(std::move(weight_name)) {
        if (size <= 0 || !(eps > 0)) fail(KIPP_E_CONFIG, "rmsnorm: size and eps must be positive");
    }
    void tensor_specs(const std::string& prefix, std::vector<TensorSpec>& out) const override {
        TensorSpec s;
        s.name = prefix + name_;
        s.shape = {size_};
        s.init = "near_one";
        out.push_back(s);
    }
    void bind(Binder& b, const std::string& prefix) override {
        // the scale keeps its storage type (bfloat16 or float32)
        wdtype_ = storage_dtype(b.stored_dtype(prefix + name_));
        weight_ = b.allocate((size_t)size_ * dtype_size(wdtype_), prefix + name_);
        b.load(prefix + name_, weight_, wdtype_, size_, 1, size_);
    }
    size_t weight_bytes() const override { return (size_t)size_ * dtype_size(wdtype_); }
    int size() const override { return size_; }
    std::optional<RmsNormSpec> rms_spec() const override { return RmsNormSpec{weight_, wdtype_, eps_, size_}; }
    void forward(StepContext& ctx, const float* x, void* out, const int* rows, int n_rows) override {
        ctx.ops->rmsnorm(out, ctx.dtype, x, weight_, wdtype_, rows, n_rows, size_, eps_);
    }

private:
    int size_;
    float eps_;
    std::string name_;
    int wdtype_ = F32;
    void* weight_ = nullptr;
};

// y = (x - mean) / sqrt(var + eps) * w + b with var the mean of the squared deviations, computed in
// float32; weight and bias are kept in float32.  `bias_name` empty: no bias.
class LayerNorm : public Norm {
public:
    LayerNorm(int size, double eps, std::string weight_name, std::string bias_name)
        : size_(size), eps_((float)eps), name_(std::move(weight_name)), bias_name_(std::move(bias_name)) {
        if (size <= 0 || !(eps > 0)) fail(KIPP_E_CONFIG, "layernorm: size and eps must be positive");
    }
    void tensor_specs(const std::string& prefix, std::vector<TensorSpec>& out) const override {
        TensorSpec s;
        s.name = prefix + name_;
        s.shape = {size_};
        s.init = "near_one";
        out.push_back(s);
        if (!bias_name_.empty()) {
            TensorSpec b;
            b.name = prefix + bias_name_;
            b.shape = {size_};
            out.push_back(b);
        }
    }
    void bind(Binder& b, const std::string& prefix) override {
        weight_ = static_cast<float*>(b.allocate((size_t)size_ * sizeof(float), prefix + name_));
        b.load(prefix + name_, weight_, F32, size_, 1, size_);
        if (!bias_name_.empty()) {
            bias_ = static_cast<float*>(b.allocate((size_t)size_ * sizeof(float), prefix + bias_name_));
            b.load(prefix + bias_name_, bias_, F32, size_, 1, size_);
        }
    }
    size_t weight_bytes() const override { return (size_t)size_ * sizeof(float) * (bias_name_.empty() ? 1 : 2); }
    int size() const override { return size_; }
    void forward(StepContext& ctx, const float* x, void* out, const int* rows, int n_rows) override {
        ctx.ops->layernorm(out, ctx.dtype, x, weight_, bias_, rows, n_rows, size_, eps_);
    }

private:
    int size_;
    float eps_;
    std::string name_, bias_name_;
    float *weight_ = nullptr, *bias_ = nullptr;
};

// ---------------------------------------------------------------------------------------------
// Rotations given by a table of frequencies: pair (i, i + rotary_dim/2) of a head turns by
// position * inv_freq[i].
class FrequencyTable : public PositionEncoding {
public:
    FrequencyTable(std::vector<float> inv_freq, std::string key, float magnitude = 1.f)
        : freq_(std::move(inv_freq)), key_(std::move(key)), magnitude_(magnitude) {}
    int rotary_dim() const override { return 2 * (int)freq_.size(); }
    float magnitude() const override { return magnitude_; }
    const float* inv_freq_device() const override { return device_; }
    std::string table_key() const override { return key_; }
    void bind(Binder& b, const std::string&) override {
        if (freq_.empty() || device_) return;
        device_ = static_cast<float*>(b.allocate(freq_.size() * sizeof(float), "rotary frequencies"));
        cuda_check(cudaMemcpy(device_, freq_.data(), freq_.size() * sizeof(float), cudaMemcpyHostToDevice),
                   "upload of rotary frequencies");
    }
    const std::vector<float>& frequencies() const { return freq_; }

private:
    std::vector<float> freq_;
    std::string key_;
    float magnitude_ = 1.f;
    float* device_ = nullptr;
};

// Half-split rotary encoding (src/kipp.c:2368-2382): the frequency of pair i is
// theta^(-2i/rot) as the reference's powf(theta, -(2.0f * i) / rot): a float32 exponent, the
// power rounded to float32 once.
// `exact`: the exponent -2i/rot in double precision instead (the power still rounded to float32
// once), for models whose frequencies are defined as the real number theta^(-2i/rot).
inline std::vector<float> rotary_frequencies(int rotary_dim, double theta, bool exact = false) {
    std::vector<float> f((size_t)rotary_dim / 2);
    const double base = exact ? theta : (double)(float)theta;
    for (int i = 0; i < rotary_dim / 2; ++i) {
        const float exponent = -(2.0f * (float)i) / (float)rotary_dim;
        f[(size_t)i] = (float)std::pow(base, exact ? -2.0 * (double)i / (double)rotary_dim : (double)exponent);
    }
    return f;
}

// Frequencies whose long wavelengths are stretched (the frequency scaling of Llama 3.1): with
// the wavelength l = 2 pi / f, f stays where l < original / high, becomes f / factor where
// l > original / low, and between the two is (1 - s) f / factor + s f with
// s = (original / l - low) / (high - low).  Formed in double precision, rounded to float32 once.
inline std::vector<float> stretched_frequencies(int rotary_dim, double theta, double factor, double low, double high,
                                                double original) {
    std::vector<float> f((size_t)rotary_dim / 2);
    const double two_pi = 6.283185307179586476925286766559;
    for (int i = 0; i < rotary_dim / 2; ++i) {
        double v = std::pow(theta, -2.0 * (double)i / (double)rotary_dim);
        const double wave = two_pi / v;
        if (wave > original / low) {
            v /= factor;
        } else if (!(wave < original / high)) {
            const double s = (original / wave - low) / (high - low);
            v = (1.0 - s) * v / factor + s * v;
        }
        f[(size_t)i] = (float)v;
    }
    return f;
}

// Frequencies scaled by a ramp over the pair index (the YaRN way of stretching a context): with
// pair(t) = dims ln(original / (2 pi t)) / (2 ln theta) the (real) pair index that makes t turns within
// `original` positions, lo = max(floor(pair(fast)), 0), hi = min(ceil(pair(slow)), dims - 1) and
// ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency of pair i is
// f_i / factor * ramp_i + f_i (1 - ramp_i): pairs that turn fast stay, slow ones are divided by the
// factor.  cos and sin are both multiplied by 0.1 ln(factor) + 1 (yarn_magnitude).  Formed in double
// precision, rounded to float32 once.
inline std::vector<float> yarn_frequencies(int rotary_dim, double theta, double factor, double original, double fast,
                                           double slow) {
    std::vector<float> f((size_t)rotary_dim / 2);
    const double two_pi = 6.283185307179586476925286766559;
    auto pair_of = [&](double turns) { return rotary_dim * std::log(original / (two_pi * turns)) / (2.0 * std::log(theta)); };
    const double lo = std::max(std::floor(pair_of(fast)), 0.0);
    const double hi = std::min(std::ceil(pair_of(slow)), (double)rotary_dim - 1.0);
    for (int i = 0; i < rotary_dim / 2; ++i) {
        const double v = std::pow(theta, -2.0 * (double)i / (double)rotary_dim);
        const double ramp = std::min(std::max(((double)i - lo) / std::max(hi - lo, 0.001), 0.0), 1.0);
        f[(size_t)i] = (float)(v / factor * ramp + v * (1.0 - ramp));
    }
    return f;
}
inline float yarn_magnitude(double factor) { return (float)(0.1 * std::log(factor) + 1.0); }

// ---------------------------------------------------------------------------------------------
// The work lists of the paged attention kernels and the rule for the decode splits.  The
// constants are those kernels': 64-token query tiles (mma.sync prompt kernel), 128-token tiles
// (tcgen05 prompt kernel), three decode CTAs resident per SM.
class AttentionPlanner : public WorkPlanner {
public:
    static constexpr int TILE = 64;
    static constexpr int CTA_FIXED_TILES = 5;   // what a decode CTA costs beside its key tiles, in 64-key tiles
    static constexpr int CTAS_PER_SM = 3;
    static constexpr double STREAM_MARGIN = 1.15;   // the stream cut must look this much better to be taken

    AttentionPlanner(int kv_heads, int sm_count, bool own_length)
        : kv_heads_(kv_heads), resident_(CTAS_PER_SM * std::max(sm_count, 1)), own_length_(own_length) {}

    static std::string key_for(int kv_heads, int sm_count, bool own_length) {
        return format("paged_attention/kv%d/sm%d/%s", kv_heads, sm_count, own_length ? "own" : "step");
    }
    std::string key() const override { return key_for(kv_heads_, resident_ / CTAS_PER_SM, own_length_); }
    int sections() const override { return 5; }

    void sizes(const StepShape& s, int* n) const override {
        int decode = 0, items = 0, all = 0, items128 = 0;
        for (int q : s.q_lens) {
            all += (q + TILE - 1) / TILE;
            if (q == 1) { ++decode; continue; }
            items += (q + TILE - 1) / TILE;
            items128 += (q + 2 * TILE - 1) / (2 * TILE);
        }
        n[0] = decode; n[1] = decode; n[2] = 2 * items; n[3] = 2 * all; n[4] = 2 * items128;
    }

    // Keys per split for the decoded tokens of a step, in whole 64-key tiles.  A CTA takes one
    // split of one (token, kv head) pair and costs its k tiles plus a fixed part (its set-up, the
    // merge of its four warps, its partial results); the CTAs run in waves of as many as the GPU
    // holds at once.  Among the numbers of tiles per split k (splits = total tiles / k, rounded
    // up, at most DECODE_MAX_SPLITS) the one with the least waves x (k + fixed part) is taken: many
    // short splits when there are few pairs (a single token's attention is bound by latency, so
    // down to one tile per split), few long ones once the pairs alone fill the GPU.  On a tie the
    // fewer splits.  The device makes the same choice between the steps of a burst
    // (kipp_attn_decode_replan): integers only, so both agree.
    int step_split_length(int decoded, int longest) const {
        if (decoded <= 0 || longest <= 0) return TILE;
        const long long pairs = (long long)decoded * kv_heads_;
        const int total = (longest + TILE - 1) / TILE;
        int best = total;
        long long best_cost = -1;
        for (int k = total; k >= 1; --k) {
            const int splits = (total + k - 1) / k;
            if (splits > Ops::DECODE_MAX_SPLITS) break;
            const long long waves = (pairs * splits + resident_ - 1) / resident_;
            const long long cost = waves * (k + CTA_FIXED_TILES);
            if (best_cost < 0 || cost < best_cost) { best = k; best_cost = cost; }
        }
        return best * TILE;
    }
    // From the token's own context only (an eighth of it): the grouping of its partial sums then
    // does not depend on what else is in the batch (the reference's lesson,
    // metal/kipp_kernels.metal:82-100).
    static int own_split_length(int kv_len) {
        const int own = (kv_len + 7) / 8;
        return std::max(TILE, (own + TILE - 1) / TILE * TILE);
    }

    void fill(const StepShape& s, int* const* sec) const override {
        int d = 0, a = 0, b = 0, c = 0, longest = 0;
        for (int i = 0; i < s.entries; ++i)
            if (s.q_lens[(size_t)i] == 1) longest = std::max(longest, s.starts[(size_t)i] + 1);
        int decoded = 0;
        for (int q : s.q_lens) decoded += q == 1;
        const int step_keys = step_split_length(decoded, longest);
        for (int i = 0; i < s.entries; ++i) {
            const int q = s.q_lens[(size_t)i];
            for (int t = 0; t < q; t += TILE) { sec[3][b++] = i; sec[3][b++] = t; }
            if (q == 1) {
                sec[0][d] = i;
                sec[1][d] = own_length_ ? own_split_length(s.starts[(size_t)i] + 1) : step_keys;
                ++d;
                continue;
            }
            for (int t = 0; t < q; t += TILE) { sec[2][a++] = i; sec[2][a++] = t; }
            for (int t = 0; t < q; t += 2 * TILE) { sec[4][c++] = i; sec[4][c++] = t; }
        }
    }

    void advance_on_device(Ops& ops, const StepShape& s, int* const* sec, const int* context_len,
                           int entries) const override {
        // (the stream cut reads the lengths itself: no keys per split to bring up to date)
        if (stream_pays(s)) return;
        ops.decode_replan(sec[1], context_len, sec[0], entries, kv_heads_, resident_, CTA_FIXED_TILES,
                          Ops::DECODE_MAX_SPLITS, own_length_ ? 1 : 0);
    }

    // Whether the decoded tokens of a step are better cut as a stream over one wave of CTAs (see
    // attn_decode_stream_kernel) than into splits of the step's length: where the splits need
    // more than one wave or leave much of one empty (64 tokens of 2,048 keys: 5.93 against 6.26
    // ms a step; 8 tokens: 2.67 against 2.49, a run then spans two pairs and pays their set-up
    // twice, hence the margin).  Never where every token's splits are to come from its own length.
    bool stream_pays(const StepShape& s) const {
        if (own_length_) return false;
        long long tiles = 0;
        int longest = 0, decoded = 0;
        for (int i = 0; i < s.entries; ++i) {
            if (s.q_lens[(size_t)i] != 1) continue;
            const int keys = s.starts[(size_t)i] + 1;
            tiles += (keys + TILE - 1) / TILE;
            longest = std::max(longest, keys);
            ++decoded;
        }
        if (decoded == 0 || !Ops::decode_stream_ok(decoded)) return false;
        const long long pairs = (long long)decoded * kv_heads_;
        const int most = (longest + TILE - 1) / TILE;
        const int k = step_split_length(decoded, longest) / TILE;
        const long long splits = (most + k - 1) / k;
        const double split_cost = (double)((pairs * splits + resident_ - 1) / resident_) * (k + CTA_FIXED_TILES);
        const long long total = tiles * kv_heads_;
        const long long per = std::max<long long>({(total + resident_ - 1) / resident_,
                                                   (most + Ops::DECODE_MAX_SPLITS - 2) / (Ops::DECODE_MAX_SPLITS - 1), 1});
        const double pieces = 1.0 + (double)per * (double)pairs / (double)total;      // pairs a run touches
        const double stream_cost = (double)per + CTA_FIXED_TILES * pieces;
        return stream_cost * STREAM_MARGIN < split_cost;
    }

    AttentionWork work_of(const StepMeta& meta) const {
        const std::string key = this->key();
        const int stream_ctas = stream_pays(meta.shape) ? resident_ : 0;
        AttentionWork w;
        auto it = meta.work.find(key);
        if (it == meta.work.end()) fail(KIPP_E_STATE, "the step carries no work lists for " + key);
        const std::vector<int*>& sec = it->second;
        const std::vector<int>& n = meta.work_sizes.at(key);
        w.decode_rows = sec[0]; w.n_decode = n[0];
        w.split_keys = sec[1];
        w.stream_ctas = stream_ctas;
        w.prefill_work = sec[2]; w.n_prefill_items = n[2] / 2;
        w.all_work = sec[3]; w.n_all_items = n[3] / 2;
        w.prefill_work128 = sec[4]; w.n_prefill_items128 = n[4] / 2;
        for (int q : meta.shape.q_lens)
            if (q > 1) w.longest_portion = std::max(w.longest_portion, q);
        w.entries = meta.shape.entries;
        w.tokens = meta.shape.tokens;
        return w;
    }

private:
    int kv_heads_, resident_;
    bool own_length_;
};

// The work list of the mixed-head attention's tensor-core prompt kernel: (entry, first token)
// per tile of `tile` tokens over every entry of the step.
class MixTilePlanner : public WorkPlanner {
public:
    explicit MixTilePlanner(int tile) : tile_(std::max(tile, 1)) {}
    static std::string key_for(int tile) { return format("attention_mix/tiles%d", tile); }
    std::string key() const override { return key_for(tile_); }
    int sections() const override { return 1; }
    void sizes(const StepShape& s, int* n) const override {
        int items = 0;
        for (int q : s.q_lens) items += (q + tile_ - 1) / tile_;
        n[0] = 2 * items;
    }
    void fill(const StepShape& s, int* const* sec) const override {
        int a = 0;
        for (int i = 0; i < s.entries; ++i)
            for (int t = 0; t < s.q_lens[(size_t)i]; t += tile_) { sec[0][a++] = i; sec[0][a++] = t; }
    }

private:
    int tile_;
};

// ---------------------------------------------------------------------------------------------
// Norms in deferred form (see NormFold, StepContext::input_scale): what a part's first product and
// its residual add pass to the kernels, and what a block runs where no residual add left the form.
inline const NormFold* fold_input(const StepContext& ctx, NormFold& f) {
    if (!ctx.input_scale.valid()) return nullptr;
    f = NormFold{};
    f.ssq_in = ctx.input_scale.ssq;
    f.ssq_in_slots = ctx.input_scale.slots;
    f.inv_n = ctx.input_scale.inv_n;
    f.eps = ctx.input_scale.eps;
    return &f;
}
inline float* fold_sums(StepContext& ctx, int hidden) {
    return ctx.workspace->get<float>("norm_ssq", (size_t)ctx.tokens() * (size_t)std::max(1, hidden / 32));
}
inline const NormFold* fold_emit(StepContext& ctx, NormFold& f, int hidden) {
    const int T = ctx.tokens();
    if (ctx.emit_for == nullptr || ctx.emit_for->size != hidden || hidden % 32 || !Ops::gemm_emit_ok(T)) return nullptr;
    f = NormFold{};
    f.norm_w = ctx.emit_for->weight;
    f.norm_w_dtype = ctx.emit_for->weight_dtype;
    f.xn = ctx.workspace->buffer("normed", (size_t)T * hidden * ctx.element());
    f.ldn = hidden;
    f.ssq_out = fold_sums(ctx, hidden);
    return &f;
}
inline RowScale deferred_norm(StepContext& ctx, const RmsNormSpec& norm, const float* x, void* h) {
    float* ssq = fold_sums(ctx, norm.size);
    ctx.ops->rmsnorm_deferred(h, ctx.dtype, ssq, x, norm.weight, norm.weight_dtype, nullptr, ctx.tokens(), norm.size);
    return RowScale{ssq, 1, 1.0f / (float)norm.size, norm.eps};
}
inline void fold_emitted(StepContext& ctx, const NormFold* f, int hidden) {
    if (f == nullptr) return;
    ctx.emitted = true;
    ctx.emitted_scale = RowScale{f->ssq_out, hidden / 32, 1.0f / (float)hidden, ctx.emit_for->eps};
}

// The step's (cos, sin) table of a position encoding: made once per forward pass and shared by
// every part that rotates alike (by token, or laid out by pair for the projection that rotates
// its own heads).
inline const float* step_rope_table(StepContext& ctx, const PositionEncoding& position, bool by_pair) {
    const int rot = position.rotary_dim(), T = ctx.tokens();
    if (rot <= 0) return nullptr;
    const std::string key = (by_pair ? "rope by pair/" : "rope/") + position.table_key();
    auto it = ctx.step_cache.find(key);
    if (it == ctx.step_cache.end()) {
        int made = 0;
        for (auto& kv : ctx.step_cache) made += kv.first.rfind("rope", 0) == 0;
        float* table = ctx.workspace->get<float>("rope_table_" + std::to_string(made), (size_t)T * rot);
        if (position.magnitude() != 1.f)
            ctx.ops->rope_table_scaled(table, ctx.meta->positions, position.inv_freq_device(), T, rot / 2, by_pair, position.magnitude());
        else if (by_pair) ctx.ops->rope_table_by_pair(table, ctx.meta->positions, position.inv_freq_device(), T, rot / 2);
        else ctx.ops->rope_table(table, ctx.meta->positions, position.inv_freq_device(), T, rot / 2);
        it = ctx.step_cache.emplace(key, table).first;
    }
    return static_cast<const float*>(it->second);
}

// Names of a part's checkpoint tensors under its prefix: the defaults, or what the plan gives.
inline std::map<std::string, std::string> tensor_names(const Json& j, std::map<std::string, std::string> defaults) {
    if (const Json* n = j.find("names"); n && n->is_object())
        for (auto& kv : n->members()) {
            if (!defaults.count(kv.first)) fail(KIPP_E_CONFIG, "unknown tensor role '" + kv.first + "' in 'names'");
            defaults[kv.first] = kv.second.as_string();
        }
    return defaults;
}

// ---------------------------------------------------------------------------------------------
// Causal grouped-query attention over the paged cache, with optional per-head q/k RMSNorm and a
// position encoding applied to q and k.  Order of operations as the reference's block
// (docs/ARCHITECTURE.md:77-92, src/kipp.c:2950-2993): q/k/v projections (no bias) -> per-head
// norm of q and k -> rotation -> keys and values into the cache -> attention -> output
// projection added to the residual stream.
//
// Options beyond that (each off by default): value heads of a size of their own (value_dim); a
// window that keeps the first keep_first positions of the sequence visible; a matrix that mixes
// the heads' scores before the softmax (head_mix: score_h <- sum_g M[h][g] score_g, a tensor
// [heads, heads]); a factor on the mixer's output (output_scale).  With any of them the step runs
// on the attention_mix kernel, which holds all heads of a query together.
//
// Further options of that path: biases of the q, k and v projections (bias); several score maps
// per head (score_maps: q has heads x maps x head_dim rows, k kv_heads x maps x head_dim, laid out
// head by head as [map 1, map 2, ...]; every map is rotated like a head and is an attention of its
// own over the head's values); and, with two maps, their combination into one head
// (combine_maps: o = a1 - lambda a2 with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + lambda_init,
// four vectors of head_dim, then o / sqrt(mean(o^2) + combine_eps) times (1 - lambda_init)).
//
// And: the q/k norm over the whole projection row instead of head by head (norm_whole: one mean
// square over all heads, weights [heads x head_dim] and [kv_heads x head_dim]); a rotation that
// pairs neighbouring dims (interleaved); blocks of positions as the mask (chunk: a query sees the
// earlier keys of its own block, counted from position 0 of the sequence); a sink in the softmax's
// denominator, learned per head or of score 0 (sink); a sigmoid gate per head from a projection of
// the mixer's input (head_gate); values that are the keys as projected (values_are_keys: no W_v);
// and a mixer without keys and values of its own that reads what another run wrote (shared_kv:
// the run order gives it that run's cache id and writes_cache false).  A cap on the scaled scores
// (softcap c: s <- c tanh(s / c)) goes with every option of this path.
struct AttentionOptions {
    int value_dim = 0, keep_first = 0;
    bool head_mix = false;
    double output_scale = 1.0;
    bool bias = false;
    int score_maps = 1;
    bool combine_maps = false;
    double lambda_init = 0.0, combine_eps = 1e-5;
    bool norm_whole = false;            // q/k norm over the whole projection row, weights of q's and k's full size
    bool interleaved = false;           // the rotation pairs dim 2i with dim 2i + 1
    int chunk = 0;                      // > 0: a query sees the keys j <= p of its own block of `chunk` positions
    int sink = 0;                       // 0 none, 1 a learned number per head (tensor), 2 a sink of score 0
    bool head_gate = false;             // head h times sigmoid(W_g h)_h, W_g [heads, hidden]
    bool values_are_keys = false;       // no W_v: the value of a key is the key as projected (before norm and rotation)
    bool shared_kv = false;             // no keys and values of its own: the run reads the cache another run wrote
    double softcap = 0.0;               // > 0: a scaled score s becomes softcap * tanh(s / softcap) before mask and softmax
    std::map<std::string, std::string> names = {{"q", "q_proj.weight"}, {"k", "k_proj.weight"}, {"v", "v_proj.weight"},
                                                {"o", "o_proj.weight"}, {"q_norm", "q_norm.weight"},
                                                {"k_norm", "k_norm.weight"}, {"head_mix", "head_mix.weight"},
                                                {"q_bias", "q_proj.bias"}, {"k_bias", "k_proj.bias"},
                                                {"v_bias", "v_proj.bias"}, {"lq1", "lambda_q1"}, {"lk1", "lambda_k1"},
                                                {"lq2", "lambda_q2"}, {"lk2", "lambda_k2"}, {"sink", "sink"},
                                                {"gate", "g_proj.weight"}};
};

class AttentionMixer : public Mixer {
public:
    AttentionMixer(int hidden, int heads, int kv_heads, int head_dim, std::unique_ptr<PositionEncoding> position,
                   std::optional<double> qk_norm_eps, int window, std::optional<double> scale,
                   AttentionOptions options = {})
        : hidden_(hidden), heads_(heads), kv_heads_(kv_heads), head_dim_(head_dim), position_(std::move(position)),
          qk_norm_(qk_norm_eps.has_value()), eps_(qk_norm_eps ? (float)*qk_norm_eps : 0.f), window_(window),
          opt_(std::move(options)) {
        if (hidden <= 0 || heads <= 0 || kv_heads <= 0 || head_dim <= 0)
            fail(KIPP_E_CONFIG, "attention: sizes must be positive");
        if (heads % kv_heads) fail(KIPP_E_CONFIG, "attention: num_heads must be a multiple of num_kv_heads");
        if (window < 0) fail(KIPP_E_CONFIG, "attention: a window must not be negative");
        if (opt_.value_dim < 0 || opt_.keep_first < 0) fail(KIPP_E_CONFIG, "attention: value_dim and keep_first must not be negative");
        if (position_->rotary_dim() > head_dim || position_->rotary_dim() % 2)
            fail(KIPP_E_CONFIG, "attention: rotary_dim must be even and at most head_dim");
        scale_ = scale ? (float)*scale : (float)(1.0 / std::sqrt((double)head_dim));
        v_dim_ = opt_.value_dim > 0 ? opt_.value_dim : head_dim;
        maps_ = opt_.score_maps;
        if (maps_ < 1) fail(KIPP_E_CONFIG, "attention: score_maps must be at least 1");
        if (opt_.combine_maps && maps_ != 2) fail(KIPP_E_CONFIG, "attention: combine_maps needs two score maps");
        if (opt_.combine_maps && !(opt_.combine_eps > 0)) fail(KIPP_E_CONFIG, "attention: combine_eps must be positive");
        if (opt_.head_mix && maps_ != 1) fail(KIPP_E_CONFIG, "attention: head_mix and score_maps do not go together");
        const bool more = opt_.norm_whole || opt_.interleaved || opt_.chunk != 0 || opt_.sink != 0 || opt_.head_gate ||
                          opt_.values_are_keys || opt_.shared_kv;
        segments_ = opt_.bias || maps_ > 1 || more;
        if ((opt_.bias || maps_ > 1) && qk_norm_) fail(KIPP_E_CONFIG, "attention: q/k norm with biases or score maps is not supported");
        if (more && (opt_.bias || maps_ > 1 || opt_.head_mix))
            fail(KIPP_E_CONFIG, "attention: norm_whole, interleaved, chunk, sink, head_gate, values_are_keys and shared_kv "
                                "do not go with biases, score maps or head_mix");
        if (opt_.norm_whole && !qk_norm_) fail(KIPP_E_CONFIG, "attention: norm_whole needs qk_norm_eps");
        if (opt_.chunk < 0 || (opt_.chunk > 0 && window_ > 0)) fail(KIPP_E_CONFIG, "attention: chunk must not be negative and excludes a window");
        if (opt_.sink < 0 || opt_.sink > 2) fail(KIPP_E_CONFIG, "attention: sink must be none, learned or unit");
        if (opt_.values_are_keys && v_dim_ != head_dim) fail(KIPP_E_CONFIG, "attention: values that are the keys have the keys' size");
        q_dim_ = heads * maps_ * head_dim;
        kv_dim_ = kv_heads * maps_ * head_dim;
        vv_dim_ = kv_heads * v_dim_;
        o_dim_ = heads * v_dim_;
        // columns of the fused projection: q, then k and v where the mixer has its own, then the gate
        k_cols_ = opt_.shared_kv ? 0 : kv_dim_;
        v_cols_ = opt_.shared_kv || opt_.values_are_keys ? 0 : vv_dim_;
        g_cols_ = opt_.head_gate ? heads : 0;
        proj_cols_ = q_dim_ + k_cols_ + v_cols_ + g_cols_;
        proj_ld_ = more ? (proj_cols_ + 7) / 8 * 8 : proj_cols_;
        if (opt_.softcap < 0) fail(KIPP_E_CONFIG, "attention: softcap must not be negative");
        mix_path_ = opt_.head_mix || (window_ > 0 && opt_.keep_first > 0) || v_dim_ != head_dim_ ||
                    opt_.output_scale != 1.0 || segments_ || opt_.softcap > 0;
    }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        auto add = [&](const char* role, std::vector<int64_t> shape, const char* init = "normal") {
            TensorSpec s;
            s.name = p + opt_.names.at(role);
            s.shape = std::move(shape);
            s.init = init;
            out.push_back(s);
        };
        add("q", {q_dim_, hidden_});
        if (k_cols_) add("k", {kv_dim_, hidden_});
        if (v_cols_) add("v", {vv_dim_, hidden_});
        add("o", {hidden_, o_dim_});
        if (qk_norm_) {
            add("q_norm", {opt_.norm_whole ? q_dim_ : head_dim_}, "near_one");
            if (k_cols_) add("k_norm", {opt_.norm_whole ? kv_dim_ : head_dim_}, "near_one");
        }
        if (opt_.sink == 1) add("sink", {heads_});
        if (opt_.head_gate) add("gate", {heads_, hidden_});
        if (opt_.head_mix) add("head_mix", {heads_, heads_}, "near_identity");
        if (opt_.bias) {
            add("q_bias", {q_dim_});
            add("k_bias", {kv_dim_});
            add("v_bias", {vv_dim_});
        }
        if (opt_.combine_maps)
            for (const char* r : {"lq1", "lk1", "lq2", "lk2"}) add(r, {head_dim_});
        position_->tensor_specs(p, out);
    }
    // (the maps of a key head lie side by side in one row of the key pages)
    std::optional<PagedKVSpec> cache_spec() const override {
        return PagedKVSpec{kv_heads_, maps_ * head_dim_, window_, v_dim_, window_ > 0 ? opt_.keep_first : 0};
    }
    std::shared_ptr<WorkPlanner> planner(const DeviceInfo& dev, bool own_length) override {
        if (mix_path_) {                          // (entry, first token) per tile of its tensor-core prompt kernel
            mix_planner_ = std::make_shared<MixTilePlanner>(Ops::attention_mix_tile());
            return mix_planner_;
        }
        auto p = std::make_shared<AttentionPlanner>(kv_heads_, dev.sm_count, own_length);
        planner_ = p;
        return p;
    }
    void bind(Binder& b, const std::string& p) override {
        dtype_ = b.compute_dtype();
        const size_t es = dtype_size(dtype_);
        const int64_t rows = proj_cols_;
        const std::string nq = p + opt_.names.at("q"), nk = p + opt_.names.at("k"), nv = p + opt_.names.at("v");
        const std::string no = p + opt_.names.at("o");
        // one matrix for q, k and v (and the gate) so that one product makes them all
        w_qkv_ = b.allocate((size_t)rows * hidden_ * es, p + "qkv");
        char* base = static_cast<char*>(w_qkv_);
        b.load(nq, base, dtype_, hidden_, q_dim_, hidden_);
        if (k_cols_) b.load(nk, base + (size_t)q_dim_ * hidden_ * es, dtype_, hidden_, kv_dim_, hidden_);
        if (v_cols_) b.load(nv, base + (size_t)(q_dim_ + k_cols_) * hidden_ * es, dtype_, hidden_, vv_dim_, hidden_);
        if (g_cols_)
            b.load(p + opt_.names.at("gate"), base + (size_t)(q_dim_ + k_cols_ + v_cols_) * hidden_ * es, dtype_, hidden_,
                   heads_, hidden_);
        w_o_ = b.allocate((size_t)hidden_ * o_dim_ * es, no);
        b.load(no, w_o_, dtype_, o_dim_, hidden_, o_dim_);
        if (qk_norm_ && segments_) {              // the head segments take their norm weights in float32
            const int64_t nqw = opt_.norm_whole ? q_dim_ : head_dim_, nkw = opt_.norm_whole ? kv_dim_ : head_dim_;
            norm_dtype_ = F32;
            q_norm_ = b.allocate((size_t)nqw * sizeof(float), p + opt_.names.at("q_norm"));
            b.load(p + opt_.names.at("q_norm"), q_norm_, F32, nqw, 1, nqw);
            if (k_cols_) {
                k_norm_ = b.allocate((size_t)nkw * sizeof(float), p + opt_.names.at("k_norm"));
                b.load(p + opt_.names.at("k_norm"), k_norm_, F32, nkw, 1, nkw);
            }
        } else if (qk_norm_) {
            const std::string qn = p + opt_.names.at("q_norm"), kn = p + opt_.names.at("k_norm");
            int qd = storage_dtype(b.stored_dtype(qn));
            int kd = storage_dtype(b.stored_dtype(kn));
            norm_dtype_ = qd == kd ? qd : F32;
            q_norm_ = b.allocate((size_t)head_dim_ * dtype_size(norm_dtype_), qn);
            k_norm_ = b.allocate((size_t)head_dim_ * dtype_size(norm_dtype_), kn);
            b.load(qn, q_norm_, norm_dtype_, head_dim_, 1, head_dim_);
            b.load(kn, k_norm_, norm_dtype_, head_dim_, 1, head_dim_);
        }
        if (opt_.head_mix) {                      // the mix runs in float32
            const std::string hm = p + opt_.names.at("head_mix");
            head_mix_ = static_cast<float*>(b.allocate((size_t)heads_ * heads_ * sizeof(float), hm));
            b.load(hm, head_mix_, F32, heads_, heads_, heads_);
        }
        auto floats = [&](const char* role, int64_t n) {
            float* d = static_cast<float*>(b.allocate((size_t)n * sizeof(float), p + opt_.names.at(role)));
            b.load(p + opt_.names.at(role), d, F32, n, 1, n);
            return d;
        };
        if (opt_.bias) {
            q_bias_ = floats("q_bias", q_dim_);
            k_bias_ = floats("k_bias", kv_dim_);
            v_bias_ = floats("v_bias", vv_dim_);
        }
        if (opt_.sink == 1) sink_ = floats("sink", heads_);
        if (opt_.sink == 2) {                     // a sink of score 0 in every head
            sink_ = static_cast<float*>(b.allocate((size_t)heads_ * sizeof(float), p + "unit sink"));
            cuda_check(cudaMemset(sink_, 0, (size_t)heads_ * sizeof(float)), "clearing the unit sink");
        }
        if (opt_.combine_maps) {
            // lambda is one number for the layer: formed once, in double precision
            double dot[2] = {0.0, 0.0};
            const char* roles[2][2] = {{"lq1", "lk1"}, {"lq2", "lk2"}};
            for (int m = 0; m < 2; ++m) {
                std::vector<float> a((size_t)head_dim_), c((size_t)head_dim_);
                const float* da = floats(roles[m][0], head_dim_);
                const float* dc = floats(roles[m][1], head_dim_);
                cuda_check(cudaDeviceSynchronize(), "reading the lambda vectors");
                cuda_check(cudaMemcpy(a.data(), da, a.size() * sizeof(float), cudaMemcpyDeviceToHost), "reading the lambda vectors");
                cuda_check(cudaMemcpy(c.data(), dc, c.size() * sizeof(float), cudaMemcpyDeviceToHost), "reading the lambda vectors");
                for (int i = 0; i < head_dim_; ++i) dot[m] += (double)a[(size_t)i] * (double)c[(size_t)i];
            }
            lambda_ = (float)(std::exp(dot[0]) - std::exp(dot[1]) + opt_.lambda_init);
        }
        position_->bind(b, p);
    }
    size_t weight_bytes() const override {
        size_t n = ((size_t)proj_cols_ * hidden_ + (size_t)hidden_ * o_dim_) * dtype_size(dtype_);
        if (qk_norm_) n += (opt_.norm_whole ? (size_t)q_dim_ + k_cols_ : 2 * (size_t)head_dim_) * dtype_size(norm_dtype_);
        if (opt_.head_mix) n += (size_t)heads_ * heads_ * sizeof(float);
        if (opt_.bias) n += (size_t)(q_dim_ + kv_dim_ + vv_dim_) * sizeof(float);
        return n;
    }
    bool folds_rms() const override { return Ops::gemm_scale_ok(dtype_, w_qkv_, hidden_, w_qkv_, hidden_); }
    void forward(StepContext& ctx, const LayerRun& run, int mixer_slot, const void* h, float* residual) override;

private:
    int hidden_, heads_, kv_heads_, head_dim_;
    std::unique_ptr<PositionEncoding> position_;
    bool qk_norm_;
    float eps_;
    int window_;
    AttentionOptions opt_;
    float scale_ = 1.f;
    int v_dim_ = 0, q_dim_ = 0, kv_dim_ = 0, vv_dim_ = 0, o_dim_ = 0, dtype_ = BF16, norm_dtype_ = F32;
    bool mix_path_ = false, segments_ = false;
    int maps_ = 1;
    float lambda_ = 0.f;
    void *w_qkv_ = nullptr, *w_o_ = nullptr, *q_norm_ = nullptr, *k_norm_ = nullptr;
    float *head_mix_ = nullptr, *q_bias_ = nullptr, *k_bias_ = nullptr, *v_bias_ = nullptr, *sink_ = nullptr;
    int k_cols_ = 0, v_cols_ = 0, g_cols_ = 0, proj_cols_ = 0, proj_ld_ = 0;
    std::shared_ptr<AttentionPlanner> planner_;
    std::shared_ptr<MixTilePlanner> mix_planner_;
};

// Dense SwiGLU feed-forward: x += W_down (silu(W_gate n) * (W_up n)) (src/kipp.c:2994-3010,
// silu src/kipp.c:2402-2404).
class SwiGLUFeedForward : public FeedForward {
public:
    SwiGLUFeedForward(int hidden, int intermediate) : hidden_(hidden), inter_(intermediate) {
        if (hidden <= 0 || intermediate <= 0) fail(KIPP_E_CONFIG, "swiglu: sizes must be positive");
    }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        auto add = [&](const char* n, std::vector<int64_t> shape) {
            TensorSpec s;
            s.name = p + n;
            s.shape = std::move(shape);
            out.push_back(s);
        };
        add("gate_proj.weight", {inter_, hidden_});
        add("up_proj.weight", {inter_, hidden_});
        add("down_proj.weight", {hidden_, inter_});
    }
    void bind(Binder& b, const std::string& p) override {
        dtype_ = b.compute_dtype();
        const size_t es = dtype_size(dtype_);
        // rows interleaved (gate_0, up_0, gate_1, up_1, ...): one product makes both, and a gate
        // sits beside its up value in the epilogue
        w_gate_up_ = b.allocate((size_t)2 * inter_ * hidden_ * es, p + "gate_up");
        char* base = static_cast<char*>(w_gate_up_);
        b.load(p + "gate_proj.weight", base, dtype_, 2 * (int64_t)hidden_, inter_, hidden_);
        b.load(p + "up_proj.weight", base + (size_t)hidden_ * es, dtype_, 2 * (int64_t)hidden_, inter_, hidden_);
        w_down_ = b.allocate((size_t)hidden_ * inter_ * es, p + "down_proj.weight");
        b.load(p + "down_proj.weight", w_down_, dtype_, inter_, hidden_, inter_);
    }
    size_t weight_bytes() const override { return (size_t)3 * inter_ * hidden_ * dtype_size(dtype_); }
    bool folds_rms() const override { return Ops::gemm_scale_ok(dtype_, w_gate_up_, hidden_, w_gate_up_, hidden_); }
    void forward(StepContext& ctx, const void* h, float* residual) override {
        const int T = ctx.tokens();
        NormFold in, out;
        void* act = ctx.workspace->buffer("ffn_act", (size_t)T * inter_ * ctx.element());
        ctx.ops->gemm(act, ctx.dtype, inter_, h, hidden_, w_gate_up_, hidden_, dtype_, T, 2 * inter_, hidden_,
                      EPI_SWIGLU, fold_input(ctx, in));
        const NormFold* emit = fold_emit(ctx, out, hidden_);
        ctx.ops->gemm(residual, F32, hidden_, act, inter_, w_down_, inter_, dtype_, T, hidden_, inter_, EPI_ADD, emit);
        fold_emitted(ctx, emit, hidden_);
    }

private:
    int hidden_, inter_, dtype_ = BF16;
    void *w_gate_up_ = nullptr, *w_down_ = nullptr;
};

// Dense feed-forward with one up projection: x += W_down act(W_up n), act one of relu, relu_squared,
// gelu_tanh, silu, applied in float32 to the projection's output.
inline int activation_code(const std::string& a) {
    if (a == "relu") return ACT_RELU;
    if (a == "relu_squared") return ACT_RELU_SQUARED;
    if (a == "gelu_tanh") return ACT_GELU_TANH;
    if (a == "silu") return ACT_SILU;
    fail(KIPP_E_CONFIG, "activation must be relu, relu_squared, gelu_tanh or silu, not '" + a + "'");
}
class DenseFeedForward : public FeedForward {
public:
    DenseFeedForward(int hidden, int intermediate, const std::string& activation, std::map<std::string, std::string> names)
        : hidden_(hidden), inter_(intermediate), act_(activation_code(activation)), names_(std::move(names)) {
        if (hidden <= 0 || intermediate <= 0) fail(KIPP_E_CONFIG, "dense_mlp: sizes must be positive");
        ld_ = (inter_ + 7) / 8 * 8;
    }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        TensorSpec up, down;
        up.name = p + names_.at("up");
        up.shape = {inter_, hidden_};
        down.name = p + names_.at("down");
        down.shape = {hidden_, inter_};
        out.push_back(up);
        out.push_back(down);
    }
    void bind(Binder& b, const std::string& p) override {
        dtype_ = b.compute_dtype();
        const size_t es = dtype_size(dtype_);
        w_up_ = b.allocate((size_t)inter_ * hidden_ * es, p + names_.at("up"));
        b.load(p + names_.at("up"), w_up_, dtype_, hidden_, inter_, hidden_);
        // rows of W_down padded to a multiple of 8 elements (zeros beyond the feed-forward's size)
        w_down_ = b.allocate((size_t)hidden_ * ld_ * es, p + names_.at("down"));
        cuda_check(cudaMemset(w_down_, 0, (size_t)hidden_ * ld_ * es), "clearing a padded weight");
        b.load(p + names_.at("down"), w_down_, dtype_, ld_, hidden_, inter_);
    }
    size_t weight_bytes() const override { return (size_t)2 * inter_ * hidden_ * dtype_size(dtype_); }
    bool folds_rms() const override { return Ops::gemm_scale_ok(dtype_, w_up_, hidden_, w_up_, hidden_); }
    void forward(StepContext& ctx, const void* h, float* residual) override {
        const int T = ctx.tokens();
        NormFold in, out;
        void* z = ctx.workspace->buffer("ffn_up", (size_t)T * ld_ * ctx.element());
        if (ld_ != inter_) cuda_check(cudaMemsetAsync(z, 0, (size_t)T * ld_ * ctx.element(), ctx.stream), "clearing the padding");
        // the activation rides in the product's epilogue where the tensor-core kernel runs it
        ctx.ops->gemm(z, ctx.dtype, ld_, h, hidden_, w_up_, hidden_, dtype_, T, inter_, hidden_, EPI_STORE, fold_input(ctx, in), act_);
        const NormFold* emit = fold_emit(ctx, out, hidden_);
        ctx.ops->gemm(residual, F32, hidden_, z, ld_, w_down_, ld_, dtype_, T, hidden_, ld_, EPI_ADD, emit);
        fold_emitted(ctx, emit, hidden_);
    }

private:
    int hidden_, inter_, act_, ld_ = 0, dtype_ = BF16;
    std::map<std::string, std::string> names_;
    void *w_up_ = nullptr, *w_down_ = nullptr;
};

// Gated dense feed-forward with limits: g = min(W_gate n + b_g, limit), u = clamp(W_up n + b_u, -limit, limit),
// x += W_down (g sigmoid(alpha g) (u + 1)) + b_d.  Biases are optional (bias), limit 0 means none.  With
// row_gate the part's output is also multiplied by sigmoid(w_r . n), one number per token (a tensor
// [1, hidden], kept in float32): the factor is applied to the hidden row before the (linear) down
// projection.  Gate and up rows lie interleaved in one matrix, so one product makes both and the
// activation runs in its epilogue on the float32 sums (tensor-core path), or in a kernel of its own
// after a stored product (32-bit, odd sizes).
class GatedFeedForward : public FeedForward {
public:
    explicit GatedFeedForward(const Json& j) {
        hidden_ = (int)j.get("hidden_size").as_int();
        inter_ = (int)j.get("intermediate_size").as_int();
        limit_ = (float)j.get_double("limit", 0.0);
        alpha_ = (float)j.get_double("alpha", 1.0);
        bias_ = j.get_bool("bias", false);
        row_gate_ = j.get_bool("row_gate", false);
        names_ = tensor_names(j, {{"gate", "gate"}, {"up", "up"}, {"down", "down"}, {"gate_bias", "gate.b"},
                                  {"up_bias", "up.b"}, {"down_bias", "down.b"}, {"row_gate", "sg"}});
        if (hidden_ <= 0 || inter_ <= 0) fail(KIPP_E_CONFIG, "gated_mlp: sizes must be positive");
        if (limit_ < 0.f || !(alpha_ > 0.f)) fail(KIPP_E_CONFIG, "gated_mlp: limit must not be negative and alpha must be positive");
        inter_ld_ = (inter_ + 7) / 8 * 8;
    }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        auto add = [&](const char* role, std::vector<int64_t> shape) {
            TensorSpec s;
            s.name = p + names_.at(role);
            s.shape = std::move(shape);
            out.push_back(s);
        };
        add("gate", {inter_, hidden_});
        add("up", {inter_, hidden_});
        add("down", {hidden_, inter_});
        if (bias_) {
            add("gate_bias", {inter_});
            add("up_bias", {inter_});
            add("down_bias", {hidden_});
        }
        if (row_gate_) add("row_gate", {1, hidden_});
    }
    void bind(Binder& b, const std::string& p) override {
        dtype_ = b.compute_dtype();
        const size_t es = dtype_size(dtype_);
        // rows interleaved (gate_0, up_0, gate_1, up_1, ...): a gate sits beside its up value in the epilogue
        w_in_ = b.allocate((size_t)2 * inter_ * hidden_ * es, p + "gate, up");
        char* base = static_cast<char*>(w_in_);
        b.load(p + names_.at("gate"), base, dtype_, 2 * (int64_t)hidden_, inter_, hidden_);
        b.load(p + names_.at("up"), base + (size_t)hidden_ * es, dtype_, 2 * (int64_t)hidden_, inter_, hidden_);
        w_down_ = b.allocate((size_t)hidden_ * inter_ld_ * es, p + names_.at("down"));
        cuda_check(cudaMemset(w_down_, 0, (size_t)hidden_ * inter_ld_ * es), "clearing a padded weight");
        b.load(p + names_.at("down"), w_down_, dtype_, inter_ld_, hidden_, inter_);
        auto floats = [&](const char* role, int64_t n, float* d, int64_t pitch) {
            if (d == nullptr) d = static_cast<float*>(b.allocate((size_t)n * pitch * sizeof(float), p + names_.at(role)));
            b.load(p + names_.at(role), d, F32, pitch, n, 1);
            return d;
        };
        if (bias_) {
            b_in_ = floats("gate_bias", inter_, nullptr, 2);         // interleaved like the rows
            floats("up_bias", inter_, b_in_ + 1, 2);
            b_down_ = floats("down_bias", hidden_, nullptr, 1);
        }
        if (row_gate_) w_row_ = floats("row_gate", hidden_, nullptr, 1);
    }
    size_t weight_bytes() const override {
        return (size_t)3 * inter_ * hidden_ * dtype_size(dtype_) + (bias_ ? (size_t)(2 * inter_ + hidden_) * 4 : 0) +
               (row_gate_ ? (size_t)hidden_ * 4 : 0);
    }
    bool folds_rms() const override { return Ops::gemm_scale_ok(dtype_, w_in_, hidden_, w_in_, hidden_); }
    void forward(StepContext& ctx, const void* h, float* residual) override {
        const int T = ctx.tokens();
        NormFold in, out;
        Ops::Glu glu;
        glu.alpha = alpha_;
        glu.limit = limit_;
        glu.bias = b_in_;
        if (row_gate_) {
            if (ctx.input_scale.valid()) fail(KIPP_E_STATE, "gated_mlp: a gate per token does not read an input in deferred form");
            float* logits = ctx.workspace->get<float>("gated_mlp_row_gate", (size_t)T);
            ctx.ops->row_dot(logits, h, hidden_, ctx.dtype, w_row_, T, hidden_);
            glu.row_gate = logits;
        }
        void* act = ctx.workspace->buffer("gated_mlp_act", (size_t)T * inter_ld_ * ctx.element());
        if (inter_ld_ != inter_) cuda_check(cudaMemsetAsync(act, 0, (size_t)T * inter_ld_ * ctx.element(), ctx.stream), "clearing the padding");
        const bool fused = Ops::gemm_tc_ok(dtype_, h, hidden_, w_in_, hidden_) && ctx.dtype == dtype_;
        void* proj = fused ? nullptr : ctx.workspace->buffer("gated_mlp_proj", (size_t)T * 2 * inter_ * ctx.element());
        ctx.ops->gemm_glu(act, ctx.dtype, inter_ld_, h, hidden_, w_in_, hidden_, dtype_, T, 2 * inter_, hidden_, glu,
                          fold_input(ctx, in), proj, 2 * inter_);
        const NormFold* emit = b_down_ == nullptr ? fold_emit(ctx, out, hidden_) : nullptr;
        ctx.ops->gemm(residual, F32, hidden_, act, inter_ld_, w_down_, inter_ld_, dtype_, T, hidden_, inter_ld_, EPI_ADD, emit);
        fold_emitted(ctx, emit, hidden_);
        if (b_down_ != nullptr) ctx.ops->add_row_bias(residual, b_down_, T, hidden_);
    }

private:
    int hidden_ = 0, inter_ = 0, inter_ld_ = 0, dtype_ = BF16;
    float limit_ = 0.f, alpha_ = 1.f;
    bool bias_ = false, row_gate_ = false;
    std::map<std::string, std::string> names_;
    void *w_in_ = nullptr, *w_down_ = nullptr;
    float *b_in_ = nullptr, *b_down_ = nullptr, *w_row_ = nullptr;
};

// x += mixer(n) + ffn(n) with n = norm(x): ONE norm whose output both sublayers read.  A block
// without a feed-forward (ffn null) has the mixer only.
class ParallelBlock : public Block {
public:
    ParallelBlock(std::unique_ptr<Norm> norm, std::unique_ptr<Mixer> mixer, std::unique_ptr<FeedForward> ffn,
                  std::vector<std::string> names)
        : norm_(std::move(norm)), mixer_(std::move(mixer)), ffn_(std::move(ffn)), names_(std::move(names)) {
        if (names_.size() != 3) fail(KIPP_E_CONFIG, "parallel_block: three name prefixes are needed");
    }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        norm_->tensor_specs(p + names_[0], out);
        mixer_->tensor_specs(p + names_[1], out);
        if (ffn_) ffn_->tensor_specs(p + names_[2], out);
    }
    void bind(Binder& b, const std::string& p) override {
        norm_->bind(b, p + names_[0]);
        mixer_->bind(b, p + names_[1]);
        if (ffn_) ffn_->bind(b, p + names_[2]);
    }
    size_t weight_bytes() const override {
        return norm_->weight_bytes() + mixer_->weight_bytes() + (ffn_ ? ffn_->weight_bytes() : 0);
    }
    bool graph_safe() const override { return norm_->graph_safe() && mixer_->graph_safe() && (!ffn_ || ffn_->graph_safe()); }
    std::vector<Mixer*> mixers() override { return mixer_->parts(); }
    void forward(StepContext& ctx, const LayerRun& run, float* x) override {
        const int T = ctx.tokens();
        // both sublayers read h, and both add to x: h must outlive the mixer, so no part may leave
        // another norm's input in its place (emit_for stays null)
        void* h = ctx.workspace->buffer("normed", (size_t)T * norm_->size() * ctx.element());
        ctx.input_scale = RowScale{};
        ctx.pending_norm = nullptr;
        ctx.emit_for = nullptr;
        ctx.emitted = false;
        norm_->forward(ctx, x, h, nullptr, T);
        mixer_->forward(ctx, run, 0, h, x);
        if (ffn_) ffn_->forward(ctx, h, x);
        ctx.emitted = false;
    }
    Norm* norm() { return norm_.get(); }
    FeedForward* feed_forward() { return ffn_.get(); }

private:
    std::unique_ptr<Norm> norm_;
    std::unique_ptr<Mixer> mixer_;
    std::unique_ptr<FeedForward> ffn_;
    std::vector<std::string> names_;
};

// x += mult * norm1(mixer(x)); x += mult * norm2(ffn(x)): the sublayers read the stream itself (rounded
// to the compute type), the norm sits on each sublayer's OUTPUT, and `mult` scales what joins the
// stream.  A sublayer adds its output into a cleared float32 buffer; the norm of that buffer and the
// addition to the stream are one float32 kernel.  The norms must be plain RMS norms.  A block
// without a feed-forward (post_norm and ffn null) has the first sublayer only.
class OutputNormBlock : public Block {
public:
    OutputNormBlock(std::unique_ptr<Norm> n1, std::unique_ptr<Mixer> mixer, std::unique_ptr<Norm> n2,
                    std::unique_ptr<FeedForward> ffn, double mult, std::vector<std::string> names)
        : n1_(std::move(n1)), mixer_(std::move(mixer)), n2_(std::move(n2)), ffn_(std::move(ffn)), mult_((float)mult),
          names_(std::move(names)) {
        if (names_.size() != 4) fail(KIPP_E_CONFIG, "output_norm_block: four name prefixes are needed");
        if ((n2_ == nullptr) != (ffn_ == nullptr))
            fail(KIPP_E_CONFIG, "output_norm_block: post_norm and ffn come together or not at all");
        if (n2_ && n1_->size() != n2_->size()) fail(KIPP_E_CONFIG, "output_norm_block: the two norms differ in size");
    }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        n1_->tensor_specs(p + names_[0], out);
        mixer_->tensor_specs(p + names_[1], out);
        if (ffn_) {
            n2_->tensor_specs(p + names_[2], out);
            ffn_->tensor_specs(p + names_[3], out);
        }
    }
    void bind(Binder& b, const std::string& p) override {
        n1_->bind(b, p + names_[0]);
        mixer_->bind(b, p + names_[1]);
        if (ffn_) {
            n2_->bind(b, p + names_[2]);
            ffn_->bind(b, p + names_[3]);
        }
        if (!n1_->rms_spec() || (n2_ && !n2_->rms_spec()))
            fail(KIPP_E_CONFIG, "output_norm_block: the norms on the sublayers' outputs must be RMS norms");
    }
    size_t weight_bytes() const override {
        return n1_->weight_bytes() + mixer_->weight_bytes() + (ffn_ ? n2_->weight_bytes() + ffn_->weight_bytes() : 0);
    }
    bool graph_safe() const override {
        return n1_->graph_safe() && mixer_->graph_safe() && (!ffn_ || (n2_->graph_safe() && ffn_->graph_safe()));
    }
    std::vector<Mixer*> mixers() override { return mixer_->parts(); }
    void forward(StepContext& ctx, const LayerRun& run, float* x) override {
        const int T = ctx.tokens(), W = n1_->size();
        // no norm runs before a sublayer here: nothing to fold into the products, nothing pending
        ctx.input_scale = RowScale{};
        ctx.pending_norm = nullptr;
        ctx.emit_for = nullptr;
        ctx.emitted = false;
        float* y = ctx.workspace->get<float>("sublayer_output", (size_t)T * W);
        // 16-bit path: a sublayer reads the stream rounded to the compute type.  The first
        // sublayer's copy is made here; the second one's leaves the kernel that adds the first
        // one's output to the stream.
        void* hc = ctx.dtype != F32 ? ctx.workspace->buffer("normed", (size_t)T * W * ctx.element()) : nullptr;
        auto sublayer = [&](const Norm& norm, bool copied, bool copy_after, auto&& run_part) {
            const void* h = x;                    // 32-bit path: the sublayer reads the stream in place
            if (hc != nullptr) {
                if (!copied) ctx.ops->convert_rows(hc, ctx.dtype, W, x, F32, W, T, W);
                h = hc;
            }
            cuda_check(cudaMemsetAsync(y, 0, (size_t)T * W * sizeof(float), ctx.stream), "clearing a sublayer's output");
            run_part(h);
            const RmsNormSpec spec = *norm.rms_spec();
            ctx.ops->rmsnorm_scaled_add(x, y, spec.weight, spec.weight_dtype, T, W, spec.eps, mult_,
                                        copy_after && ctx.dtype == BF16 ? hc : nullptr);
        };
        const bool hand_on = ffn_ != nullptr && ctx.dtype == BF16;
        sublayer(*n1_, false, hand_on, [&](const void* h) { mixer_->forward(ctx, run, 0, h, y); });
        if (ffn_) sublayer(*n2_, hand_on, false, [&](const void* h) { ffn_->forward(ctx, h, y); });
        ctx.emitted = false;
    }
    Norm* mixer_norm() { return n1_.get(); }
    Norm* post_norm() { return n2_.get(); }
    FeedForward* feed_forward() { return ffn_.get(); }

private:
    std::unique_ptr<Norm> n1_;
    std::unique_ptr<Mixer> mixer_;
    std::unique_ptr<Norm> n2_;
    std::unique_ptr<FeedForward> ffn_;
    float mult_;
    std::vector<std::string> names_;
};

// x += mixer(norm1(x)); x += ffn(norm2(x)): the un-normed x is the residual stream
// (src/kipp.c:2948, 2994).  A block without a feed-forward (post_norm and ffn null) has the
// first sublayer only.
class PreNormBlock : public Block {
public:
    PreNormBlock(std::unique_ptr<Norm> n1, std::unique_ptr<Mixer> mixer, std::unique_ptr<Norm> n2,
                 std::unique_ptr<FeedForward> ffn, std::vector<std::string> names)
        : n1_(std::move(n1)), mixer_(std::move(mixer)), n2_(std::move(n2)), ffn_(std::move(ffn)), names_(std::move(names)) {
        if (names_.size() != 4) fail(KIPP_E_CONFIG, "pre_norm_block: four name prefixes are needed");
        if ((n2_ == nullptr) != (ffn_ == nullptr))
            fail(KIPP_E_CONFIG, "pre_norm_block: post_norm and ffn come together or not at all");
        if (n2_ && n1_->size() != n2_->size()) fail(KIPP_E_CONFIG, "pre_norm_block: the two norms differ in size");
    }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        n1_->tensor_specs(p + names_[0], out);
        mixer_->tensor_specs(p + names_[1], out);
        if (ffn_) {
            n2_->tensor_specs(p + names_[2], out);
            ffn_->tensor_specs(p + names_[3], out);
        }
    }
    void bind(Binder& b, const std::string& p) override {
        n1_->bind(b, p + names_[0]);
        mixer_->bind(b, p + names_[1]);
        if (ffn_) {
            n2_->bind(b, p + names_[2]);
            ffn_->bind(b, p + names_[3]);
        }
    }
    size_t weight_bytes() const override {
        return n1_->weight_bytes() + mixer_->weight_bytes() + (ffn_ ? n2_->weight_bytes() + ffn_->weight_bytes() : 0);
    }
    bool graph_safe() const override {
        return n1_->graph_safe() && mixer_->graph_safe() && (!ffn_ || (n2_->graph_safe() && ffn_->graph_safe()));
    }
    std::vector<Mixer*> mixers() override { return mixer_->parts(); }
    const Norm* deferred_first_norm() const override {
        return mixer_->folds_rms() && n1_->rms_spec() ? n1_.get() : nullptr;
    }
    // A plain RMSNorm before a part that folds it runs in deferred form, at every size of step:
    // the part's input is bf16(x * weight), the row factor goes into its first product.  In steps
    // of few tokens the residual add BEFORE the norm leaves that form itself (two launches fewer
    // per layer, where a launch costs more than the norm's arithmetic); otherwise one kernel makes
    // it.  Both give the same bits, so the logits do not depend on which ran.
    void forward(StepContext& ctx, const LayerRun& run, float* x) override {
        const int T = ctx.tokens();
        void* h = ctx.workspace->buffer("normed", (size_t)T * n1_->size() * ctx.element());
        const std::optional<RmsNormSpec> spec1 = n1_->rms_spec(), spec2 = ffn_ ? n2_->rms_spec() : std::nullopt;
        const bool defer1 = spec1 && mixer_->folds_rms(), defer2 = ffn_ && spec2 && ffn_->folds_rms();
        // the norm the next block starts with, if the last residual add of this one may leave its form
        const Norm* next = ctx.following_norm;
        const std::optional<RmsNormSpec> spec_next = next ? next->rms_spec() : std::nullopt;
        const bool next_fits = spec_next && next->size() == n1_->size();
        // -- norm 1 and the mixer
        ctx.input_scale = RowScale{};
        if (defer1 && ctx.pending_norm == n1_.get()) ctx.input_scale = ctx.pending_scale;   // h is made already
        else if (defer1) ctx.input_scale = deferred_norm(ctx, *spec1, x, h);
        else n1_->forward(ctx, x, h, nullptr, T);
        ctx.pending_norm = nullptr;
        ctx.emit_for = defer2 ? &*spec2 : (!ffn_ && next_fits && mixer_->folds_rms() ? &*spec_next : nullptr);
        ctx.emitted = false;
        mixer_->forward(ctx, run, 0, h, x);
        if (ffn_) {
            // -- norm 2 and the feed-forward
            ctx.input_scale = RowScale{};
            if (defer2 && ctx.emitted) ctx.input_scale = ctx.emitted_scale;
            else if (defer2) ctx.input_scale = deferred_norm(ctx, *spec2, x, h);
            else n2_->forward(ctx, x, h, nullptr, T);
            ctx.emit_for = next_fits && ffn_->folds_rms() ? &*spec_next : nullptr;
            ctx.emitted = false;
            ffn_->forward(ctx, h, x);
        }
        if (ctx.emitted) {
            ctx.pending_norm = next;
            ctx.pending_scale = ctx.emitted_scale;
        }
        ctx.input_scale = RowScale{};
        ctx.emit_for = nullptr;
        ctx.emitted = false;
    }
    Norm* input_norm() { return n1_.get(); }
    Norm* post_norm() { return n2_.get(); }
    FeedForward* feed_forward() { return ffn_.get(); }

private:
    std::unique_ptr<Norm> n1_;
    std::unique_ptr<Mixer> mixer_;
    std::unique_ptr<Norm> n2_;
    std::unique_ptr<FeedForward> ffn_;
    std::vector<std::string> names_;
};

// Hyper-connections: the residual stream is `streams` copies x_1 .. x_S (all equal to the embedding
// output at the start, summed at the end).  Sublayer q (1 the mixer, 2 the feed-forward) reads
// u = sum_s in_q[s] x_s through its RMS norm, and its output y joins every copy at once:
// x_t <- sum_s mix_q[s, t] x_s + mult * out_q[t] * y.  Three small tensors per sublayer (in [S], out [S],
// mix [S, S] indexed [from, to]) under the prefixes names[4], names[5].  Without connections
// (connections false: no such tensors) the block is the plain pre-norm x <- x + mult * sublayer(norm(x))
// on one stream.  The kernel between two sublayers updates the copies and forms the next sublayer's
// input in one pass; everything of it is float32.  A block without a feed-forward has the mixer only.
class HyperConnectionBlock : public Block {
public:
    HyperConnectionBlock(const Json& j, std::unique_ptr<Norm> n1, std::unique_ptr<Mixer> mixer, std::unique_ptr<Norm> n2,
                         std::unique_ptr<FeedForward> ffn)
        : n1_(std::move(n1)), mixer_(std::move(mixer)), n2_(std::move(n2)), ffn_(std::move(ffn)) {
        streams_ = (int)j.get_int("streams", 1);
        connections_ = j.get_bool("connections", true);
        mult_ = (float)j.get_double("residual_mult", 1.0);
        for (auto& n : j.get("names").items()) names_.push_back(n.as_string());
        if (names_.size() != 6) fail(KIPP_E_CONFIG, "hyper_connection_block: six name prefixes are needed");
        if (streams_ < 1) fail(KIPP_E_CONFIG, "hyper_connection_block: streams must be at least 1");
        if (!connections_ && streams_ != 1) fail(KIPP_E_CONFIG, "hyper_connection_block: several streams need their connections");
        if ((n2_ == nullptr) != (ffn_ == nullptr))
            fail(KIPP_E_CONFIG, "hyper_connection_block: post_norm and ffn come together or not at all");
        if (n2_ && n1_->size() != n2_->size()) fail(KIPP_E_CONFIG, "hyper_connection_block: the two norms differ in size");
    }
    int streams() const override { return streams_; }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        n1_->tensor_specs(p + names_[0], out);
        mixer_->tensor_specs(p + names_[1], out);
        if (ffn_) {
            n2_->tensor_specs(p + names_[2], out);
            ffn_->tensor_specs(p + names_[3], out);
        }
        if (!connections_) return;
        for (int q = 0; q < (ffn_ ? 2 : 1); ++q) {
            auto add = [&](const char* name, std::vector<int64_t> shape, const char* init) {
                TensorSpec s;
                s.name = p + names_[4 + (size_t)q] + name;
                s.shape = std::move(shape);
                s.init = init;
                out.push_back(s);
            };
            add("in", {streams_}, "near_one");
            add("out", {streams_}, "near_one");
            add("mix", {streams_, streams_}, "near_identity");
        }
    }
    void bind(Binder& b, const std::string& p) override {
        n1_->bind(b, p + names_[0]);
        mixer_->bind(b, p + names_[1]);
        if (ffn_) {
            n2_->bind(b, p + names_[2]);
            ffn_->bind(b, p + names_[3]);
        }
        if (!n1_->rms_spec() || (n2_ && !n2_->rms_spec()))
            fail(KIPP_E_CONFIG, "hyper_connection_block: the norms must be RMS norms");
        if (streams_ > Ops::hyper_connection_max_streams())
            fail(KIPP_E_UNSUPPORTED, format("hyper_connection_block: at most %d streams", Ops::hyper_connection_max_streams()));
        if (!connections_) return;
        // in [S], out [S], mix [S, S] of each sublayer, float32, one after another
        const size_t per = (size_t)streams_ * (streams_ + 2);
        coef_ = static_cast<float*>(b.allocate(2 * per * sizeof(float), p + "connections"));
        for (int q = 0; q < (ffn_ ? 2 : 1); ++q) {
            float* c = coef_ + (size_t)q * per;
            const std::string hp = p + names_[4 + (size_t)q];
            b.load(hp + "in", c, F32, streams_, 1, streams_);
            b.load(hp + "out", c + streams_, F32, streams_, 1, streams_);
            b.load(hp + "mix", c + 2 * streams_, F32, streams_, streams_, streams_);
        }
    }
    size_t weight_bytes() const override {
        return n1_->weight_bytes() + mixer_->weight_bytes() + (ffn_ ? n2_->weight_bytes() + ffn_->weight_bytes() : 0) +
               (connections_ ? (size_t)2 * streams_ * (streams_ + 2) * 4 : 0);
    }
    bool graph_safe() const override {
        return n1_->graph_safe() && mixer_->graph_safe() && (!ffn_ || (n2_->graph_safe() && ffn_->graph_safe()));
    }
    std::vector<Mixer*> mixers() override { return mixer_->parts(); }
    void forward(StepContext& ctx, const LayerRun& run, float* x) override {
        const int T = ctx.tokens(), W = n1_->size(), S = streams_;
        const long long stride = (long long)T * W;
        Ops& ops = *ctx.ops;
        // the norms run inside the connection kernel: nothing to fold into the products, nothing pending
        ctx.input_scale = RowScale{};
        ctx.pending_norm = nullptr;
        ctx.emit_for = nullptr;
        ctx.emitted = false;
        void* h = ctx.workspace->buffer("normed", (size_t)T * W * ctx.element());
        float* y = ctx.workspace->get<float>("sublayer_output", (size_t)T * W);
        const size_t per = (size_t)S * (S + 2);
        auto in_w = [&](int q) { return connections_ ? coef_ + (size_t)q * per : nullptr; };
        auto out_w = [&](int q) { return connections_ ? coef_ + (size_t)q * per + S : nullptr; };
        auto mix = [&](int q) { return connections_ ? coef_ + (size_t)q * per + 2 * S : nullptr; };
        const RmsNormSpec s1 = *n1_->rms_spec();
        // (the block before may have formed this block's first input while it wrote the streams)
        const bool ready = ctx.input_ready_for == this;
        ctx.input_ready_for = nullptr;
        // y, the float32 buffer a sublayer adds its output into: in steps of few tokens the kernel that reads it
        // leaves it zeroed (a launch less per sublayer, where launches are what a step costs) and only a block
        // that starts on its own (the first of a step) clears it itself; in prompt-sized steps a memset does
        // (measured at 2,048 tokens: the kernel that also clears took 51 against 36 us a launch)
        const bool kernel_clears = T < 1024;
        auto clear = [&] { cuda_check(cudaMemsetAsync(y, 0, (size_t)T * W * sizeof(float), ctx.stream), "clearing a sublayer's output"); };
        if (!ready)
            ops.hyper_connection(x, stride, S, nullptr, false, nullptr, nullptr, 0.f, in_w(0), s1.weight, s1.weight_dtype, s1.eps,
                                 h, ctx.dtype, T, W);
        if (!ready || !kernel_clears) clear();
        mixer_->forward(ctx, run, 0, h, y);
        // the last update of this block also reads the streams for the block that runs next, if that is
        // one of this kind on as many streams
        const HyperConnectionBlock* next = dynamic_cast<const HyperConnectionBlock*>(ctx.following_block);
        if (next != nullptr && (next->streams_ != S || next->n1_->size() != W || !next->n1_->rms_spec())) next = nullptr;
        auto last_update = [&](int q) {
            if (next == nullptr) {
                ops.hyper_connection(x, stride, S, y, false, mix(q), out_w(q), mult_, nullptr, nullptr, 0, 0.f, nullptr, ctx.dtype,
                                     T, W);
                return;
            }
            const RmsNormSpec sn = *next->n1_->rms_spec();
            ops.hyper_connection(x, stride, S, y, kernel_clears, mix(q), out_w(q), mult_, next->connections_ ? next->coef_ : nullptr,
                                 sn.weight, sn.weight_dtype, sn.eps, h, ctx.dtype, T, W);
            ctx.input_ready_for = next;
        };
        if (ffn_) {
            const RmsNormSpec s2 = *n2_->rms_spec();
            ops.hyper_connection(x, stride, S, y, kernel_clears, mix(0), out_w(0), mult_, in_w(1), s2.weight, s2.weight_dtype, s2.eps, h,
                                 ctx.dtype, T, W);
            if (!kernel_clears) clear();
            ffn_->forward(ctx, h, y);
            last_update(1);
        } else {
            last_update(0);
        }
        ctx.emitted = false;
    }
    Norm* input_norm() { return n1_.get(); }
    Norm* post_norm() { return n2_.get(); }
    FeedForward* feed_forward() { return ffn_.get(); }

private:
    std::unique_ptr<Norm> n1_;
    std::unique_ptr<Mixer> mixer_;
    std::unique_ptr<Norm> n2_;
    std::unique_ptr<FeedForward> ffn_;
    int streams_ = 1;
    bool connections_ = true;
    float mult_ = 1.f;
    std::vector<std::string> names_;
    float* coef_ = nullptr;
};

// ---------------------------------------------------------------------------------------------
// Parts whose forward pass the caller supplies (kipp_external_part).  The plan declares what
// the engine has to know without calling them: their tensors (so that a checkpoint is checked
// as a whole), a mixer's per-request state, and whether a captured graph may hold their work.
struct ExternalCommon {
    kipp_external_part hook{};
    std::vector<TensorSpec> specs;
    bool graph_safe = false;
    int size = 0;

    void read(const Json& j, const BuildContext& ctx) {
        const long long index = j.get("index").as_int();
        if (index < 0 || index >= ctx.n_external || !ctx.external || !ctx.external[index].forward)
            fail(KIPP_E_CONFIG, format("the plan names external part %lld, which the caller did not supply", index));
        hook = ctx.external[index];
        if (const Json* t = j.find("tensors"))
            for (auto& s : t->items()) specs.push_back(TensorSpec::from_json(s));
        graph_safe = j.get_bool("graph_safe", false);
        size = (int)j.get_int("size", 0);
    }
    void fill(kipp_external_call& c, StepContext& ctx, int role) const {
        const StepMeta& m = *ctx.meta;
        c = kipp_external_call{};
        c.role = role;
        c.tokens = m.shape.tokens;
        c.entries = m.shape.entries;
        c.token_ids = m.token_ids;
        c.positions = m.positions;
        c.entry_of_token = m.entry_of_token;
        c.q_start = m.q_start;
        c.context_len = m.context_len;
        c.slots = m.slots;
        c.host_q_lens = m.shape.q_lens.data();
        c.host_context_len = m.shape.starts.data();
        c.host_slots = m.shape.slots.data();
        c.input_dtype = ctx.dtype;
        c.max_requests = ctx.max_requests();
        c.stream = ctx.stream;
    }
    void call(const kipp_external_call& c, const char* what) const {
        const int rc = hook.forward(hook.user, &c);
        if (rc) fail(KIPP_E_KERNEL, format("the external %s failed with code %d", what, rc));
    }
};

class ExternalMixer : public Mixer {
public:
    ExternalMixer(const Json& j, const BuildContext& ctx) {
        common_.read(j, ctx);
        hidden_ = j.get("hidden_size").as_int();
        if (const Json* s = j.find("state"); s && !s->is_null()) {
            StateSpec spec;
            for (auto& d : s->get("shape").items()) spec.shape.push_back(d.as_int());
            const std::string dt = s->get_string("dtype", "float32");
            spec.dtype = dt == "float32" ? F32 : dt == "bfloat16" ? BF16 : dt == "int32" ? I32 : -1;
            if (spec.dtype < 0) fail(KIPP_E_CONFIG, "external mixer: state dtype must be float32, bfloat16 or int32");
            state_ = spec;
        }
    }
    void tensor_specs(const std::string&, std::vector<TensorSpec>& out) const override {
        out.insert(out.end(), common_.specs.begin(), common_.specs.end());
    }
    std::optional<StateSpec> state_spec() const override { return state_; }
    bool graph_safe() const override { return common_.graph_safe; }
    void forward(StepContext& ctx, const LayerRun& run, int mixer_slot, const void* h, float* residual) override {
        kipp_external_call c;
        common_.fill(c, ctx, 2);
        c.layer = run.layer;
        c.cache = run.cache;
        c.writes_cache = run.writes_cache ? 1 : 0;
        c.input = h;
        c.input_cols = hidden_;
        c.residual = residual;
        c.hidden = hidden_;
        if (state_) {
            size_t bytes = 0;
            c.state = ctx.state_view(run, mixer_slot, &bytes);
            c.state_bytes = (long long)bytes;
        }
        common_.call(c, "mixer");
    }

private:
    ExternalCommon common_;
    long long hidden_ = 0;
    std::optional<StateSpec> state_;
};

class ExternalFeedForward : public FeedForward {
public:
    ExternalFeedForward(const Json& j, const BuildContext& ctx) {
        common_.read(j, ctx);
        hidden_ = j.get("hidden_size").as_int();
    }
    void tensor_specs(const std::string&, std::vector<TensorSpec>& out) const override {
        out.insert(out.end(), common_.specs.begin(), common_.specs.end());
    }
    bool graph_safe() const override { return common_.graph_safe; }
    void forward(StepContext& ctx, const void* h, float* residual) override {
        kipp_external_call c;
        common_.fill(c, ctx, 3);
        c.input = h;
        c.input_cols = hidden_;
        c.residual = residual;
        c.hidden = hidden_;
        common_.call(c, "feed-forward");
    }

private:
    ExternalCommon common_;
    long long hidden_ = 0;
};

class ExternalEmbeddingStage : public EmbeddingStage {
public:
    ExternalEmbeddingStage(const Json& j, const BuildContext& ctx) {
        common_.read(j, ctx);
        hidden_ = j.get("hidden_size").as_int();
    }
    void tensor_specs(const std::string&, std::vector<TensorSpec>& out) const override {
        out.insert(out.end(), common_.specs.begin(), common_.specs.end());
    }
    bool graph_safe() const override { return common_.graph_safe; }
    void forward(StepContext& ctx, float* x) override {
        kipp_external_call c;
        common_.fill(c, ctx, 0);
        c.residual = x;
        c.hidden = hidden_;
        common_.call(c, "embedding stage");
    }

private:
    ExternalCommon common_;
    long long hidden_ = 0;
};

class ExternalNorm : public Norm {
public:
    ExternalNorm(const Json& j, const BuildContext& ctx) {
        common_.read(j, ctx);
        if (common_.size <= 0) fail(KIPP_E_CONFIG, "external norm: 'size' is needed");
    }
    void tensor_specs(const std::string&, std::vector<TensorSpec>& out) const override {
        out.insert(out.end(), common_.specs.begin(), common_.specs.end());
    }
    bool graph_safe() const override { return common_.graph_safe; }
    int size() const override { return common_.size; }
    void forward(StepContext& ctx, const float* x, void* out, const int* rows, int n_rows) override {
        kipp_external_call c;
        common_.fill(c, ctx, 1);
        c.residual = const_cast<float*>(x);
        c.hidden = common_.size;
        c.output = out;
        c.rows = rows;
        c.n_rows = n_rows;
        common_.call(c, "norm");
    }

private:
    ExternalCommon common_;
};

// ---------------------------------------------------------------------------------------------
inline std::unique_ptr<PositionEncoding> make_position(const Json& j, const BuildContext& ctx) {
    return Registry::get().make_as<PositionEncoding>(j, ctx, "a position encoding");
}
void register_recurrent_parts(Registry& r);     // recurrent_parts.hpp
void register_latent_parts(Registry& r);        // latent_parts.hpp
void register_expert_parts(Registry& r);        // expert_parts.hpp

inline void register_builtin_parts() {
    Registry& r = Registry::get();
    r.add_part_kind("token_embedding", [](const Json& j, const BuildContext&) -> std::unique_ptr<Part> {
        return std::make_unique<TokenEmbedding>((int)j.get("vocab_size").as_int(), (int)j.get("hidden_size").as_int(),
                                                j.get_string("weight_name", "weight"));
    });
    r.add_part_kind("output_head", [](const Json& j, const BuildContext&) -> std::unique_ptr<Part> {
        return std::make_unique<OutputHead>((int)j.get("vocab_size").as_int(), (int)j.get("hidden_size").as_int(),
                                            j.get_string("tied_to", ""), j.get_string("weight_name", "weight"),
                                            j.get_double("logit_scale", 1.0), j.get_double("logit_softcap", 0.0));
    });
    r.add_part_kind("hashed_pair_embedding", [](const Json& j, const BuildContext&) -> std::unique_ptr<Part> {
        return std::make_unique<HashedPairEmbedding>((int)j.get("vocab_size").as_int(), (int)j.get("hidden_size").as_int(),
                                                     j.get("buckets").as_int(), j.get("mul_prev").as_int(),
                                                     j.get("mul_cur").as_int(), j.get_string("weight_name", "weight"));
    });
    r.add_part_kind("rmsnorm", [](const Json& j, const BuildContext&) -> std::unique_ptr<Part> {
        return std::make_unique<RMSNorm>((int)j.get("size").as_int(), j.get("eps").as_double(),
                                         j.get_string("weight_name", "weight"));
    });
    r.add_part_kind("layernorm", [](const Json& j, const BuildContext&) -> std::unique_ptr<Part> {
        return std::make_unique<LayerNorm>((int)j.get("size").as_int(), j.get("eps").as_double(),
                                           j.get_string("weight_name", "weight"), j.get_string("bias_name", "bias"));
    });
    r.add_part_kind("stretched_rotary", [](const Json& j, const BuildContext&) -> std::unique_ptr<Part> {
        const int head_dim = (int)j.get("head_dim").as_int();
        const int rot = (int)j.get_int("rotary_dim", head_dim);
        const double theta = j.get("theta").as_double(), factor = j.get("factor").as_double();
        const double low = j.get("low").as_double(), high = j.get("high").as_double(), original = j.get("original").as_double();
        if (rot % 2 || rot <= 0 || rot > head_dim)
            fail(KIPP_E_CONFIG, format("rotary_dim %d must be even, positive and at most head_dim %d", rot, head_dim));
        if (!(theta > 0) || !(factor > 0) || !(low > 0) || !(high > low) || !(original > 0))
            fail(KIPP_E_CONFIG, "stretched_rotary: theta, factor, low and original must be positive and high above low");
        return std::make_unique<FrequencyTable>(stretched_frequencies(rot, theta, factor, low, high, original),
                                                format("stretched/%.17g/%d/%.17g/%.17g/%.17g/%.17g", theta, rot, factor, low, high, original));
    });
    r.add_part_kind("yarn_rotary", [](const Json& j, const BuildContext&) -> std::unique_ptr<Part> {
        const int head_dim = (int)j.get("head_dim").as_int();
        const int rot = (int)j.get_int("rotary_dim", head_dim);
        const double theta = j.get("theta").as_double(), factor = j.get("factor").as_double();
        const double original = j.get("original").as_double(), fast = j.get("fast").as_double(), slow = j.get("slow").as_double();
        if (rot % 2 || rot <= 0 || rot > head_dim)
            fail(KIPP_E_CONFIG, format("rotary_dim %d must be even, positive and at most head_dim %d", rot, head_dim));
        if (!(theta > 0) || theta == 1.0 || !(factor > 0) || !(original > 0) || !(fast > 0) || !(slow > 0))
            fail(KIPP_E_CONFIG, "yarn_rotary: theta (not 1), factor, original, fast and slow must be positive");
        return std::make_unique<FrequencyTable>(yarn_frequencies(rot, theta, factor, original, fast, slow),
                                                format("yarn/%.17g/%d/%.17g/%.17g/%.17g/%.17g", theta, rot, factor, original, fast, slow),
                                                yarn_magnitude(factor));
    });
    r.add_part_kind("gated_mlp", [](const Json& j, const BuildContext&) -> std::unique_ptr<Part> {
        return std::make_unique<GatedFeedForward>(j);
    });
    r.add_part_kind("hyper_connection_block", [](const Json& j, const BuildContext& ctx) -> std::unique_ptr<Part> {
        const Registry& reg = Registry::get();
        const Json* n2 = j.find("post_norm");
        const Json* ff = j.find("ffn");
        const bool has_ffn = ff != nullptr && !ff->is_null();
        if (has_ffn && (n2 == nullptr || n2->is_null())) fail(KIPP_E_CONFIG, "hyper_connection_block: a feed-forward needs its post_norm");
        return std::make_unique<HyperConnectionBlock>(
            j, reg.make_as<Norm>(j.get("input_norm"), ctx, "a norm"), reg.make_as<Mixer>(j.get("mixer"), ctx, "a mixer"),
            has_ffn ? reg.make_as<Norm>(*n2, ctx, "a norm") : nullptr,
            has_ffn ? reg.make_as<FeedForward>(*ff, ctx, "a feed-forward") : nullptr);
    });
    r.add_part_kind("dense_mlp", [](const Json& j, const BuildContext&) -> std::unique_ptr<Part> {
        return std::make_unique<DenseFeedForward>((int)j.get("hidden_size").as_int(), (int)j.get("intermediate_size").as_int(),
                                                  j.get_string("activation", "relu_squared"),
                                                  tensor_names(j, {{"up", "up"}, {"down", "down"}}));
    });
    r.add_part_kind("parallel_block", [](const Json& j, const BuildContext& ctx) -> std::unique_ptr<Part> {
        const Registry& reg = Registry::get();
        std::vector<std::string> names;
        for (auto& n : j.get("names").items()) names.push_back(n.as_string());
        const Json* ff = j.find("ffn");
        return std::make_unique<ParallelBlock>(reg.make_as<Norm>(j.get("norm"), ctx, "a norm"),
                                               reg.make_as<Mixer>(j.get("mixer"), ctx, "a mixer"),
                                               ff && !ff->is_null() ? reg.make_as<FeedForward>(*ff, ctx, "a feed-forward") : nullptr,
                                               names);
    });
    r.add_part_kind("rotary", [](const Json& j, const BuildContext&) -> std::unique_ptr<Part> {
        const int head_dim = (int)j.get("head_dim").as_int();
        const int rot = (int)j.get_int("rotary_dim", head_dim);
        const double theta = j.get("theta").as_double();
        if (rot % 2 || rot < 0 || rot > head_dim)
            fail(KIPP_E_CONFIG, format("rotary_dim %d must be even and at most head_dim %d", rot, head_dim));
        if (!(theta > 0)) fail(KIPP_E_CONFIG, "rotary: theta must be positive");
        const bool exact = j.get_bool("exact_exponent", false);
        return std::make_unique<FrequencyTable>(rotary_frequencies(rot, theta, exact),
                                                format("rotary/%.17g/%d%s", exact ? theta : (double)(float)theta, rot,
                                                       exact ? "/exact" : ""));
    });
    r.add_part_kind("frequency_table", [](const Json& j, const BuildContext&) -> std::unique_ptr<Part> {
        std::vector<float> f;
        for (auto& v : j.get("inv_freq").items()) f.push_back((float)v.as_double());
        return std::make_unique<FrequencyTable>(std::move(f), j.get("key").as_string());
    });
    r.add_part_kind("no_position", [](const Json&, const BuildContext&) -> std::unique_ptr<Part> {
        return std::make_unique<FrequencyTable>(std::vector<float>{}, "none");
    });
    r.add_part_kind("attention", [](const Json& j, const BuildContext& ctx) -> std::unique_ptr<Part> {
        std::optional<double> eps, scale;
        if (const Json* e = j.find("qk_norm_eps"); e && !e->is_null()) eps = e->as_double();
        if (const Json* s = j.find("scale"); s && !s->is_null()) scale = s->as_double();
        AttentionOptions options;
        options.value_dim = (int)j.get_int("value_dim", 0);
        options.keep_first = (int)j.get_int("keep_first", 0);
        options.head_mix = j.get_bool("head_mix", false);
        options.output_scale = j.get_double("output_scale", 1.0);
        options.bias = j.get_bool("bias", false);
        options.score_maps = (int)j.get_int("score_maps", 1);
        options.combine_maps = j.get_bool("combine_maps", false);
        options.lambda_init = j.get_double("lambda_init", 0.0);
        options.combine_eps = j.get_double("combine_eps", 1e-5);
        options.norm_whole = j.get_bool("norm_whole", false);
        options.interleaved = j.get_bool("interleaved", false);
        options.chunk = (int)j.get_int("chunk", 0);
        const std::string sink = j.get_string("sink", "none");
        if (sink != "none" && sink != "learned" && sink != "unit")
            fail(KIPP_E_CONFIG, "attention: sink must be none, learned or unit, not '" + sink + "'");
        options.sink = sink == "learned" ? 1 : sink == "unit" ? 2 : 0;
        options.head_gate = j.get_bool("head_gate", false);
        options.values_are_keys = j.get_bool("values_are_keys", false);
        options.shared_kv = j.get_bool("shared_kv", false);
        options.softcap = j.get_double("softcap", 0.0);
        options.names = tensor_names(j, options.names);
        return std::make_unique<AttentionMixer>(
            (int)j.get("hidden_size").as_int(), (int)j.get("num_heads").as_int(), (int)j.get("num_kv_heads").as_int(),
            (int)j.get("head_dim").as_int(), make_position(j.get("position"), ctx), eps, (int)j.get_int("window", 0),
            scale, std::move(options));
    });
    r.add_part_kind("swiglu", [](const Json& j, const BuildContext&) -> std::unique_ptr<Part> {
        return std::make_unique<SwiGLUFeedForward>((int)j.get("hidden_size").as_int(),
                                                   (int)j.get("intermediate_size").as_int());
    });
    r.add_part_kind("pre_norm_block", [](const Json& j, const BuildContext& ctx) -> std::unique_ptr<Part> {
        const Registry& reg = Registry::get();
        std::vector<std::string> names;
        for (auto& n : j.get("names").items()) names.push_back(n.as_string());
        const Json* n2 = j.find("post_norm");
        const Json* ff = j.find("ffn");
        const bool has_ffn = ff != nullptr && !ff->is_null();
        if (has_ffn && (n2 == nullptr || n2->is_null())) fail(KIPP_E_CONFIG, "pre_norm_block: a feed-forward needs its post_norm");
        return std::make_unique<PreNormBlock>(
            reg.make_as<Norm>(j.get("input_norm"), ctx, "a norm"), reg.make_as<Mixer>(j.get("mixer"), ctx, "a mixer"),
            has_ffn ? reg.make_as<Norm>(*n2, ctx, "a norm") : nullptr,
            has_ffn ? reg.make_as<FeedForward>(*ff, ctx, "a feed-forward") : nullptr, names);
    });
    r.add_part_kind("output_norm_block", [](const Json& j, const BuildContext& ctx) -> std::unique_ptr<Part> {
        const Registry& reg = Registry::get();
        std::vector<std::string> names;
        for (auto& n : j.get("names").items()) names.push_back(n.as_string());
        const Json* n2 = j.find("post_norm");
        const Json* ff = j.find("ffn");
        const bool has_ffn = ff != nullptr && !ff->is_null();
        if (has_ffn && (n2 == nullptr || n2->is_null())) fail(KIPP_E_CONFIG, "output_norm_block: a feed-forward needs its post_norm");
        return std::make_unique<OutputNormBlock>(
            reg.make_as<Norm>(j.get("mixer_norm"), ctx, "a norm"), reg.make_as<Mixer>(j.get("mixer"), ctx, "a mixer"),
            has_ffn ? reg.make_as<Norm>(*n2, ctx, "a norm") : nullptr,
            has_ffn ? reg.make_as<FeedForward>(*ff, ctx, "a feed-forward") : nullptr, j.get_double("residual_mult", 1.0),
            names);
    });
    register_recurrent_parts(r);
    register_latent_parts(r);
    register_expert_parts(r);
    r.add_part_kind("external", [](const Json& j, const BuildContext& ctx) -> std::unique_ptr<Part> {
        const std::string role = j.get("role").as_string();
        if (role == "mixer") return std::make_unique<ExternalMixer>(j, ctx);
        if (role == "feed_forward") return std::make_unique<ExternalFeedForward>(j, ctx);
        if (role == "embedding") return std::make_unique<ExternalEmbeddingStage>(j, ctx);
        if (role == "norm") return std::make_unique<ExternalNorm>(j, ctx);
        fail(KIPP_E_CONFIG, "external part: role must be mixer, feed_forward, embedding or norm, not '" + role + "'");
    });
}

}  // namespace kipp
