// A feed-forward made of many small experts of which every token uses a few.
//
//   expert_mixture   z = W_router h + b in float32; the `top` largest logits are chosen and their
//                    weights are the softmax over the chosen logits only; the output is the weighted
//                    sum of the chosen experts' W_down act(W_up h)
//
//
// Options: routing by scores (routing "scores": s = softmax(z) over all outputs of the router, the choice
// by s + a learned correction per output, the weights s of the chosen divided by their sum and times
// weight_scale); identity experts (identity n: the router has n more outputs whose expert hands the
// token's input on, without tensors); gated experts (gated: W_down (g sigmoid(alpha g) (u + 1)) with
// g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit)); a shared feed-forward (shared: any
// feed-forward part, under shared_prefix) that runs for every token and is added.
//
// Sizes, the number of experts and of choices, the activation and every tensor name are parameters
// of the plan.  The routing happens on the device (moe.cu): a step's launches do not depend on which
// experts its tokens chose, so a captured graph replays them.
#pragma once
#include "recurrent_parts.hpp"

namespace kipp {

class ExpertMixture : public FeedForward {
public:
    ExpertMixture(const Json& j, const BuildContext& ctx) {
        const std::string routing = j.get_string("routing", "chosen_softmax");
        if (routing != "chosen_softmax" && routing != "scores")
            fail(KIPP_E_CONFIG, "expert_mixture: routing must be chosen_softmax or scores, not '" + routing + "'");
        by_scores_ = routing == "scores";
        identity_ = (int)j.get_int("identity", 0);
        weight_scale_ = (float)j.get_double("weight_scale", 1.0);
        correction_ = j.get_bool("correction", false);
        gated_ = j.get_bool("gated", false);
        limit_ = (float)j.get_double("limit", 0.0);
        alpha_ = (float)j.get_double("alpha", 1.0);
        if (identity_ < 0 || limit_ < 0.f) fail(KIPP_E_CONFIG, "expert_mixture: identity and limit must not be negative");
        if ((identity_ > 0 || correction_) && !by_scores_)
            fail(KIPP_E_CONFIG, "expert_mixture: identity experts and a correction go with routing by scores");
        if (const Json* sh = j.find("shared"); sh && !sh->is_null()) {
            shared_ = Registry::get().make_as<FeedForward>(*sh, ctx, "a feed-forward");
            shared_prefix_ = j.get_string("shared_prefix", "shared.");
        }
        hidden_ = (int)j.get("hidden_size").as_int();
        inter_ = (int)j.get("intermediate_size").as_int();
        experts_ = (int)j.get("experts").as_int();
        top_ = (int)j.get("top").as_int();
        act_ = activation_code(j.get_string("activation", "relu_squared"));
        router_bias_ = j.get_bool("router_bias", !by_scores_);
        if (router_bias_ && by_scores_) fail(KIPP_E_CONFIG, "expert_mixture: routing by scores has a correction, not a bias");
        expert_prefix_ = j.get_string("expert_prefix", "e");        // expert i's tensors: <prefix><i>.<up|down>
        names_ = tensor_names(j, {{"up", "up"}, {"down", "down"}, {"gate", "gate"}, {"router", "router"},
                                  {"router_bias", "router.b"}, {"correction", "correction"}});
        if (hidden_ <= 0 || inter_ <= 0 || experts_ <= 0) fail(KIPP_E_CONFIG, "expert_mixture: sizes must be positive");
        outputs_ = experts_ + identity_;
        if (top_ <= 0 || top_ > outputs_) fail(KIPP_E_CONFIG, "expert_mixture: top must lie between 1 and the number of experts");
        if (outputs_ > 2048) fail(KIPP_E_UNSUPPORTED, "expert_mixture: at most 2048 experts");
        up_rows_ = gated_ ? 2 * inter_ : inter_;
    }
    std::string expert_name(int e, const char* role) const {
        return expert_prefix_ + std::to_string(e) + "." + names_.at(role);
    }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        auto add = [&](const std::string& name, std::vector<int64_t> shape) {
            TensorSpec s;
            s.name = p + name;
            s.shape = std::move(shape);
            out.push_back(s);
        };
        for (int e = 0; e < experts_; ++e) {
            if (gated_) add(expert_name(e, "gate"), {inter_, hidden_});
            add(expert_name(e, "up"), {inter_, hidden_});
            add(expert_name(e, "down"), {hidden_, inter_});
        }
        add(names_.at("router"), {outputs_, hidden_});
        if (router_bias_) add(names_.at("router_bias"), {experts_});
        if (correction_) add(names_.at("correction"), {outputs_});
        if (shared_) shared_->tensor_specs(p + shared_prefix_, out);
    }
    void bind(Binder& b, const std::string& p) override {
        dtype_ = b.compute_dtype();
        const size_t es = dtype_size(dtype_);
        // the experts' matrices one after another, so that a tile finds its expert's by an offset
        // (a gated expert: its gate's and its up projection's rows interleaved, gate_0, up_0, gate_1, ...)
        const size_t one = (size_t)inter_ * hidden_, first = (size_t)up_rows_ * hidden_;
        w_up_ = b.allocate((size_t)experts_ * first * es, p + "experts up");
        w_down_ = b.allocate((size_t)experts_ * one * es, p + "experts down");
        for (int e = 0; e < experts_; ++e) {
            char* up = static_cast<char*>(w_up_) + (size_t)e * first * es;
            if (gated_) {
                b.load(p + expert_name(e, "gate"), up, dtype_, 2 * (int64_t)hidden_, inter_, hidden_);
                b.load(p + expert_name(e, "up"), up + (size_t)hidden_ * es, dtype_, 2 * (int64_t)hidden_, inter_, hidden_);
            } else {
                b.load(p + expert_name(e, "up"), up, dtype_, hidden_, inter_, hidden_);
            }
            b.load(p + expert_name(e, "down"), static_cast<char*>(w_down_) + (size_t)e * one * es, dtype_, inter_, hidden_, inter_);
        }
        // the router works in float32
        router_ = load_f32_matrix(b, p + names_.at("router"), outputs_, hidden_);
        if (router_bias_) bias_ = load_f32(b, p + names_.at("router_bias"), experts_);
        if (correction_) bias_ = load_f32(b, p + names_.at("correction"), outputs_);
        if (shared_) shared_->bind(b, p + shared_prefix_);
    }
    // bytes one step reads at most: every expert's matrices (a step of few tokens reads top per token)
    size_t weight_bytes() const override {
        return (size_t)(up_rows_ + inter_) * experts_ * hidden_ * dtype_size(dtype_) + (size_t)outputs_ * (hidden_ + 1) * 4 +
               (shared_ ? shared_->weight_bytes() : 0);
    }
    bool graph_safe() const override { return !shared_ || shared_->graph_safe(); }
    // z, the choice and the weights (float32); identity experts get negative ids
    void route(StepContext& ctx, int* expert_of, float* weight_of, const void* h, int T) {
        if (by_scores_)
            ctx.ops->moe_route_scores(expert_of, weight_of, h, hidden_, ctx.dtype, router_, bias_, T, hidden_, outputs_, experts_,
                                      top_, weight_scale_);
        else
            ctx.ops->moe_route(expert_of, weight_of, h, hidden_, ctx.dtype, router_, bias_, T, hidden_, experts_, top_);
    }
    void combine(StepContext& ctx, float* residual, const float* rows, const float* weight_of, const int* expert_of,
                 const void* h, int T, const int* place) {
        if (identity_ > 0)
            ctx.ops->moe_combine_identity(residual, rows, weight_of, expert_of, h, hidden_, ctx.dtype, T, hidden_, top_, place);
        else
            ctx.ops->moe_combine(residual, rows, weight_of, T, hidden_, top_, place);
    }
    void forward(StepContext& ctx, const void* h, float* residual) override {
        const int T = ctx.tokens(), pairs = T * top_;
        Ops& ops = *ctx.ops;
        if (shared_) {
            // the shared feed-forward reads the same input without a norm of its own to fold
            const RowScale keep = ctx.input_scale;
            const RmsNormSpec* emit = ctx.emit_for;
            ctx.emit_for = nullptr;
            shared_->forward(ctx, h, residual);
            ctx.input_scale = keep;
            ctx.emit_for = emit;
            ctx.emitted = false;
        }
        if (ops.moe_tensor_core && ctx.dtype == dtype_ && Ops::moe_grouped_ok(dtype_, hidden_, inter_)) {
            // bfloat16: the pairs' rows sorted by expert and padded to whole tiles, each projection
            // ONE grouped product on the tcgen05 kernels (tiles of 128 rows for prompt-sized steps,
            // of 16 for few tokens)
            const int tile = Ops::grouped_tile_rows(T, pairs, experts_);
            const int cap = Ops::moe_max_padded_tiles(pairs, experts_, tile), rows_cap = cap * tile;
            int* expert_of = ctx.workspace->get<int>("moe_expert_of", (size_t)pairs);
            float* weight_of = ctx.workspace->get<float>("moe_weight_of", (size_t)pairs);
            int* place = ctx.workspace->get<int>("moe_place_of_pair", (size_t)pairs);
            int* tile_expert = ctx.workspace->get<int>("moe_expert_of_tile", (size_t)cap + 1);
            int* n_tiles = tile_expert + cap;
            void* in = ctx.workspace->buffer("moe_input_rows", (size_t)rows_cap * hidden_ * ctx.element());
            void* act = ctx.workspace->buffer("moe_hidden_rows", (size_t)rows_cap * inter_ * ctx.element());
            float* rows = ctx.workspace->get<float>("moe_output_rows", (size_t)rows_cap * hidden_);
            route(ctx, expert_of, weight_of, h, T);
            ops.moe_padded_lists(place, tile_expert, n_tiles, expert_of, pairs, experts_, tile);
            ops.moe_gather_rows(in, h, hidden_, place, pairs, top_, hidden_);
            if (gated_) {                           // the gated activation in the grouped product's epilogue
                Ops::Glu glu;
                glu.alpha = alpha_;
                glu.limit = limit_;
                ops.gemm_grouped_glu(act, ctx.dtype, inter_, in, hidden_, w_up_, rows_cap, up_rows_, hidden_, experts_, glu,
                                     tile_expert, n_tiles, tile);
            } else {
                ops.gemm_grouped(act, ctx.dtype, inter_, in, hidden_, w_up_, rows_cap, inter_, hidden_, experts_, act_, tile_expert,
                                 n_tiles, tile);
            }
            ops.gemm_grouped(rows, F32, hidden_, act, inter_, w_down_, rows_cap, hidden_, inter_, experts_, -1, tile_expert,
                             n_tiles, tile);
            combine(ctx, residual, rows, weight_of, expert_of, h, T, place);
            return;
        }
        const int max_tiles = Ops::moe_max_tiles(pairs, experts_);
        int* expert_of = ctx.workspace->get<int>("moe_expert_of", (size_t)pairs);
        float* weight_of = ctx.workspace->get<float>("moe_weight_of", (size_t)pairs);
        int* sorted = ctx.workspace->get<int>("moe_sorted_pairs", (size_t)pairs);
        int* tiles = ctx.workspace->get<int>("moe_tiles", (size_t)3 * max_tiles + 1);
        int* n_tiles = tiles + (size_t)3 * max_tiles;
        void* act = ctx.workspace->buffer("moe_hidden", (size_t)pairs * inter_ * ctx.element());
        float* rows = ctx.workspace->get<float>("moe_rows", (size_t)pairs * hidden_);
        route(ctx, expert_of, weight_of, h, T);
        ops.moe_lists(sorted, tiles, n_tiles, expert_of, pairs, experts_);
        const long long one = (long long)inter_ * hidden_;
        // up: the rows of a tile are gathered from their tokens; the hidden rows lie in sorted order
        if (gated_) {
            void* both = ctx.workspace->buffer("moe_gate_up", (size_t)pairs * up_rows_ * ctx.element());
            ops.moe_gemm(both, ctx.dtype, up_rows_, h, hidden_, w_up_, (long long)up_rows_ * hidden_, dtype_, up_rows_, hidden_, top_,
                         true, false, -1, sorted, tiles, n_tiles, pairs, experts_);
            Ops::Glu glu;
            glu.alpha = alpha_;
            glu.limit = limit_;
            ops.glu_limited(act, inter_, both, up_rows_, ctx.dtype, pairs, inter_, glu);
        } else
        ops.moe_gemm(act, ctx.dtype, inter_, h, hidden_, w_up_, one, dtype_, inter_, hidden_, top_, true, false, act_, sorted,
                     tiles, n_tiles, pairs, experts_);
        // down: one float32 row per (token, choice) pair, at the pair's own place
        ops.moe_gemm(rows, F32, hidden_, act, inter_, w_down_, one, dtype_, hidden_, inter_, top_, false, true, -1, sorted,
                     tiles, n_tiles, pairs, experts_);
        combine(ctx, residual, rows, weight_of, expert_of, h, T, nullptr);
    }

private:
    static float* load_f32_matrix(Binder& b, const std::string& name, int64_t rows, int64_t cols) {
        float* d = static_cast<float*>(b.allocate((size_t)rows * cols * sizeof(float), name));
        b.load(name, d, F32, cols, rows, cols);
        return d;
    }
    int hidden_ = 0, inter_ = 0, experts_ = 0, top_ = 0, act_ = 0, dtype_ = BF16;
    int identity_ = 0, outputs_ = 0, up_rows_ = 0;
    bool router_bias_ = true, by_scores_ = false, correction_ = false, gated_ = false;
    float weight_scale_ = 1.f, limit_ = 0.f, alpha_ = 1.f;
    std::unique_ptr<FeedForward> shared_;
    std::string shared_prefix_;
    std::string expert_prefix_;
    std::map<std::string, std::string> names_;
    void *w_up_ = nullptr, *w_down_ = nullptr;
    float *router_ = nullptr, *bias_ = nullptr;
};

inline void register_expert_parts(Registry& r) {
    r.add_part_kind("expert_mixture", [](const Json& j, const BuildContext& ctx) -> std::unique_ptr<Part> {
        return std::make_unique<ExpertMixture>(j, ctx);
    });
}

}  // namespace kipp
