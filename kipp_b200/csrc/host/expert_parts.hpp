// A feed-forward made of many small experts of which every token uses a few.
//
//   expert_mixture   z = W_router h + b in float32; the `top` largest logits are chosen and their
//                    weights are the softmax over the chosen logits only; the output is the weighted
//                    sum of the chosen experts' W_down act(W_up h)
//
// Sizes, the number of experts and of choices, the activation and every tensor name are parameters
// of the plan.  The routing happens on the device (moe.cu): a step's launches do not depend on which
// experts its tokens chose, so a captured graph replays them.
#pragma once
#include "recurrent_parts.hpp"

namespace kipp {

class ExpertMixture : public FeedForward {
public:
    ExpertMixture(const Json& j, const BuildContext&) {
        hidden_ = (int)j.get("hidden_size").as_int();
        inter_ = (int)j.get("intermediate_size").as_int();
        experts_ = (int)j.get("experts").as_int();
        top_ = (int)j.get("top").as_int();
        act_ = activation_code(j.get_string("activation", "relu_squared"));
        router_bias_ = j.get_bool("router_bias", true);
        expert_prefix_ = j.get_string("expert_prefix", "e");        // expert i's tensors: <prefix><i>.<up|down>
        names_ = tensor_names(j, {{"up", "up"}, {"down", "down"}, {"router", "router"}, {"router_bias", "router.b"}});
        if (hidden_ <= 0 || inter_ <= 0 || experts_ <= 0) fail(KIPP_E_CONFIG, "expert_mixture: sizes must be positive");
        if (top_ <= 0 || top_ > experts_) fail(KIPP_E_CONFIG, "expert_mixture: top must lie between 1 and the number of experts");
        if (experts_ > 2048) fail(KIPP_E_UNSUPPORTED, "expert_mixture: at most 2048 experts");
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
            add(expert_name(e, "up"), {inter_, hidden_});
            add(expert_name(e, "down"), {hidden_, inter_});
        }
        add(names_.at("router"), {experts_, hidden_});
        if (router_bias_) add(names_.at("router_bias"), {experts_});
    }
    void bind(Binder& b, const std::string& p) override {
        dtype_ = b.compute_dtype();
        const size_t es = dtype_size(dtype_);
        // the experts' matrices one after another, so that a tile finds its expert's by an offset
        const size_t one = (size_t)inter_ * hidden_;
        w_up_ = b.allocate((size_t)experts_ * one * es, p + "experts up");
        w_down_ = b.allocate((size_t)experts_ * one * es, p + "experts down");
        for (int e = 0; e < experts_; ++e) {
            b.load(p + expert_name(e, "up"), static_cast<char*>(w_up_) + (size_t)e * one * es, dtype_, hidden_, inter_, hidden_);
            b.load(p + expert_name(e, "down"), static_cast<char*>(w_down_) + (size_t)e * one * es, dtype_, inter_, hidden_, inter_);
        }
        // the router works in float32
        router_ = load_f32_matrix(b, p + names_.at("router"), experts_, hidden_);
        if (router_bias_) bias_ = load_f32(b, p + names_.at("router_bias"), experts_);
    }
    // bytes one step reads at most: every expert's matrices (a step of few tokens reads top per token)
    size_t weight_bytes() const override {
        return (size_t)2 * experts_ * inter_ * hidden_ * dtype_size(dtype_) + (size_t)experts_ * (hidden_ + 1) * 4;
    }
    void forward(StepContext& ctx, const void* h, float* residual) override {
        const int T = ctx.tokens(), pairs = T * top_;
        Ops& ops = *ctx.ops;
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
            ops.moe_route(expert_of, weight_of, h, hidden_, ctx.dtype, router_, bias_, T, hidden_, experts_, top_);
            ops.moe_padded_lists(place, tile_expert, n_tiles, expert_of, pairs, experts_, tile);
            ops.moe_gather_rows(in, h, hidden_, place, pairs, top_, hidden_);
            ops.gemm_grouped(act, ctx.dtype, inter_, in, hidden_, w_up_, rows_cap, inter_, hidden_, experts_, act_, tile_expert,
                             n_tiles, tile);
            ops.gemm_grouped(rows, F32, hidden_, act, inter_, w_down_, rows_cap, hidden_, inter_, experts_, -1, tile_expert,
                             n_tiles, tile);
            ops.moe_combine(residual, rows, weight_of, T, hidden_, top_, place);
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
        ops.moe_route(expert_of, weight_of, h, hidden_, ctx.dtype, router_, bias_, T, hidden_, experts_, top_);
        ops.moe_lists(sorted, tiles, n_tiles, expert_of, pairs, experts_);
        const long long one = (long long)inter_ * hidden_;
        // up: the rows of a tile are gathered from their tokens; the hidden rows lie in sorted order
        ops.moe_gemm(act, ctx.dtype, inter_, h, hidden_, w_up_, one, dtype_, inter_, hidden_, top_, true, false, act_, sorted,
                     tiles, n_tiles, pairs, experts_);
        // down: one float32 row per (token, choice) pair, at the pair's own place
        ops.moe_gemm(rows, F32, hidden_, act, inter_, w_down_, one, dtype_, hidden_, inter_, top_, false, true, -1, sorted,
                     tiles, n_tiles, pairs, experts_);
        ops.moe_combine(residual, rows, weight_of, T, hidden_, top_);
    }

private:
    static float* load_f32_matrix(Binder& b, const std::string& name, int64_t rows, int64_t cols) {
        float* d = static_cast<float*>(b.allocate((size_t)rows * cols * sizeof(float), name));
        b.load(name, d, F32, cols, rows, cols);
        return d;
    }
    int hidden_ = 0, inter_ = 0, experts_ = 0, top_ = 0, act_ = 0, dtype_ = BF16;
    bool router_bias_ = true;
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
