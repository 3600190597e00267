// Zunilorn: a decoder whose layers are listed one by one in its config.json, each with one of two
// mixers and a feed-forward (dense, a mixture of experts, or none), joined to a residual stream of
// several copies by hyper-connections.
//
//   mamba2      the selective state space layer in its matrix-state form (state_space,
//               recurrent_parts.hpp): a short causal convolution, a decay and a step size per head and
//               token, B and C shared by the heads of a group, a gate before a grouped norm
//   attention   grouped-query attention with value heads of their own size, a rotation of the first
//               dims of every head (pair i with i + dims/2) whose slow pairs may be stretched
//               (yarn_rotary), a cap on the scaled scores, a learned sink per head in the softmax's
//               denominator and a sigmoid gate per head read from the mixer's input
//
// Feed-forwards: gated with limits, g sigmoid(1.702 g) (u + 1) (gated_mlp), dense with biases, or as
// experts chosen by softmax scores plus a correction, with identity experts and a shared expert
// behind a sigmoid gate per token (expert_mixture).  A span of layers may run several times in a row,
// every pass with a cache and state of its own.  The logits come from the embedding table and are
// capped.
//
// config.json keys: architecture, vocab, width, norm.eps, residual_mult, streams, logit_softcap,
// loop.{start, stop, times}, layers[i].{type, mixer, mlp}.
// Tensor names: embed, l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.*, l<i>.hc1.*, l<i>.hc2.*, final.norm.
#pragma once
#include "zasudra.hpp"

namespace kipp {
namespace zunilorn {

using venizen::need;
using venizen::need_int;
using venizen::need_number;
using zasudra::optional_number;

constexpr double GLU_ALPHA = 1.702;       // the design's constant in g sigmoid(alpha g)

inline bool present(const Json& o, const char* key) {
    const Json* v = o.is_object() ? o.find(key) : nullptr;
    return v && !v->is_null();
}

// rot: {base, dims, scaling: {factor, original, fast, slow}}; absent or dims 0 = no rotation
inline Json rotation(const Json& mixer, long long dim, const std::string& where) {
    Json out = venizen::rotation(mixer, dim, where);
    out.set("scaling", nullptr);
    const Json* rot = mixer.find("rot");
    if (out.get("dims").as_int() == 0 || !rot || !present(*rot, "scaling")) return out;
    const Json& sc = rot->get("scaling");
    const std::string ws = where + "rot.scaling.";
    Json s = Json::object();
    for (const char* key : {"factor", "original", "fast", "slow"}) {
        const double v = need_number(sc, key, ws);
        if (!(v > 0)) fail(KIPP_E_CONFIG, "config key '" + ws + key + "' must be positive");
        s.set(key, v);
    }
    if (out.get("base").as_double() == 1.0) fail(KIPP_E_CONFIG, "config key '" + where + "rot.base' must not be 1 with a scaling");
    out.set("scaling", std::move(s));
    return out;
}

inline Json gated_sizes(const Json& o, const std::string& where) {
    Json f = Json::object();
    f.set("ff", need_int(o, "ff", where));
    const double limit = optional_number(o, "limit", where, 0.0);
    if (limit < 0) fail(KIPP_E_CONFIG, "config key '" + where + "limit' must not be negative");
    f.set("limit", limit);
    return f;
}

// The keys after checks; every size and constant a model of this design can choose is kept.
inline Json normalize(const Json& c) {
    if (!c.is_object()) fail(KIPP_E_CONFIG, "config.json must hold a JSON object");
    Json out = Json::object();
    out.set("architecture", architecture_of(c));
    out.set("vocab", need_int(c, "vocab", ""));
    const long long width = need_int(c, "width", "");
    out.set("width", width);
    const double eps = need_number(need(c, "norm", ""), "eps", "norm.");
    if (!(eps > 0)) fail(KIPP_E_CONFIG, "norm.eps must be positive");
    Json norm = Json::object();
    norm.set("eps", eps);
    out.set("norm", std::move(norm));
    out.set("residual_mult", optional_number(c, "residual_mult", "", 1.0));
    const double cap = optional_number(c, "logit_softcap", "", 0.0);
    if (cap < 0) fail(KIPP_E_CONFIG, "logit_softcap must not be negative");
    out.set("logit_softcap", cap);
    // streams absent: one stream without connection tensors (the plain residual sum)
    if (present(c, "streams")) out.set("streams", need_int(c, "streams", ""));
    else out.set("streams", nullptr);

    const Json& layers = need(c, "layers", "");
    if (!layers.is_array() || layers.size() == 0) fail(KIPP_E_CONFIG, "config key 'layers' must be a list of layers");
    Json ls = Json::array();
    for (size_t i = 0; i < layers.size(); ++i) {
        const Json& l = layers.at(i);
        const std::string where = format("layers[%zu].", i), wm = where + "mixer.";
        const Json& type = need(l, "type", where);
        if (!type.is_string()) fail(KIPP_E_CONFIG, "config key '" + where + "type' must be a string");
        const std::string kind = type.as_string();
        const Json& mx = need(l, "mixer", where);
        Json layer = Json::object(), mixer = Json::object();
        layer.set("type", kind);
        if (kind == "attention") {
            const long long heads = need_int(mx, "heads", wm);
            const long long kv = present(mx, "kv_heads") ? need_int(mx, "kv_heads", wm) : heads;
            const long long dim = need_int(mx, "dim", wm);
            if (heads % kv) fail(KIPP_E_CONFIG, "config key '" + wm + "heads' must be a multiple of kv_heads");
            mixer.set("heads", heads);
            mixer.set("kv_heads", kv);
            mixer.set("dim", dim);
            mixer.set("vdim", present(mx, "vdim") ? need_int(mx, "vdim", wm) : dim);
            mixer.set("scale", need_number(mx, "scale", wm));
            const double softcap = optional_number(mx, "softcap", wm, 0.0);
            if (softcap < 0) fail(KIPP_E_CONFIG, "config key '" + wm + "softcap' must not be negative");
            mixer.set("softcap", softcap);
            mixer.set("rot", rotation(mx, dim, wm));
        } else if (kind == "mamba2") {
            const long long heads = need_int(mx, "heads", wm), groups = present(mx, "groups") ? need_int(mx, "groups", wm) : 1;
            const long long vdim = need_int(mx, "vdim", wm);
            const long long parts = present(mx, "norm_groups") ? need_int(mx, "norm_groups", wm) : 1;
            if (heads % groups) fail(KIPP_E_CONFIG, "config key '" + wm + "heads' must be a multiple of groups");
            if ((heads * vdim) % parts) fail(KIPP_E_CONFIG, "config key '" + wm + "norm_groups' must divide heads * vdim");
            mixer.set("heads", heads);
            mixer.set("groups", groups);
            mixer.set("vdim", vdim);
            mixer.set("state", need_int(mx, "state", wm));
            mixer.set("conv", need_int(mx, "conv", wm));
            mixer.set("norm_groups", parts);
        } else {
            fail(KIPP_E_CONFIG, "unknown layer type '" + kind + "' (attention, mamba2)");
        }
        layer.set("mixer", std::move(mixer));
        const Json* mlp = l.find("mlp");
        if (mlp && !mlp->is_null()) {
            const std::string wf = where + "mlp.";
            const Json& fkind = need(*mlp, "kind", wf);
            const std::string fk = fkind.is_string() ? fkind.as_string() : "";
            Json f = Json::object();
            f.set("kind", fk);
            if (fk == "dense") {
                const Json sizes = gated_sizes(*mlp, wf);
                f.set("ff", sizes.get("ff").as_int());
                f.set("limit", sizes.get("limit").as_double());
            } else if (fk == "moe") {
                const Json& router = need(*mlp, "router", wf);
                const std::string wr = wf + "router.";
                Json r = Json::object();
                const long long experts = need_int(router, "experts", wr), top = need_int(router, "top", wr);
                const long long identity = present(router, "identity") ? need_int(router, "identity", wr, 0) : 0;
                if (top > experts + identity) fail(KIPP_E_CONFIG, "config key '" + wr + "top' must not exceed the router's outputs");
                r.set("experts", experts);
                r.set("identity", identity);
                r.set("top", top);
                r.set("scale", optional_number(router, "scale", wr, 1.0));
                f.set("router", std::move(r));
                f.set("expert", gated_sizes(need(*mlp, "expert", wf), wf + "expert."));
                if (present(*mlp, "shared")) f.set("shared", gated_sizes(mlp->get("shared"), wf + "shared."));
                else f.set("shared", nullptr);
            } else {
                fail(KIPP_E_CONFIG, "config key '" + wf + "kind' must be dense or moe");
            }
            layer.set("mlp", std::move(f));
        } else {
            layer.set("mlp", nullptr);
        }
        ls.push(std::move(layer));
    }
    // layers start .. stop-1 run `times` times in a row
    if (present(c, "loop")) {
        const Json& lp = c.get("loop");
        const long long start = need_int(lp, "start", "loop.", 0), stop = need_int(lp, "stop", "loop.", 0);
        const long long times = need_int(lp, "times", "loop.", 1);
        if (start > stop || stop > (long long)ls.size()) fail(KIPP_E_CONFIG, "loop.start .. loop.stop must be a span of the layers");
        Json loop = Json::object();
        loop.set("start", start);
        loop.set("stop", stop);
        loop.set("times", times);
        out.set("loop", std::move(loop));
    } else {
        out.set("loop", nullptr);
    }
    out.set("layers", std::move(ls));
    return out;
}

inline Json gated_part(long long width, const Json& sizes, bool bias, bool row_gate) {
    Json f = Json::object();
    f.set("kind", "gated_mlp");
    f.set("hidden_size", width);
    f.set("intermediate_size", sizes.get("ff").as_int());
    f.set("limit", sizes.get("limit").as_double());
    f.set("alpha", GLU_ALPHA);
    f.set("bias", bias);
    f.set("row_gate", row_gate);
    return f;
}

inline Json plan(const Json& c) {
    const long long width = c.get("width").as_int(), vocab = c.get("vocab").as_int();
    const double eps = c.get("norm").get("eps").as_double();
    const bool connections = !c.get("streams").is_null();
    const long long streams = connections ? c.get("streams").as_int() : 1;
    Json p = Json::object();
    p.set("hidden_size", width);
    p.set("vocab_size", vocab);
    p.set("max_positions", 0LL);
    p.set("streams", streams);
    p.set("config", c);
    Json stages = Json::array();
    {
        Json emb = Json::object();
        emb.set("kind", "token_embedding");
        emb.set("vocab_size", vocab);
        emb.set("hidden_size", width);
        emb.set("weight_name", "embed");
        Json stage = Json::object();
        stage.set("prefix", "");
        stage.set("part", std::move(emb));
        stages.push(std::move(stage));
    }
    p.set("embedding", std::move(stages));

    Json blocks = Json::array();
    const Json& layers = c.get("layers");
    for (size_t i = 0; i < layers.size(); ++i) {
        const Json& l = layers.at(i);
        const Json& mx = l.get("mixer");
        Json mixer = Json::object();
        if (l.get("type").as_string() == "mamba2") {
            mixer.set("kind", "state_space");
            mixer.set("hidden_size", width);
            mixer.set("num_heads", mx.get("heads").as_int());
            mixer.set("value_dim", mx.get("vdim").as_int());
            mixer.set("state_dim", mx.get("state").as_int());
            mixer.set("groups", mx.get("groups").as_int());
            mixer.set("conv", mx.get("conv").as_int());
            mixer.set("norm_groups", mx.get("norm_groups").as_int());
            mixer.set("eps", eps);
        } else {
            const Json& rot = mx.get("rot");
            Json position = venizen::rotary_part(rot, mx.get("dim").as_int());
            if (!rot.get("scaling").is_null()) {
                const Json& sc = rot.get("scaling");
                position = Json::object();
                position.set("kind", "yarn_rotary");
                position.set("head_dim", mx.get("dim").as_int());
                position.set("rotary_dim", rot.get("dims").as_int());
                position.set("theta", rot.get("base").as_double());
                for (const char* key : {"factor", "original", "fast", "slow"}) position.set(key, sc.get(key).as_double());
            }
            mixer.set("kind", "attention");
            mixer.set("hidden_size", width);
            mixer.set("num_heads", mx.get("heads").as_int());
            mixer.set("num_kv_heads", mx.get("kv_heads").as_int());
            mixer.set("head_dim", mx.get("dim").as_int());
            mixer.set("value_dim", mx.get("vdim").as_int());
            mixer.set("position", std::move(position));
            mixer.set("scale", mx.get("scale").as_double());
            mixer.set("softcap", mx.get("softcap").as_double());
            mixer.set("sink", "learned");
            mixer.set("head_gate", true);
            mixer.set("names", venizen::names_of({{"q", "q"}, {"k", "k"}, {"v", "v"}, {"o", "o"}, {"sink", "sink"}, {"gate", "g"}}));
        }
        Json block = Json::object();
        block.set("kind", "hyper_connection_block");
        Json names = Json::array();
        for (const char* n : {"", "mix.", "", "mlp.", "hc1.", "hc2."}) names.push(n);
        block.set("names", std::move(names));
        block.set("streams", streams);
        block.set("connections", connections);
        block.set("residual_mult", c.get("residual_mult").as_double());
        block.set("input_norm", venizen::rmsnorm_part(width, eps, "norm1"));
        block.set("mixer", std::move(mixer));
        const Json& f = l.get("mlp");
        if (!f.is_null()) {
            Json ffn;
            if (f.get("kind").as_string() == "dense") {
                ffn = gated_part(width, f, true, false);
            } else {
                const Json& r = f.get("router");
                ffn = Json::object();
                ffn.set("kind", "expert_mixture");
                ffn.set("hidden_size", width);
                ffn.set("intermediate_size", f.get("expert").get("ff").as_int());
                ffn.set("experts", r.get("experts").as_int());
                ffn.set("identity", r.get("identity").as_int());
                ffn.set("top", r.get("top").as_int());
                ffn.set("routing", "scores");
                ffn.set("correction", true);
                ffn.set("weight_scale", r.get("scale").as_double());
                ffn.set("gated", true);
                ffn.set("limit", f.get("expert").get("limit").as_double());
                ffn.set("alpha", GLU_ALPHA);
                if (!f.get("shared").is_null()) {
                    ffn.set("shared", gated_part(width, f.get("shared"), false, true));
                    ffn.set("shared_prefix", "shared.");
                }
            }
            block.set("post_norm", venizen::rmsnorm_part(width, eps, "norm2"));
            block.set("ffn", std::move(ffn));
        } else {
            block.set("post_norm", nullptr);
            block.set("ffn", nullptr);
        }
        Json layer = Json::object();
        layer.set("prefix", format("l%zu.", i));
        layer.set("part", std::move(block));
        blocks.push(std::move(layer));
    }
    p.set("layers", std::move(blocks));

    // every run has a cache id of its own: a layer that runs again has other pages and another state
    Json order = Json::array();
    long long cache = 0;
    auto run = [&](long long layer) {
        Json r = Json::object();
        r.set("layer", layer);
        r.set("cache", cache++);
        r.set("writes_cache", true);
        order.push(std::move(r));
    };
    const long long n = (long long)layers.size();
    const Json& loop = c.get("loop");
    const long long start = loop.is_null() ? n : loop.get("start").as_int(), stop = loop.is_null() ? n : loop.get("stop").as_int();
    const long long times = loop.is_null() ? 1 : loop.get("times").as_int();
    for (long long i = 0; i < start; ++i) run(i);
    for (long long k = 0; k < times; ++k)
        for (long long i = start; i < stop; ++i) run(i);
    for (long long i = stop; i < n; ++i) run(i);
    p.set("order", std::move(order));

    Json fn = Json::object();
    fn.set("prefix", "");
    fn.set("part", venizen::rmsnorm_part(width, eps, "final.norm"));
    p.set("final_norm", std::move(fn));
    Json head = Json::object();
    head.set("kind", "output_head");
    head.set("vocab_size", vocab);
    head.set("hidden_size", width);
    head.set("tied_to", "embed");
    head.set("weight_name", "head");
    head.set("logit_softcap", c.get("logit_softcap").as_double());
    Json hd = Json::object();
    hd.set("prefix", "");
    hd.set("part", std::move(head));
    p.set("head", std::move(hd));
    return p;
}

}  // namespace zunilorn

inline void register_zunilorn() {
    Registry::get().add_architecture("Zunilorn", Architecture{zunilorn::normalize, zunilorn::plan});
}

}  // namespace kipp
