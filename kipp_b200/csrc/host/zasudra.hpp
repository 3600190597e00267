// Zasudra: a decoder whose layers are listed one by one in its config.json, each with one of
// three mixers and a feed-forward of routed experts (or none).
//
//   attention     grouped-query attention whose values are the keys as projected (no W_v); an RMS
//                 norm over the whole q and the whole k projection; an interleaved rotation of the
//                 first dims of every head; blocks of positions as the mask (a query sees the
//                 earlier keys of its own block); a learned sink per head in the softmax's denominator
//   attention_2   grouped-query attention with W_v, the same whole-projection norms, no rotation,
//                 the causal mask, a sink of score 0 and a sigmoid gate per head; with 'kv_from': j
//                 the layer has no keys and values of its own and reads what layer j cached
//   wkv           time mixing with a per-token decay (recurrent_parts.hpp)
//
// The token embedding is joined by a table addressed by a hash of the token pair.  A layer is
// x <- x + m norm1(mixer(x)), x <- x + m norm2(ff(x)): the norm sits on the sublayer's output
// (output_norm_block).  Then the model's norm, the output head and a scale on the logits.
//
// config.json keys: architecture, vocab, width, norm.eps, residual_mult, logit_scale,
// embedding.bigram.{buckets, mul_prev, mul_cur}, layers[i].{type, mixer, mlp}.
// Tensor names: embed, bigram, l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.*, final.norm, head.
#pragma once
#include "varunex.hpp"

namespace kipp {
namespace zasudra {

using venizen::need;
using venizen::need_int;
using venizen::need_number;

inline double optional_number(const Json& o, const char* key, const std::string& where, double fallback) {
    const Json* v = o.find(key);
    return v && !v->is_null() ? need_number(o, key, where) : fallback;
}

// The keys after checks; every size and constant a model of this design can choose is kept.
inline Json normalize(const Json& c) {
    if (!c.is_object()) fail(KIPP_E_CONFIG, "config.json must hold a JSON object");
    Json out = Json::object();
    out.set("architecture", architecture_of(c));
    out.set("vocab", need_int(c, "vocab", ""));
    out.set("width", need_int(c, "width", ""));
    const double eps = need_number(need(c, "norm", ""), "eps", "norm.");
    if (!(eps > 0)) fail(KIPP_E_CONFIG, "norm.eps must be positive");
    Json norm = Json::object();
    norm.set("eps", eps);
    out.set("norm", std::move(norm));
    out.set("residual_mult", optional_number(c, "residual_mult", "", 1.0));
    out.set("logit_scale", optional_number(c, "logit_scale", "", 1.0));
    // the hashed pair table is there when the configuration names it
    Json embedding = Json::object();
    const Json* emb = c.find("embedding");
    const Json* bigram = emb && emb->is_object() ? emb->find("bigram") : nullptr;
    if (bigram && !bigram->is_null()) {
        Json b = Json::object();
        b.set("buckets", need_int(*bigram, "buckets", "embedding.bigram."));
        b.set("mul_prev", need_int(*bigram, "mul_prev", "embedding.bigram.", 0));
        b.set("mul_cur", need_int(*bigram, "mul_cur", "embedding.bigram.", 0));
        embedding.set("bigram", std::move(b));
    } else {
        embedding.set("bigram", nullptr);
    }
    out.set("embedding", std::move(embedding));

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
        if (kind == "attention" || kind == "attention_2") {
            const long long heads = need_int(mx, "heads", wm), kv = need_int(mx, "kv_heads", wm);
            const long long dim = need_int(mx, "dim", wm);
            if (heads % kv) fail(KIPP_E_CONFIG, "config key '" + wm + "heads' must be a multiple of kv_heads");
            const long long vdim = mx.has("vdim") && !mx.get("vdim").is_null() ? need_int(mx, "vdim", wm) : dim;
            if (kind == "attention" && vdim != dim)
                fail(KIPP_E_CONFIG, "config key '" + wm + "vdim' must equal dim where the values are the keys");
            mixer.set("heads", heads);
            mixer.set("kv_heads", kv);
            mixer.set("dim", dim);
            mixer.set("vdim", vdim);
            mixer.set("scale", need_number(mx, "scale", wm));
            mixer.set("rot", venizen::rotation(mx, dim, wm));
            long long chunk = 0;
            if (const Json* m = mx.find("mask"); m && !m->is_null()) chunk = need_int(*m, "size", wm + "mask.");
            Json mask = Json::object();
            mask.set("size", chunk);                     // 0: every earlier token is seen
            mixer.set("mask", std::move(mask));
            if (const Json* from = mx.find("kv_from"); from && !from->is_null()) {
                const long long j = need_int(mx, "kv_from", wm, 0);
                if (j >= (long long)i) fail(KIPP_E_CONFIG, "config key '" + wm + "kv_from' must name an earlier layer");
                mixer.set("kv_from", j);
            } else {
                mixer.set("kv_from", nullptr);
            }
        } else if (kind == "wkv") {
            mixer.set("heads", need_int(mx, "heads", wm));
            mixer.set("dim", need_int(mx, "dim", wm));
            // the width of the decay's bottleneck is the shape of its tensors unless a key gives it
            // (the random-weights writer needs it)
            if (const Json* r = mx.find("decay_rank"); r && !r->is_null())
                mixer.set("decay_rank", need_int(mx, "decay_rank", wm));
        } else {
            fail(KIPP_E_CONFIG, "unknown layer type '" + kind + "' (attention, attention_2, wkv)");
        }
        layer.set("mixer", std::move(mixer));
        const Json* mlp = l.find("mlp");
        if (mlp && !mlp->is_null()) {
            const std::string wf = where + "mlp.";
            const std::string fk = mlp->get_string("kind", "moe");
            if (fk != "moe") fail(KIPP_E_CONFIG, "feed-forward kind '" + fk + "' is not supported (moe)");
            const Json& router = need(*mlp, "router", wf);
            Json f = Json::object(), e = Json::object(), r = Json::object();
            e.set("ff", need_int(need(*mlp, "expert", wf), "ff", wf + "expert."));
            const long long experts = need_int(router, "experts", wf + "router."), top = need_int(router, "top", wf + "router.");
            if (top > experts) fail(KIPP_E_CONFIG, "config key '" + wf + "router.top' must not exceed the number of experts");
            r.set("experts", experts);
            r.set("top", top);
            f.set("kind", fk);
            f.set("expert", std::move(e));
            f.set("router", std::move(r));
            layer.set("mlp", std::move(f));
        } else {
            layer.set("mlp", nullptr);
        }
        ls.push(std::move(layer));
    }
    // a layer that borrows keys and values: the lender has its own, of the same form
    for (size_t i = 0; i < ls.size(); ++i) {
        const Json& mx = ls.at(i).get("mixer");
        const Json* from = mx.find("kv_from");
        if (!from || from->is_null()) continue;
        const Json& other = ls.at((size_t)from->as_int());
        const std::string where = format("layers[%zu].mixer.kv_from", i);
        const std::string t = other.get("type").as_string();
        if (t != "attention" && t != "attention_2") fail(KIPP_E_CONFIG, "config key '" + where + "' must name an attention layer");
        const Json& om = other.get("mixer");
        if (!om.get("kv_from").is_null()) fail(KIPP_E_CONFIG, "config key '" + where + "' must name a layer with keys of its own");
        for (const char* key : {"kv_heads", "dim", "vdim"})
            if (om.get(key).as_int() != mx.get(key).as_int())
                fail(KIPP_E_CONFIG, "config key '" + where + "': the two layers differ in '" + key + "'");
    }
    out.set("layers", std::move(ls));
    return out;
}

inline Json plan(const Json& c) {
    const long long width = c.get("width").as_int(), vocab = c.get("vocab").as_int();
    const double eps = c.get("norm").get("eps").as_double();
    Json p = Json::object();
    p.set("hidden_size", width);
    p.set("vocab_size", vocab);
    p.set("max_positions", 0LL);
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
    if (const Json& b = c.get("embedding").get("bigram"); !b.is_null()) {
        Json pair = Json::object();
        pair.set("kind", "hashed_pair_embedding");
        pair.set("vocab_size", vocab);
        pair.set("hidden_size", width);
        pair.set("buckets", b.get("buckets").as_int());
        pair.set("mul_prev", b.get("mul_prev").as_int());
        pair.set("mul_cur", b.get("mul_cur").as_int());
        pair.set("weight_name", "bigram");
        Json stage = Json::object();
        stage.set("prefix", "");
        stage.set("part", std::move(pair));
        stages.push(std::move(stage));
    }
    p.set("embedding", std::move(stages));

    Json blocks = Json::array(), order = Json::array();
    const Json& layers = c.get("layers");
    for (size_t i = 0; i < layers.size(); ++i) {
        const Json& l = layers.at(i);
        const Json& mx = l.get("mixer");
        const std::string type = l.get("type").as_string();
        Json mixer = Json::object();
        long long cache = (long long)i;
        bool writes = true;
        if (type == "wkv") {
            mixer.set("kind", "wkv");
            mixer.set("hidden_size", width);
            mixer.set("num_heads", mx.get("heads").as_int());
            mixer.set("head_dim", mx.get("dim").as_int());
            mixer.set("decay_rank", mx.get_int("decay_rank", 0));
            mixer.set("eps", eps);
            mixer.set("gate", "silu");
        } else {
            const bool second = type == "attention_2";
            const bool borrows = !mx.get("kv_from").is_null();
            mixer.set("kind", "attention");
            mixer.set("hidden_size", width);
            mixer.set("num_heads", mx.get("heads").as_int());
            mixer.set("num_kv_heads", mx.get("kv_heads").as_int());
            mixer.set("head_dim", mx.get("dim").as_int());
            mixer.set("value_dim", mx.get("vdim").as_int());
            mixer.set("position", venizen::rotary_part(mx.get("rot"), mx.get("dim").as_int()));
            mixer.set("qk_norm_eps", eps);
            mixer.set("scale", mx.get("scale").as_double());
            mixer.set("norm_whole", true);
            mixer.set("interleaved", true);
            mixer.set("chunk", mx.get("mask").get("size").as_int());
            mixer.set("sink", second ? "unit" : "learned");
            mixer.set("head_gate", second);
            mixer.set("values_are_keys", !second);
            mixer.set("shared_kv", borrows);
            mixer.set("names", venizen::names_of({{"q", "q"}, {"k", "k"}, {"v", "v"}, {"o", "o"}, {"q_norm", "q.norm"},
                                                  {"k_norm", "k.norm"}, {"sink", "sink"}, {"gate", "g"}}));
            if (borrows) {
                cache = mx.get("kv_from").as_int();
                writes = false;
            }
        }
        Json block = Json::object();
        block.set("kind", "output_norm_block");
        Json names = Json::array();
        for (const char* n : {"", "mix.", "", "mlp."}) names.push(n);
        block.set("names", std::move(names));
        block.set("residual_mult", c.get("residual_mult").as_double());
        block.set("mixer_norm", venizen::rmsnorm_part(width, eps, "norm1"));
        block.set("mixer", std::move(mixer));
        if (!l.get("mlp").is_null()) {
            const Json& f = l.get("mlp");
            Json ffn = Json::object();
            ffn.set("kind", "expert_mixture");
            ffn.set("hidden_size", width);
            ffn.set("intermediate_size", f.get("expert").get("ff").as_int());
            ffn.set("experts", f.get("router").get("experts").as_int());
            ffn.set("top", f.get("router").get("top").as_int());
            ffn.set("activation", "relu_squared");
            ffn.set("router_bias", true);
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
        Json run = Json::object();
        run.set("layer", (long long)i);
        run.set("cache", cache);
        run.set("writes_cache", writes);
        order.push(std::move(run));
    }
    p.set("layers", std::move(blocks));
    p.set("order", std::move(order));

    Json fn = Json::object();
    fn.set("prefix", "");
    fn.set("part", venizen::rmsnorm_part(width, eps, "final.norm"));
    p.set("final_norm", std::move(fn));
    Json head = Json::object();
    head.set("kind", "output_head");
    head.set("vocab_size", vocab);
    head.set("hidden_size", width);
    head.set("tied_to", nullptr);
    head.set("weight_name", "head");
    head.set("logit_scale", c.get("logit_scale").as_double());
    Json hd = Json::object();
    hd.set("prefix", "");
    hd.set("part", std::move(head));
    p.set("head", std::move(hd));
    return p;
}

}  // namespace zasudra

inline void register_zasudra() {
    Registry::get().add_architecture("Zasudra", Architecture{zasudra::normalize, zasudra::plan});
}

}  // namespace kipp
