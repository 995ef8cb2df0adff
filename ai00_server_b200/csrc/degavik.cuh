// Degavik model family: sequential blocks with the norm on the sublayer's OUTPUT,
//     x += rms(Mixer(x)) * w1;    x += rms(FF(x)) * w2        (the sublayers read the residual itself; FF may be absent)
// mixers = retention (retention.cuh), gated delta rule behind short convolutions (delta_rule.cuh), or windowed softmax
// attention with kept first tokens, capped scores and mixed head weights over a paged cache (window_attn.cuh); feed-forward =
// one gated unit silu(g) * u, or routed experts (top logits, softmax over the chosen) plus an always-on shared expert
// (moe.cuh); a layer may use another layer's tensors with sequence memory of its own.  Every size and constant that can
// differ between models comes from config.json / the tensor shapes.  The family shares the sequence-model engine of the
// Kemirax family (kemirax.cuh: configuration structs, slot / page / snapshot plumbing); this file reads its configuration.
#pragma once

namespace b200 {

static KxConfig dg_parse_config(const JVal& root) {
    KxConfig c;
    c.family = KX_FAMILY_DEGAVIK;
    c.vocab = root.integer("vocab");
    c.width = root.integer("width");
    c.eps = (float)root.at("norm").number("eps");
    const JVal& ls = root.at("layers");
    REQUIRE(ls.kind == JVal::ARR && !ls.arr.empty(), B200RWKV_ERR_INVALID, "config: layers");
    for (const JVal& l : ls.arr) {
        KxLayerCfg k;
        REQUIRE(l.kind == JVal::OBJ && l.has("type") && l.at("type").kind == JVal::STR, B200RWKV_ERR_INVALID, "config: layer without a type");
        const std::string type = l.at("type").str;
        const JVal& m = l.at("mixer");
        k.heads = m.integer("heads"); k.dim = m.integer("dim"); k.vdim = m.integer("vdim");
        k.kv_heads = m.has("kv_heads") ? m.integer("kv_heads") : k.heads;
        if (l.has("weights_of")) k.weights_of = l.integer("weights_of");
        auto rot = [&]() {
            const JVal& r = m.at("rot");
            k.rot.dims = r.integer("dims"); k.rot.base = r.number("base");
            REQUIRE(k.rot.dims % 2 == 0 && k.rot.dims <= k.dim, B200RWKV_ERR_INVALID, "config: rot.dims must be even and <= dim");
        };
        if (type == "retention") {
            k.mixer = KX_RETENTION;
            rot();
            const JVal& d = m.at("decay");
            REQUIRE(d.kind == JVal::ARR && (int)d.arr.size() == k.heads, B200RWKV_ERR_INVALID, "config: decay must list one number per head");
            for (const JVal& v : d.arr) {
                REQUIRE(v.kind == JVal::NUM, B200RWKV_ERR_INVALID, "config: decay entries must be numbers");
                k.decay.push_back(v.num);
            }
        } else if (type == "channel_delta") {
            k.mixer = KX_DELTA;
            k.taps = m.integer("conv");
            REQUIRE(k.taps >= 1, B200RWKV_ERR_INVALID, "config: conv must be >= 1");
        } else if (type == "attention") {
            k.mixer = KX_WINDOW;
            rot();
            k.scale = (float)m.number("scale");
            k.softcap = m.has("softcap") ? (float)m.number("softcap") : 0.f;
            const JVal& mk = m.at("mask");
            k.window = mk.integer("size");
            k.keep_first = mk.has("keep_first") ? mk.integer("keep_first") : 0;
            REQUIRE(k.window >= 1, B200RWKV_ERR_INVALID, "config: mask.size must be >= 1");
        } else {
            throw Error(B200RWKV_ERR_UNSUPPORTED, "config: unknown layer type '" + type + "'");
        }
        REQUIRE(k.kv_heads >= 1 && k.heads % k.kv_heads == 0, B200RWKV_ERR_INVALID, "config: heads must be a multiple of kv_heads");
        if (l.has("mlp")) {
            const JVal& f = l.at("mlp");
            const std::string kind = f.at("kind").str;
            k.has_mlp = true;
            if (kind == "dense") {
                k.mlp_dense = true;
                k.ff = f.integer("ff");
            } else if (kind == "moe") {
                const JVal& r = f.at("router");
                k.experts = r.integer("experts"); k.top = r.integer("top");
                k.ff = f.at("expert").integer("ff");
                if (f.has("shared")) { k.has_shared = true; k.sff = f.at("shared").integer("ff"); }
            } else {
                throw Error(B200RWKV_ERR_UNSUPPORTED, "config: unknown mlp kind '" + kind + "'");
            }
        }
        c.layers.push_back(k);
    }
    const int nl = (int)c.layers.size();
    for (int i = 0; i < nl; ++i) {              // a named layer that itself names another: follow to the layer that owns the tensors
        int j = c.layers[i].weights_of;
        for (int hops = 0; j >= 0 && j < nl && c.layers[j].weights_of >= 0; ++hops) {
            REQUIRE(hops < nl, B200RWKV_ERR_INVALID, "config: weights_of forms a cycle");
            j = c.layers[j].weights_of;
        }
        if (c.layers[i].weights_of < 0) continue;
        REQUIRE(j >= 0 && j < nl && j != i, B200RWKV_ERR_INVALID, "config: weights_of must name a layer that has tensors of its own");
        REQUIRE(c.layers[j].mixer == c.layers[i].mixer, B200RWKV_ERR_INVALID, "config: weights_of names a layer of another type");
        c.layers[i].weights_of = j;
    }
    return c;
}

}  // namespace b200
