// Sovezen: a decoder whose layers run attention over a low-rank latent of keys and values beside their
// feed-forward, both on one normed input.
//
// config.json (all sizes and every constant that differs between models come from it):
//   architecture  "Sovezen"
//   vocab, width, logit_scale
//   norm.eps
//   layers[i]     {type, mixer: {...}, mlp: {...} | null, weights_of: j | absent}
//     type "latent_attention"     mixer {heads, dim, rot_dim, vdim, kv_rank, scale, rot {dims, base}}: queries straight
//                                 from the input, each head [dim plain | rot_dim rotated]; one rotated key part for all
//                                 heads; a sink per head in the softmax
//     type "latent_attention_2"   mixer {heads, dim, vdim, kv_rank, q_rank, scale}: no positions, no sink; queries pass
//                                 a normed latent of q_rank entries
//     mlp {kind: "dense", ff}                                  down(silu(gate h) * (up h))
//         {kind: "moe", expert {ff}, router {experts, top}}    `top` of `experts` small feed-forwards down(relu(up h)^2),
//                                                              weighted by the softmax over the chosen router logits
//     weights_of j: the layer uses layer j's tensors (norm, mixer, feed-forward) with a cache of its own
//
// A layer is h = norm1(x); x += ls1 * mixer(h) + ls2 * ff(h), ls1 and ls2 a learned factor per channel.  The output
// is the final norm, the embedding table as the head, times logit_scale.
// Tensors: embed, final.norm, and per layer l<i>.norm1, l<i>.ls1, l<i>.ls2, l<i>.mix.{q | dq, dq.norm, uq}, dkv,
// dkv.norm, uk, uv, o, sink, l<i>.mlp.{gate, up, down | router, router.b, e<k>.up, e<k>.down}; linear weights [out, in].
//
// The typed configuration below checks the file; `describe` turns it into parts of parts_latent.cpp and
// parts_hybrid.cpp.  Nothing else in the engine knows this architecture.
#include <cmath>

#include "config.h"
#include "errors.h"

namespace sandy {

namespace {

[[noreturn]] void bad(const std::string& where, const std::string& what) { throw ConfigError("config.json: " + where + ": " + what); }

const Json& need(const Json& o, const std::string& where, const std::string& key) {
    const Json* v = o.is_object() ? o.find(key) : nullptr;
    if (!v || v->is_null()) bad(where, "required key '" + key + "' is missing");
    return *v;
}
int64_t need_int(const Json& o, const std::string& where, const std::string& key) {
    const Json& v = need(o, where, key);
    if (!v.is_int()) bad(where, "'" + key + "' must be int, got " + v.dump());
    return v.as_int();
}
double need_num(const Json& o, const std::string& where, const std::string& key) {
    const Json& v = need(o, where, key);
    if (!v.is_number()) bad(where, "'" + key + "' must be a number, got " + v.dump());
    return v.as_double();
}
const Json& need_obj(const Json& o, const std::string& where, const std::string& key) {
    const Json& v = need(o, where, key);
    if (!v.is_object()) bad(where, "'" + key + "' must be an object, got " + v.dump());
    return v;
}
const Json* maybe_obj(const Json& o, const std::string& where, const std::string& key) {
    const Json* v = o.find(key);
    if (!v || v->is_null()) return nullptr;
    if (!v->is_object()) bad(where, "'" + key + "' must be an object or null, got " + v->dump());
    return v;
}
void positive(int64_t v, const std::string& where, const std::string& key) {
    if (v <= 0) bad(where, "'" + key + "' must be > 0, got " + std::to_string(v));
}

constexpr const char* kWithRotation = "latent_attention";
constexpr const char* kWithQueryLatent = "latent_attention_2";

}  // namespace

SovezenConfig SovezenConfig::from_json(const Json& raw) {
    if (!raw.is_object()) throw ConfigError("config.json: top level must be a JSON object");
    SovezenConfig c;
    c.vocab = need_int(raw, "top level", "vocab");
    c.width = need_int(raw, "top level", "width");
    c.norm_eps = need_num(need_obj(raw, "top level", "norm"), "norm", "eps");
    c.logit_scale = need_num(raw, "top level", "logit_scale");
    const Json& layers = need(raw, "top level", "layers");
    if (!layers.is_array() || layers.size() == 0) bad("layers", "must be a non-empty list");
    int i = 0;
    for (const Json& lj : layers.items()) {
        const std::string at = "layers[" + std::to_string(i++) + "]";
        if (!lj.is_object()) bad(at, "must be an object");
        Layer l;
        const Json& type = need(lj, at, "type");
        if (!type.is_string()) bad(at, "'type' must be a string");
        l.type = type.as_string();
        const Json& m = need_obj(lj, at, "mixer");
        const std::string ma = at + ".mixer";
        if (l.type != kWithRotation && l.type != kWithQueryLatent)
            bad(at, "unknown layer type '" + l.type + "'; one of ['latent_attention', 'latent_attention_2']");
        l.heads = need_int(m, ma, "heads");
        l.dim = need_int(m, ma, "dim");
        l.vdim = need_int(m, ma, "vdim");
        l.kv_rank = need_int(m, ma, "kv_rank");
        l.scale = need_num(m, ma, "scale");
        if (l.type == kWithRotation) {
            l.rot_dim = need_int(m, ma, "rot_dim");
            const Json& rot = need_obj(m, ma, "rot");
            l.rot_dims = need_int(rot, ma + ".rot", "dims");
            l.rot_base = need_num(rot, ma + ".rot", "base");
        } else {
            l.q_rank = need_int(m, ma, "q_rank");
        }
        if (const Json* mlp = maybe_obj(lj, at, "mlp")) {
            const std::string fa = at + ".mlp";
            const Json& kind = need(*mlp, fa, "kind");
            if (!kind.is_string()) bad(fa, "'kind' must be a string");
            l.mlp = kind.as_string();
            if (l.mlp == "dense") {
                l.ff = need_int(*mlp, fa, "ff");
            } else if (l.mlp == "moe") {
                l.ff = need_int(need_obj(*mlp, fa, "expert"), fa + ".expert", "ff");
                const Json& router = need_obj(*mlp, fa, "router");
                l.experts = need_int(router, fa + ".router", "experts");
                l.top = need_int(router, fa + ".router", "top");
            } else {
                bad(fa, "'kind' must be 'dense' or 'moe', got " + kind.dump());
            }
        }
        if (const Json* of = lj.find("weights_of")) {
            if (!of->is_null()) {
                if (!of->is_int()) bad(at, "'weights_of' must be int, got " + of->dump());
                l.weights_of = of->as_int();
            }
        }
        c.layers.push_back(l);
    }
    return c;
}

Json SovezenConfig::to_json() const {
    Json j = Json::object();
    j["architecture"] = kArchitecture;
    Json ls = Json::array();
    for (const Layer& l : layers) {
        Json lj = Json::object();
        Json m = Json::object();
        m["dim"] = (long long)l.dim;
        m["heads"] = (long long)l.heads;
        m["kv_rank"] = (long long)l.kv_rank;
        if (l.type == kWithRotation) {
            Json rot = Json::object();
            rot["base"] = l.rot_base;
            rot["dims"] = (long long)l.rot_dims;
            m["rot"] = rot;
            m["rot_dim"] = (long long)l.rot_dim;
        } else {
            m["q_rank"] = (long long)l.q_rank;
        }
        m["scale"] = l.scale;
        m["vdim"] = (long long)l.vdim;
        lj["mixer"] = m;
        if (l.mlp == "dense") {
            Json mlp = Json::object();
            mlp["ff"] = (long long)l.ff;
            mlp["kind"] = "dense";
            lj["mlp"] = mlp;
        } else if (l.mlp == "moe") {
            Json mlp = Json::object(), expert = Json::object(), router = Json::object();
            expert["ff"] = (long long)l.ff;
            router["experts"] = (long long)l.experts;
            router["top"] = (long long)l.top;
            mlp["expert"] = expert;
            mlp["kind"] = "moe";
            mlp["router"] = router;
            lj["mlp"] = mlp;
        } else {
            lj["mlp"] = Json();
        }
        lj["type"] = l.type;
        if (l.weights_of >= 0) lj["weights_of"] = (long long)l.weights_of;
        ls.push(lj);
    }
    j["layers"] = ls;
    j["logit_scale"] = logit_scale;
    Json norm = Json::object();
    norm["eps"] = norm_eps;
    j["norm"] = norm;
    j["vocab"] = (long long)vocab;
    j["width"] = (long long)width;
    return j;
}

int SovezenConfig::owner(int layer) const {
    int at = layer;
    for (size_t hops = 0; hops <= layers.size(); hops++) {
        const int64_t next = layers.at((size_t)at).weights_of;
        if (next < 0) return at;
        if (next >= (int64_t)layers.size()) break;
        at = (int)next;
    }
    bad("layers[" + std::to_string(layer) + "]", "'weights_of' leads to no layer with tensors of its own");
}

void SovezenConfig::validate() const {
    positive(vocab, "top level", "vocab");
    positive(width, "top level", "width");
    if (!(norm_eps > 0.0)) bad("norm", "'eps' must be > 0");
    if (!std::isfinite(logit_scale)) bad("top level", "'logit_scale' must be a finite number");
    for (size_t i = 0; i < layers.size(); i++) {
        const Layer& l = layers[i];
        const std::string at = "layers[" + std::to_string(i) + "]";
        positive(l.heads, at, "heads");
        positive(l.dim, at, "dim");
        positive(l.vdim, at, "vdim");
        positive(l.kv_rank, at, "kv_rank");
        if (l.type == kWithRotation) {
            if (l.rot_dim < 0) bad(at, "'rot_dim' must be >= 0");
            if (l.rot_dims < 0 || l.rot_dims > l.rot_dim || l.rot_dims % 2) bad(at + ".rot", "'dims' must be even and at most rot_dim");
            if (l.rot_dims && !(l.rot_base > 0.0)) bad(at + ".rot", "'base' must be > 0");
        } else {
            positive(l.q_rank, at, "q_rank");
        }
        if (l.kv_rank + l.rot_dim > 640) bad(at, "kv_rank + rot_dim is at most 640 (the attention kernels' widest head)");
        if (l.mlp == "dense") positive(l.ff, at + ".mlp", "ff");
        if (l.mlp == "moe") {
            positive(l.ff, at + ".mlp.expert", "ff");
            positive(l.experts, at + ".mlp.router", "experts");
            if (l.top < 1 || l.top > l.experts) bad(at + ".mlp.router", "'top' must be 1 .. experts");
            if (l.experts > 2048) bad(at + ".mlp.router", "'experts' is at most 2048");
        }
        if (l.weights_of >= 0) {
            if (l.weights_of >= (int64_t)layers.size() || l.weights_of == (int64_t)i) bad(at, "'weights_of' must name another layer");
            const Layer& o = layers[(size_t)owner((int)i)];
            if (o.type != l.type || o.heads != l.heads || o.dim != l.dim || o.vdim != l.vdim || o.kv_rank != l.kv_rank ||
                o.rot_dim != l.rot_dim || o.q_rank != l.q_rank || o.mlp != l.mlp || o.ff != l.ff || o.experts != l.experts ||
                o.top != l.top || o.scale != l.scale || o.rot_dims != l.rot_dims || o.rot_base != l.rot_base)
                bad(at, "a layer that uses another layer's tensors must have that layer's type, sizes and constants");
        }
    }
}

// The description: which parts every layer is made of, the run order (a layer that uses another's tensors is a second
// call of that layer's parts with a cache entry of its own), and the tensor names.
ModelSpec describe_sovezen(const SovezenConfig& cfg) {
    ModelSpec s;
    s.architecture = cfg.architecture();
    s.width = cfg.width;
    s.vocab_size = cfg.vocab;
    auto norm = [&](const std::string& name) {
        PartSpec p;
        p.kind = "rmsnorm";
        p.params["width"] = (long long)cfg.width;
        p.params["eps"] = cfg.norm_eps;
        p.tensors = {{"weight", name}};
        return p;
    };
    auto channel_scale = [&](const std::string& name) {
        PartSpec p;
        p.kind = "channel_scale";
        p.params["width"] = (long long)cfg.width;
        p.tensors = {{"weight", name}};
        return p;
    };
    std::vector<int> spec_of((size_t)cfg.layers.size(), -1);     // config layer -> entry of s.layers, for owners
    for (size_t i = 0; i < cfg.layers.size(); i++) {
        if (cfg.owner((int)i) != (int)i) continue;
        const SovezenConfig::Layer& c = cfg.layers[i];
        const std::string p = "l" + std::to_string(i) + ".";
        LayerSpec l;
        l.block = "parallel_branches";
        PartSpec& m = l.mixer;
        m.kind = "latent_attention";
        m.params["width"] = (long long)cfg.width;
        m.params["eps"] = cfg.norm_eps;
        m.params["n_heads"] = (long long)c.heads;
        m.params["qk_dim"] = (long long)c.dim;
        m.params["v_dim"] = (long long)c.vdim;
        m.params["kv_rank"] = (long long)c.kv_rank;
        m.params["scale"] = c.scale;
        const std::string x = p + "mix.";
        m.tensors = {{"dkv", x + "dkv"}, {"dkv_norm", x + "dkv.norm"}, {"uk", x + "uk"}, {"uv", x + "uv"}, {"o", x + "o"}};
        if (c.type == kWithRotation) {
            m.params["rot_dim"] = (long long)c.rot_dim;
            m.params["rot_dims"] = (long long)c.rot_dims;
            m.params["rot_base"] = c.rot_base;
            m.params["rot_pairs"] = "neighbours";
            m.params["sink"] = true;
            m.params["q_rank"] = 0LL;
            m.tensors["q"] = x + "q";
            m.tensors["sink"] = x + "sink";
        } else {
            m.params["rot_dim"] = 0LL;
            m.params["sink"] = false;
            m.params["q_rank"] = (long long)c.q_rank;
            m.tensors["dq"] = x + "dq";
            m.tensors["dq_norm"] = x + "dq.norm";
            m.tensors["uq"] = x + "uq";
        }
        l.norms["input"] = norm(p + "norm1");
        l.norms["mixer_scale"] = channel_scale(p + "ls1");
        PartSpec& f = l.feed_forward;
        if (c.mlp == "dense") {
            f.kind = "gated_mlp";
            f.params["width"] = (long long)cfg.width;
            f.params["inner"] = (long long)c.ff;
            f.params["activation"] = "silu";
            f.tensors = {{"gate", p + "mlp.gate"}, {"up", p + "mlp.up"}, {"down", p + "mlp.down"}};
        } else if (c.mlp == "moe") {
            f.kind = "routed_experts";
            f.params["width"] = (long long)cfg.width;
            f.params["inner"] = (long long)c.ff;
            f.params["n_experts"] = (long long)c.experts;
            f.params["top"] = (long long)c.top;
            f.params["activation"] = "relu_squared";
            f.params["router_bias"] = true;
            f.tensors = {{"router", p + "mlp.router"}, {"router_bias", p + "mlp.router.b"}};
            for (int64_t e = 0; e < c.experts; e++) {
                f.tensors["up." + std::to_string(e)] = p + "mlp.e" + std::to_string(e) + ".up";
                f.tensors["down." + std::to_string(e)] = p + "mlp.e" + std::to_string(e) + ".down";
            }
        } else {
            f.kind = "none";
        }
        if (!c.mlp.empty()) l.norms["feed_forward_scale"] = channel_scale(p + "ls2");
        else s.ignored_tensors.push_back("^l" + std::to_string(i) + R"(\.ls2$)");      // a factor with nothing to scale, if the file has one
        spec_of[i] = (int)s.layers.size();
        s.layers.push_back(std::move(l));
    }
    for (size_t i = 0; i < cfg.layers.size(); i++) {
        LayerCall c;
        c.layer = spec_of[(size_t)cfg.owner((int)i)];
        c.cache = (int)i;
        s.schedule.push_back(c);
    }
    s.embedding.kind = "token_embedding";
    s.embedding.params["vocab_size"] = (long long)cfg.vocab;
    s.embedding.params["width"] = (long long)cfg.width;
    s.embedding.tensors = {{"weight", "embed"}};
    s.position.kind = "none";
    s.final_norm = norm("final.norm");
    s.head.kind = "output_head";
    s.head.params["vocab_size"] = (long long)cfg.vocab;
    s.head.params["width"] = (long long)cfg.width;
    s.head.params["tied"] = true;
    s.head.params["logit_scale"] = cfg.logit_scale;
    return s;
}

}  // namespace sandy
