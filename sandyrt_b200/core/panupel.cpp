// Panupel: a decoder whose layers mix softmax attention with recurrences.
//
// config.json (all sizes and every constant that differs between models come from it):
//   architecture  "Panupel"
//   vocab, width
//   norm.eps, residual_mult
//   layers[i]     {type: "parallel" | "delta", mixer: {...}, mlp: {kind: "dense", ff} | null}
//     delta       mixer {heads, kv_heads, dim, vdim, conv}
//     parallel    mixer {left {heads, kv_heads, dim, vdim, scale, rot {dims, base, scaling {factor, low, high,
//                 original} | absent} | absent}, right {heads, dim, vdim, gate_cap}, left_scale, right_scale}
//   loop          {start, stop, times} | absent: layers start .. stop - 1 run `times` times in a row on the same
//                 weights, each pass with a cache and state of its own, and each pass is entered through
//                 x <- W_in [x; x0] (x0 the embedding's output)
//
// A layer is x += m norm1b(mixer(norm1(x))); x += m norm2b(ff(norm2(x))) with RMS norms and m = residual_mult.
// Tensors: embed, head, final.norm, loop.in, and per layer l<i>.norm1 / norm1b / norm2 / norm2b, l<i>.mix.* and
// l<i>.mlp.gate / up / down; linear weights are [out, in].
//
// The typed configuration below checks the file; `describe` turns it into parts of parts_hybrid.cpp.  Nothing
// else in the engine knows this architecture.
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

}  // namespace

PanupelConfig PanupelConfig::from_json(const Json& raw) {
    if (!raw.is_object()) throw ConfigError("config.json: top level must be a JSON object");
    PanupelConfig c;
    c.vocab = need_int(raw, "top level", "vocab");
    c.width = need_int(raw, "top level", "width");
    c.norm_eps = need_num(need_obj(raw, "top level", "norm"), "norm", "eps");
    c.residual_mult = need_num(raw, "top level", "residual_mult");
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
        if (l.type == "delta") {
            l.heads = need_int(m, at + ".mixer", "heads");
            l.kv_heads = need_int(m, at + ".mixer", "kv_heads");
            l.dim = need_int(m, at + ".mixer", "dim");
            l.vdim = need_int(m, at + ".mixer", "vdim");
            l.conv = need_int(m, at + ".mixer", "conv");
        } else if (l.type == "parallel") {
            const Json& a = need_obj(m, at + ".mixer", "left");
            const std::string la = at + ".mixer.left";
            l.heads = need_int(a, la, "heads");
            l.kv_heads = need_int(a, la, "kv_heads");
            l.dim = need_int(a, la, "dim");
            l.vdim = need_int(a, la, "vdim");
            l.scale = need_num(a, la, "scale");
            if (const Json* rot = maybe_obj(a, la, "rot")) {
                l.rot_dims = need_int(*rot, la + ".rot", "dims");
                l.rot_base = need_num(*rot, la + ".rot", "base");
                if (const Json* sc = maybe_obj(*rot, la + ".rot", "scaling")) {
                    l.rot_scaling = true;
                    l.rot_factor = need_num(*sc, la + ".rot.scaling", "factor");
                    l.rot_low = need_num(*sc, la + ".rot.scaling", "low");
                    l.rot_high = need_num(*sc, la + ".rot.scaling", "high");
                    l.rot_original = need_num(*sc, la + ".rot.scaling", "original");
                }
            }
            const Json& r = need_obj(m, at + ".mixer", "right");
            const std::string ra = at + ".mixer.right";
            l.right_heads = need_int(r, ra, "heads");
            l.right_dim = need_int(r, ra, "dim");
            l.right_vdim = need_int(r, ra, "vdim");
            l.gate_cap = need_num(r, ra, "gate_cap");
            l.left_scale = need_num(m, at + ".mixer", "left_scale");
            l.right_scale = need_num(m, at + ".mixer", "right_scale");
        } else {
            bad(at, "unknown layer type '" + l.type + "'; one of ['parallel', 'delta']");
        }
        if (const Json* mlp = maybe_obj(lj, at, "mlp")) {
            const Json& kind = need(*mlp, at + ".mlp", "kind");
            if (!kind.is_string() || kind.as_string() != "dense") bad(at + ".mlp", "'kind' must be 'dense', got " + kind.dump());
            l.ff = need_int(*mlp, at + ".mlp", "ff");
        }
        c.layers.push_back(l);
    }
    if (const Json* loop = maybe_obj(raw, "top level", "loop")) {
        c.has_loop = true;
        c.loop_start = need_int(*loop, "loop", "start");
        c.loop_stop = need_int(*loop, "loop", "stop");
        c.loop_times = need_int(*loop, "loop", "times");
    }
    return c;
}

Json PanupelConfig::to_json() const {
    Json j = Json::object();
    j["architecture"] = kArchitecture;
    Json ls = Json::array();
    for (const Layer& l : layers) {
        Json lj = Json::object();
        Json m = Json::object();
        if (l.type == "delta") {
            m["conv"] = (long long)l.conv;
            m["dim"] = (long long)l.dim;
            m["heads"] = (long long)l.heads;
            m["kv_heads"] = (long long)l.kv_heads;
            m["vdim"] = (long long)l.vdim;
        } else {
            Json a = Json::object();
            a["dim"] = (long long)l.dim;
            a["heads"] = (long long)l.heads;
            a["kv_heads"] = (long long)l.kv_heads;
            if (l.rot_dims) {
                Json rot = Json::object();
                rot["base"] = l.rot_base;
                rot["dims"] = (long long)l.rot_dims;
                if (l.rot_scaling) {
                    Json sc = Json::object();
                    sc["factor"] = l.rot_factor;
                    sc["high"] = l.rot_high;
                    sc["low"] = l.rot_low;
                    sc["original"] = l.rot_original;
                    rot["scaling"] = sc;
                }
                a["rot"] = rot;
            }
            a["scale"] = l.scale;
            a["vdim"] = (long long)l.vdim;
            m["left"] = a;
            m["left_scale"] = l.left_scale;
            Json r = Json::object();
            r["dim"] = (long long)l.right_dim;
            r["gate_cap"] = l.gate_cap;
            r["heads"] = (long long)l.right_heads;
            r["vdim"] = (long long)l.right_vdim;
            m["right"] = r;
            m["right_scale"] = l.right_scale;
        }
        lj["mixer"] = m;
        if (l.ff) {
            Json mlp = Json::object();
            mlp["ff"] = (long long)l.ff;
            mlp["kind"] = "dense";
            lj["mlp"] = mlp;
        } else {
            lj["mlp"] = Json();
        }
        lj["type"] = l.type;
        ls.push(lj);
    }
    j["layers"] = ls;
    if (has_loop) {
        Json loop = Json::object();
        loop["start"] = (long long)loop_start;
        loop["stop"] = (long long)loop_stop;
        loop["times"] = (long long)loop_times;
        j["loop"] = loop;
    }
    Json norm = Json::object();
    norm["eps"] = norm_eps;
    j["norm"] = norm;
    j["residual_mult"] = residual_mult;
    j["vocab"] = (long long)vocab;
    j["width"] = (long long)width;
    return j;
}

void PanupelConfig::validate() const {
    positive(vocab, "top level", "vocab");
    positive(width, "top level", "width");
    if (!(norm_eps > 0.0)) bad("norm", "'eps' must be > 0");
    for (size_t i = 0; i < layers.size(); i++) {
        const Layer& l = layers[i];
        const std::string at = "layers[" + std::to_string(i) + "]";
        positive(l.heads, at, "heads");
        positive(l.kv_heads, at, "kv_heads");
        positive(l.dim, at, "dim");
        positive(l.vdim, at, "vdim");
        if (l.heads % l.kv_heads) bad(at, std::to_string(l.heads) + " heads do not divide into " + std::to_string(l.kv_heads) + " kv_heads");
        if (l.type == "delta") {
            if (l.conv < 1 || l.conv > 8) bad(at, "'conv' must be 1 to 8 taps, got " + std::to_string(l.conv));
            if (l.dim > 256) bad(at, "'dim' is at most 256");
        } else {
            positive(l.right_heads, at + ".right", "heads");
            positive(l.right_dim, at + ".right", "dim");
            positive(l.right_vdim, at + ".right", "vdim");
            if (!(l.gate_cap > 0.0)) bad(at + ".right", "'gate_cap' must be > 0");
            if (l.rot_dims < 0 || l.rot_dims > l.dim || l.rot_dims % 2) bad(at + ".left.rot", "'dims' must be even and at most the head's dim");
            if (l.rot_dims && !(l.rot_base > 0.0)) bad(at + ".left.rot", "'base' must be > 0");
            if (l.rot_scaling && (!(l.rot_factor > 0.0) || l.rot_high == l.rot_low || !(l.rot_original > 0.0)))
                bad(at + ".left.rot.scaling", "needs factor > 0, original > 0 and high != low");
            if (std::max(l.dim, l.vdim) > 256 || l.right_dim > 256) bad(at, "head sizes are at most 256");
        }
        if (l.ff < 0) bad(at + ".mlp", "'ff' must be > 0");
    }
    if (has_loop) {
        if (loop_start < 0 || loop_stop <= loop_start || loop_stop > (int64_t)layers.size())
            bad("loop", "needs 0 <= start < stop <= " + std::to_string(layers.size()));
        if (loop_times < 1) bad("loop", "'times' must be >= 1");
    }
}

// The description: which parts every layer is made of, the run order (a looped span appears once per pass, each
// pass with cache entries of its own and entered through the stream mix), and the tensor names.
ModelSpec describe_panupel(const PanupelConfig& cfg) {
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
    for (size_t i = 0; i < cfg.layers.size(); i++) {
        const PanupelConfig::Layer& c = cfg.layers[i];
        const std::string p = "l" + std::to_string(i) + ".";
        LayerSpec l;
        l.block = "sandwich_norm";
        l.block_params["residual_mult"] = cfg.residual_mult;
        PartSpec& m = l.mixer;
        m.params["width"] = (long long)cfg.width;
        m.params["eps"] = cfg.norm_eps;
        if (c.type == "delta") {
            m.kind = "gated_delta";
            m.params["n_heads"] = (long long)c.heads;
            m.params["n_qk_heads"] = (long long)c.kv_heads;
            m.params["qk_dim"] = (long long)c.dim;
            m.params["v_dim"] = (long long)c.vdim;
            m.params["conv_taps"] = (long long)c.conv;
            const std::string x = p + "mix.";
            m.tensors = {{"q", x + "q"}, {"k", x + "k"}, {"v", x + "v"}, {"gate", x + "g"}, {"o", x + "o"},
                         {"q_conv", x + "q.conv"}, {"k_conv", x + "k.conv"}, {"v_conv", x + "v.conv"},
                         {"beta", x + "b"}, {"decay", x + "a"}, {"a_log", x + "A_log"}, {"dt_bias", x + "dt_bias"},
                         {"norm", x + "norm"}};
        } else {
            m.kind = "attention_beside_matrix_memory";
            m.params["left_scale"] = c.left_scale;
            m.params["right_scale"] = c.right_scale;
            m.params["left.n_heads"] = (long long)c.heads;
            m.params["left.n_kv_heads"] = (long long)c.kv_heads;
            m.params["left.qk_dim"] = (long long)c.dim;
            m.params["left.v_dim"] = (long long)c.vdim;
            m.params["left.scale"] = c.scale;
            m.params["left.qk_norm"] = true;
            m.params["left.sink"] = true;
            m.params["left.rot_dims"] = (long long)c.rot_dims;
            if (c.rot_dims) {
                m.params["left.rot_base"] = c.rot_base;
                if (c.rot_scaling) {
                    Json sc = Json::object();
                    sc["factor"] = c.rot_factor;
                    sc["low"] = c.rot_low;
                    sc["high"] = c.rot_high;
                    sc["original"] = c.rot_original;
                    m.params["left.rot_scaling"] = sc;
                }
            }
            m.params["right.n_heads"] = (long long)c.right_heads;
            m.params["right.qk_dim"] = (long long)c.right_dim;
            m.params["right.v_dim"] = (long long)c.right_vdim;
            m.params["right.gate_cap"] = c.gate_cap;
            const std::string a = p + "mix.left.", r = p + "mix.right.";
            m.tensors = {{"left.q", a + "q"}, {"left.k", a + "k"}, {"left.v", a + "v"}, {"left.o", a + "o"},
                         {"left.q_norm", a + "q.norm"}, {"left.k_norm", a + "k.norm"}, {"left.sink", a + "sink"},
                         {"left.gate", a + "g"},
                         {"right.q", r + "q"}, {"right.k", r + "k"}, {"right.v", r + "v"}, {"right.gate", r + "g"},
                         {"right.o", r + "o"}, {"right.norm", r + "norm"}, {"right.i", r + "i"}, {"right.i_bias", r + "i.b"},
                         {"right.f", r + "f"}, {"right.f_bias", r + "f.b"}};
        }
        l.norms["mixer"] = norm(p + "norm1");
        l.norms["mixer_out"] = norm(p + "norm1b");
        if (c.ff) {
            l.feed_forward.kind = "gated_mlp";
            l.feed_forward.params["width"] = (long long)cfg.width;
            l.feed_forward.params["inner"] = (long long)c.ff;
            l.feed_forward.params["activation"] = "silu";
            l.feed_forward.tensors = {{"gate", p + "mlp.gate"}, {"up", p + "mlp.up"}, {"down", p + "mlp.down"}};
            l.norms["feed_forward"] = norm(p + "norm2");
            l.norms["feed_forward_out"] = norm(p + "norm2b");
        } else {
            l.feed_forward.kind = "none";
        }
        s.layers.push_back(std::move(l));
    }
    // run order
    const int n = (int)cfg.layers.size();
    int cache = 0;
    auto call = [&](int layer, int remix) {
        LayerCall c;
        c.layer = layer;
        c.cache = cache++;
        c.remix = remix;
        s.schedule.push_back(c);
    };
    if (cfg.has_loop) {
        PartSpec in;
        in.kind = "concat_linear";
        in.params["width"] = (long long)cfg.width;
        in.tensors = {{"weight", "loop.in"}};
        s.remixes.push_back(in);
        for (int i = 0; i < (int)cfg.loop_start; i++) call(i, -1);
        for (int64_t pass = 0; pass < cfg.loop_times; pass++)
            for (int i = (int)cfg.loop_start; i < (int)cfg.loop_stop; i++) call(i, i == (int)cfg.loop_start ? 0 : -1);
        for (int i = (int)cfg.loop_stop; i < n; i++) call(i, -1);
    } else {
        for (int i = 0; i < n; i++) call(i, -1);
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
    s.head.params["tied"] = false;
    s.head.tensors = {{"weight", "head"}};
    return s;
}

}  // namespace sandy
