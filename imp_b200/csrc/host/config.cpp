#include "config.hpp"

#include <sys/stat.h>

#include <cmath>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>

#include "parts.hpp"

namespace imp {

namespace {
[[noreturn]] void bad(const std::string& msg) { fail(IMP_ERROR_INVALID_MODEL, msg); }

const Json& require(const Json& d, const std::string& key, const std::string& where) {
    const Json* v = d.find(key);
    if (!v) bad(where + ": missing required key '" + key + "'");
    return *v;
}
int64_t require_int(const Json& d, const std::string& key, const std::string& where) {
    const Json& v = require(d, key, where);
    if (!v.is_int()) bad(where + ": key '" + key + "' must be int, got " + v.type_name());
    return v.as_int();
}
double require_float(const Json& d, const std::string& key, const std::string& where) {
    const Json& v = require(d, key, where);
    if (!v.is_number()) bad(where + ": key '" + key + "' must be float, got " + v.type_name());
    return v.as_double();
}
int64_t positive(const std::string& name, int64_t v, const std::string& where) {
    if (v <= 0) bad(where + ": '" + name + "' must be positive, got " + std::to_string(v));
    return v;
}
}  // namespace

// ------------------------------------------------------------------------------- base config
void ModelConfig::read_base(ModelConfig& c, const Json& d, const std::string& where) {
    const Json* archs = d.find("architectures");
    if (!archs || !archs->is_array() || archs->size() == 0 || !(*archs)[0].is_string())
        bad(where + ": 'architectures' must be a list that names the model class");
    c.architecture = (*archs)[0].as_string();
    c.vocab_size = positive("vocab_size", require_int(d, "vocab_size", where), where);
    c.hidden_size = positive("hidden_size", require_int(d, "hidden_size", where), where);
    c.num_hidden_layers = positive("num_hidden_layers", require_int(d, "num_hidden_layers", where), where);
    c.max_position_embeddings = positive("max_position_embeddings", d.get_int("max_position_embeddings", 4096), where);
    c.torch_dtype = d.get_string("torch_dtype", d.get_string("dtype", "bfloat16"));
    if (const Json* eos = d.find("eos_token_id")) {
        if (eos->is_array()) {
            for (const auto& e : eos->items())
                if (e.is_int()) c.eos_token_ids.push_back((int)e.as_int());
        } else if (eos->is_int()) {
            c.eos_token_ids.push_back((int)eos->as_int());
        }
    }
    c.bos_token_id = d.get_int("bos_token_id", -1);
    c.raw = d;
}

Json ModelConfig::to_json() const {
    Json j = raw.is_object() ? raw : Json::object();
    j["architectures"] = Json::array_of(std::vector<std::string>{architecture});
    j["vocab_size"] = vocab_size;
    j["hidden_size"] = hidden_size;
    j["num_hidden_layers"] = num_hidden_layers;
    j["max_position_embeddings"] = max_position_embeddings;
    j["torch_dtype"] = torch_dtype;
    if (eos_token_ids.size() == 1) j["eos_token_id"] = eos_token_ids[0];
    else if (!eos_token_ids.empty()) j["eos_token_id"] = Json::array_of(eos_token_ids);
    if (bos_token_id >= 0) j["bos_token_id"] = bos_token_id;
    j.erase("dtype");
    return j;
}

// ------------------------------------------------------------------------------------- Qwen3
Qwen3Config Qwen3Config::from_json(const Json& d, const std::string& where) {
    Qwen3Config c;
    // hidden_size and the head counts first, so that a missing one is named before anything derived from it
    const int64_t hidden = positive("hidden_size", require_int(d, "hidden_size", where), where);
    const int64_t heads = positive("num_attention_heads", require_int(d, "num_attention_heads", where), where);
    read_base(c, d, where);
    c.num_attention_heads = heads;
    const Json* kv = d.find("num_key_value_heads");
    c.num_key_value_heads = (kv && kv->is_int()) ? kv->as_int() : heads;
    const Json* hd = d.find("head_dim");
    if (hd && hd->is_int()) {
        c.head_dim = hd->as_int();
    } else {
        if (hidden % heads)
            bad(where + ": no 'head_dim' and hidden_size " + std::to_string(hidden) +
                " is not a multiple of num_attention_heads " + std::to_string(heads));
        c.head_dim = hidden / heads;
    }
    c.intermediate_size = positive("intermediate_size", require_int(d, "intermediate_size", where), where);
    c.rms_norm_eps = require_float(d, "rms_norm_eps", where);
    c.rope_theta = d.get_double("rope_theta", 10000.0);
    c.tie_word_embeddings = d.get_bool("tie_word_embeddings", false);
    c.attention_bias = d.get_bool("attention_bias", false);
    c.hidden_act = d.get_string("hidden_act", "silu");
    c.use_sliding_window = d.get_bool("use_sliding_window", false);
    c.sliding_window = d.get_int("sliding_window", 0);
    c.max_window_layers = d.get_int("max_window_layers", -1);
    if (const Json* lt = d.find("layer_types"))
        if (lt->is_array())
            for (const auto& t : lt->items()) c.layer_types.push_back(t.is_string() ? t.as_string() : std::string("?"));
    if (const Json* rs = d.find("rope_scaling"))
        if (!rs->is_null() && !(rs->is_object() && rs->size() == 0))
            bad(where + ": rope_scaling " + rs->dump() + " is not supported (only the plain rotary encoding)");
    c.validate(where);
    return c;
}

void Qwen3Config::validate(const std::string& where) const {
    if (num_key_value_heads <= 0 || num_attention_heads % num_key_value_heads)
        bad(where + ": num_attention_heads " + std::to_string(num_attention_heads) +
            " must be a positive multiple of num_key_value_heads " + std::to_string(num_key_value_heads));
    if (head_dim <= 0 || head_dim % 16) bad(where + ": head_dim " + std::to_string(head_dim) + " must be a positive multiple of 16");
    if (head_dim > 256) bad(where + ": head_dim " + std::to_string(head_dim) + " exceeds the kernels' limit of 256");
    if (attention_bias) bad(where + ": attention_bias=true is not supported for " + architecture);
    if (hidden_act != "silu") bad(where + ": hidden_act '" + hidden_act + "' is not supported (silu only)");
    if (!(rms_norm_eps > 0)) bad(where + ": rms_norm_eps must be positive");
    if (!(rope_theta > 0)) bad(where + ": rope_theta must be positive");
    if (torch_dtype != "bfloat16" && torch_dtype != "float32")
        bad(where + ": torch_dtype '" + torch_dtype + "' is not supported (bfloat16 or float32)");
    bool any_sliding = false;
    if (!layer_types.empty()) {
        if ((int64_t)layer_types.size() != num_hidden_layers)
            bad(where + ": layer_types has " + std::to_string(layer_types.size()) + " entries for " +
                std::to_string(num_hidden_layers) + " layers");
        for (const auto& t : layer_types) {
            if (t != "full_attention" && t != "sliding_attention") bad(where + ": unknown layer type '" + t + "' in layer_types");
            any_sliding = any_sliding || t == "sliding_attention";
        }
    }
    if ((use_sliding_window || any_sliding) && sliding_window <= 0)
        bad(where + ": sliding window in use but 'sliding_window' is not a positive size");
}

int64_t Qwen3Config::window_of_layer(int layer) const {
    if (!layer_types.empty()) return layer_types[(size_t)layer] == "sliding_attention" ? sliding_window : 0;
    if (!use_sliding_window) return 0;
    const int64_t first = max_window_layers >= 0 ? max_window_layers : 0;
    return layer >= first ? sliding_window : 0;
}

Json Qwen3Config::to_json() const {
    Json j = ModelConfig::to_json();
    j["model_type"] = j.get_string("model_type", "qwen3");
    j["num_attention_heads"] = num_attention_heads;
    j["num_key_value_heads"] = num_key_value_heads;
    j["head_dim"] = head_dim;
    j["intermediate_size"] = intermediate_size;
    j["rms_norm_eps"] = rms_norm_eps;
    j["rope_theta"] = rope_theta;
    j["tie_word_embeddings"] = tie_word_embeddings;
    j["attention_bias"] = attention_bias;
    j["hidden_act"] = hidden_act;
    j["use_sliding_window"] = use_sliding_window;
    if (sliding_window > 0) j["sliding_window"] = sliding_window;
    if (max_window_layers >= 0) j["max_window_layers"] = max_window_layers;
    if (!layer_types.empty()) j["layer_types"] = Json::array_of(layer_types);
    return j;
}

// The Qwen3 dense decoder as a plan of parts: pre-norm blocks of grouped-query attention (per-head
// RMSNorm on q and k before the rotary encoding, no bias, head size independent of the width) and a
// SwiGLU feed-forward; final RMSNorm; output head tied to the embedding or its own (the reference's
// forward pass for this family: src/graph/executor_forward.cu:2701-3140; tensor names:
// src/model/safetensors_loader.cpp:366-401 and, for the q/k norms that binder lacks, the GGUF twins
// at src/model/gguf_loader.cpp:387-388).  Everything here is data.
ModelPlan qwen3_plan(const Qwen3Config& cfg) {
    const int64_t d = cfg.hidden_size;
    Json rotary = Json::object();
    rotary["kind"] = "rotary";
    rotary["params"]["head_dim"] = cfg.head_dim;
    rotary["params"]["theta"] = cfg.rope_theta;
    rotary["params"]["max_positions"] = cfg.max_position_embeddings;
    ModelPlan plan;
    plan.architecture = cfg.architecture;
    plan.hidden_size = d;
    plan.vocab_size = cfg.vocab_size;
    plan.max_positions = cfg.max_position_embeddings;
    auto norm = [&](const std::string& tensor) {
        PartSpec n;
        n.kind = "rmsnorm";
        n.params["size"] = d;
        n.params["eps"] = cfg.rms_norm_eps;
        n.tensors = {{"weight", tensor}};
        return n;
    };
    for (int i = 0; i < cfg.num_hidden_layers; ++i) {
        const std::string p = "model.layers." + std::to_string(i) + ".";
        PartSpec attn;
        attn.kind = "gqa_attention";
        attn.params["hidden_size"] = d;
        attn.params["num_heads"] = cfg.num_attention_heads;
        attn.params["num_kv_heads"] = cfg.num_key_value_heads;
        attn.params["head_dim"] = cfg.head_dim;
        attn.params["window"] = cfg.window_of_layer(i);
        attn.params["qk_norm"] = true;
        attn.params["qk_norm_eps"] = cfg.rms_norm_eps;
        attn.params["position"] = rotary;
        attn.tensors = {{"q_proj", p + "self_attn.q_proj.weight"}, {"k_proj", p + "self_attn.k_proj.weight"},
                        {"v_proj", p + "self_attn.v_proj.weight"}, {"o_proj", p + "self_attn.o_proj.weight"},
                        {"q_norm", p + "self_attn.q_norm.weight"}, {"k_norm", p + "self_attn.k_norm.weight"}};
        PartSpec ffn;
        ffn.kind = "swiglu";
        ffn.params["hidden_size"] = d;
        ffn.params["intermediate_size"] = cfg.intermediate_size;
        ffn.tensors = {{"gate_proj", p + "mlp.gate_proj.weight"}, {"up_proj", p + "mlp.up_proj.weight"},
                       {"down_proj", p + "mlp.down_proj.weight"}};
        LayerSpec layer;
        layer.block = "prenorm";
        layer.parts = {{"mixer_norm", norm(p + "input_layernorm.weight")}, {"mixer", attn},
                       {"ffn_norm", norm(p + "post_attention_layernorm.weight")}, {"feed_forward", ffn}};
        plan.layers.push_back(layer);
    }
    plan.embedding.kind = "token_embedding";
    plan.embedding.params["vocab_size"] = cfg.vocab_size;
    plan.embedding.params["hidden_size"] = d;
    plan.embedding.tensors = {{"weight", "model.embed_tokens.weight"}};
    plan.final_norm = norm("model.norm.weight");
    plan.head.kind = "linear_head";
    plan.head.params["vocab_size"] = cfg.vocab_size;
    plan.head.params["hidden_size"] = d;
    plan.head.tensors = {{"weight", cfg.tie_word_embeddings ? "model.embed_tokens.weight" : "lm_head.weight"}};
    // Published tied checkpoints of this family also store the head; the reference binds it when present and
    // aliases the embedding when absent (src/model/weight_map.cpp:182, 330).  With a tied configuration the
    // stored copy is not read.
    if (cfg.tie_word_embeddings) plan.ignored_tensors.push_back("lm_head.weight");
    return plan;
}

// ------------------------------------------------------------------------------------ Kazedra
namespace {
const Json& require_object(const Json& d, const std::string& key, const std::string& where) {
    const Json& v = require(d, key, where);
    if (!v.is_object()) bad(where + ": key '" + key + "' must be an object, got " + v.type_name());
    return v;
}
}  // namespace

KazedraConfig KazedraConfig::from_json(const Json& d, const std::string& where) {
    KazedraConfig c;
    c.architecture = d.get_string("architecture", "Kazedra");
    c.vocab_size = positive("vocab", require_int(d, "vocab", where), where);
    c.hidden_size = positive("width", require_int(d, "width", where), where);
    c.max_position_embeddings = positive("max_positions", d.get_int("max_positions", 1 << 20), where);
    c.torch_dtype = d.get_string("torch_dtype", d.get_string("dtype", "bfloat16"));
    if (c.torch_dtype != "bfloat16" && c.torch_dtype != "float32")
        bad(where + ": torch_dtype '" + c.torch_dtype + "' is not supported (bfloat16 or float32)");
    if (const Json* eos = d.find("eos_token_id")) {
        if (eos->is_array()) {
            for (const auto& e : eos->items())
                if (e.is_int()) c.eos_token_ids.push_back((int)e.as_int());
        } else if (eos->is_int()) {
            c.eos_token_ids.push_back((int)eos->as_int());
        }
    }
    c.bos_token_id = d.get_int("bos_token_id", -1);
    c.raw = d;
    c.norm_eps = require_float(require_object(d, "norm", where), "eps", where + ": norm");
    if (!(c.norm_eps > 0)) bad(where + ": norm.eps must be positive");
    c.logit_scale = d.get_double("logit_scale", 1.0);
    const Json& layers = require(d, "layers", where);
    if (!layers.is_array() || layers.size() == 0) bad(where + ": 'layers' must be a non-empty list");
    int i = 0;
    for (const Json& lj : layers.items()) {
        const std::string lw = where + ": layers[" + std::to_string(i++) + "]";
        if (!lj.is_object()) bad(lw + " must be an object");
        Layer l;
        l.type = lj.get_string("type", "");
        if (l.type != "parallel") bad(lw + ": unknown layer type '" + l.type + "' (known: parallel)");
        const Json& m = require_object(lj, "mixer", lw);
        const Json& a = require_object(m, "left", lw + ".mixer");
        const std::string aw = lw + ".mixer.left", bw = lw + ".mixer.right";
        l.left.heads = positive("heads", require_int(a, "heads", aw), aw);
        l.left.kv_heads = positive("kv_heads", require_int(a, "kv_heads", aw), aw);
        l.left.dim = positive("dim", require_int(a, "dim", aw), aw);
        l.left.vdim = positive("vdim", a.get_int("vdim", l.left.dim), aw);
        l.left.bias_max = positive("bias_max", require_int(a, "bias_max", aw), aw);
        l.left.scale = require_float(a, "scale", aw);
        if (const Json* qt = a.find("q_temp")) {
            if (qt->is_object()) {
                l.left.temp_coef = require_float(*qt, "coef", aw + ".q_temp");
                l.left.temp_every = positive("every", require_int(*qt, "every", aw + ".q_temp"), aw + ".q_temp");
            }
        }
        if (l.left.heads % l.left.kv_heads) bad(aw + ": heads " + std::to_string(l.left.heads) + " must be a multiple of kv_heads " + std::to_string(l.left.kv_heads));
        if (l.left.vdim != l.left.dim) bad(aw + ": the values are the keys, so vdim " + std::to_string(l.left.vdim) + " must equal dim " + std::to_string(l.left.dim));
        const Json& b = require_object(m, "right", lw + ".mixer");
        l.right.heads = positive("heads", require_int(b, "heads", bw), bw);
        l.right.kv_heads = positive("kv_heads", require_int(b, "kv_heads", bw), bw);
        l.right.dim = positive("dim", require_int(b, "dim", bw), bw);
        l.right.vdim = positive("vdim", require_int(b, "vdim", bw), bw);
        l.right.conv = positive("conv", require_int(b, "conv", bw), bw);
        if (l.right.heads % l.right.kv_heads) bad(bw + ": heads " + std::to_string(l.right.heads) + " must be a multiple of kv_heads " + std::to_string(l.right.kv_heads));
        l.left_scale = require_float(m, "left_scale", lw + ".mixer");
        l.right_scale = require_float(m, "right_scale", lw + ".mixer");
        if (const Json* f = lj.find("mlp")) {
            if (f->is_object()) {
                const std::string kind = f->get_string("kind", "");
                if (kind != "dense") bad(lw + ".mlp: unknown kind '" + kind + "' (known: dense)");
                l.ff = positive("ff", require_int(*f, "ff", lw + ".mlp"), lw + ".mlp");
            } else if (!f->is_null()) {
                bad(lw + ".mlp must be an object or null");
            }
        }
        c.layers.push_back(l);
    }
    c.num_hidden_layers = (int64_t)c.layers.size();
    return c;
}

Json KazedraConfig::to_json() const {
    Json j = raw.is_object() ? raw : Json::object();
    j["architecture"] = architecture;
    j["vocab"] = vocab_size;
    j["width"] = hidden_size;
    j["torch_dtype"] = torch_dtype;
    j.erase("dtype");
    return j;
}

// Layer i's tensors are 'l<i>.norm1', 'l<i>.mix.left.*', 'l<i>.mix.right.*', 'l<i>.norm2', 'l<i>.mlp.*'; the
// norm weights are stored around zero (weight_offset 1).  A model-wide `bias_buckets` key, when present, fixes
// the rows of the distance-bias tables (random weights need it); otherwise the checkpoint's tables decide.
ModelPlan kazedra_plan(const KazedraConfig& cfg) {
    const int64_t d = cfg.hidden_size;
    ModelPlan plan;
    plan.architecture = cfg.architecture;
    plan.hidden_size = d;
    plan.vocab_size = cfg.vocab_size;
    plan.max_positions = cfg.max_position_embeddings;
    auto norm = [&](const std::string& tensor) {
        PartSpec n;
        n.kind = "rmsnorm";
        n.params["size"] = d;
        n.params["eps"] = cfg.norm_eps;
        n.params["weight_offset"] = 1.0;
        n.tensors = {{"weight", tensor}};
        return n;
    };
    const int64_t buckets = cfg.raw.is_object() ? cfg.raw.get_int("bias_buckets", 0) : 0;
    for (size_t i = 0; i < cfg.layers.size(); ++i) {
        const KazedraConfig::Layer& l = cfg.layers[i];
        const std::string p = "l" + std::to_string(i) + ".", a = p + "mix.left.", b = p + "mix.right.";
        PartSpec left;
        left.kind = "sink_bias_attention";
        left.params["hidden_size"] = d;
        left.params["num_heads"] = l.left.heads;
        left.params["num_kv_heads"] = l.left.kv_heads;
        left.params["head_dim"] = l.left.dim;
        left.params["scale"] = l.left.scale;
        left.params["norm_eps"] = cfg.norm_eps;
        left.params["q_temp_coef"] = l.left.temp_coef;
        left.params["q_temp_every"] = l.left.temp_every;
        left.params["bias_max_distance"] = l.left.bias_max;
        left.params["bias_buckets"] = buckets;
        left.tensors = {{"q_proj", a + "q"}, {"q_bias", a + "q.b"}, {"k_proj", a + "k"}, {"k_bias", a + "k.b"}, {"q_norm", a + "q.norm"},
                        {"k_norm", a + "k.norm"}, {"rel_bias", a + "rel"}, {"sink", a + "sink"}, {"o_proj", a + "o"}, {"o_bias", a + "o.b"}};
        PartSpec right;
        right.kind = "gated_delta_rule";
        right.params["hidden_size"] = d;
        right.params["num_heads"] = l.right.heads;
        right.params["num_kv_heads"] = l.right.kv_heads;
        right.params["key_dim"] = l.right.dim;
        right.params["value_dim"] = l.right.vdim;
        right.params["conv_taps"] = l.right.conv;
        right.params["norm_eps"] = cfg.norm_eps;
        right.tensors = {{"q_proj", b + "q"}, {"q_conv", b + "q.conv"}, {"k_proj", b + "k"}, {"k_conv", b + "k.conv"}, {"v_proj", b + "v"},
                         {"v_conv", b + "v.conv"}, {"beta_proj", b + "b"}, {"a_log", b + "A_log"}, {"out_norm", b + "norm"}, {"a_proj", b + "a"},
                         {"dt_bias", b + "dt_bias"}, {"gate_proj", b + "g"}, {"o_proj", b + "o"}};
        LayerSpec layer;
        layer.block = "parallel_prenorm";
        layer.block_params["left_scale"] = l.left_scale;
        layer.block_params["right_scale"] = l.right_scale;
        layer.block_params["has_ffn"] = l.ff > 0;
        layer.parts = {{"mixer_norm", norm(p + "norm1")}, {"left", left}, {"right", right}};
        if (l.ff > 0) {
            PartSpec ffn;
            ffn.kind = "swiglu";
            ffn.params["hidden_size"] = d;
            ffn.params["intermediate_size"] = l.ff;
            ffn.tensors = {{"gate_proj", p + "mlp.gate"}, {"up_proj", p + "mlp.up"}, {"down_proj", p + "mlp.down"}};
            layer.parts.emplace_back("ffn_norm", norm(p + "norm2"));
            layer.parts.emplace_back("feed_forward", ffn);
        }
        plan.layers.push_back(layer);
    }
    plan.embedding.kind = "token_embedding";
    plan.embedding.params["vocab_size"] = cfg.vocab_size;
    plan.embedding.params["hidden_size"] = d;
    plan.embedding.tensors = {{"weight", "embed"}};
    plan.final_norm = norm("final.norm");
    plan.head.kind = "linear_head";
    plan.head.params["vocab_size"] = cfg.vocab_size;
    plan.head.params["hidden_size"] = d;
    plan.head.params["scale"] = cfg.logit_scale;
    plan.head.tensors = {{"weight", "head"}};
    return plan;
}

// ------------------------------------------------------------------------------------ Kuzipel
KuzipelConfig KuzipelConfig::from_json(const Json& d, const std::string& where) {
    KuzipelConfig c;
    c.architecture = d.get_string("architecture", "Kuzipel");
    c.vocab_size = positive("vocab", require_int(d, "vocab", where), where);
    c.hidden_size = positive("width", require_int(d, "width", where), where);
    c.max_position_embeddings = positive("max_positions", d.get_int("max_positions", 1 << 16), where);
    c.torch_dtype = d.get_string("torch_dtype", d.get_string("dtype", "bfloat16"));
    if (c.torch_dtype != "bfloat16" && c.torch_dtype != "float32")
        bad(where + ": torch_dtype '" + c.torch_dtype + "' is not supported (bfloat16 or float32)");
    if (const Json* eos = d.find("eos_token_id")) {
        if (eos->is_array()) {
            for (const auto& e : eos->items())
                if (e.is_int()) c.eos_token_ids.push_back((int)e.as_int());
        } else if (eos->is_int()) {
            c.eos_token_ids.push_back((int)eos->as_int());
        }
    }
    c.bos_token_id = d.get_int("bos_token_id", -1);
    c.raw = d;
    c.norm_eps = require_float(require_object(d, "norm", where), "eps", where + ": norm");
    if (!(c.norm_eps > 0)) bad(where + ": norm.eps must be positive");
    c.residual_mult = d.get_double("residual_mult", 1.0);
    const Json& layers = require(d, "layers", where);
    if (!layers.is_array() || layers.size() == 0) bad(where + ": 'layers' must be a non-empty list");
    int i = 0;
    for (const Json& lj : layers.items()) {
        const std::string lw = where + ": layers[" + std::to_string(i++) + "]";
        if (!lj.is_object()) bad(lw + " must be an object");
        Layer l;
        l.type = lj.get_string("type", "");
        const Json& m = require_object(lj, "mixer", lw);
        const std::string mw = lw + ".mixer";
        l.heads = positive("heads", require_int(m, "heads", mw), mw);
        l.dim = positive("dim", require_int(m, "dim", mw), mw);
        if (l.type == "latent_attention") {
            l.rot_dim = positive("rot_dim", require_int(m, "rot_dim", mw), mw);
            l.vdim = positive("vdim", require_int(m, "vdim", mw), mw);
            l.kv_rank = positive("kv_rank", require_int(m, "kv_rank", mw), mw);
            l.q_rank = positive("q_rank", require_int(m, "q_rank", mw), mw);
            l.scale = require_float(m, "scale", mw);
            const Json& rot = require_object(m, "rot", mw);
            l.rot_base = require_float(rot, "base", mw + ".rot");
            l.rot_dims = positive("dims", rot.get_int("dims", l.rot_dim), mw + ".rot");
            if (!(l.rot_base > 0)) bad(mw + ".rot: base must be positive");
            if (l.rot_dims % 2 || l.rot_dims > l.rot_dim)
                bad(mw + ".rot: dims " + std::to_string(l.rot_dims) + " must be even and at most rot_dim " + std::to_string(l.rot_dim));
        } else if (l.type == "wkv") {
            l.decay_rank = m.get_int("decay_rank", 0);
            if (l.decay_rank < 0) bad(mw + ": decay_rank must not be negative");
        } else {
            bad(lw + ": unknown layer type '" + l.type + "' (known: latent_attention, wkv)");
        }
        if (const Json* f = lj.find("mlp")) {
            if (f->is_object()) {
                const std::string fw = lw + ".mlp", kind = f->get_string("kind", "");
                if (kind != "moe") bad(fw + ": unknown kind '" + kind + "' (known: moe)");
                l.has_mlp = true;
                l.expert_ff = positive("ff", require_int(require_object(*f, "expert", fw), "ff", fw + ".expert"), fw + ".expert");
                const Json& r = require_object(*f, "router", fw);
                l.experts = positive("experts", require_int(r, "experts", fw + ".router"), fw + ".router");
                l.top = positive("top", require_int(r, "top", fw + ".router"), fw + ".router");
                if (l.top > l.experts) bad(fw + ".router: top " + std::to_string(l.top) + " exceeds the " + std::to_string(l.experts) + " experts");
                if (const Json* s = f->find("shared")) {
                    if (s->is_object()) l.shared_ff = positive("ff", require_int(*s, "ff", fw + ".shared"), fw + ".shared");
                    else if (!s->is_null()) bad(fw + ".shared must be an object or null");
                }
            } else if (!f->is_null()) {
                bad(lw + ".mlp must be an object or null");
            }
        }
        c.layers.push_back(l);
    }
    c.num_hidden_layers = (int64_t)c.layers.size();
    if (const Json* lp = d.find("loop")) {
        if (lp->is_object()) {
            c.has_loop = true;
            c.loop_start = require_int(*lp, "start", where + ": loop");
            c.loop_stop = require_int(*lp, "stop", where + ": loop");
            c.loop_times = positive("times", require_int(*lp, "times", where + ": loop"), where + ": loop");
            if (c.loop_start < 0 || c.loop_stop <= c.loop_start || c.loop_stop > c.num_hidden_layers)
                bad(where + ": loop: 0 <= start < stop <= " + std::to_string(c.num_hidden_layers) + " is required, got " +
                    std::to_string(c.loop_start) + " and " + std::to_string(c.loop_stop));
        } else if (!lp->is_null()) {
            bad(where + ": 'loop' must be an object or null");
        }
    }
    return c;
}

Json KuzipelConfig::to_json() const {
    Json j = raw.is_object() ? raw : Json::object();
    j["architecture"] = architecture;
    j["vocab"] = vocab_size;
    j["width"] = hidden_size;
    j["torch_dtype"] = torch_dtype;
    j.erase("dtype");
    return j;
}

std::vector<int> KuzipelConfig::run_order() const {
    std::vector<int> o;
    const int L = (int)layers.size();
    if (!has_loop) {
        for (int i = 0; i < L; ++i) o.push_back(i);
        return o;
    }
    for (int i = 0; i < (int)loop_start; ++i) o.push_back(i);
    for (int64_t pass = 0; pass < loop_times; ++pass) {
        o.push_back(L);
        for (int i = (int)loop_start; i < (int)loop_stop; ++i) o.push_back(i);
    }
    for (int i = (int)loop_stop; i < L; ++i) o.push_back(i);
    return o;
}

// Layer i's tensors are 'l<i>.norm1', 'l<i>.mix.*', 'l<i>.norm2', 'l<i>.mlp.*', 'l<i>.ls1', 'l<i>.ls2'; the map before
// every pass of a repeated run is 'loop.in'.  A layer that runs several times gets a cache per run.
ModelPlan kuzipel_plan(const KuzipelConfig& cfg) {
    const int64_t d = cfg.hidden_size;
    ModelPlan plan;
    plan.architecture = cfg.architecture;
    plan.hidden_size = d;
    plan.vocab_size = cfg.vocab_size;
    plan.max_positions = cfg.max_position_embeddings;
    auto norm = [&](const std::string& tensor) {
        PartSpec n;
        n.kind = "layernorm";
        n.params["size"] = d;
        n.params["eps"] = cfg.norm_eps;
        n.tensors = {{"weight", tensor}};
        return n;
    };
    for (size_t i = 0; i < cfg.layers.size(); ++i) {
        const KuzipelConfig::Layer& l = cfg.layers[i];
        const std::string p = "l" + std::to_string(i) + ".", a = p + "mix.", f = p + "mlp.";
        PartSpec mixer;
        mixer.params["hidden_size"] = d;
        mixer.params["num_heads"] = l.heads;
        mixer.params["head_dim"] = l.dim;
        mixer.params["norm_eps"] = cfg.norm_eps;
        if (l.type == "latent_attention") {
            mixer.kind = "latent_attention";
            mixer.params["rot_dim"] = l.rot_dim;
            mixer.params["value_dim"] = l.vdim;
            mixer.params["kv_rank"] = l.kv_rank;
            mixer.params["q_rank"] = l.q_rank;
            mixer.params["scale"] = l.scale;
            mixer.params["rot_base"] = l.rot_base;
            mixer.params["rot_dims"] = l.rot_dims;
            mixer.params["max_positions"] = cfg.max_position_embeddings;
            mixer.tensors = {{"q_down", a + "dq"}, {"q_norm", a + "dq.norm"}, {"q_up", a + "uq"}, {"kv_down", a + "dkv"},
                             {"kv_norm", a + "dkv.norm"}, {"k_up", a + "uk"}, {"v_up", a + "uv"}, {"o_proj", a + "o"}};
        } else {
            mixer.kind = "wkv";
            mixer.params["decay_rank"] = l.decay_rank;
            mixer.tensors = {{"mu_r", a + "mu.r"}, {"mu_k", a + "mu.k"}, {"mu_v", a + "mu.v"}, {"mu_g", a + "mu.g"}, {"mu_w", a + "mu.w"},
                             {"r_proj", a + "r"}, {"k_proj", a + "k"}, {"v_proj", a + "v"}, {"g_proj", a + "g"}, {"decay_down", a + "w1"},
                             {"decay_up", a + "w2"}, {"decay_bias", a + "w0"}, {"bonus", a + "u"}, {"out_norm", a + "norm"}, {"o_proj", a + "o"}};
        }
        LayerSpec layer;
        layer.block = "scaled_prenorm";
        layer.block_params["hidden_size"] = d;
        layer.block_params["residual_mult"] = cfg.residual_mult;
        layer.block_params["has_ffn"] = l.has_mlp;
        layer.block_tensors = {{"mixer_scale", p + "ls1"}};
        layer.parts = {{"mixer_norm", norm(p + "norm1")}, {"mixer", mixer}};
        if (l.has_mlp) {
            PartSpec ffn;
            ffn.kind = "routed_experts";
            ffn.params["hidden_size"] = d;
            ffn.params["num_experts"] = l.experts;
            ffn.params["top_k"] = l.top;
            ffn.params["expert_size"] = l.expert_ff;
            ffn.params["shared_size"] = l.shared_ff;
            ffn.tensors = {{"router", f + "router"}, {"router_bias", f + "router.b"}};
            for (int64_t e = 0; e < l.experts; ++e) {
                const std::string n = std::to_string(e), t = f + "e" + n + ".";
                ffn.tensors.emplace_back("gate_" + n, t + "gate");
                ffn.tensors.emplace_back("up_" + n, t + "up");
                ffn.tensors.emplace_back("down_" + n, t + "down");
            }
            if (l.shared_ff > 0) {
                ffn.tensors.emplace_back("shared_gate", f + "shared.gate");
                ffn.tensors.emplace_back("shared_up", f + "shared.up");
                ffn.tensors.emplace_back("shared_down", f + "shared.down");
                ffn.tensors.emplace_back("shared_mix", f + "shared.sg");
            }
            layer.block_tensors.emplace_back("ffn_scale", p + "ls2");
            layer.parts.emplace_back("ffn_norm", norm(p + "norm2"));
            layer.parts.emplace_back("feed_forward", ffn);
        }
        plan.layers.push_back(layer);
    }
    if (cfg.has_loop) {
        LayerSpec inject;
        inject.block = "stream_reinject";
        inject.block_params["hidden_size"] = d;
        inject.block_tensors = {{"weight", "loop.in"}};
        plan.layers.push_back(inject);
        plan.has_order = true;
        plan.order = cfg.run_order();
    }
    plan.embedding.kind = "token_embedding";
    plan.embedding.params["vocab_size"] = cfg.vocab_size;
    plan.embedding.params["hidden_size"] = d;
    plan.embedding.tensors = {{"weight", "embed"}};
    plan.final_norm = norm("final.norm");
    plan.head.kind = "linear_head";
    plan.head.params["vocab_size"] = cfg.vocab_size;
    plan.head.params["hidden_size"] = d;
    plan.head.tensors = {{"weight", "head"}};
    return plan;
}

// ------------------------------------------------------------------------------------ Pemidra
PemidraConfig PemidraConfig::from_json(const Json& d, const std::string& where) {
    PemidraConfig c;
    c.architecture = d.get_string("architecture", "Pemidra");
    c.vocab_size = positive("vocab", require_int(d, "vocab", where), where);
    c.hidden_size = positive("width", require_int(d, "width", where), where);
    c.max_position_embeddings = positive("max_positions", d.get_int("max_positions", 1 << 20), where);
    c.torch_dtype = d.get_string("torch_dtype", d.get_string("dtype", "bfloat16"));
    if (c.torch_dtype != "bfloat16" && c.torch_dtype != "float32")
        bad(where + ": torch_dtype '" + c.torch_dtype + "' is not supported (bfloat16 or float32)");
    if (const Json* eos = d.find("eos_token_id")) {
        if (eos->is_array()) {
            for (const auto& e : eos->items())
                if (e.is_int()) c.eos_token_ids.push_back((int)e.as_int());
        } else if (eos->is_int()) {
            c.eos_token_ids.push_back((int)eos->as_int());
        }
    }
    c.bos_token_id = d.get_int("bos_token_id", -1);
    c.raw = d;
    c.norm_eps = require_float(require_object(d, "norm", where), "eps", where + ": norm");
    if (!(c.norm_eps > 0)) bad(where + ": norm.eps must be positive");
    c.postln_alpha = require_float(d, "postln_alpha", where);
    const Json& layers = require(d, "layers", where);
    if (!layers.is_array() || layers.size() == 0) bad(where + ": 'layers' must be a non-empty list");
    int i = 0;
    for (const Json& lj : layers.items()) {
        const std::string lw = where + ": layers[" + std::to_string(i++) + "]";
        if (!lj.is_object()) bad(lw + " must be an object");
        Layer l;
        l.type = lj.get_string("type", "");
        const Json& m = require_object(lj, "mixer", lw);
        const std::string mw = lw + ".mixer";
        if (l.type == "retention") {
            l.heads = positive("heads", require_int(m, "heads", mw), mw);
            l.dim = positive("dim", require_int(m, "dim", mw), mw);
            l.vdim = positive("vdim", m.get_int("vdim", l.dim), mw);
            const Json& dec = require(m, "decay", mw);
            if (!dec.is_array() || (int64_t)dec.size() != l.heads) bad(mw + ": 'decay' must list a number per head (" + std::to_string(l.heads) + ")");
            for (const Json& e : dec.items()) {
                if (!e.is_number()) bad(mw + ": 'decay' must list numbers");
                l.decay.push_back(e.as_double());
            }
        } else if (l.type == "general_delta") {
            l.heads = positive("heads", require_int(m, "heads", mw), mw);
            l.dim = positive("dim", require_int(m, "dim", mw), mw);
            l.vdim = l.dim;
            l.decay_rank = m.get_int("decay_rank", 0);
        } else if (l.type == "parallel") {
            const Json& a = require_object(m, "left", mw);
            const Json& b = require_object(m, "right", mw);
            const std::string aw = mw + ".left", bw = mw + ".right";
            l.left.heads = positive("heads", require_int(a, "heads", aw), aw);
            l.left.kv_heads = positive("kv_heads", a.get_int("kv_heads", l.left.heads), aw);
            l.left.dim = positive("dim", require_int(a, "dim", aw), aw);
            l.left.vdim = positive("vdim", a.get_int("vdim", l.left.dim), aw);
            l.left.scale = require_float(a, "scale", aw);
            if (!(l.left.scale > 0)) bad(aw + ": scale must be positive");
            if (l.left.heads % l.left.kv_heads) bad(aw + ": heads " + std::to_string(l.left.heads) + " must be a multiple of kv_heads " + std::to_string(l.left.kv_heads));
            if (const Json* mask = a.find("mask"))
                if (mask->is_object()) l.left.chunk = positive("size", require_int(*mask, "size", aw + ".mask"), aw + ".mask");
            if (const Json* rot = a.find("rot"))
                if (rot->is_object()) {
                    l.left.rot_dims = positive("dims", require_int(*rot, "dims", aw + ".rot"), aw + ".rot");
                    l.left.rot_base = require_float(*rot, "base", aw + ".rot");
                    if (l.left.rot_dims % 2 || l.left.rot_dims > l.left.dim) bad(aw + ".rot: dims " + std::to_string(l.left.rot_dims) + " must be even and within dim " + std::to_string(l.left.dim));
                }
            l.right.heads = positive("heads", require_int(b, "heads", bw), bw);
            l.right.kv_heads = positive("kv_heads", b.get_int("kv_heads", l.right.heads), bw);
            l.right.dim = positive("dim", require_int(b, "dim", bw), bw);
            l.right.vdim = positive("vdim", b.get_int("vdim", l.right.dim), bw);
            l.right.conv = positive("conv", require_int(b, "conv", bw), bw);
            l.right.decay_rank = b.get_int("decay_rank", 0);
            l.right.gate_rank = b.get_int("gate_rank", 0);
            if (l.right.heads % l.right.kv_heads) bad(bw + ": heads " + std::to_string(l.right.heads) + " must be a multiple of kv_heads " + std::to_string(l.right.kv_heads));
        } else {
            bad(lw + ": unknown layer type '" + l.type + "' (known: retention, general_delta, parallel)");
        }
        if (const Json* f = lj.find("mlp")) {
            if (f->is_object()) {
                const std::string kind = f->get_string("kind", "");
                if (kind != "dense") bad(lw + ".mlp: unknown kind '" + kind + "' (known: dense)");
                l.ff = positive("ff", require_int(*f, "ff", lw + ".mlp"), lw + ".mlp");
            } else if (!f->is_null()) {
                bad(lw + ".mlp must be an object or null");
            }
        }
        c.layers.push_back(l);
    }
    c.num_hidden_layers = (int64_t)c.layers.size();
    return c;
}

Json PemidraConfig::to_json() const {
    Json j = raw.is_object() ? raw : Json::object();
    j["architecture"] = architecture;
    j["vocab"] = vocab_size;
    j["width"] = hidden_size;
    j["torch_dtype"] = torch_dtype;
    j.erase("dtype");
    return j;
}

// Layer i's tensors are 'l<i>.norm1' (+ '.b'), 'l<i>.ls1', 'l<i>.mix.*', and with a feed-forward 'l<i>.norm2' (+ '.b'),
// 'l<i>.ls2', 'l<i>.mlp.*'; a pair's mixers live under 'mix.left.' and 'mix.right.'.
ModelPlan pemidra_plan(const PemidraConfig& cfg) {
    const int64_t d = cfg.hidden_size;
    ModelPlan plan;
    plan.architecture = cfg.architecture;
    plan.hidden_size = d;
    plan.vocab_size = cfg.vocab_size;
    plan.max_positions = cfg.max_position_embeddings;
    auto norm = [&](const std::string& tensor) {
        PartSpec n;
        n.kind = "layernorm";
        n.params["size"] = d;
        n.params["eps"] = cfg.norm_eps;
        n.params["bias"] = true;
        n.tensors = {{"weight", tensor}, {"bias", tensor + ".b"}};
        return n;
    };
    for (size_t i = 0; i < cfg.layers.size(); ++i) {
        const PemidraConfig::Layer& l = cfg.layers[i];
        const std::string p = "l" + std::to_string(i) + ".", a = p + "mix.";
        LayerSpec layer;
        layer.block = "postnorm";
        layer.block_params["hidden_size"] = d;
        layer.block_params["residual_mult"] = cfg.postln_alpha;
        layer.block_params["has_ffn"] = l.ff > 0;
        layer.block_params["pair"] = l.type == "parallel";
        layer.block_params["pair_eps"] = cfg.norm_eps;
        layer.block_tensors = {{"mixer_scale", p + "ls1"}};
        layer.parts = {{"mixer_norm", norm(p + "norm1")}};
        if (l.type == "retention") {
            PartSpec m;
            m.kind = "retention";
            m.params["hidden_size"] = d;
            m.params["num_heads"] = l.heads;
            m.params["key_dim"] = l.dim;
            m.params["value_dim"] = l.vdim;
            m.params["norm_eps"] = cfg.norm_eps;
            Json dec = Json::array();
            for (double v : l.decay) dec.push(Json(v));
            m.params["decay"] = dec;
            m.tensors = {{"q_proj", a + "q"}, {"k_proj", a + "k"}, {"v_proj", a + "v"}, {"gate_proj", a + "g"}, {"o_proj", a + "o"}};
            layer.parts.emplace_back("mixer", m);
        } else if (l.type == "general_delta") {
            PartSpec m;
            m.kind = "general_delta";
            m.params["hidden_size"] = d;
            m.params["num_heads"] = l.heads;
            m.params["head_dim"] = l.dim;
            m.params["norm_eps"] = cfg.norm_eps;
            m.params["decay_rank"] = l.decay_rank;
            m.tensors = {{"r_proj", a + "r"}, {"k_proj", a + "k"}, {"v_proj", a + "v"}, {"gate_proj", a + "g"}, {"a_proj", a + "a"},
                         {"a_bias", a + "a.b"}, {"decay_down", a + "w1"}, {"decay_up", a + "w2"}, {"decay_bias", a + "w0"},
                         {"out_norm", a + "norm"}, {"o_proj", a + "o"}};
            layer.parts.emplace_back("mixer", m);
        } else {
            const std::string la = a + "left.", rb = a + "right.";
            PartSpec left;
            left.kind = "gated_head_attention";
            left.params["hidden_size"] = d;
            left.params["num_heads"] = l.left.heads;
            left.params["num_kv_heads"] = l.left.kv_heads;
            left.params["head_dim"] = l.left.dim;
            left.params["value_dim"] = l.left.vdim;
            left.params["scale"] = l.left.scale;
            left.params["norm_eps"] = cfg.norm_eps;
            left.params["qk_norm"] = true;
            left.params["value_norm"] = true;
            left.params["rot_dims"] = l.left.rot_dims;
            left.params["rot_base"] = l.left.rot_base;
            left.params["head_temp"] = true;
            left.params["chunk"] = l.left.chunk;
            left.params["sink"] = true;
            left.params["head_gate"] = true;
            left.tensors = {{"q_proj", la + "q"}, {"k_proj", la + "k"}, {"v_proj", la + "v"}, {"q_norm", la + "q.norm"}, {"k_norm", la + "k.norm"},
                            {"head_temp", la + "temp"}, {"gate_proj", la + "g"}, {"o_proj", la + "o"}};
            PartSpec right;
            right.kind = "channel_delta_rule";
            right.params["hidden_size"] = d;
            right.params["num_heads"] = l.right.heads;
            right.params["num_kv_heads"] = l.right.kv_heads;
            right.params["key_dim"] = l.right.dim;
            right.params["value_dim"] = l.right.vdim;
            right.params["conv_taps"] = l.right.conv;
            right.params["norm_eps"] = cfg.norm_eps;
            right.params["decay_rank"] = l.right.decay_rank;
            right.params["gate_rank"] = l.right.gate_rank;
            right.tensors = {{"q_proj", rb + "q"}, {"q_conv", rb + "q.conv"}, {"k_proj", rb + "k"}, {"k_conv", rb + "k.conv"}, {"v_proj", rb + "v"},
                             {"v_conv", rb + "v.conv"}, {"beta_proj", rb + "b"}, {"a_log", rb + "A_log"}, {"out_norm", rb + "norm"},
                             {"decay_down", rb + "a1"}, {"decay_up", rb + "a2"}, {"dt_bias", rb + "dt_bias"}, {"gate_down", rb + "g1"},
                             {"gate_up", rb + "g2"}, {"o_proj", rb + "o"}};
            layer.parts.emplace_back("left", left);
            layer.parts.emplace_back("right", right);
            layer.block_tensors.emplace_back("left_out", la + "out");
            layer.block_tensors.emplace_back("right_out", rb + "out");
        }
        if (l.ff > 0) {
            PartSpec ffn;
            ffn.kind = "gated_mlp";
            ffn.params["hidden_size"] = d;
            ffn.params["intermediate_size"] = l.ff;
            ffn.params["activation"] = "gelu_tanh";
            ffn.tensors = {{"gate_proj", p + "mlp.gate"}, {"up_proj", p + "mlp.up"}, {"down_proj", p + "mlp.down"}};
            layer.block_tensors.emplace_back("ffn_scale", p + "ls2");
            layer.parts.emplace_back("ffn_norm", norm(p + "norm2"));
            layer.parts.emplace_back("feed_forward", ffn);
        }
        plan.layers.push_back(layer);
    }
    plan.embedding.kind = "token_embedding";
    plan.embedding.params["vocab_size"] = cfg.vocab_size;
    plan.embedding.params["hidden_size"] = d;
    plan.embedding.tensors = {{"weight", "embed"}};
    plan.final_norm = norm("final.norm");
    plan.head.kind = "linear_head";
    plan.head.params["vocab_size"] = cfg.vocab_size;
    plan.head.params["hidden_size"] = d;
    plan.head.tensors = {{"weight", "head"}};
    return plan;
}

// ------------------------------------------------------------------------------------ Nizorax
NizoraxConfig NizoraxConfig::from_json(const Json& d, const std::string& where) {
    NizoraxConfig c;
    c.architecture = d.get_string("architecture", "Nizorax");
    c.vocab_size = positive("vocab", require_int(d, "vocab", where), where);
    c.hidden_size = positive("width", require_int(d, "width", where), where);
    c.max_position_embeddings = positive("max_positions", d.get_int("max_positions", 1 << 20), where);
    c.torch_dtype = d.get_string("torch_dtype", d.get_string("dtype", "bfloat16"));
    if (c.torch_dtype != "bfloat16" && c.torch_dtype != "float32")
        bad(where + ": torch_dtype '" + c.torch_dtype + "' is not supported (bfloat16 or float32)");
    if (const Json* eos = d.find("eos_token_id")) {
        if (eos->is_array()) {
            for (const auto& e : eos->items())
                if (e.is_int()) c.eos_token_ids.push_back((int)e.as_int());
        } else if (eos->is_int()) {
            c.eos_token_ids.push_back((int)eos->as_int());
        }
    }
    c.bos_token_id = d.get_int("bos_token_id", -1);
    c.raw = d;
    c.norm_eps = require_float(require_object(d, "norm", where), "eps", where + ": norm");
    if (!(c.norm_eps > 0)) bad(where + ": norm.eps must be positive");
    auto optional_object = [&](const Json& in, const char* key, const std::string& w) -> const Json* {
        const Json* v = in.find(key);
        if (!v || v->is_null()) return nullptr;
        if (!v->is_object()) bad(w + ": '" + key + "' must be an object or null");
        return v;
    };
    if (const Json* e = optional_object(d, "embedding", where)) c.embedding_scale = e->get_double("scale", 1.0);
    c.logit_scale = d.get_double("logit_scale", 1.0);
    if (const Json* cn = optional_object(d, "canon", where)) {
        c.canon_taps = positive("taps", require_int(*cn, "taps", where + ": canon"), where + ": canon");
        if (c.canon_taps > 64) bad(where + ": canon.taps must be at most 64");
    }
    const Json& layers = require(d, "layers", where);
    if (!layers.is_array() || layers.size() == 0) bad(where + ": 'layers' must be a non-empty list");
    int i = 0;
    for (const Json& lj : layers.items()) {
        const std::string lw = where + ": layers[" + std::to_string(i++) + "]";
        if (!lj.is_object()) bad(lw + " must be an object");
        Layer l;
        l.type = lj.get_string("type", "");
        const Json& m = require_object(lj, "mixer", lw);
        const std::string mw = lw + ".mixer";
        l.heads = positive("heads", require_int(m, "heads", mw), mw);
        l.dim = positive("dim", require_int(m, "dim", mw), mw);
        l.vdim = positive("vdim", m.get_int("vdim", l.dim), mw);
        if (l.type == "attention") {
            l.kv_heads = positive("kv_heads", m.get_int("kv_heads", l.heads), mw);
            if (l.heads % l.kv_heads) bad(mw + ": " + std::to_string(l.heads) + " heads are not a multiple of " + std::to_string(l.kv_heads) + " kv_heads");
            l.diff = require_float(m, "diff", mw);
            l.scale = m.find("scale") ? require_float(m, "scale", mw) : 1.0 / std::sqrt((double)l.dim);
            if (!(l.scale > 0)) bad(mw + ": scale must be positive");
            if (const Json* mask = optional_object(m, "mask", mw)) l.window = positive("size", require_int(*mask, "size", mw + ".mask"), mw + ".mask");
            if (const Json* rot = optional_object(m, "rot", mw)) {
                const std::string rw = mw + ".rot";
                l.rot_base = require_float(*rot, "base", rw);
                l.rot_dims = positive("dims", require_int(*rot, "dims", rw), rw);
                if (!(l.rot_base > 0)) bad(rw + ": base must be positive");
                if (l.rot_dims % 2 || l.rot_dims > l.dim) bad(rw + ": dims " + std::to_string(l.rot_dims) + " must be even and at most dim " + std::to_string(l.dim));
                if (const Json* sc = optional_object(*rot, "scaling", rw)) {
                    const std::string sw = rw + ".scaling";
                    l.rot_scaled = true;
                    l.rot_factor = require_float(*sc, "factor", sw);
                    l.rot_low = require_float(*sc, "low", sw);
                    l.rot_high = require_float(*sc, "high", sw);
                    l.rot_original = require_float(*sc, "original", sw);
                    if (!(l.rot_factor > 0) || !(l.rot_low > 0) || !(l.rot_high > l.rot_low) || !(l.rot_original > 0))
                        bad(sw + ": factor > 0, 0 < low < high and original > 0 are required");
                }
            }
        } else if (l.type == "lightning") {
            l.kv_heads = l.heads;
            const Json& dj = require(m, "decay", mw);
            if (!dj.is_array() || (int64_t)dj.size() != l.heads) bad(mw + ": 'decay' must list a number per head");
            for (const Json& e : dj.items()) {
                if (!e.is_number()) bad(mw + ": 'decay' must list numbers");
                l.decay.push_back(e.as_double());
            }
        } else {
            bad(lw + ": unknown layer type '" + l.type + "' (known: attention, lightning)");
        }
        if (const Json* f = optional_object(lj, "mlp", lw)) {
            const std::string fw = lw + ".mlp";
            l.mlp = f->get_string("kind", "");
            if (l.mlp == "dense") {
                l.ff = positive("ff", require_int(*f, "ff", fw), fw);
            } else if (l.mlp == "moe") {
                l.expert_ff = positive("ff", require_int(require_object(*f, "expert", fw), "ff", fw + ".expert"), fw + ".expert");
                const Json& r = require_object(*f, "router", fw);
                const std::string rw = fw + ".router";
                l.experts = positive("experts", require_int(r, "experts", rw), rw);
                l.top = positive("top", require_int(r, "top", rw), rw);
                if (l.top > l.experts) bad(rw + ": top " + std::to_string(l.top) + " exceeds the " + std::to_string(l.experts) + " experts");
                l.route_scale = r.get_double("scale", 1.0);
                if (const Json* g = optional_object(r, "groups", rw)) {
                    l.groups = positive("count", require_int(*g, "count", rw + ".groups"), rw + ".groups");
                    l.keep = positive("keep", require_int(*g, "keep", rw + ".groups"), rw + ".groups");
                    if (l.experts % l.groups || l.keep > l.groups || l.top > l.keep * (l.experts / l.groups))
                        bad(rw + ".groups: count must divide the experts, keep be at most count, and the kept groups hold `top` experts");
                }
                if (const Json* sh = optional_object(*f, "shared", fw)) l.shared_ff = positive("ff", require_int(*sh, "ff", fw + ".shared"), fw + ".shared");
            } else {
                bad(fw + ": unknown kind '" + l.mlp + "' (known: dense, moe)");
            }
        }
        c.layers.push_back(l);
    }
    c.num_hidden_layers = (int64_t)c.layers.size();
    if (const Json* lp = optional_object(d, "loop", where)) {
        c.has_loop = true;
        c.loop_start = require_int(*lp, "start", where + ": loop");
        c.loop_stop = require_int(*lp, "stop", where + ": loop");
        c.loop_times = positive("times", require_int(*lp, "times", where + ": loop"), where + ": loop");
        if (c.loop_start < 0 || c.loop_stop <= c.loop_start || c.loop_stop > c.num_hidden_layers)
            bad(where + ": loop: 0 <= start < stop <= " + std::to_string(c.num_hidden_layers) + " is required, got " + std::to_string(c.loop_start) +
                " and " + std::to_string(c.loop_stop));
    }
    return c;
}

Json NizoraxConfig::to_json() const {
    Json j = raw.is_object() ? raw : Json::object();
    j["architecture"] = architecture;
    j["vocab"] = vocab_size;
    j["width"] = hidden_size;
    j["torch_dtype"] = torch_dtype;
    j.erase("dtype");
    return j;
}

std::vector<int> NizoraxConfig::run_order() const {
    std::vector<int> o;
    const int L = (int)layers.size();
    const int a = has_loop ? (int)loop_start : L, b = has_loop ? (int)loop_stop : L;
    for (int i = 0; i < a; ++i) o.push_back(i);
    for (int64_t pass = 0; has_loop && pass < loop_times; ++pass)
        for (int i = a; i < b; ++i) o.push_back(i);
    for (int i = b; i < L; ++i) o.push_back(i);
    return o;
}

// Layer i's tensors are 'l<i>.norm1', 'l<i>.norm1b' (the norms before and after the mixer, each with '.b'), 'l<i>.canon1',
// 'l<i>.mix.*', and with a feed-forward 'l<i>.norm2', 'l<i>.norm2b', 'l<i>.canon2', 'l<i>.mlp.*'.  A layer that runs
// several times gets a cache and a state per run.
ModelPlan nizorax_plan(const NizoraxConfig& cfg) {
    const int64_t d = cfg.hidden_size;
    ModelPlan plan;
    plan.architecture = cfg.architecture;
    plan.hidden_size = d;
    plan.vocab_size = cfg.vocab_size;
    plan.max_positions = cfg.max_position_embeddings;
    auto norm = [&](const std::string& tensor) {
        PartSpec n;
        n.kind = "layernorm";
        n.params["size"] = d;
        n.params["eps"] = cfg.norm_eps;
        n.params["bias"] = true;
        n.tensors = {{"weight", tensor}, {"bias", tensor + ".b"}};
        return n;
    };
    auto conv = [&](const std::string& tensor) {
        PartSpec c;
        c.kind = "residual_conv";
        c.params["hidden_size"] = d;
        c.params["taps"] = cfg.canon_taps;
        c.tensors = {{"weight", tensor}};
        return c;
    };
    const bool has_conv = cfg.canon_taps > 0;
    for (size_t i = 0; i < cfg.layers.size(); ++i) {
        const NizoraxConfig::Layer& l = cfg.layers[i];
        const std::string p = "l" + std::to_string(i) + ".", a = p + "mix.", f = p + "mlp.";
        PartSpec mixer;
        mixer.params["hidden_size"] = d;
        mixer.params["num_heads"] = l.heads;
        mixer.params["value_dim"] = l.vdim;
        mixer.params["norm_eps"] = cfg.norm_eps;
        if (l.type == "attention") {
            mixer.kind = "differential_attention";
            mixer.params["num_kv_heads"] = l.kv_heads;
            mixer.params["head_dim"] = l.dim;
            mixer.params["scale"] = l.scale;
            mixer.params["lambda_init"] = l.diff;
            mixer.params["window"] = l.window;
            mixer.params["rot_dims"] = l.rot_dims;
            mixer.params["rot_base"] = l.rot_base;
            mixer.params["rot_pairing"] = "neighbours";
            if (l.rot_scaled) {
                Json sc = Json::object();
                sc["factor"] = l.rot_factor;
                sc["low"] = l.rot_low;
                sc["high"] = l.rot_high;
                sc["original"] = l.rot_original;
                mixer.params["rot_scaling"] = sc;
            }
            mixer.tensors = {{"q_proj", a + "q"}, {"k_proj", a + "k"}, {"v_proj", a + "v"}, {"lambda_q1", a + "lq1"}, {"lambda_k1", a + "lk1"},
                             {"lambda_q2", a + "lq2"}, {"lambda_k2", a + "lk2"}, {"o_proj", a + "o"}};
        } else {
            mixer.kind = "retention";
            mixer.params["key_dim"] = l.dim;
            Json dec = Json::array();
            for (double v : l.decay) dec.push(v);
            mixer.params["decay"] = dec;
            mixer.params["key_scale"] = 1.0;
            mixer.params["qkv_act"] = "silu";
            mixer.params["gate_act"] = "sigmoid";
            mixer.params["norm_over"] = "row";
            mixer.params["out_norm"] = true;
            mixer.tensors = {{"q_proj", a + "q"}, {"k_proj", a + "k"}, {"v_proj", a + "v"}, {"gate_proj", a + "g"}, {"out_norm", a + "norm"}, {"o_proj", a + "o"}};
        }
        LayerSpec layer;
        layer.block = "sandwich";
        layer.block_params["has_ffn"] = !l.mlp.empty();
        layer.block_params["input_conv"] = has_conv;
        layer.parts = {{"mixer_norm", norm(p + "norm1")}};
        if (has_conv) layer.parts.emplace_back("mixer_conv", conv(p + "canon1"));
        layer.parts.emplace_back("mixer", mixer);
        layer.parts.emplace_back("mixer_post_norm", norm(p + "norm1b"));
        if (!l.mlp.empty()) {
            PartSpec ffn;
            ffn.params["hidden_size"] = d;
            if (l.mlp == "dense") {
                ffn.kind = "polynorm_mlp";
                ffn.params["intermediate_size"] = l.ff;
                ffn.params["norm_eps"] = cfg.norm_eps;
                ffn.tensors = {{"up_proj", f + "up"}, {"down_proj", f + "down"}, {"coef", f + "act"}};
            } else {
                ffn.kind = "routed_experts";
                ffn.params["num_experts"] = l.experts;
                ffn.params["top_k"] = l.top;
                ffn.params["expert_size"] = l.expert_ff;
                ffn.params["shared_size"] = l.shared_ff;
                ffn.params["router_bias"] = false;
                ffn.params["shared_gate"] = false;
                ffn.params["scores"] = "sigmoid";
                ffn.params["weight_scale"] = l.route_scale;
                ffn.params["num_groups"] = l.groups;
                ffn.params["keep_groups"] = l.keep;
                ffn.tensors = {{"router", f + "router"}};
                for (int64_t e = 0; e < l.experts; ++e) {
                    const std::string n = std::to_string(e), t = f + "e" + n + ".";
                    ffn.tensors.emplace_back("gate_" + n, t + "gate");
                    ffn.tensors.emplace_back("up_" + n, t + "up");
                    ffn.tensors.emplace_back("down_" + n, t + "down");
                }
                if (l.shared_ff > 0) {
                    ffn.tensors.emplace_back("shared_gate", f + "shared.gate");
                    ffn.tensors.emplace_back("shared_up", f + "shared.up");
                    ffn.tensors.emplace_back("shared_down", f + "shared.down");
                }
            }
            layer.parts.emplace_back("ffn_norm", norm(p + "norm2"));
            if (has_conv) layer.parts.emplace_back("ffn_conv", conv(p + "canon2"));
            layer.parts.emplace_back("feed_forward", ffn);
            layer.parts.emplace_back("ffn_post_norm", norm(p + "norm2b"));
        }
        plan.layers.push_back(layer);
    }
    if (cfg.has_loop) {
        plan.has_order = true;
        plan.order = cfg.run_order();
    }
    plan.embedding.kind = "token_embedding";
    plan.embedding.params["vocab_size"] = cfg.vocab_size;
    plan.embedding.params["hidden_size"] = d;
    plan.embedding.params["scale"] = cfg.embedding_scale;
    plan.embedding.tensors = {{"weight", "embed"}};
    plan.final_norm = norm("final.norm");
    plan.head.kind = "linear_head";
    plan.head.params["vocab_size"] = cfg.vocab_size;
    plan.head.params["hidden_size"] = d;
    plan.head.params["scale"] = cfg.logit_scale;
    plan.head.tensors = {{"weight", "head"}};
    return plan;
}

// ------------------------------------------------------------------------------------ registry
namespace {
std::mutex g_arch_mutex;
std::map<std::string, Architecture>& archs() {
    static std::map<std::string, Architecture> a;
    return a;
}
void ensure_builtin_archs() {
    static std::once_flag once;
    std::call_once(once, [] {
        Architecture q;
        q.name = "Qwen3ForCausalLM";
        q.parse_config = [](const Json& d, const std::string& where) -> std::shared_ptr<ModelConfig> {
            return std::make_shared<Qwen3Config>(Qwen3Config::from_json(d, where));
        };
        q.plan = [](const Json& d) { return qwen3_plan(Qwen3Config::from_json(d, "config.json")); };
        archs()[q.name] = q;
        Architecture k;
        k.name = "Kazedra";
        k.parse_config = [](const Json& d, const std::string& where) -> std::shared_ptr<ModelConfig> {
            return std::make_shared<KazedraConfig>(KazedraConfig::from_json(d, where));
        };
        k.plan = [](const Json& d) { return kazedra_plan(KazedraConfig::from_json(d, "config.json")); };
        archs()[k.name] = k;
        Architecture z;
        z.name = "Kuzipel";
        z.parse_config = [](const Json& d, const std::string& where) -> std::shared_ptr<ModelConfig> {
            return std::make_shared<KuzipelConfig>(KuzipelConfig::from_json(d, where));
        };
        z.plan = [](const Json& d) { return kuzipel_plan(KuzipelConfig::from_json(d, "config.json")); };
        archs()[z.name] = z;
        Architecture pm;
        pm.name = "Pemidra";
        pm.parse_config = [](const Json& d, const std::string& where) -> std::shared_ptr<ModelConfig> {
            return std::make_shared<PemidraConfig>(PemidraConfig::from_json(d, where));
        };
        pm.plan = [](const Json& d) { return pemidra_plan(PemidraConfig::from_json(d, "config.json")); };
        archs()[pm.name] = pm;
        Architecture nz;
        nz.name = "Nizorax";
        nz.parse_config = [](const Json& d, const std::string& where) -> std::shared_ptr<ModelConfig> {
            return std::make_shared<NizoraxConfig>(NizoraxConfig::from_json(d, where));
        };
        nz.plan = [](const Json& d) { return nizorax_plan(NizoraxConfig::from_json(d, "config.json")); };
        archs()[nz.name] = nz;
    });
}
}  // namespace

void register_architecture(Architecture a, bool replace) {
    ensure_builtin_archs();
    std::lock_guard<std::mutex> lock(g_arch_mutex);
    if (archs().count(a.name) && !replace) fail(IMP_ERROR_INVALID_ARG, "architecture '" + a.name + "' is already registered");
    archs()[a.name] = std::move(a);
}

void unregister_architecture(const std::string& name) {
    std::lock_guard<std::mutex> lock(g_arch_mutex);
    archs().erase(name);
}

std::vector<std::string> known_architectures() {
    ensure_builtin_archs();
    std::lock_guard<std::mutex> lock(g_arch_mutex);
    std::vector<std::string> out;
    for (const auto& kv : archs()) out.push_back(kv.first);
    return out;
}

const Architecture& architecture(const std::string& name) {
    ensure_builtin_archs();
    std::lock_guard<std::mutex> lock(g_arch_mutex);
    auto it = archs().find(name);
    if (it == archs().end()) {
        std::string known;
        for (const auto& kv : archs()) known += (known.empty() ? "" : ", ") + kv.first;
        bad("unknown architecture '" + name + "'; known: " + (known.empty() ? "(none)" : known));
    }
    return it->second;
}

const Architecture& architecture_of(const Json& config, const std::string& where) {
    if (!config.is_object()) bad(where + ": top level must be an object");
    const Json* a = config.find("architectures");
    if (a && a->is_array() && a->size() > 0 && (*a)[0].is_string()) return architecture((*a)[0].as_string());
    // families that name themselves with a single string
    const Json* one = config.find("architecture");
    if (!a && one && one->is_string()) return architecture(one->as_string());
    bad(where + ": 'architectures' must be a list that names the model class");
}

Json read_config_json(const std::string& path_or_text, std::string* where, std::string* folder) {
    size_t first = path_or_text.find_first_not_of(" \t\r\n");
    if (first != std::string::npos && path_or_text[first] == '{') {
        if (where) *where = "config";
        if (folder) folder->clear();
        try {
            return Json::parse(path_or_text, "config");
        } catch (const std::exception& e) {
            bad(e.what());
        }
    }
    std::string path = path_or_text;
    struct stat st;
    if (stat(path.c_str(), &st) == 0 && S_ISDIR(st.st_mode)) {
        if (folder) *folder = path;
        path += "/config.json";
    } else if (folder) {
        size_t slash = path.find_last_of('/');
        *folder = slash == std::string::npos ? "." : path.substr(0, slash);
    }
    std::ifstream f(path, std::ios::binary);
    if (!f) fail(IMP_ERROR_FILE_NOT_FOUND, "no config.json at " + path);
    std::stringstream ss;
    ss << f.rdbuf();
    if (where) *where = path;
    try {
        Json j = Json::parse(ss.str(), path);
        if (!j.is_object()) bad(path + ": top level must be an object");
        return j;
    } catch (const Error&) {
        throw;
    } catch (const std::exception& e) {
        bad(e.what());
    }
}

// ------------------------------------------------------------------------------ engine config
void validate_engine_config(const ImpConfig& c) {
    auto arg = [](const std::string& m) { fail(IMP_ERROR_INVALID_ARG, m); };
    if (c.compute_dtype != IMP_COMPUTE_BF16 && c.compute_dtype != IMP_COMPUTE_FP32)
        arg("compute_dtype must be bfloat16 or float32");
    if (c.max_batch_size <= 0) arg("max_batch_size must be positive");
    if (c.max_seq_len <= 0) arg("max_seq_len must be positive");
    if (c.kv_block_size <= 0) arg("kv_block_size must be positive");
    if (c.max_batch_tokens <= 0) arg("max_batch_tokens must be positive");
    if (c.prefill_chunk_size < 0) arg("prefill_chunk_size must be >= 0");
    if (c.max_batch_tokens < c.max_batch_size)
        arg("max_batch_tokens must be at least max_batch_size (one token per decoding request)");
    if (c.device_id < 0) arg("device_id must be >= 0");
    if (c.state_slots < 0) arg("state_slots must be >= 0");
    if (!(c.gpu_memory_fraction > 0.f) || c.gpu_memory_fraction > 1.f) arg("gpu_memory_fraction must be in (0, 1]");
}

}  // namespace imp
