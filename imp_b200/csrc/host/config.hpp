// Typed model configurations read from an architecture's own config.json keys, the registry from
// an architecture's name to its configuration class and plan function, and the engine settings.
//
// Every size and constant of a model comes from here; no kernel, part or engine file holds a model
// size of its own.  The reference keeps one struct for every family with defaults in the
// declaration (src/model/model.h:28-76), maps an architecture string to an enum
// (src/model/model.cpp:70-103) and, on the safetensors route, guesses the family from tensor names
// and never reads config.json (src/model/safetensors_loader.cpp:238-263, 297-359); this engine reads
// config.json and refuses what it cannot run.
#pragma once

#include <functional>
#include <string>
#include <vector>

#include "plan.hpp"

namespace imp {

// The keys every decoder has.
struct ModelConfig {
    std::string architecture;
    int64_t vocab_size = 0, hidden_size = 0, num_hidden_layers = 0, max_position_embeddings = 4096;
    std::string torch_dtype = "bfloat16";
    std::vector<int> eos_token_ids;        // config.json's eos_token_id: one id or a list
    int64_t bos_token_id = -1;
    Json raw = Json::object();             // config.json as read (architectures registered from outside read their own keys)

    virtual ~ModelConfig() = default;
    virtual Json to_json() const;          // the typed fields, plus the keys this configuration did not interpret
    static void read_base(ModelConfig& c, const Json& d, const std::string& where);
};

// The Qwen3 dense decoder (architectures[0] == "Qwen3ForCausalLM").  Keys follow the HF config.json
// of this architecture.  The reference reads the GGUF twins of the same fields
// (src/model/gguf_loader.cpp:726-738: block_count, embedding_length, head counts,
// attention.key_length, feed_forward_length, rope.freq_base, layer_norm_rms_epsilon; sliding window
// at :821) into src/model/model.h:28-76.
struct Qwen3Config : ModelConfig {
    int64_t num_attention_heads = 0, num_key_value_heads = 0, head_dim = 0, intermediate_size = 0;
    double rms_norm_eps = 1e-6, rope_theta = 10000.0;
    bool tie_word_embeddings = false, attention_bias = false, use_sliding_window = false;
    std::string hidden_act = "silu";
    int64_t sliding_window = 0;            // 0 = none given
    int64_t max_window_layers = -1;        // -1 = not given
    std::vector<std::string> layer_types;  // empty = not given

    static Qwen3Config from_json(const Json& d, const std::string& where);
    void validate(const std::string& where) const;
    // Window in tokens of `layer` (0 = attends to all earlier tokens).  A query at position p sees keys
    // j with 0 <= p - j < window, the mask of the reference's kernels (src/compute/attention.cu:167;
    // decode: src/compute/attention_paged.cu:163-164).
    int64_t window_of_layer(int layer) const;
    Json to_json() const override;
};

ModelPlan qwen3_plan(const Qwen3Config& cfg);

// Kazedra ("architecture": "Kazedra"): a pre-norm decoder whose layers run two mixers side by side on the same
// normalised input, softmax attention with a sink and a bias by distance (left) and the gated delta rule (right),
// added with fixed weights, followed by an optional gated feed-forward.  Its config.json lists the layers one by
// one, each with its own sizes and constants; the keys are this family's own.
struct KazedraConfig : ModelConfig {
    struct Left {
        int64_t heads = 0, kv_heads = 0, dim = 0, vdim = 0, bias_max = 0, temp_every = 0;
        double scale = 0, temp_coef = 0;
    };
    struct Right {
        int64_t heads = 0, kv_heads = 0, dim = 0, vdim = 0, conv = 0;
    };
    struct Layer {
        std::string type;
        Left left;
        Right right;
        double left_scale = 1, right_scale = 1;
        int64_t ff = 0;            // 0 = the layer has no feed-forward
    };
    std::vector<Layer> layers;
    double norm_eps = 1e-6, logit_scale = 1.0;

    static KazedraConfig from_json(const Json& d, const std::string& where);
    Json to_json() const override;
};

// Every size is in config.json except the rows of each layer's distance-bias table, which the checkpoint's tensor
// gives; an optional model-wide `bias_buckets` key fixes them (random weights need it).
ModelPlan kazedra_plan(const KazedraConfig& cfg);

// Kuzipel ("architecture": "Kuzipel"): a pre-norm decoder with layer norms (weight, no bias), one mixer per layer
// (latent attention or the wkv recurrence), routed experts with a shared expert as feed-forward (or none), a learned
// factor per channel and one constant on every branch, and optionally a run of layers that is repeated with the same
// weights, the stream being re-made from itself and the embedding's output before every pass.  config.json lists
// the layers one by one; the keys are this family's own.
struct KuzipelConfig : ModelConfig {
    struct Layer {
        std::string type;                       // "latent_attention" | "wkv"
        int64_t heads = 0, dim = 0;             // both mixers
        int64_t rot_dim = 0, vdim = 0, kv_rank = 0, q_rank = 0, rot_dims = 0;   // latent attention
        double scale = 0, rot_base = 10000.0;
        int64_t decay_rank = 0;                 // wkv: 0 = the checkpoint's tensor decides
        bool has_mlp = false;
        int64_t experts = 0, top = 0, expert_ff = 0, shared_ff = 0;   // shared_ff 0 = no shared expert
    };
    std::vector<Layer> layers;
    double norm_eps = 1e-5, residual_mult = 1.0;
    bool has_loop = false;
    int64_t loop_start = 0, loop_stop = 0, loop_times = 1;

    static KuzipelConfig from_json(const Json& d, const std::string& where);
    Json to_json() const override;
    // Layer indices in the order they run: those before the repeated run once, the run `times` times, the rest once.
    // With a repeated run, the index num_hidden_layers stands for the map that re-makes the stream before every pass.
    std::vector<int> run_order() const;
};

ModelPlan kuzipel_plan(const KuzipelConfig& cfg);

// Pemidra ("architecture": "Pemidra"): a post-norm decoder, x <- LN(alpha x + s1 (.) mixer(x)) and, where the layer has
// one, x <- LN(alpha x + s2 (.) ffn(x)), with layer norms that have a weight and a bias.  A layer's mixer is retention, the
// generalised delta rule, or a pair side by side (softmax attention with normalised, partly rotated, chunk-masked and gated
// heads beside the delta rule with a decay per key channel) whose outputs are each RMS-normalised and averaged.  The
// feed-forward is gated with the tanh form of gelu.  config.json lists the layers one by one; the keys are this family's own.
struct PemidraConfig : ModelConfig {
    struct Left {
        int64_t heads = 0, kv_heads = 0, dim = 0, vdim = 0, chunk = 0, rot_dims = 0;
        double scale = 0, rot_base = 10000.0;
    };
    struct Right {
        int64_t heads = 0, kv_heads = 0, dim = 0, vdim = 0, conv = 0, decay_rank = 0, gate_rank = 0;
    };
    struct Layer {
        std::string type;                       // "retention" | "general_delta" | "parallel"
        int64_t heads = 0, dim = 0, vdim = 0;   // retention, general_delta
        std::vector<double> decay;              // retention: a number per head
        int64_t decay_rank = 0;                 // general_delta: 0 = the checkpoint's tensor decides
        Left left;
        Right right;
        int64_t ff = 0;                         // 0 = the layer has no feed-forward
    };
    std::vector<Layer> layers;
    double norm_eps = 1e-6, postln_alpha = 1.0;

    static PemidraConfig from_json(const Json& d, const std::string& where);
    Json to_json() const override;
};

// The inner sizes of the low-rank products are no config keys: the checkpoint's tensors give them; optional `decay_rank`
// and `gate_rank` keys of a mixer fix them (random weights need them).
ModelPlan pemidra_plan(const PemidraConfig& cfg);

// Nizorax ("architecture": "Nizorax"): every sublayer stands between two layer norms (weight and bias),
// x <- x + ln_b(sublayer(c(ln_a(x)))), and what it reads first gets a short causal convolution per channel added to itself
// (c(u) = u + conv(u), `canon.taps` taps).  A layer's mixer is differential attention (two softmax maps per head over the
// same values, grouped key/value heads, a sliding window, a rotation of neighbouring pairs with slowed long wavelengths) or
// lightning (linear attention with a fixed decay per head).  The feed-forward is dense with a normalised polynomial as
// activation, a mixture of gated experts (sigmoid scores, groups of experts, a shared expert), or absent.  A run of layers
// may be repeated with the same weights.  config.json lists the layers one by one; the keys are this family's own.
struct NizoraxConfig : ModelConfig {
    struct Layer {
        std::string type;                         // "attention" | "lightning"
        int64_t heads = 0, kv_heads = 0, dim = 0, vdim = 0;
        // attention
        double diff = 0, scale = 0, rot_base = 10000.0;
        int64_t window = 0, rot_dims = 0;         // 0: no window / no rotation
        bool rot_scaled = false;
        double rot_factor = 1, rot_low = 1, rot_high = 1, rot_original = 1;
        // lightning
        std::vector<double> decay;                // a number per head
        // feed-forward
        std::string mlp;                          // "" (none) | "dense" | "moe"
        int64_t ff = 0;                           // dense
        int64_t experts = 0, top = 0, expert_ff = 0, shared_ff = 0, groups = 0, keep = 0;   // moe; groups 0: none; shared_ff 0: none
        double route_scale = 1.0;
    };
    std::vector<Layer> layers;
    double norm_eps = 1e-5, embedding_scale = 1.0, logit_scale = 1.0;
    int64_t canon_taps = 0;                       // 0: no convolution on the sublayers' inputs
    bool has_loop = false;
    int64_t loop_start = 0, loop_stop = 0, loop_times = 1;

    static NizoraxConfig from_json(const Json& d, const std::string& where);
    Json to_json() const override;
    // Layer indices in the order they run: those before the repeated run once, the run `times` times, the rest once.
    std::vector<int> run_order() const;
};

ModelPlan nizorax_plan(const NizoraxConfig& cfg);

// ------------------------------------------------------------------------------------ registry
struct Architecture {
    std::string name;
    // config.json (parsed) -> typed, validated configuration
    std::function<std::shared_ptr<ModelConfig>(const Json& d, const std::string& where)> parse_config;
    // config.json (parsed) -> plan
    std::function<ModelPlan(const Json& d)> plan;
};

void register_architecture(Architecture a, bool replace = false);
void unregister_architecture(const std::string& name);
std::vector<std::string> known_architectures();
const Architecture& architecture(const std::string& name);    // throws, listing known names
const Architecture& architecture_of(const Json& config, const std::string& where);

// Reads `path` (a folder holding config.json, or the file itself) or takes `text` as JSON.
Json read_config_json(const std::string& path_or_text, std::string* where, std::string* folder);

// ------------------------------------------------------------------------------ engine config
void validate_engine_config(const ImpConfig& c);

}  // namespace imp
