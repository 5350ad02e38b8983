// Qwen2ForCausalLM, the Qwen2.5 dense decoder: its config.json, typed, and how it turns
// into parts.
//
// Keys and defaults follow the reference's reading of the same hyper-parameters from GGUF
// metadata (model_config.cpp:35-54): kv heads default to the head count (:43), the head
// size to hidden/heads (:50), the norm's eps is required (:46), the rotary base defaults
// to 10000 (:47).  Its checks (model_config.cpp:56-63) are kept, except the restriction
// to a head size of 128.  The reference has no window and no scaling of the rotary base;
// a non-null `rope_scaling` is refused by name (running without it would give wrong
// logits), and `max_window_layers` must be given whenever `use_sliding_window` is true
// (Hugging Face's own default for it is a layer count of one particular model).
//
// The model: token table; per layer a pre-norm block of grouped-query attention (biased
// q/k/v, rotary NeoX encoding, optional window) and a SwiGLU feed-forward, RMSNorm
// before each; final RMSNorm; head (own matrix, or the token table when
// tie_word_embeddings).  Tensor names are the Hugging Face ones; the reference's GGUF
// names map to them one to one (token_embd -> model.embed_tokens, blk.L.attn_norm ->
// model.layers.L.input_layernorm, attn_q/k/v -> self_attn.q/k/v_proj, attn_output ->
// self_attn.o_proj, ffn_norm -> post_attention_layernorm, ffn_gate/up/down ->
// mlp.gate/up/down_proj, output_norm -> model.norm, output -> lm_head;
// transformer.cpp:299-362, 1000-1005).
#include "friday/config.h"
#include "friday/parts.h"

namespace friday {

namespace {
const char* kName = "Qwen2ForCausalLM";

const std::vector<Key>& qwen2_keys() {
    static const std::vector<Key> keys = {
        Key::required_key("vocab_size", Key::Int, json_positive, "must be positive"),
        Key::required_key("hidden_size", Key::Int, json_positive, "must be positive"),
        Key::required_key("intermediate_size", Key::Int, json_positive, "must be positive"),
        Key::required_key("num_hidden_layers", Key::Int, json_positive, "must be positive"),
        Key::required_key("num_attention_heads", Key::Int, json_positive, "must be positive"),
        Key::derived_key("num_key_value_heads", Key::Int, [](const Json& v) { return v.at("num_attention_heads"); },
                         json_positive, "must be positive"),
        Key::derived_key("head_dim", Key::Int,
                         [](const Json& v) { return Json(v.at("hidden_size").as_int() / v.at("num_attention_heads").as_int()); },
                         json_positive, "must be positive"),
        Key::required_key("max_position_embeddings", Key::Int, json_positive, "must be positive"),
        Key::required_key("rms_norm_eps", Key::Float, json_positive, "must be positive"),
        Key::optional_key("rope_theta", Key::Float, Json(10000.0), [](const Json& v) { return v.as_double() > 1.0; },
                          "must be greater than 1"),
        Key::optional_key("tie_word_embeddings", Key::Bool, Json(false)),
        Key::optional_key("use_sliding_window", Key::Bool, Json(false)),
        Key::optional_key("sliding_window", Key::Int, Json(), json_positive, "must be positive"),
        Key::optional_key("max_window_layers", Key::Int, Json(), [](const Json& v) { return v.as_int() >= 0; },
                          "must not be negative"),
        Key::optional_key("torch_dtype", Key::String, Json("bfloat16")),
        Key::optional_key("hidden_act", Key::String, Json("silu"), [](const Json& v) { return v.as_string() == "silu"; },
                          "this architecture has silu only"),
    };
    return keys;
}
}  // namespace

Json Qwen2Config::read(const Json& d) {
    Json v = read_keys(d, qwen2_keys(), {"rope_scaling"});
    const int64_t heads = v.at("num_attention_heads").as_int(), kv = v.at("num_key_value_heads").as_int();
    if (heads % kv != 0)
        throw ConfigError(format("config.json: 'num_attention_heads' (%lld) must be a multiple of 'num_key_value_heads' (%lld)",
                                 (long long)heads, (long long)kv));
    if (v.at("head_dim").as_int() % 2 != 0)
        throw ConfigError(format("config.json: 'head_dim' (%lld) must be even: the rotary encoding pairs its halves",
                                 (long long)v.at("head_dim").as_int()));
    if (v.at("use_sliding_window").as_bool()) {
        if (v.at("sliding_window").is_null())
            throw ConfigError("config.json: 'use_sliding_window' is true but 'sliding_window' is missing");
        if (v.at("max_window_layers").is_null())
            throw ConfigError("config.json: 'use_sliding_window' is true but 'max_window_layers' is missing: layers at "
                              "or above it have the window, those below see every key (0: all layers have it)");
    } else if (v.at("max_window_layers").is_null()) {
        v.set("max_window_layers", v.at("num_hidden_layers"));         // no layer has a window
    }
    std::string name = kName;
    const Json* archs = d.find("architectures");
    if (archs && archs->is_array() && archs->size() && (*archs)[0].is_string())
        name = (*archs)[0].as_string();                                  // another registered name may reuse these keys
    Json a = Json::array();
    a.push(Json(name));
    v.set("architectures", a);
    v.set("model_type", Json("qwen2"));
    return v;
}

Qwen2Config Qwen2Config::from_typed(const Json& v) {
    Qwen2Config c;
    c.vocab_size = v.at("vocab_size").as_int();
    c.hidden_size = v.at("hidden_size").as_int();
    c.intermediate_size = v.at("intermediate_size").as_int();
    c.num_hidden_layers = v.at("num_hidden_layers").as_int();
    c.num_attention_heads = v.at("num_attention_heads").as_int();
    c.num_key_value_heads = v.at("num_key_value_heads").as_int();
    c.head_dim = v.at("head_dim").as_int();
    c.max_position_embeddings = v.at("max_position_embeddings").as_int();
    c.rms_norm_eps = v.at("rms_norm_eps").as_double();
    c.rope_theta = v.at("rope_theta").as_double();
    c.tie_word_embeddings = v.at("tie_word_embeddings").as_bool();
    c.use_sliding_window = v.at("use_sliding_window").as_bool();
    c.sliding_window = v.at("sliding_window").is_null() ? 0 : v.at("sliding_window").as_int();
    c.max_window_layers = v.at("max_window_layers").as_int();
    c.torch_dtype = v.at("torch_dtype").as_string();
    c.hidden_act = v.at("hidden_act").as_string();
    c.architecture = architecture_name_of(v);
    return c;
}

ModelSpec qwen2_spec(const Json& typed) {
    const Qwen2Config c = Qwen2Config::from_typed(typed);
    ModelSpec spec;
    spec.architecture = c.architecture;
    spec.vocab_size = c.vocab_size;
    spec.width = c.hidden_size;
    spec.max_positions = c.max_position_embeddings;
    spec.embedding = "model.embed_tokens.weight";
    for (int64_t l = 0; l < c.num_hidden_layers; ++l) {
        Json pos = Json::object();
        pos.set("theta", Json(c.rope_theta));
        pos.set("head_dim", Json(c.head_dim));
        Json att = Json::object();
        att.set("n_heads", Json(c.num_attention_heads));
        att.set("n_kv_heads", Json(c.num_key_value_heads));
        att.set("head_dim", Json(c.head_dim));
        att.set("qkv_bias", Json(true));
        att.set("out_bias", Json(false));
        att.set("window", Json(c.window_of(l)));
        PartSpec mixer("gqa_attention", att, "self_attn.");
        mixer.parts["position"] = PartSpec("rotary_neox", pos);
        Json ffn = Json::object();
        ffn.set("inner", Json(c.intermediate_size));
        Json norm = Json::object();
        norm.set("eps", Json(c.rms_norm_eps));
        PartSpec block("prenorm", Json::object(), format("model.layers.%lld.", (long long)l));
        block.parts["norm1"] = PartSpec("rmsnorm", norm, "input_layernorm.");
        block.parts["mixer"] = mixer;
        block.parts["norm2"] = PartSpec("rmsnorm", norm, "post_attention_layernorm.");
        block.parts["feed_forward"] = PartSpec("swiglu", ffn, "mlp.");
        spec.layers.push_back(block);
        LayerCall call;
        call.layer = (int)l;
        call.cache = (int)l;
        spec.program.push_back(call);
    }
    Json norm = Json::object();
    norm.set("eps", Json(c.rms_norm_eps));
    spec.final_norm = PartSpec("rmsnorm", norm, "model.norm.");
    if (c.tie_word_embeddings) spec.ignorable.push_back("lm_head.weight");   // a tied checkpoint may still carry a copy
    else spec.head = "lm_head.weight";
    return spec;
}

namespace {
struct RegisterQwen2 {
    RegisterQwen2() { register_architecture({kName, Qwen2Config::read, qwen2_spec}); }
} register_qwen2;
}  // namespace

}  // namespace friday
