// Typed reading of config.json, and the one registry from an architecture's name to its
// configuration reader and its model description.
//
// An architecture declares its keys once (name, kind, default or "required", a check);
// read_keys turns config.json's object into a complete object of typed values and
// reports every problem with the name of the key.  The registry then gives, for
// config.json's `architectures[0]`, the function that reads the keys and the function
// that turns them into a ModelSpec (parts.h).  An unknown name is refused with the list
// of known names, as the reference refuses an unknown GGUF architecture
// (model_config.cpp:56-58).
#pragma once
#include <functional>
#include <string>
#include <vector>

#include "friday/base.h"
#include "friday/json.h"

namespace friday {

struct ModelSpec;

struct Key {
    enum Kind { Int, Float, Bool, String };
    std::string name;
    Kind kind;
    bool required = false;
    Json fallback;                                          // used when absent and not required (null: "none")
    std::function<Json(const Json& so_far)> derive;         // if set, computes the default from earlier keys
    std::function<bool(const Json&)> check;                 // if set, must hold for a non-null value
    std::string rule;                                       // said in the error when `check` fails

    static Key required_key(const std::string& n, Kind k, std::function<bool(const Json&)> check = nullptr,
                            const std::string& rule = "");
    static Key optional_key(const std::string& n, Kind k, const Json& fallback,
                            std::function<bool(const Json&)> check = nullptr, const std::string& rule = "");
    static Key derived_key(const std::string& n, Kind k, std::function<Json(const Json&)> derive,
                           std::function<bool(const Json&)> check = nullptr, const std::string& rule = "");
};

bool json_positive(const Json& v);

// Values for `keys` from config.json's object `d`, defaults filled in the order of `keys`.
// Keys in `refused` must be absent or null: they change the model's arithmetic in a way the
// architecture's parts do not implement, so running without them would give wrong logits.
Json read_keys(const Json& d, const std::vector<Key>& keys, const std::vector<std::string>& refused = {});

struct Architecture {
    std::string name;
    std::function<Json(const Json& config_json)> read_config;       // typed, complete, checked
    std::function<ModelSpec(const Json& typed_config)> build_spec;
};

void register_architecture(const Architecture& arch);
Architecture architecture(const std::string& name);                  // ConfigError listing the known names
std::vector<std::string> registered_architectures();
std::string architecture_name_of(const Json& config_json);           // architectures[0]

// config.json of a model folder (ConfigError if absent or not JSON).
Json read_config_file(const std::string& model_dir);

// ---- the Qwen2.5 dense decoder's configuration, typed (src: config/qwen2.cpp)
struct Qwen2Config {
    int64_t vocab_size, hidden_size, intermediate_size, num_hidden_layers, num_attention_heads, num_key_value_heads,
        head_dim, max_position_embeddings;
    double rms_norm_eps, rope_theta;
    bool tie_word_embeddings, use_sliding_window;
    int64_t sliding_window;              // 0: none given
    int64_t max_window_layers;
    std::string torch_dtype, hidden_act, architecture;

    static Json read(const Json& config_json);                       // the registry's read_config
    static Qwen2Config from_typed(const Json& typed);
    // Keys that a query of `layer` may see (itself included); 0 for all of them.
    int64_t window_of(int64_t layer) const {
        return (use_sliding_window && layer >= max_window_layers) ? sliding_window : 0;
    }
};
ModelSpec qwen2_spec(const Json& typed_config);

}  // namespace friday
