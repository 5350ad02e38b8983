// Typed reading of config.json and the registry of architectures (config.h).
#include "friday/config.h"

#include <stdio.h>

#include <fstream>
#include <map>
#include <mutex>
#include <sstream>

#include "friday/parts.h"

namespace friday {

Key Key::required_key(const std::string& n, Kind k, std::function<bool(const Json&)> check, const std::string& rule) {
    Key key;
    key.name = n;
    key.kind = k;
    key.required = true;
    key.check = std::move(check);
    key.rule = rule;
    return key;
}

Key Key::optional_key(const std::string& n, Kind k, const Json& fallback, std::function<bool(const Json&)> check,
                      const std::string& rule) {
    Key key;
    key.name = n;
    key.kind = k;
    key.fallback = fallback;
    key.check = std::move(check);
    key.rule = rule;
    return key;
}

Key Key::derived_key(const std::string& n, Kind k, std::function<Json(const Json&)> derive,
                     std::function<bool(const Json&)> check, const std::string& rule) {
    Key key;
    key.name = n;
    key.kind = k;
    key.derive = std::move(derive);
    key.check = std::move(check);
    key.rule = rule;
    return key;
}

bool json_positive(const Json& v) { return v.is_number() && v.as_double() > 0; }

namespace {
const char* kind_name(Key::Kind k) {
    return k == Key::Int ? "int" : k == Key::Float ? "float" : k == Key::Bool ? "bool" : "str";
}

Json coerce(const Key& key, const Json& v) {
    switch (key.kind) {
        case Key::Bool:
            if (v.is_bool()) return v;
            break;
        case Key::Int:
            if (v.is_int()) return v;
            if (v.type() == Json::Float && v.as_double() == (double)(int64_t)v.as_double()) return Json((int64_t)v.as_double());
            break;
        case Key::Float:
            if (v.is_number()) return Json(v.as_double());
            break;
        case Key::String:
            if (v.is_string()) return v;
            break;
    }
    throw ConfigError("config.json: '" + key.name + "' must be " + kind_name(key.kind) + ", got " + v.dump());
}
}  // namespace

Json read_keys(const Json& d, const std::vector<Key>& keys, const std::vector<std::string>& refused) {
    if (!d.is_object()) throw ConfigError("config.json: the top level must be an object");
    for (const auto& name : refused) {
        const Json* v = d.find(name);
        if (v && !v->is_null())
            throw ConfigError("config.json: '" + name + "' = " + v->dump() + " is not supported: it changes the model's "
                              "arithmetic in a way this library does not implement, and ignoring it would give wrong "
                              "logits; remove the key or set it to null to run without it");
    }
    Json out = Json::object();
    for (const auto& key : keys) {
        const Json* v = d.find(key.name);
        Json value;
        if (v && !v->is_null()) value = coerce(key, *v);
        else if (key.required) throw ConfigError("config.json: required key '" + key.name + "' is missing");
        else if (key.derive) value = key.derive(out);
        else value = key.fallback;
        if (key.check && !value.is_null() && !key.check(value))
            throw ConfigError("config.json: '" + key.name + "' = " + value.dump() + ": " + key.rule);
        out.set(key.name, value);
    }
    return out;
}

namespace {
std::mutex& registry_mutex() { static std::mutex m; return m; }
std::map<std::string, Architecture>& registry() { static std::map<std::string, Architecture> r; return r; }
}  // namespace

void register_architecture(const Architecture& arch) {
    std::lock_guard<std::mutex> lock(registry_mutex());
    registry()[arch.name] = arch;
}

std::vector<std::string> registered_architectures() {
    std::lock_guard<std::mutex> lock(registry_mutex());
    std::vector<std::string> names;
    for (const auto& kv : registry()) names.push_back(kv.first);
    return names;
}

Architecture architecture(const std::string& name) {
    std::lock_guard<std::mutex> lock(registry_mutex());
    auto it = registry().find(name);
    if (it == registry().end()) {
        std::string known;
        for (const auto& kv : registry()) known += (known.empty() ? "" : ", ") + kv.first;
        throw ConfigError("unsupported architecture '" + name + "' (supported: " + (known.empty() ? "none" : known) + ")");
    }
    return it->second;
}

std::string architecture_name_of(const Json& d) {
    const Json* a = d.is_object() ? d.find("architectures") : nullptr;
    if (a && a->is_array() && a->size() > 0 && (*a)[0].is_string()) return (*a)[0].as_string();
    throw ConfigError("config.json: 'architectures' must be a list whose first item names the model class");
}

Json read_config_file(const std::string& model_dir) {
    const std::string path = model_dir + "/config.json";
    std::ifstream f(path);
    if (!f) throw ConfigError(model_dir + ": no config.json in the model folder");
    std::stringstream ss;
    ss << f.rdbuf();
    try {
        return Json::parse(ss.str());
    } catch (const std::invalid_argument& e) {
        throw ConfigError(path + ": not JSON: " + e.what());
    }
}

}  // namespace friday
