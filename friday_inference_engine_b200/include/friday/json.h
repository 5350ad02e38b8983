// A small JSON value: what config.json, a safetensors header, a shard index and a part's
// parameters are made of.  Numbers keep whether they were written as integers.
#pragma once
#include <stdint.h>

#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace friday {

class Json {
public:
    enum Type { Null, Bool, Int, Float, String, Array, Object };
    typedef std::vector<std::pair<std::string, Json>> Members;      // an object keeps the order of its keys

    Json() : type_(Null) {}
    Json(bool b) : type_(Bool), i_(b) {}
    Json(int v) : type_(Int), i_(v) {}
    Json(int64_t v) : type_(Int), i_(v) {}
    Json(double v) : type_(Float), d_(v) {}
    Json(const char* s) : type_(String), s_(s) {}
    Json(const std::string& s) : type_(String), s_(s) {}
    static Json array() { Json j; j.type_ = Array; return j; }
    static Json object() { Json j; j.type_ = Object; return j; }

    Type type() const { return type_; }
    bool is_null() const { return type_ == Null; }
    bool is_bool() const { return type_ == Bool; }
    bool is_int() const { return type_ == Int; }
    bool is_number() const { return type_ == Int || type_ == Float; }
    bool is_string() const { return type_ == String; }
    bool is_array() const { return type_ == Array; }
    bool is_object() const { return type_ == Object; }

    bool as_bool() const { return i_ != 0; }
    int64_t as_int() const { return type_ == Float ? (int64_t)d_ : i_; }
    double as_double() const { return type_ == Float ? d_ : (double)i_; }
    const std::string& as_string() const { return s_; }

    // arrays
    size_t size() const { return type_ == Array ? a_.size() : (type_ == Object ? o_.size() : 0); }
    const Json& operator[](size_t i) const { return a_[i]; }
    void push(const Json& v) { a_.push_back(v); }
    const std::vector<Json>& items() const { return a_; }

    // objects
    const Json* find(const std::string& key) const;
    bool has(const std::string& key) const { return find(key) != nullptr; }
    const Json& at(const std::string& key) const;               // throws std::out_of_range
    void set(const std::string& key, const Json& v);
    const Members& members() const { return o_; }

    // Typed reads of an object's member with a default (used by parts for their parameters).
    int64_t get_int(const std::string& key, int64_t fallback) const;
    double get_double(const std::string& key, double fallback) const;
    bool get_bool(const std::string& key, bool fallback) const;
    std::string get_string(const std::string& key, const std::string& fallback) const;

    static Json parse(const std::string& text);                   // throws std::invalid_argument with the offset
    std::string dump(int indent = -1) const;                      // indent < 0: one line

private:
    void dump_to(std::string& out, int indent, int depth) const;
    Type type_;
    int64_t i_ = 0;
    double d_ = 0;
    std::string s_;
    std::vector<Json> a_;
    Members o_;
};

}  // namespace friday
