// Parser and printer of friday::Json (include/friday/json.h).
#include "friday/json.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <stdexcept>

namespace friday {

const Json* Json::find(const std::string& key) const {
    for (const auto& m : o_)
        if (m.first == key) return &m.second;
    return nullptr;
}

const Json& Json::at(const std::string& key) const {
    const Json* j = find(key);
    if (!j) throw std::out_of_range("no key '" + key + "'");
    return *j;
}

void Json::set(const std::string& key, const Json& v) {
    if (type_ != Object) { *this = object(); }
    for (auto& m : o_)
        if (m.first == key) { m.second = v; return; }
    o_.emplace_back(key, v);
}

int64_t Json::get_int(const std::string& key, int64_t fallback) const {
    const Json* j = find(key);
    return (j && j->is_number()) ? j->as_int() : fallback;
}
double Json::get_double(const std::string& key, double fallback) const {
    const Json* j = find(key);
    return (j && j->is_number()) ? j->as_double() : fallback;
}
bool Json::get_bool(const std::string& key, bool fallback) const {
    const Json* j = find(key);
    return (j && j->is_bool()) ? j->as_bool() : fallback;
}
std::string Json::get_string(const std::string& key, const std::string& fallback) const {
    const Json* j = find(key);
    return (j && j->is_string()) ? j->as_string() : fallback;
}

namespace {

struct Reader {
    const char* p;
    const char* begin;
    const char* end;

    [[noreturn]] void fail(const char* what) const {
        char buf[160];
        snprintf(buf, sizeof buf, "%s at offset %ld", what, (long)(p - begin));
        throw std::invalid_argument(buf);
    }
    void skip() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool eat(char c) { skip(); if (p < end && *p == c) { ++p; return true; } return false; }
    void need(char c) { if (!eat(c)) { char w[32]; snprintf(w, sizeof w, "expected '%c'", c); fail(w); } }

    static void utf8(std::string& out, unsigned cp) {
        if (cp < 0x80) out += (char)cp;
        else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
        else { out += (char)(0xF0 | (cp >> 18)); out += (char)(0x80 | ((cp >> 12) & 0x3F)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
    }
    unsigned hex4() {
        if (end - p < 4) fail("short \\u escape");
        unsigned v = 0;
        for (int i = 0; i < 4; ++i) {
            char c = *p++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= c - '0';
            else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
            else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
            else fail("bad \\u escape");
        }
        return v;
    }
    std::string string() {
        need('"');
        std::string out;
        while (true) {
            if (p >= end) fail("unterminated string");
            char c = *p++;
            if (c == '"') break;
            if (c != '\\') { out += c; continue; }
            if (p >= end) fail("unterminated escape");
            char e = *p++;
            switch (e) {
                case 'n': out += '\n'; break;
                case 't': out += '\t'; break;
                case 'r': out += '\r'; break;
                case 'b': out += '\b'; break;
                case 'f': out += '\f'; break;
                case 'u': {
                    unsigned cp = hex4();
                    if (cp >= 0xD800 && cp < 0xDC00 && end - p >= 6 && p[0] == '\\' && p[1] == 'u') {
                        p += 2;
                        unsigned lo = hex4();
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    utf8(out, cp);
                    break;
                }
                default: out += e;
            }
        }
        return out;
    }
    Json value(int depth) {
        if (depth > 200) fail("nested too deeply");
        skip();
        if (p >= end) fail("unexpected end");
        char c = *p;
        if (c == '{') {
            ++p;
            Json o = Json::object();
            if (eat('}')) return o;
            do {
                skip();
                std::string k = string();
                need(':');
                o.set(k, value(depth + 1));
            } while (eat(','));
            need('}');
            return o;
        }
        if (c == '[') {
            ++p;
            Json a = Json::array();
            if (eat(']')) return a;
            do { a.push(value(depth + 1)); } while (eat(','));
            need(']');
            return a;
        }
        if (c == '"') return Json(string());
        if (!strncmp(p, "true", end - p < 4 ? end - p : 4) && end - p >= 4) { p += 4; return Json(true); }
        if (end - p >= 5 && !strncmp(p, "false", 5)) { p += 5; return Json(false); }
        if (end - p >= 4 && !strncmp(p, "null", 4)) { p += 4; return Json(); }
        if (end - p >= 3 && !strncmp(p, "NaN", 3)) { p += 3; return Json((double)NAN); }
        if (end - p >= 8 && !strncmp(p, "Infinity", 8)) { p += 8; return Json((double)INFINITY); }
        if (end - p >= 9 && !strncmp(p, "-Infinity", 9)) { p += 9; return Json((double)-INFINITY); }
        const char* s = p;
        bool integral = true;
        if (p < end && (*p == '-' || *p == '+')) ++p;
        while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '-' || *p == '+')) {
            if (*p == '.' || *p == 'e' || *p == 'E') integral = false;
            ++p;
        }
        if (p == s) fail("unexpected character");
        std::string num(s, p);
        if (integral && num.size() < 19) return Json((int64_t)strtoll(num.c_str(), nullptr, 10));
        return Json(strtod(num.c_str(), nullptr));
    }
};

void escape_to(std::string& out, const std::string& s) {
    out += '"';
    for (unsigned char c : s) {
        switch (c) {
            case '"': out += "\\\""; break;
            case '\\': out += "\\\\"; break;
            case '\n': out += "\\n"; break;
            case '\t': out += "\\t"; break;
            case '\r': out += "\\r"; break;
            default:
                if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); out += b; }
                else out += (char)c;
        }
    }
    out += '"';
}

}  // namespace

Json Json::parse(const std::string& text) {
    Reader r{text.data(), text.data(), text.data() + text.size()};
    Json v = r.value(0);
    r.skip();
    if (r.p != r.end) r.fail("trailing characters");
    return v;
}

void Json::dump_to(std::string& out, int indent, int depth) const {
    auto newline = [&](int d) {
        if (indent < 0) return;
        out += '\n';
        out.append((size_t)(indent * d), ' ');
    };
    switch (type_) {
        case Null: out += "null"; break;
        case Bool: out += i_ ? "true" : "false"; break;
        case Int: out += std::to_string(i_); break;
        case Float: {
            if (d_ != d_) { out += "NaN"; break; }
            if (isinf(d_)) { out += d_ > 0 ? "Infinity" : "-Infinity"; break; }
            char b[40];
            snprintf(b, sizeof b, "%.17g", d_);
            if (!strpbrk(b, ".eE")) strcat(b, ".0");
            out += b;
            break;
        }
        case String: escape_to(out, s_); break;
        case Array:
            out += '[';
            for (size_t i = 0; i < a_.size(); ++i) {
                if (i) out += indent < 0 ? ", " : ",";
                newline(depth + 1);
                a_[i].dump_to(out, indent, depth + 1);
            }
            if (!a_.empty()) newline(depth);
            out += ']';
            break;
        case Object:
            out += '{';
            for (size_t i = 0; i < o_.size(); ++i) {
                if (i) out += indent < 0 ? ", " : ",";
                newline(depth + 1);
                escape_to(out, o_[i].first);
                out += ": ";
                o_[i].second.dump_to(out, indent, depth + 1);
            }
            if (!o_.empty()) newline(depth);
            out += '}';
            break;
    }
}

std::string Json::dump(int indent) const {
    std::string out;
    dump_to(out, indent, 0);
    return out;
}

}  // namespace friday
