// Minimal JSON DOM parser for converted model files.
//
// The reference parses model files with nlohmann::json (model.hpp:227-228).  Model files are
// dominated by long arrays of base64 strings (weights), so this parser keeps string values as
// views into the source text whenever they contain no escapes and parses numbers lazily cheap.
#pragma once

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace fdk {

class Json {
public:
    enum Type { Null, Bool, Number, String, Array, Object };

    Type type = Null;
    bool b = false;
    double num = 0.0;
    bool is_integer = false;
    // String payload: view into the source buffer (no escapes) or owned (with escapes).
    const char* sptr = nullptr;
    size_t slen = 0;
    std::shared_ptr<std::string> owned;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;

    bool is_null() const { return type == Null; }
    bool is_bool() const { return type == Bool; }
    bool is_number() const { return type == Number; }
    bool is_string() const { return type == String; }
    bool is_array() const { return type == Array; }
    bool is_object() const { return type == Object; }

    size_t size() const { return type == Array ? arr.size() : type == Object ? obj.size() : 0; }
    bool empty() const { return size() == 0; }

    const Json* find(const std::string& key) const {
        if (type != Object) return nullptr;
        for (const auto& kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    bool contains(const std::string& key) const { return find(key) != nullptr; }
    const Json& at(const std::string& key) const {
        const Json* j = find(key);
        if (!j) throw std::runtime_error("json: missing key '" + key + "'");
        return *j;
    }
    // Missing keys read as null, like nlohmann's operator[] on a mutable object.
    const Json& operator[](const std::string& key) const {
        static const Json null_json;
        const Json* j = find(key);
        return j ? *j : null_json;
    }
    const Json& operator[](const char* key) const { return (*this)[std::string(key)]; }
    const Json& operator[](size_t i) const {
        if (type != Array || i >= arr.size()) throw std::runtime_error("json: array index out of range");
        return arr[i];
    }
    const Json& operator[](int i) const { return (*this)[(size_t)i]; }

    std::string str() const {
        if (type != String) throw std::runtime_error("json: value is not a string");
        return std::string(sptr, slen);
    }
    double number() const {
        if (type != Number) throw std::runtime_error("json: value is not a number");
        return num;
    }
    int64_t integer() const { return (int64_t)number(); }
    bool boolean() const {
        if (type != Bool) throw std::runtime_error("json: value is not a bool");
        return b;
    }
    bool get_bool(const std::string& key, bool def) const {
        const Json* j = find(key);
        return (j && j->is_bool()) ? j->b : def;
    }
    std::string get_str(const std::string& key, const std::string& def) const {
        const Json* j = find(key);
        return (j && j->is_string()) ? j->str() : def;
    }

    // `text` must outlive the returned value (string views point into it).
    static Json parse(const char* text, size_t len) {
        Parser p{text, text + len};
        p.skip_ws();
        Json j = p.value(0);
        p.skip_ws();
        if (p.cur != p.end) p.err("trailing characters");
        return j;
    }

private:
    struct Parser {
        const char* cur;
        const char* end;
        [[noreturn]] void err(const char* m) const { throw std::runtime_error(std::string("json parse error: ") + m); }
        void skip_ws() {
            while (cur < end && (*cur == ' ' || *cur == '\n' || *cur == '\t' || *cur == '\r')) ++cur;
        }
        Json value(int depth) {
            if (depth > 256) err("nesting too deep");
            if (cur >= end) err("unexpected end");
            switch (*cur) {
                case '{': return object(depth);
                case '[': return array(depth);
                case '"': return string_value();
                case 't': return literal("true", Bool, true);
                case 'f': return literal("false", Bool, false);
                case 'n': return literal("null", Null, false);
                default: return number_value();
            }
        }
        Json literal(const char* w, Type t, bool v) {
            const size_t n = std::strlen(w);
            if ((size_t)(end - cur) < n || std::memcmp(cur, w, n) != 0) err("bad literal");
            cur += n;
            Json j;
            j.type = t;
            j.b = v;
            return j;
        }
        Json number_value() {
            const char* s = cur;
            bool integral = true;
            if (cur < end && (*cur == '-' || *cur == '+')) ++cur;
            while (cur < end) {
                const char c = *cur;
                if (c >= '0' && c <= '9') { ++cur; continue; }
                if (c == '.' || c == 'e' || c == 'E' || c == '+' || c == '-') { integral = false; ++cur; continue; }
                break;
            }
            if (cur == s) err("bad number");
            char buf[64];
            const size_t n = (size_t)(cur - s);
            if (n >= sizeof(buf)) err("number too long");
            std::memcpy(buf, s, n);
            buf[n] = 0;
            Json j;
            j.type = Number;
            j.num = std::strtod(buf, nullptr);
            j.is_integer = integral;
            return j;
        }
        Json string_value() {
            ++cur;  // opening quote
            const char* s = cur;
            const char* q = (const char*)std::memchr(cur, '"', (size_t)(end - cur));
            if (!q) err("unterminated string");
            Json j;
            j.type = String;
            if (!std::memchr(s, '\\', (size_t)(q - s))) {  // fast path: no escapes
                j.sptr = s;
                j.slen = (size_t)(q - s);
                cur = q + 1;
                return j;
            }
            auto out = std::make_shared<std::string>();
            while (cur < end && *cur != '"') {
                if (*cur == '\\') {
                    ++cur;
                    if (cur >= end) err("bad escape");
                    switch (*cur) {
                        case 'n': out->push_back('\n'); break;
                        case 't': out->push_back('\t'); break;
                        case 'r': out->push_back('\r'); break;
                        case 'b': out->push_back('\b'); break;
                        case 'f': out->push_back('\f'); break;
                        case 'u': {
                            if (end - cur < 5) err("bad unicode escape");
                            char hex[5] = {cur[1], cur[2], cur[3], cur[4], 0};
                            const unsigned cp = (unsigned)std::strtoul(hex, nullptr, 16);
                            if (cp < 0x80) out->push_back((char)cp);
                            else if (cp < 0x800) { out->push_back((char)(0xC0 | (cp >> 6))); out->push_back((char)(0x80 | (cp & 0x3F))); }
                            else { out->push_back((char)(0xE0 | (cp >> 12))); out->push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out->push_back((char)(0x80 | (cp & 0x3F))); }
                            cur += 4;
                            break;
                        }
                        default: out->push_back(*cur);
                    }
                    ++cur;
                } else {
                    out->push_back(*cur++);
                }
            }
            if (cur >= end) err("unterminated string");
            ++cur;
            j.owned = out;
            j.sptr = out->data();
            j.slen = out->size();
            return j;
        }
        Json array(int depth) {
            ++cur;
            Json j;
            j.type = Array;
            skip_ws();
            if (cur < end && *cur == ']') { ++cur; return j; }
            for (;;) {
                skip_ws();
                j.arr.push_back(value(depth + 1));
                skip_ws();
                if (cur >= end) err("unterminated array");
                if (*cur == ',') { ++cur; continue; }
                if (*cur == ']') { ++cur; break; }
                err("expected , or ]");
            }
            return j;
        }
        Json object(int depth) {
            ++cur;
            Json j;
            j.type = Object;
            skip_ws();
            if (cur < end && *cur == '}') { ++cur; return j; }
            for (;;) {
                skip_ws();
                if (cur >= end || *cur != '"') err("expected key");
                Json k = string_value();
                skip_ws();
                if (cur >= end || *cur != ':') err("expected :");
                ++cur;
                skip_ws();
                j.obj.emplace_back(k.str(), value(depth + 1));
                skip_ws();
                if (cur >= end) err("unterminated object");
                if (*cur == ',') { ++cur; continue; }
                if (*cur == '}') { ++cur; break; }
                err("expected , or }");
            }
            return j;
        }
    };
};

}  // namespace fdk
