// Minimal JSON reader for the three small documents the inference path parses:
// config.json, the safetensors header, tokenizer.json / generation_config.json.
// (The reference uses nlohmann::json for the same files: inference/src/model/qwen.cu:21-63,
// inference/src/io/safetensors.cpp:51-77, inference/src/io/tokenizer.cpp:16-84.)
// Objects keep insertion order; lookups are linear except through the optional index.
#pragma once
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace tffn {

struct JsonValue {
    enum Type { Null, Bool, Number, String, Array, Object } type = Null;
    bool b = false;
    double num = 0;
    bool is_int = false;
    int64_t inum = 0;
    std::string str;
    std::vector<JsonValue> arr;
    std::vector<std::pair<std::string, JsonValue>> obj;

    bool is_null() const { return type == Null; }
    bool is_number() const { return type == Number; }
    bool is_array() const { return type == Array; }
    bool is_object() const { return type == Object; }
    bool is_string() const { return type == String; }

    const JsonValue* find(const std::string& key) const {
        if (type != Object) return nullptr;
        for (auto& kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    bool contains(const std::string& key) const { return find(key) != nullptr; }
    int64_t as_int() const { return is_int ? inum : (int64_t)num; }
    double as_double() const { return is_int ? (double)inum : num; }

    int64_t value_int(const std::string& key, int64_t def) const {
        auto* v = find(key);
        return (v && v->type == Number) ? v->as_int() : def;
    }
    double value_double(const std::string& key, double def) const {
        auto* v = find(key);
        return (v && v->type == Number) ? v->as_double() : def;
    }
    bool value_bool(const std::string& key, bool def) const {
        auto* v = find(key);
        return (v && v->type == Bool) ? v->b : def;
    }
};

class JsonParser {
public:
    JsonParser(const char* data, size_t len) : p_(data), end_(data + len) {}
    JsonValue parse() {
        JsonValue v = value(0);
        ws();
        if (p_ != end_) fail("trailing characters");
        return v;
    }

private:
    const char* p_;
    const char* end_;
    [[noreturn]] void fail(const char* what) { throw std::runtime_error(std::string("JSON: ") + what); }
    void ws() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\r' || *p_ == '\t')) ++p_;
    }
    JsonValue value(int depth) {
        if (depth > 64) fail("nesting too deep");
        ws();
        if (p_ >= end_) fail("unexpected end");
        JsonValue v;
        char c = *p_;
        if (c == '{') {
            ++p_;
            v.type = JsonValue::Object;
            ws();
            if (p_ < end_ && *p_ == '}') { ++p_; return v; }
            for (;;) {
                ws();
                if (p_ >= end_ || *p_ != '"') fail("expected key");
                std::string k = string();
                ws();
                if (p_ >= end_ || *p_ != ':') fail("expected ':'");
                ++p_;
                v.obj.emplace_back(std::move(k), value(depth + 1));
                ws();
                if (p_ >= end_) fail("unexpected end in object");
                if (*p_ == ',') { ++p_; continue; }
                if (*p_ == '}') { ++p_; break; }
                fail("expected ',' or '}'");
            }
        } else if (c == '[') {
            ++p_;
            v.type = JsonValue::Array;
            ws();
            if (p_ < end_ && *p_ == ']') { ++p_; return v; }
            for (;;) {
                v.arr.push_back(value(depth + 1));
                ws();
                if (p_ >= end_) fail("unexpected end in array");
                if (*p_ == ',') { ++p_; continue; }
                if (*p_ == ']') { ++p_; break; }
                fail("expected ',' or ']'");
            }
        } else if (c == '"') {
            v.type = JsonValue::String;
            v.str = string();
        } else if (c == 't' && end_ - p_ >= 4 && !memcmp(p_, "true", 4)) {
            v.type = JsonValue::Bool; v.b = true; p_ += 4;
        } else if (c == 'f' && end_ - p_ >= 5 && !memcmp(p_, "false", 5)) {
            v.type = JsonValue::Bool; v.b = false; p_ += 5;
        } else if (c == 'n' && end_ - p_ >= 4 && !memcmp(p_, "null", 4)) {
            p_ += 4;
        } else if (c == '-' || (c >= '0' && c <= '9')) {
            const char* s = p_;
            bool is_int = true;
            if (*p_ == '-') ++p_;
            while (p_ < end_ && ((*p_ >= '0' && *p_ <= '9') || *p_ == '.' || *p_ == 'e' || *p_ == 'E' || *p_ == '+' || *p_ == '-')) {
                if (*p_ == '.' || *p_ == 'e' || *p_ == 'E') is_int = false;
                ++p_;
            }
            std::string t(s, p_ - s);
            v.type = JsonValue::Number;
            v.is_int = is_int;
            if (is_int) v.inum = strtoll(t.c_str(), nullptr, 10);
            v.num = strtod(t.c_str(), nullptr);
        } else {
            fail("unexpected character");
        }
        return v;
    }
    static void utf8(std::string& out, uint32_t cp) {
        if (cp < 0x80) out += (char)cp;
        else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
        else { out += (char)(0xF0 | (cp >> 18)); out += (char)(0x80 | ((cp >> 12) & 0x3F)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
    }
    uint32_t hex4() {
        if (end_ - p_ < 4) fail("bad \\u escape");
        uint32_t v = 0;
        for (int i = 0; i < 4; ++i) {
            char c = *p_++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= c - '0';
            else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
            else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
            else fail("bad \\u escape");
        }
        return v;
    }
    std::string string() {
        ++p_;  // opening quote
        std::string out;
        while (p_ < end_ && *p_ != '"') {
            char c = *p_++;
            if (c != '\\') { out += c; continue; }
            if (p_ >= end_) fail("bad escape");
            char e = *p_++;
            switch (e) {
                case '"': out += '"'; break;
                case '\\': out += '\\'; break;
                case '/': out += '/'; break;
                case 'b': out += '\b'; break;
                case 'f': out += '\f'; break;
                case 'n': out += '\n'; break;
                case 'r': out += '\r'; break;
                case 't': out += '\t'; break;
                case 'u': {
                    uint32_t cp = hex4();
                    if (cp >= 0xD800 && cp < 0xDC00 && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
                        p_ += 2;
                        uint32_t lo = hex4();
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    utf8(out, cp);
                    break;
                }
                default: fail("bad escape");
            }
        }
        if (p_ >= end_) fail("unterminated string");
        ++p_;
        return out;
    }
};

inline JsonValue json_parse(const std::string& s) { return JsonParser(s.data(), s.size()).parse(); }
inline JsonValue json_parse(const char* d, size_t n) { return JsonParser(d, n).parse(); }

}  // namespace tffn
