// Minimal JSON reader for the three JSON inputs of the decode path: the model.bin header,
// the vocabulary (array of strings) and tokenised stories (array of arrays of strings).
// The reference links cJSON for these (load_model.cu:6, main.cu:25); this is an independent
// recursive-descent parser that keeps object members in file order.
#pragma once
#include <cstdint>
#include <cstdlib>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace mlb {

struct JsonValue {
    enum Type { Null, Bool, Number, String, Array, Object } type = Null;
    bool b = false;
    double num = 0.0;
    std::string str;
    std::vector<JsonValue> items;                               // Array
    std::vector<std::pair<std::string, JsonValue>> members;     // Object, in file order

    const JsonValue* get(const char* key) const {
        if (type != Object) return nullptr;
        for (const auto& m : members)
            if (m.first == key) return &m.second;
        return nullptr;
    }
    bool is(Type t) const { return type == t; }
};

class JsonParser {
public:
    JsonParser(const char* data, size_t len) : p_(data), end_(data + len) {}

    // Returns false (and sets error()) on malformed input; never throws.
    bool parse(JsonValue* out) {
        skip_ws();
        if (!value(out, 0)) return false;
        skip_ws();
        if (p_ != end_) return fail("trailing characters after JSON value");
        return true;
    }
    const std::string& error() const { return err_; }

private:
    const char* p_;
    const char* end_;
    std::string err_;

    bool fail(const char* msg) {
        if (err_.empty()) err_ = msg;
        return false;
    }
    void skip_ws() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\t' || *p_ == '\n' || *p_ == '\r')) ++p_;
    }
    bool literal(const char* s) {
        const char* q = p_;
        while (*s) {
            if (q >= end_ || *q != *s) return false;
            ++q; ++s;
        }
        p_ = q;
        return true;
    }
    static void append_utf8(std::string* s, uint32_t cp) {
        if (cp < 0x80) {
            s->push_back(static_cast<char>(cp));
        } else if (cp < 0x800) {
            s->push_back(static_cast<char>(0xC0 | (cp >> 6)));
            s->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
        } else if (cp < 0x10000) {
            s->push_back(static_cast<char>(0xE0 | (cp >> 12)));
            s->push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
            s->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
        } else {
            s->push_back(static_cast<char>(0xF0 | (cp >> 18)));
            s->push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
            s->push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
            s->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
        }
    }
    bool hex4(uint32_t* out) {
        if (end_ - p_ < 4) return fail("truncated \\u escape");
        uint32_t v = 0;
        for (int i = 0; i < 4; ++i) {
            char c = p_[i];
            v <<= 4;
            if (c >= '0' && c <= '9') v |= static_cast<uint32_t>(c - '0');
            else if (c >= 'a' && c <= 'f') v |= static_cast<uint32_t>(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= static_cast<uint32_t>(c - 'A' + 10);
            else return fail("bad hex digit in \\u escape");
        }
        p_ += 4;
        *out = v;
        return true;
    }
    bool string(std::string* out) {
        if (p_ >= end_ || *p_ != '"') return fail("expected string");
        ++p_;
        out->clear();
        while (p_ < end_) {
            char c = *p_++;
            if (c == '"') return true;
            if (c != '\\') {
                out->push_back(c);
                continue;
            }
            if (p_ >= end_) break;
            char e = *p_++;
            switch (e) {
                case '"': out->push_back('"'); break;
                case '\\': out->push_back('\\'); break;
                case '/': out->push_back('/'); break;
                case 'b': out->push_back('\b'); break;
                case 'f': out->push_back('\f'); break;
                case 'n': out->push_back('\n'); break;
                case 'r': out->push_back('\r'); break;
                case 't': out->push_back('\t'); break;
                case 'u': {
                    uint32_t cp;
                    if (!hex4(&cp)) return false;
                    if (cp >= 0xD800 && cp <= 0xDBFF && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
                        p_ += 2;
                        uint32_t lo;
                        if (!hex4(&lo)) return false;
                        if (lo >= 0xDC00 && lo <= 0xDFFF) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    append_utf8(out, cp);
                    break;
                }
                default: return fail("bad escape in string");
            }
        }
        return fail("unterminated string");
    }
    bool value(JsonValue* out, int depth) {
        if (depth > 64) return fail("JSON nested too deeply");
        skip_ws();
        if (p_ >= end_) return fail("unexpected end of JSON");
        char c = *p_;
        if (c == '{') {
            ++p_;
            out->type = JsonValue::Object;
            skip_ws();
            if (p_ < end_ && *p_ == '}') { ++p_; return true; }
            for (;;) {
                skip_ws();
                std::string key;
                if (!string(&key)) return false;
                skip_ws();
                if (p_ >= end_ || *p_ != ':') return fail("expected ':' in object");
                ++p_;
                out->members.emplace_back(std::move(key), JsonValue());
                if (!value(&out->members.back().second, depth + 1)) return false;
                skip_ws();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == '}') { ++p_; return true; }
                return fail("expected ',' or '}' in object");
            }
        }
        if (c == '[') {
            ++p_;
            out->type = JsonValue::Array;
            skip_ws();
            if (p_ < end_ && *p_ == ']') { ++p_; return true; }
            for (;;) {
                out->items.emplace_back();
                if (!value(&out->items.back(), depth + 1)) return false;
                skip_ws();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == ']') { ++p_; return true; }
                return fail("expected ',' or ']' in array");
            }
        }
        if (c == '"') {
            out->type = JsonValue::String;
            return string(&out->str);
        }
        if (literal("true")) { out->type = JsonValue::Bool; out->b = true; return true; }
        if (literal("false")) { out->type = JsonValue::Bool; out->b = false; return true; }
        if (literal("null")) { out->type = JsonValue::Null; return true; }
        // number
        const char* start = p_;
        while (p_ < end_ && ((*p_ >= '0' && *p_ <= '9') || *p_ == '-' || *p_ == '+' || *p_ == '.' ||
                             *p_ == 'e' || *p_ == 'E'))
            ++p_;
        if (p_ == start) return fail("unexpected character in JSON");
        std::string tmp(start, p_);
        char* endp = nullptr;
        out->num = std::strtod(tmp.c_str(), &endp);
        if (endp == tmp.c_str()) return fail("bad number");
        out->type = JsonValue::Number;
        return true;
    }
};

}  // namespace mlb
