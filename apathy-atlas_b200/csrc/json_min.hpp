// A small JSON reader for the two documents the adapter ingest meets: PEFT's adapter_config.json and the header of a
// safetensors file.  Values are kept as a tree; numbers keep their text so that integers beyond 2^53 (byte offsets)
// and the int-or-float forms PEFT writes both survive.  Host only.
#pragma once

#include <cstdint>
#include <cstdlib>
#include <map>
#include <string>
#include <vector>

namespace atlas {
namespace json {

struct Value {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    std::string text;                                   // Number: the literal; String: the decoded text
    std::vector<Value> items;                           // Array
    std::vector<std::pair<std::string, Value>> members; // Object, in document order

    const Value* get(const std::string& key) const {
        if (kind != Object) return nullptr;
        for (const auto& m : members)
            if (m.first == key) return &m.second;
        return nullptr;
    }
    bool is_integer() const {
        if (kind != Number || text.empty()) return false;
        size_t i = text[0] == '-' ? 1 : 0;
        if (i >= text.size()) return false;
        for (; i < text.size(); ++i)
            if (text[i] < '0' || text[i] > '9') return false;
        return true;
    }
    double as_double() const { return kind == Number ? std::strtod(text.c_str(), nullptr) : 0.0; }
    uint64_t as_u64() const { return kind == Number ? std::strtoull(text.c_str(), nullptr, 10) : 0ull; }
    // compact re-serialisation, for error messages that quote the offending value
    std::string dump() const {
        switch (kind) {
            case Null: return "null";
            case Bool: return b ? "true" : "false";
            case Number: return text;
            case String: return "\"" + text + "\"";
            case Array: {
                std::string s = "[";
                for (size_t i = 0; i < items.size(); ++i) s += (i ? "," : "") + items[i].dump();
                return s + "]";
            }
            case Object: {
                std::string s = "{";
                for (size_t i = 0; i < members.size(); ++i) s += (i ? "," : "") + ("\"" + members[i].first + "\":") + members[i].second.dump();
                return s + "}";
            }
        }
        return "";
    }
};

class Parser {
public:
    Parser(const char* p, size_t n) : p_(p), end_(p + n) {}
    // false (with `error` set) on malformed input or trailing garbage
    bool parse(Value& out, std::string& error) {
        if (!value(out, 0)) { error = err_.empty() ? "malformed JSON" : err_; return false; }
        ws();
        if (p_ != end_) { error = "trailing characters after the JSON value"; return false; }
        return true;
    }

private:
    const char* p_;
    const char* end_;
    std::string err_;

    void ws() { while (p_ < end_ && (*p_ == ' ' || *p_ == '\t' || *p_ == '\n' || *p_ == '\r')) ++p_; }
    bool fail(const char* m) { if (err_.empty()) err_ = m; return false; }
    bool lit(const char* s) {
        const char* q = p_;
        for (; *s; ++s, ++q)
            if (q >= end_ || *q != *s) return false;
        p_ = q;
        return true;
    }
    static void utf8(std::string& o, uint32_t c) {
        if (c < 0x80) o += char(c);
        else if (c < 0x800) { o += char(0xC0 | (c >> 6)); o += char(0x80 | (c & 0x3F)); }
        else if (c < 0x10000) { o += char(0xE0 | (c >> 12)); o += char(0x80 | ((c >> 6) & 0x3F)); o += char(0x80 | (c & 0x3F)); }
        else { o += char(0xF0 | (c >> 18)); o += char(0x80 | ((c >> 12) & 0x3F)); o += char(0x80 | ((c >> 6) & 0x3F)); o += char(0x80 | (c & 0x3F)); }
    }
    bool hex4(uint32_t& v) {
        if (end_ - p_ < 4) return false;
        v = 0;
        for (int i = 0; i < 4; ++i) {
            const char c = *p_++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= uint32_t(c - '0');
            else if (c >= 'a' && c <= 'f') v |= uint32_t(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= uint32_t(c - 'A' + 10);
            else return false;
        }
        return true;
    }
    bool string(std::string& out) {
        if (p_ >= end_ || *p_ != '"') return fail("expected a string");
        ++p_;
        out.clear();
        while (p_ < end_) {
            const char c = *p_++;
            if (c == '"') return true;
            if (c != '\\') { out += c; continue; }
            if (p_ >= end_) break;
            const char e = *p_++;
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
                    uint32_t cp;
                    if (!hex4(cp)) return fail("bad \\u escape");
                    if (cp >= 0xD800 && cp < 0xDC00 && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
                        p_ += 2;
                        uint32_t lo;
                        if (!hex4(lo)) return fail("bad \\u escape");
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    utf8(out, cp);
                    break;
                }
                default: return fail("bad escape in string");
            }
        }
        return fail("unterminated string");
    }
    bool number(Value& out) {
        const char* s = p_;
        if (p_ < end_ && *p_ == '-') ++p_;
        if (p_ >= end_ || *p_ < '0' || *p_ > '9') return fail("bad number");
        while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        if (p_ < end_ && *p_ == '.') { ++p_; while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_; }
        if (p_ < end_ && (*p_ == 'e' || *p_ == 'E')) {
            ++p_;
            if (p_ < end_ && (*p_ == '+' || *p_ == '-')) ++p_;
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        out.kind = Value::Number;
        out.text.assign(s, p_);
        return true;
    }
    bool value(Value& out, int depth) {
        if (depth > 64) return fail("nesting too deep");
        ws();
        if (p_ >= end_) return fail("unexpected end of document");
        const char c = *p_;
        if (c == '{') {
            ++p_;
            out.kind = Value::Object;
            ws();
            if (p_ < end_ && *p_ == '}') { ++p_; return true; }
            while (true) {
                ws();
                std::string key;
                if (!string(key)) return false;
                ws();
                if (p_ >= end_ || *p_ != ':') return fail("expected ':'");
                ++p_;
                Value v;
                if (!value(v, depth + 1)) return false;
                out.members.emplace_back(std::move(key), std::move(v));
                ws();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == '}') { ++p_; return true; }
                return fail("expected ',' or '}'");
            }
        }
        if (c == '[') {
            ++p_;
            out.kind = Value::Array;
            ws();
            if (p_ < end_ && *p_ == ']') { ++p_; return true; }
            while (true) {
                Value v;
                if (!value(v, depth + 1)) return false;
                out.items.push_back(std::move(v));
                ws();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == ']') { ++p_; return true; }
                return fail("expected ',' or ']'");
            }
        }
        if (c == '"') { out.kind = Value::String; return string(out.text); }
        if (lit("true")) { out.kind = Value::Bool; out.b = true; return true; }
        if (lit("false")) { out.kind = Value::Bool; out.b = false; return true; }
        if (lit("null")) { out.kind = Value::Null; return true; }
        return number(out);
    }
};

}  // namespace json
}  // namespace atlas
