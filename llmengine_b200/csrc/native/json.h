// A small JSON reader: enough for config.json, a safetensors header and the kernel manifest.
#pragma once

#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace llmengine_b200 {
namespace json {

struct Value {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0;
    std::string str;
    std::vector<Value> arr;
    std::vector<std::pair<std::string, Value>> obj;      // in file order

    const Value* find(const std::string& key) const {
        if (kind != Object) return nullptr;
        for (auto& kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    bool is_null() const { return kind == Null; }
};

class Parser {
public:
    Parser(const char* p, size_t n) : p_(p), end_(p + n) {}
    Value parse() {
        Value v = value();
        ws();
        if (p_ != end_) fail("text after the value");
        return v;
    }

private:
    const char *p_, *end_;
    [[noreturn]] void fail(const std::string& what) { throw std::runtime_error("JSON: " + what); }
    void ws() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
    }
    bool eat(const char* word) {
        size_t n = strlen(word);
        if ((size_t)(end_ - p_) >= n && !strncmp(p_, word, n)) {
            p_ += n;
            return true;
        }
        return false;
    }
    std::string string() {
        if (p_ >= end_ || *p_ != '"') fail("a string was expected");
        ++p_;
        std::string out;
        while (p_ < end_ && *p_ != '"') {
            char c = *p_++;
            if (c != '\\') {
                out += c;
                continue;
            }
            if (p_ >= end_) fail("unfinished escape");
            char e = *p_++;
            switch (e) {
                case 'n': out += '\n'; break;
                case 't': out += '\t'; break;
                case 'r': out += '\r'; break;
                case 'b': out += '\b'; break;
                case 'f': out += '\f'; break;
                case 'u': {
                    if (end_ - p_ < 4) fail("unfinished \\u escape");
                    unsigned cp = (unsigned)strtoul(std::string(p_, 4).c_str(), nullptr, 16);
                    p_ += 4;
                    if (cp < 0x80) out += (char)cp;
                    else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
                    else { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
                    break;
                }
                default: out += e;
            }
        }
        if (p_ >= end_) fail("unfinished string");
        ++p_;
        return out;
    }
    Value value() {
        ws();
        if (p_ >= end_) fail("unexpected end");
        Value v;
        if (*p_ == '{') {
            ++p_;
            v.kind = Value::Object;
            ws();
            if (p_ < end_ && *p_ == '}') { ++p_; return v; }
            for (;;) {
                ws();
                std::string k = string();
                ws();
                if (p_ >= end_ || *p_ != ':') fail("':' was expected");
                ++p_;
                v.obj.emplace_back(std::move(k), value());
                ws();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == '}') { ++p_; return v; }
                fail("',' or '}' was expected");
            }
        }
        if (*p_ == '[') {
            ++p_;
            v.kind = Value::Array;
            ws();
            if (p_ < end_ && *p_ == ']') { ++p_; return v; }
            for (;;) {
                v.arr.push_back(value());
                ws();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == ']') { ++p_; return v; }
                fail("',' or ']' was expected");
            }
        }
        if (*p_ == '"') {
            v.kind = Value::String;
            v.str = string();
            return v;
        }
        if (eat("true")) { v.kind = Value::Bool; v.b = true; return v; }
        if (eat("false")) { v.kind = Value::Bool; return v; }
        if (eat("null")) return v;
        char* stop = nullptr;
        std::string text(p_, (size_t)(end_ - p_) < 64 ? (size_t)(end_ - p_) : 64);
        v.num = strtod(text.c_str(), &stop);
        if (stop == text.c_str()) fail("a value was expected");
        p_ += stop - text.c_str();
        v.kind = Value::Number;
        return v;
    }
};

inline Value parse(const std::string& text) { return Parser(text.data(), text.size()).parse(); }

}  // namespace json
}  // namespace llmengine_b200
