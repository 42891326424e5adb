// A small JSON value and parser (objects keep insertion order); used for safetensors headers,
// META.json, config.json and option strings.
#pragma once
#include <map>
#include <memory>
#include <vector>

#include "common.hpp"

namespace qwh {

class Json {
public:
    enum Kind { Null, Bool, Num, Str, Arr, Obj };
    Kind kind = Null;
    bool b = false;
    double num = 0;
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;

    static Json parse(const std::string &text) {
        size_t i = 0;
        Json v = value(text, i);
        ws(text, i);
        if (i != text.size()) fail("json: trailing characters");
        return v;
    }
    bool has(const std::string &k) const {
        for (auto &kv : obj) if (kv.first == k) return true;
        return false;
    }
    const Json &operator[](const std::string &k) const {
        for (auto &kv : obj) if (kv.first == k) return kv.second;
        fail("json: missing key " + k);
    }
    const Json &operator[](size_t i) const { QWH_CHECK(kind == Arr && i < arr.size(), "json index"); return arr[i]; }
    size_t size() const { return kind == Arr ? arr.size() : obj.size(); }
    int64_t as_int() const { QWH_CHECK(kind == Num, "json: not a number"); return int64_t(num); }
    double as_double() const { QWH_CHECK(kind == Num, "json: not a number"); return num; }
    const std::string &as_str() const { QWH_CHECK(kind == Str, "json: not a string"); return str; }
    bool as_bool() const { QWH_CHECK(kind == Bool, "json: not a bool"); return b; }

private:
    static void ws(const std::string &s, size_t &i) { while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i; }
    static Json value(const std::string &s, size_t &i) {
        ws(s, i);
        if (i >= s.size()) fail("json: unexpected end");
        Json v;
        const char c = s[i];
        if (c == '{') {
            v.kind = Obj;
            ++i; ws(s, i);
            if (i < s.size() && s[i] == '}') { ++i; return v; }
            for (;;) {
                ws(s, i);
                Json k = string(s, i);
                ws(s, i);
                if (i >= s.size() || s[i] != ':') fail("json: expected ':'");
                ++i;
                v.obj.emplace_back(k.str, value(s, i));
                ws(s, i);
                if (i < s.size() && s[i] == ',') { ++i; continue; }
                if (i < s.size() && s[i] == '}') { ++i; return v; }
                fail("json: expected ',' or '}'");
            }
        }
        if (c == '[') {
            v.kind = Arr;
            ++i; ws(s, i);
            if (i < s.size() && s[i] == ']') { ++i; return v; }
            for (;;) {
                v.arr.push_back(value(s, i));
                ws(s, i);
                if (i < s.size() && s[i] == ',') { ++i; continue; }
                if (i < s.size() && s[i] == ']') { ++i; return v; }
                fail("json: expected ',' or ']'");
            }
        }
        if (c == '"') return string(s, i);
        if (s.compare(i, 4, "true") == 0) { i += 4; v.kind = Bool; v.b = true; return v; }
        if (s.compare(i, 5, "false") == 0) { i += 5; v.kind = Bool; return v; }
        if (s.compare(i, 4, "null") == 0) { i += 4; return v; }
        size_t j = i;
        while (j < s.size() && (std::isdigit((unsigned char)s[j]) || s[j] == '-' || s[j] == '+' || s[j] == '.' || s[j] == 'e' || s[j] == 'E')) ++j;
        if (j == i) fail("json: unexpected character");
        v.kind = Num;
        v.num = std::stod(s.substr(i, j - i));
        i = j;
        return v;
    }
    static void utf8(std::string &out, unsigned cp) {
        if (cp < 0x80) out += char(cp);
        else if (cp < 0x800) { out += char(0xc0 | (cp >> 6)); out += char(0x80 | (cp & 0x3f)); }
        else if (cp < 0x10000) { out += char(0xe0 | (cp >> 12)); out += char(0x80 | ((cp >> 6) & 0x3f)); out += char(0x80 | (cp & 0x3f)); }
        else { out += char(0xf0 | (cp >> 18)); out += char(0x80 | ((cp >> 12) & 0x3f)); out += char(0x80 | ((cp >> 6) & 0x3f)); out += char(0x80 | (cp & 0x3f)); }
    }
    static Json string(const std::string &s, size_t &i) {
        if (i >= s.size() || s[i] != '"') fail("json: expected string");
        Json v;
        v.kind = Str;
        for (++i; i < s.size(); ++i) {
            char c = s[i];
            if (c == '"') { ++i; return v; }
            if (c != '\\') { v.str += c; continue; }
            if (++i >= s.size()) break;
            switch (s[i]) {
                case 'n': v.str += '\n'; break;
                case 't': v.str += '\t'; break;
                case 'r': v.str += '\r'; break;
                case 'b': v.str += '\b'; break;
                case 'f': v.str += '\f'; break;
                case 'u': {
                    if (i + 4 >= s.size()) fail("json: bad \\u escape");
                    unsigned cp = unsigned(std::stoul(s.substr(i + 1, 4), nullptr, 16));
                    i += 4;
                    if (cp >= 0xd800 && cp < 0xdc00 && i + 6 < s.size() && s[i + 1] == '\\' && s[i + 2] == 'u') {
                        unsigned lo = unsigned(std::stoul(s.substr(i + 3, 4), nullptr, 16));
                        cp = 0x10000 + ((cp - 0xd800) << 10) + (lo - 0xdc00);
                        i += 6;
                    }
                    utf8(v.str, cp);
                    break;
                }
                default: v.str += s[i];
            }
        }
        fail("json: unterminated string");
    }
};

}  // namespace qwh
