// Minimal JSON reader/writer for plan and tensor descriptions.
// (The reference uses nlohmann/json for the same files, ark/model/model_json.hpp:7.)
#pragma once
#include <cstdint>
#include <cstdlib>
#include <map>
#include <sstream>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace arkb {

class Json {
   public:
    enum Type { Null, Bool, Int, Float, String, Array, Object };
    Type type = Null;
    bool b = false;
    int64_t i = 0;
    double d = 0;
    std::string s;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;

    static Json parse(const std::string &text) {
        size_t pos = 0;
        Json v = parse_value(text, pos);
        skip_ws(text, pos);
        if (pos != text.size()) throw std::runtime_error("json: trailing characters at " + std::to_string(pos));
        return v;
    }

    bool is_null() const { return type == Null; }
    bool is_object() const { return type == Object; }
    bool is_array() const { return type == Array; }
    bool is_string() const { return type == String; }
    bool is_number() const { return type == Int || type == Float; }
    bool contains(const std::string &k) const {
        for (auto &kv : obj)
            if (kv.first == k) return true;
        return false;
    }
    const Json &at(const std::string &k) const {
        for (auto &kv : obj)
            if (kv.first == k) return kv.second;
        throw std::runtime_error("json: missing key '" + k + "'");
    }
    const Json &at(size_t idx) const {
        if (type != Array || idx >= arr.size()) throw std::runtime_error("json: bad array index");
        return arr[idx];
    }
    size_t size() const { return type == Array ? arr.size() : obj.size(); }
    int64_t as_int() const {
        if (type == Int) return i;
        if (type == Float) return (int64_t)d;
        if (type == Bool) return b ? 1 : 0;
        throw std::runtime_error("json: not a number");
    }
    double as_float() const {
        if (type == Float) return d;
        if (type == Int) return (double)i;
        throw std::runtime_error("json: not a number");
    }
    bool as_bool() const {
        if (type == Bool) return b;
        if (type == Int) return i != 0;
        throw std::runtime_error("json: not a bool");
    }
    const std::string &as_string() const {
        if (type != String) throw std::runtime_error("json: not a string");
        return s;
    }
    std::vector<int64_t> as_int_vec() const {
        if (type != Array) throw std::runtime_error("json: not an array");
        std::vector<int64_t> v;
        for (auto &e : arr) v.push_back(e.as_int());
        return v;
    }

   private:
    static void skip_ws(const std::string &t, size_t &p) {
        while (p < t.size() && (t[p] == ' ' || t[p] == '\n' || t[p] == '\t' || t[p] == '\r')) ++p;
    }
    static Json parse_value(const std::string &t, size_t &p) {
        skip_ws(t, p);
        if (p >= t.size()) throw std::runtime_error("json: unexpected end");
        char c = t[p];
        Json v;
        if (c == '{') {
            v.type = Object;
            ++p;
            skip_ws(t, p);
            if (p < t.size() && t[p] == '}') {
                ++p;
                return v;
            }
            for (;;) {
                skip_ws(t, p);
                Json k = parse_string(t, p);
                skip_ws(t, p);
                if (p >= t.size() || t[p] != ':') throw std::runtime_error("json: expected ':' at " + std::to_string(p));
                ++p;
                Json e = parse_value(t, p);
                v.obj.emplace_back(k.s, std::move(e));
                skip_ws(t, p);
                if (p < t.size() && t[p] == ',') {
                    ++p;
                    continue;
                }
                if (p < t.size() && t[p] == '}') {
                    ++p;
                    return v;
                }
                throw std::runtime_error("json: expected ',' or '}' at " + std::to_string(p));
            }
        }
        if (c == '[') {
            v.type = Array;
            ++p;
            skip_ws(t, p);
            if (p < t.size() && t[p] == ']') {
                ++p;
                return v;
            }
            for (;;) {
                v.arr.push_back(parse_value(t, p));
                skip_ws(t, p);
                if (p < t.size() && t[p] == ',') {
                    ++p;
                    continue;
                }
                if (p < t.size() && t[p] == ']') {
                    ++p;
                    return v;
                }
                throw std::runtime_error("json: expected ',' or ']' at " + std::to_string(p));
            }
        }
        if (c == '"') return parse_string(t, p);
        if (t.compare(p, 4, "true") == 0) {
            v.type = Bool;
            v.b = true;
            p += 4;
            return v;
        }
        if (t.compare(p, 5, "false") == 0) {
            v.type = Bool;
            v.b = false;
            p += 5;
            return v;
        }
        if (t.compare(p, 4, "null") == 0) {
            p += 4;
            return v;
        }
        // number
        size_t q = p;
        bool is_float = false;
        if (q < t.size() && (t[q] == '-' || t[q] == '+')) ++q;
        while (q < t.size() && (isdigit((unsigned char)t[q]) || t[q] == '.' || t[q] == 'e' || t[q] == 'E' || t[q] == '-' ||
                                t[q] == '+')) {
            if (t[q] == '.' || t[q] == 'e' || t[q] == 'E') is_float = true;
            ++q;
        }
        if (q == p) throw std::runtime_error("json: unexpected character at " + std::to_string(p));
        std::string num = t.substr(p, q - p);
        p = q;
        if (is_float) {
            v.type = Float;
            v.d = strtod(num.c_str(), nullptr);
        } else {
            v.type = Int;
            v.i = strtoll(num.c_str(), nullptr, 10);
        }
        return v;
    }
    static Json parse_string(const std::string &t, size_t &p) {
        if (p >= t.size() || t[p] != '"') throw std::runtime_error("json: expected string at " + std::to_string(p));
        ++p;
        Json v;
        v.type = String;
        while (p < t.size() && t[p] != '"') {
            if (t[p] == '\\' && p + 1 < t.size()) {
                char e = t[p + 1];
                switch (e) {
                    case 'n': v.s += '\n'; break;
                    case 't': v.s += '\t'; break;
                    case 'r': v.s += '\r'; break;
                    case 'b': v.s += '\b'; break;
                    case 'f': v.s += '\f'; break;
                    case 'u': {
                        unsigned code = (unsigned)strtoul(t.substr(p + 2, 4).c_str(), nullptr, 16);
                        v.s += (char)(code & 0x7f);
                        p += 4;
                        break;
                    }
                    default: v.s += e; break;
                }
                p += 2;
            } else {
                v.s += t[p++];
            }
        }
        if (p >= t.size()) throw std::runtime_error("json: unterminated string");
        ++p;
        return v;
    }
};

}  // namespace arkb
