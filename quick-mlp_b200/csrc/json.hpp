// Minimal JSON value + recursive-descent reader/writer for the network specification.
// The reference takes nlohmann::json in its constructors (src_cpp/include/qmlp/fused_network.h:156); that library
// is not vendored, so the spec text is parsed here. Supports objects, arrays, strings (with \uXXXX escapes),
// numbers, booleans, null and // or /* */ comments (the reference README's example spec carries one).
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace qmlp {

class configuration_error : public std::runtime_error {
public:
    explicit configuration_error(const std::string& m) : std::runtime_error(m) {}
};

class Json {
public:
    enum Type { Null, Bool, Number, String, Array, Object };

    Json() : type_(Null) {}
    static Json boolean(bool b) { Json j; j.type_ = Bool; j.bool_ = b; return j; }
    static Json number(double d) { Json j; j.type_ = Number; j.num_ = d; j.isInt_ = std::floor(d) == d && std::fabs(d) < 9e15; return j; }
    static Json string(const std::string& s) { Json j; j.type_ = String; j.str_ = s; return j; }
    static Json array() { Json j; j.type_ = Array; return j; }
    static Json object() { Json j; j.type_ = Object; return j; }

    Type type() const { return type_; }
    bool isNull() const { return type_ == Null; }
    bool isBool() const { return type_ == Bool; }
    bool isNumber() const { return type_ == Number; }
    bool isString() const { return type_ == String; }
    bool isArray() const { return type_ == Array; }
    bool isObject() const { return type_ == Object; }

    bool contains(const std::string& key) const {
        if (type_ != Object) return false;
        for (const auto& kv : obj_) if (kv.first == key) return true;
        return false;
    }
    const Json& at(const std::string& key) const {
        if (type_ != Object) throw configuration_error("json: object expected when reading key '" + key + "'");
        for (const auto& kv : obj_) if (kv.first == key) return kv.second;
        throw configuration_error("json: key '" + key + "' not found");
    }
    const Json& at(size_t i) const {
        if (type_ != Array || i >= arr_.size()) throw configuration_error("json: array index out of range");
        return arr_[i];
    }
    size_t size() const { return type_ == Array ? arr_.size() : (type_ == Object ? obj_.size() : 0); }
    bool empty() const { return size() == 0; }
    const std::vector<Json>& items() const { return arr_; }
    const std::vector<std::pair<std::string, Json>>& members() const { return obj_; }

    int asInt() const {
        if (type_ != Number) throw configuration_error("json: number expected");
        return static_cast<int>(num_);
    }
    double asDouble() const {
        if (type_ != Number) throw configuration_error("json: number expected");
        return num_;
    }
    bool asBool() const {
        if (type_ != Bool) throw configuration_error("json: boolean expected");
        return bool_;
    }
    const std::string& asString() const {
        if (type_ != String) throw configuration_error("json: string expected");
        return str_;
    }
    int valueInt(const std::string& key, int def) const { return contains(key) ? at(key).asInt() : def; }
    bool valueBool(const std::string& key, bool def) const { return contains(key) ? at(key).asBool() : def; }
    std::vector<float> valueFloats(const std::string& key) const {
        std::vector<float> v;
        if (!contains(key)) return v;
        const Json& a = at(key);
        if (!a.isArray()) throw configuration_error("json: array expected for '" + key + "'");
        for (const auto& e : a.items()) v.push_back(static_cast<float>(e.asDouble()));
        return v;
    }

    void push(Json v) { arr_.push_back(std::move(v)); }
    void set(const std::string& key, Json v) {
        for (auto& kv : obj_) if (kv.first == key) { kv.second = std::move(v); return; }
        obj_.emplace_back(key, std::move(v));
    }

    std::string dump() const { std::ostringstream o; write(o); return o.str(); }

    static Json parse(const std::string& text) {
        Parser p{text, 0};
        Json j = p.value();
        p.skip();
        if (p.pos != text.size()) p.fail("trailing characters");
        return j;
    }

private:
    Type type_;
    bool bool_ = false;
    double num_ = 0;
    bool isInt_ = false;
    std::string str_;
    std::vector<Json> arr_;
    std::vector<std::pair<std::string, Json>> obj_;

    static void writeString(std::ostream& o, const std::string& s) {
        o << '"';
        for (unsigned char c : s) {
            switch (c) {
            case '"': o << "\\\""; break;
            case '\\': o << "\\\\"; break;
            case '\n': o << "\\n"; break;
            case '\r': o << "\\r"; break;
            case '\t': o << "\\t"; break;
            default:
                if (c < 0x20) { char b[8]; std::snprintf(b, sizeof b, "\\u%04x", c); o << b; }
                else o << c;
            }
        }
        o << '"';
    }
    void write(std::ostream& o) const {
        switch (type_) {
        case Null: o << "null"; break;
        case Bool: o << (bool_ ? "true" : "false"); break;
        case Number:
            // formatted with snprintf, not with the stream's numeric inserter: that one goes through locale facets, which
            // fail in a process that holds a second copy of the C++ runtime (an extension linked against a static libstdc++)
            char b[40];
            if (isInt_) std::snprintf(b, sizeof b, "%lld", static_cast<long long>(num_));
            else std::snprintf(b, sizeof b, "%.9g", num_);
            o << b;
            break;
        case String: writeString(o, str_); break;
        case Array: {
            o << '[';
            for (size_t i = 0; i < arr_.size(); ++i) { if (i) o << ','; arr_[i].write(o); }
            o << ']';
        } break;
        case Object: {
            o << '{';
            for (size_t i = 0; i < obj_.size(); ++i) {
                if (i) o << ',';
                writeString(o, obj_[i].first); o << ':'; obj_[i].second.write(o);
            }
            o << '}';
        } break;
        }
    }

    struct Parser {
        const std::string& s;
        size_t pos;
        [[noreturn]] void fail(const std::string& what) const {
            throw configuration_error("json parse error at offset " + std::to_string(pos) + ": " + what);
        }
        void skip() {
            for (;;) {
                while (pos < s.size() && (s[pos] == ' ' || s[pos] == '\t' || s[pos] == '\n' || s[pos] == '\r')) ++pos;
                if (pos + 1 < s.size() && s[pos] == '/' && s[pos + 1] == '/') {
                    while (pos < s.size() && s[pos] != '\n') ++pos;
                } else if (pos + 1 < s.size() && s[pos] == '/' && s[pos + 1] == '*') {
                    pos += 2;
                    while (pos + 1 < s.size() && !(s[pos] == '*' && s[pos + 1] == '/')) ++pos;
                    pos = pos + 2 <= s.size() ? pos + 2 : s.size();
                } else break;
            }
        }
        Json value() {
            skip();
            if (pos >= s.size()) fail("unexpected end");
            char c = s[pos];
            if (c == '{') return object();
            if (c == '[') return array();
            if (c == '"') return Json::string(str());
            if (c == 't' && s.compare(pos, 4, "true") == 0) { pos += 4; return Json::boolean(true); }
            if (c == 'f' && s.compare(pos, 5, "false") == 0) { pos += 5; return Json::boolean(false); }
            if (c == 'n' && s.compare(pos, 4, "null") == 0) { pos += 4; return Json(); }
            if (c == '-' || (c >= '0' && c <= '9')) return num();
            fail(std::string("unexpected character '") + c + "'");
        }
        Json num() {
            const char* b = s.c_str() + pos;
            char* e = nullptr;
            double d = std::strtod(b, &e);
            if (e == b) fail("bad number");
            pos += static_cast<size_t>(e - b);
            return Json::number(d);
        }
        std::string str() {
            ++pos; // opening quote
            std::string o;
            while (pos < s.size() && s[pos] != '"') {
                char c = s[pos++];
                if (c != '\\') { o += c; continue; }
                if (pos >= s.size()) fail("bad escape");
                char e = s[pos++];
                switch (e) {
                case '"': o += '"'; break;
                case '\\': o += '\\'; break;
                case '/': o += '/'; break;
                case 'b': o += '\b'; break;
                case 'f': o += '\f'; break;
                case 'n': o += '\n'; break;
                case 'r': o += '\r'; break;
                case 't': o += '\t'; break;
                case 'u': {
                    if (pos + 4 > s.size()) fail("bad \\u escape");
                    unsigned cp = static_cast<unsigned>(std::strtoul(s.substr(pos, 4).c_str(), nullptr, 16));
                    pos += 4;
                    if (cp < 0x80) o += static_cast<char>(cp);
                    else if (cp < 0x800) { o += static_cast<char>(0xC0 | (cp >> 6)); o += static_cast<char>(0x80 | (cp & 0x3F)); }
                    else { o += static_cast<char>(0xE0 | (cp >> 12)); o += static_cast<char>(0x80 | ((cp >> 6) & 0x3F)); o += static_cast<char>(0x80 | (cp & 0x3F)); }
                } break;
                default: fail("bad escape");
                }
            }
            if (pos >= s.size()) fail("unterminated string");
            ++pos; // closing quote
            return o;
        }
        Json array() {
            ++pos;
            Json a = Json::array();
            skip();
            if (pos < s.size() && s[pos] == ']') { ++pos; return a; }
            for (;;) {
                a.push(value());
                skip();
                if (pos < s.size() && s[pos] == ',') { ++pos; continue; }
                if (pos < s.size() && s[pos] == ']') { ++pos; return a; }
                fail("',' or ']' expected");
            }
        }
        Json object() {
            ++pos;
            Json o = Json::object();
            skip();
            if (pos < s.size() && s[pos] == '}') { ++pos; return o; }
            for (;;) {
                skip();
                if (pos >= s.size() || s[pos] != '"') fail("string key expected");
                std::string k = str();
                skip();
                if (pos >= s.size() || s[pos] != ':') fail("':' expected");
                ++pos;
                o.set(k, value());
                skip();
                if (pos < s.size() && s[pos] == ',') { ++pos; continue; }
                if (pos < s.size() && s[pos] == '}') { ++pos; return o; }
                fail("',' or '}' expected");
            }
        }
    };
};

} // namespace qmlp
