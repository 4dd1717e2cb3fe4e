// Minimal JSON document model + recursive-descent parser for package manifests.
// Numbers keep their source text so that integers up to 2^63 and floats both
// round-trip; objects keep insertion order.
#pragma once

#include <cstdint>
#include <cstdlib>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace nerve {

class Json {
public:
    enum class Kind { Null, Bool, Number, String, Array, Object };

    Json() = default;

    Kind kind() const { return kind_; }
    bool is_null() const { return kind_ == Kind::Null; }
    bool is_object() const { return kind_ == Kind::Object; }
    bool is_array() const { return kind_ == Kind::Array; }
    bool is_string() const { return kind_ == Kind::String; }
    bool is_number() const { return kind_ == Kind::Number; }
    bool is_bool() const { return kind_ == Kind::Bool; }

    bool as_bool() const {
        require(Kind::Bool, "bool");
        return bool_;
    }
    double as_double() const {
        require(Kind::Number, "number");
        return std::strtod(text_.c_str(), nullptr);
    }
    int64_t as_int() const {
        require(Kind::Number, "number");
        if (text_.find_first_of(".eE") != std::string::npos) return static_cast<int64_t>(as_double());
        return std::strtoll(text_.c_str(), nullptr, 10);
    }
    const std::string &as_string() const {
        require(Kind::String, "string");
        return text_;
    }
    const std::vector<Json> &items() const {
        require(Kind::Array, "array");
        return array_;
    }
    const std::vector<std::pair<std::string, Json>> &members() const {
        require(Kind::Object, "object");
        return object_;
    }
    size_t size() const { return kind_ == Kind::Array ? array_.size() : object_.size(); }

    bool has(const std::string &key) const { return kind_ == Kind::Object && find(key) != nullptr; }
    // Missing keys yield a shared null value so that optional fields chain.
    const Json &operator[](const std::string &key) const {
        static const Json null_value;
        if (kind_ != Kind::Object) return null_value;
        const Json *found = find(key);
        return found ? *found : null_value;
    }
    const Json &operator[](size_t index) const {
        require(Kind::Array, "array");
        if (index >= array_.size()) throw std::runtime_error("json: array index out of range");
        return array_[index];
    }
    const Json &at(const std::string &key) const {
        const Json *found = kind_ == Kind::Object ? find(key) : nullptr;
        if (!found) throw std::runtime_error("json: missing key \"" + key + "\"");
        return *found;
    }

    static Json parse(const std::string &text) {
        Parser parser{text, 0};
        Json value = parser.value();
        parser.skip_space();
        if (parser.pos != text.size()) parser.fail("trailing characters");
        return value;
    }

private:
    struct Parser {
        const std::string &text;
        size_t pos;

        [[noreturn]] void fail(const char *what) const {
            throw std::runtime_error(std::string("json: ") + what + " at byte " + std::to_string(pos));
        }
        void skip_space() {
            while (pos < text.size() && (text[pos] == ' ' || text[pos] == '\n' || text[pos] == '\t' || text[pos] == '\r')) pos++;
        }
        bool consume(const char *literal) {
            size_t n = std::char_traits<char>::length(literal);
            if (text.compare(pos, n, literal) == 0) {
                pos += n;
                return true;
            }
            return false;
        }
        static void append_utf8(std::string &out, uint32_t cp) {
            if (cp < 0x80) out.push_back(static_cast<char>(cp));
            else if (cp < 0x800) {
                out.push_back(static_cast<char>(0xC0 | (cp >> 6)));
                out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
            } else if (cp < 0x10000) {
                out.push_back(static_cast<char>(0xE0 | (cp >> 12)));
                out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
                out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
            } else {
                out.push_back(static_cast<char>(0xF0 | (cp >> 18)));
                out.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
                out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
                out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
            }
        }
        uint32_t hex4() {
            if (pos + 4 > text.size()) fail("short \\u escape");
            uint32_t value = 0;
            for (int i = 0; i < 4; i++) {
                char c = text[pos++];
                value <<= 4;
                if (c >= '0' && c <= '9') value |= static_cast<uint32_t>(c - '0');
                else if (c >= 'a' && c <= 'f') value |= static_cast<uint32_t>(c - 'a' + 10);
                else if (c >= 'A' && c <= 'F') value |= static_cast<uint32_t>(c - 'A' + 10);
                else fail("bad \\u escape");
            }
            return value;
        }
        std::string string() {
            if (text[pos] != '"') fail("expected string");
            pos++;
            std::string out;
            while (true) {
                if (pos >= text.size()) fail("unterminated string");
                char c = text[pos++];
                if (c == '"') break;
                if (c != '\\') {
                    out.push_back(c);
                    continue;
                }
                if (pos >= text.size()) fail("unterminated escape");
                char e = text[pos++];
                switch (e) {
                case '"': out.push_back('"'); break;
                case '\\': out.push_back('\\'); break;
                case '/': out.push_back('/'); break;
                case 'b': out.push_back('\b'); break;
                case 'f': out.push_back('\f'); break;
                case 'n': out.push_back('\n'); break;
                case 'r': out.push_back('\r'); break;
                case 't': out.push_back('\t'); break;
                case 'u': {
                    uint32_t cp = hex4();
                    if (cp >= 0xD800 && cp < 0xDC00 && text.compare(pos, 2, "\\u") == 0) {
                        pos += 2;
                        uint32_t low = hex4();
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (low - 0xDC00);
                    }
                    append_utf8(out, cp);
                    break;
                }
                default: fail("bad escape");
                }
            }
            return out;
        }
        Json value() {
            skip_space();
            if (pos >= text.size()) fail("unexpected end");
            Json out;
            char c = text[pos];
            if (c == '{') {
                pos++;
                out.kind_ = Kind::Object;
                skip_space();
                if (pos < text.size() && text[pos] == '}') {
                    pos++;
                    return out;
                }
                while (true) {
                    skip_space();
                    std::string key = string();
                    skip_space();
                    if (pos >= text.size() || text[pos] != ':') fail("expected ':'");
                    pos++;
                    out.object_.emplace_back(std::move(key), value());
                    skip_space();
                    if (pos < text.size() && text[pos] == ',') {
                        pos++;
                        continue;
                    }
                    if (pos < text.size() && text[pos] == '}') {
                        pos++;
                        break;
                    }
                    fail("expected ',' or '}'");
                }
                return out;
            }
            if (c == '[') {
                pos++;
                out.kind_ = Kind::Array;
                skip_space();
                if (pos < text.size() && text[pos] == ']') {
                    pos++;
                    return out;
                }
                while (true) {
                    out.array_.push_back(value());
                    skip_space();
                    if (pos < text.size() && text[pos] == ',') {
                        pos++;
                        continue;
                    }
                    if (pos < text.size() && text[pos] == ']') {
                        pos++;
                        break;
                    }
                    fail("expected ',' or ']'");
                }
                return out;
            }
            if (c == '"') {
                out.kind_ = Kind::String;
                out.text_ = string();
                return out;
            }
            if (consume("true")) {
                out.kind_ = Kind::Bool;
                out.bool_ = true;
                return out;
            }
            if (consume("false")) {
                out.kind_ = Kind::Bool;
                out.bool_ = false;
                return out;
            }
            if (consume("null")) return out;
            size_t start = pos;
            while (pos < text.size() && (std::string("+-0123456789.eE").find(text[pos]) != std::string::npos)) pos++;
            if (pos == start) fail("unexpected character");
            out.kind_ = Kind::Number;
            out.text_ = text.substr(start, pos - start);
            return out;
        }
    };

    void require(Kind kind, const char *name) const {
        if (kind_ != kind) throw std::runtime_error(std::string("json: value is not a ") + name);
    }
    const Json *find(const std::string &key) const {
        for (const auto &member : object_)
            if (member.first == key) return &member.second;
        return nullptr;
    }

    Kind kind_ = Kind::Null;
    bool bool_ = false;
    std::string text_;
    std::vector<Json> array_;
    std::vector<std::pair<std::string, Json>> object_;
};

}  // namespace nerve
