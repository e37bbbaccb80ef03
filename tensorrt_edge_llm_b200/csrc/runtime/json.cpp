#include "json.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>

namespace telb {

class JsonParser {
  public:
    explicit JsonParser(const std::string& t) : t_(t) {}
    Json run() {
        Json v = value();
        ws();
        if (p_ != t_.size()) fail("trailing characters");
        return v;
    }

  private:
    const std::string& t_;
    size_t p_ = 0;

    [[noreturn]] void fail(const char* what) const {
        throw std::runtime_error(std::string("JSON parse error at byte ") + std::to_string(p_) + ": " + what);
    }
    void ws() {
        while (p_ < t_.size() && (t_[p_] == ' ' || t_[p_] == '\n' || t_[p_] == '\t' || t_[p_] == '\r')) ++p_;
    }
    Json value() {
        ws();
        if (p_ >= t_.size()) fail("unexpected end");
        const char c = t_[p_];
        if (c == '{') return object();
        if (c == '[') return array();
        if (c == '"') return Json(string());
        if (c == 't') { expect("true"); return Json(true); }
        if (c == 'f') { expect("false"); return Json(false); }
        if (c == 'n') { expect("null"); return Json(); }
        return number();
    }
    void expect(const char* lit) {
        for (const char* q = lit; *q; ++q, ++p_)
            if (p_ >= t_.size() || t_[p_] != *q) fail("bad literal");
    }
    Json number() {
        const size_t s = p_;
        bool is_int = true;
        if (p_ < t_.size() && (t_[p_] == '-' || t_[p_] == '+')) ++p_;
        while (p_ < t_.size()) {
            const char c = t_[p_];
            if (c >= '0' && c <= '9') { ++p_; }
            else if (c == '.' || c == 'e' || c == 'E' || c == '-' || c == '+') { is_int = false; ++p_; }
            else break;
        }
        if (s == p_) fail("bad number");
        const std::string tok = t_.substr(s, p_ - s);
        if (is_int && tok.size() < 18) return Json(static_cast<int64_t>(std::strtoll(tok.c_str(), nullptr, 10)));
        return Json(std::strtod(tok.c_str(), nullptr));
    }
    static void put_utf8(std::string& o, uint32_t cp) {
        if (cp < 0x80) o += static_cast<char>(cp);
        else if (cp < 0x800) { o += static_cast<char>(0xC0 | (cp >> 6)); o += static_cast<char>(0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) {
            o += static_cast<char>(0xE0 | (cp >> 12)); o += static_cast<char>(0x80 | ((cp >> 6) & 0x3F));
            o += static_cast<char>(0x80 | (cp & 0x3F));
        } else {
            o += static_cast<char>(0xF0 | (cp >> 18)); o += static_cast<char>(0x80 | ((cp >> 12) & 0x3F));
            o += static_cast<char>(0x80 | ((cp >> 6) & 0x3F)); o += static_cast<char>(0x80 | (cp & 0x3F));
        }
    }
    uint32_t hex4() {
        if (p_ + 4 > t_.size()) fail("bad \\u escape");
        uint32_t v = 0;
        for (int i = 0; i < 4; ++i) {
            const char c = t_[p_++];
            v <<= 4;
            if (c >= '0' && c <= '9') v |= c - '0';
            else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
            else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
            else fail("bad hex digit");
        }
        return v;
    }
    std::string string() {
        ++p_;   // opening quote
        std::string o;
        while (true) {
            if (p_ >= t_.size()) fail("unterminated string");
            const char c = t_[p_++];
            if (c == '"') break;
            if (c != '\\') { o += c; continue; }
            if (p_ >= t_.size()) fail("bad escape");
            const char e = t_[p_++];
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
                    uint32_t cp = hex4();
                    if (cp >= 0xD800 && cp <= 0xDBFF && p_ + 1 < t_.size() && t_[p_] == '\\' && t_[p_ + 1] == 'u') {
                        p_ += 2;
                        const uint32_t lo = hex4();
                        if (lo >= 0xDC00 && lo <= 0xDFFF) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    put_utf8(o, cp);
                    break;
                }
                default: fail("unknown escape");
            }
        }
        return o;
    }
    Json array() {
        ++p_;
        Json a = Json::array();
        ws();
        if (p_ < t_.size() && t_[p_] == ']') { ++p_; return a; }
        while (true) {
            a.push_back(value());
            ws();
            if (p_ >= t_.size()) fail("unterminated array");
            if (t_[p_] == ',') { ++p_; continue; }
            if (t_[p_] == ']') { ++p_; break; }
            fail("expected , or ]");
        }
        return a;
    }
    Json object() {
        ++p_;
        Json o = Json::object();
        ws();
        if (p_ < t_.size() && t_[p_] == '}') { ++p_; return o; }
        while (true) {
            ws();
            if (p_ >= t_.size() || t_[p_] != '"') fail("expected key");
            std::string k = string();
            ws();
            if (p_ >= t_.size() || t_[p_] != ':') fail("expected :");
            ++p_;
            o.o_.emplace_back(std::move(k), value());
            ws();
            if (p_ >= t_.size()) fail("unterminated object");
            if (t_[p_] == ',') { ++p_; continue; }
            if (t_[p_] == '}') { ++p_; break; }
            fail("expected , or }");
        }
        return o;
    }
};

Json Json::parse(const std::string& text) { return JsonParser(text).run(); }

static void dump_string(const std::string& s, std::string& o) {
    o += '"';
    for (unsigned char c : s) {
        switch (c) {
            case '"': o += "\\\""; break;
            case '\\': o += "\\\\"; break;
            case '\n': o += "\\n"; break;
            case '\r': o += "\\r"; break;
            case '\t': o += "\\t"; break;
            default:
                if (c < 0x20) {
                    char buf[8];
                    snprintf(buf, sizeof(buf), "\\u%04x", c);
                    o += buf;
                } else {
                    o += static_cast<char>(c);
                }
        }
    }
    o += '"';
}

static void dump_value(const Json& j, std::string& o) {
    switch (j.type()) {
        case Json::Type::Null: o += "null"; break;
        case Json::Type::Bool: o += j.as_bool() ? "true" : "false"; break;
        case Json::Type::Number: {
            const double d = j.as_double();
            char buf[40];
            if (std::floor(d) == d && std::fabs(d) < 9e15) snprintf(buf, sizeof(buf), "%lld", static_cast<long long>(j.as_int()));
            else snprintf(buf, sizeof(buf), "%.17g", d);
            o += buf;
            break;
        }
        case Json::Type::String: dump_string(j.as_string(), o); break;
        case Json::Type::Array: {
            o += '[';
            bool first = true;
            for (const auto& v : j.items()) {
                if (!first) o += ',';
                first = false;
                dump_value(v, o);
            }
            o += ']';
            break;
        }
        case Json::Type::Object: {
            o += '{';
            bool first = true;
            for (const auto& kv : j.members()) {
                if (!first) o += ',';
                first = false;
                dump_string(kv.first, o);
                o += ':';
                dump_value(kv.second, o);
            }
            o += '}';
            break;
        }
    }
}

std::string Json::dump() const {
    std::string o;
    dump_value(*this, o);
    return o;
}

}  // namespace telb
