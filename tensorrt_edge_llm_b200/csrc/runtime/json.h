// Minimal JSON value + recursive-descent parser / serialiser for the runtime (engine config,
// tokenizer.json, request files).  UTF-8 in, UTF-8 out; \uXXXX escapes incl. surrogate pairs.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace telb {

class Json {
  public:
    enum class Type { Null, Bool, Number, String, Array, Object };
    using Array = std::vector<Json>;
    using Object = std::vector<std::pair<std::string, Json>>;   // keeps insertion order

    Json() = default;
    Json(bool b) : type_(Type::Bool), b_(b) {}
    Json(double d) : type_(Type::Number), n_(d) {}
    Json(int64_t i) : type_(Type::Number), n_(static_cast<double>(i)), is_int_(true), i_(i) {}
    Json(int i) : Json(static_cast<int64_t>(i)) {}
    Json(const std::string& s) : type_(Type::String), s_(s) {}
    Json(const char* s) : type_(Type::String), s_(s) {}
    static Json array() { Json j; j.type_ = Type::Array; return j; }
    static Json object() { Json j; j.type_ = Type::Object; return j; }

    Type type() const { return type_; }
    bool is_null() const { return type_ == Type::Null; }
    bool is_object() const { return type_ == Type::Object; }
    bool is_array() const { return type_ == Type::Array; }
    bool is_string() const { return type_ == Type::String; }
    bool is_number() const { return type_ == Type::Number; }
    bool is_bool() const { return type_ == Type::Bool; }

    bool as_bool(bool dflt = false) const { return type_ == Type::Bool ? b_ : dflt; }
    double as_double(double dflt = 0.0) const { return type_ == Type::Number ? n_ : dflt; }
    int64_t as_int(int64_t dflt = 0) const { return type_ == Type::Number ? (is_int_ ? i_ : static_cast<int64_t>(n_)) : dflt; }
    const std::string& as_string() const {
        static const std::string empty;
        return type_ == Type::String ? s_ : empty;
    }
    const Array& items() const { return a_; }
    Array& items() { return a_; }
    const Object& members() const { return o_; }

    bool contains(const std::string& k) const { return find(k) != nullptr; }
    const Json* find(const std::string& k) const {
        if (type_ != Type::Object) return nullptr;
        for (const auto& kv : o_)
            if (kv.first == k) return &kv.second;
        return nullptr;
    }
    const Json& operator[](const std::string& k) const {
        static const Json null_json;
        const Json* p = find(k);
        return p ? *p : null_json;
    }
    const Json& operator[](size_t i) const { return a_.at(i); }
    size_t size() const { return type_ == Type::Array ? a_.size() : (type_ == Type::Object ? o_.size() : 0); }
    void set(const std::string& k, Json v) {
        if (type_ != Type::Object) { type_ = Type::Object; o_.clear(); }
        for (auto& kv : o_)
            if (kv.first == k) { kv.second = std::move(v); return; }
        o_.emplace_back(k, std::move(v));
    }
    void push_back(Json v) {
        if (type_ != Type::Array) { type_ = Type::Array; a_.clear(); }
        a_.push_back(std::move(v));
    }

    static Json parse(const std::string& text);
    std::string dump() const;

  private:
    Type type_ = Type::Null;
    bool b_ = false;
    double n_ = 0.0;
    bool is_int_ = false;
    int64_t i_ = 0;
    std::string s_;
    Array a_;
    Object o_;
    friend class JsonParser;
};

}  // namespace telb
