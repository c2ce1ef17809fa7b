// A small JSON value with a parser and a writer: what config.json, the safetensors header, model
// plans and the introspection strings of the C API need.  Objects keep the order of their keys.
// The reference carries its own parser for the safetensors header
// (src/model/safetensors_loader.cpp:34-208) and never reads config.json.
#pragma once

#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace imp {

class Json {
public:
    enum Type { Null, Bool, Int, Float, String, Array, Object };
    using Member = std::pair<std::string, Json>;

    Json() = default;
    Json(std::nullptr_t) {}
    Json(bool b) : type_(Bool), b_(b) {}
    Json(int v) : type_(Int), i_(v) {}
    Json(int64_t v) : type_(Int), i_(v) {}
    Json(size_t v) : type_(Int), i_((int64_t)v) {}
    Json(double v) : type_(Float), d_(v) {}
    Json(const char* s) : type_(String), s_(s) {}
    Json(std::string s) : type_(String), s_(std::move(s)) {}

    static Json array() { Json j; j.type_ = Array; return j; }
    static Json object() { Json j; j.type_ = Object; return j; }
    template <typename T> static Json array_of(const std::vector<T>& v) {
        Json j = array();
        for (const auto& x : v) j.push(Json(x));
        return j;
    }

    Type type() const { return type_; }
    bool is_null() const { return type_ == Null; }
    bool is_bool() const { return type_ == Bool; }
    bool is_int() const { return type_ == Int; }
    bool is_number() const { return type_ == Int || type_ == Float; }
    bool is_string() const { return type_ == String; }
    bool is_array() const { return type_ == Array; }
    bool is_object() const { return type_ == Object; }
    const char* type_name() const;

    bool as_bool() const { need(Bool); return b_; }
    int64_t as_int() const;            // integers, and floats with an integral value
    double as_double() const { if (type_ == Int) return (double)i_; need(Float); return d_; }
    const std::string& as_string() const { need(String); return s_; }
    const std::vector<Json>& items() const { need(Array); return a_; }
    std::vector<Json>& items() { need(Array); return a_; }
    const std::vector<Member>& members() const { need(Object); return o_; }
    std::vector<Member>& members() { need(Object); return o_; }
    size_t size() const { return type_ == Array ? a_.size() : type_ == Object ? o_.size() : 0; }

    // Object access.  find: nullptr when absent.  at: throws when absent.  operator[]: inserts.
    const Json* find(const std::string& key) const;
    Json* find(const std::string& key);
    bool has(const std::string& key) const { return find(key) != nullptr; }
    const Json& at(const std::string& key) const;
    Json& operator[](const std::string& key);
    const Json& operator[](size_t i) const { need(Array); return a_.at(i); }
    void push(Json v) { need(Array); a_.push_back(std::move(v)); }
    void erase(const std::string& key);

    // Typed reads with defaults, for parameter dictionaries.
    int64_t get_int(const std::string& key, int64_t dflt) const;
    double get_double(const std::string& key, double dflt) const;
    bool get_bool(const std::string& key, bool dflt) const;
    std::string get_string(const std::string& key, const std::string& dflt) const;

    std::string dump(int indent = -1) const;
    static Json parse(const std::string& text, const std::string& where = "JSON");   // throws std::runtime_error

    bool operator==(const Json& o) const;
    bool operator!=(const Json& o) const { return !(*this == o); }

private:
    void need(Type t) const;
    void write(std::string& out, int indent, int depth) const;
    Type type_ = Null;
    bool b_ = false;
    int64_t i_ = 0;
    double d_ = 0.0;
    std::string s_;
    std::vector<Json> a_;
    std::vector<Member> o_;
};

}  // namespace imp
