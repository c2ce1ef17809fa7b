#include "json.hpp"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace imp {

const char* Json::type_name() const {
    switch (type_) {
        case Null: return "null";
        case Bool: return "bool";
        case Int: return "int";
        case Float: return "float";
        case String: return "string";
        case Array: return "array";
        case Object: return "object";
    }
    return "?";
}

void Json::need(Type t) const {
    if (type_ != t) {
        static const char* names[] = {"null", "bool", "int", "float", "string", "array", "object"};
        throw std::runtime_error(std::string("JSON value is ") + type_name() + ", expected " + names[t]);
    }
}

int64_t Json::as_int() const {
    if (type_ == Int) return i_;
    if (type_ == Float && std::floor(d_) == d_ && std::fabs(d_) < 9.0e18) return (int64_t)d_;
    need(Int);
    return 0;
}

const Json* Json::find(const std::string& key) const {
    if (type_ != Object) return nullptr;
    for (const auto& m : o_)
        if (m.first == key) return &m.second;
    return nullptr;
}

Json* Json::find(const std::string& key) {
    return const_cast<Json*>(static_cast<const Json*>(this)->find(key));
}

const Json& Json::at(const std::string& key) const {
    const Json* j = find(key);
    if (!j) throw std::runtime_error("JSON object has no key '" + key + "'");
    return *j;
}

Json& Json::operator[](const std::string& key) {
    if (type_ == Null) type_ = Object;
    need(Object);
    if (Json* j = find(key)) return *j;
    o_.emplace_back(key, Json());
    return o_.back().second;
}

void Json::erase(const std::string& key) {
    if (type_ != Object) return;
    for (size_t i = 0; i < o_.size(); ++i)
        if (o_[i].first == key) {
            o_.erase(o_.begin() + (long)i);
            return;
        }
}

int64_t Json::get_int(const std::string& key, int64_t dflt) const {
    const Json* j = find(key);
    return (j && !j->is_null()) ? j->as_int() : dflt;
}
double Json::get_double(const std::string& key, double dflt) const {
    const Json* j = find(key);
    return (j && !j->is_null()) ? j->as_double() : dflt;
}
bool Json::get_bool(const std::string& key, bool dflt) const {
    const Json* j = find(key);
    if (!j || j->is_null()) return dflt;
    if (j->is_bool()) return j->as_bool();
    return j->as_int() != 0;
}
std::string Json::get_string(const std::string& key, const std::string& dflt) const {
    const Json* j = find(key);
    return (j && j->is_string()) ? j->as_string() : dflt;
}

bool Json::operator==(const Json& o) const {
    if (is_number() && o.is_number()) return as_double() == o.as_double();
    if (type_ != o.type_) return false;
    switch (type_) {
        case Null: return true;
        case Bool: return b_ == o.b_;
        case String: return s_ == o.s_;
        case Array: return a_ == o.a_;
        case Object: {
            if (o_.size() != o.o_.size()) return false;
            for (const auto& m : o_) {
                const Json* other = o.find(m.first);
                if (!other || !(*other == m.second)) return false;
            }
            return true;
        }
        default: return false;
    }
}

// ------------------------------------------------------------------------------------- writer
static void write_string(std::string& out, const std::string& s) {
    out.push_back('"');
    for (unsigned char c : s) {
        switch (c) {
            case '"': out += "\\\""; break;
            case '\\': out += "\\\\"; break;
            case '\n': out += "\\n"; break;
            case '\r': out += "\\r"; break;
            case '\t': out += "\\t"; break;
            default:
                if (c < 0x20) {
                    char buf[8];
                    snprintf(buf, sizeof buf, "\\u%04x", c);
                    out += buf;
                } else {
                    out.push_back((char)c);
                }
        }
    }
    out.push_back('"');
}

void Json::write(std::string& out, int indent, int depth) const {
    auto newline = [&](int d) {
        if (indent < 0) return;
        out.push_back('\n');
        out.append((size_t)(indent * d), ' ');
    };
    switch (type_) {
        case Null: out += "null"; break;
        case Bool: out += b_ ? "true" : "false"; break;
        case Int: out += std::to_string(i_); break;
        case Float: {
            if (!std::isfinite(d_)) { out += "null"; break; }
            char buf[40];
            snprintf(buf, sizeof buf, "%.17g", d_);
            out += buf;
            if (!strpbrk(buf, ".eEn")) out += ".0";
            break;
        }
        case String: write_string(out, s_); break;
        case Array:
            out.push_back('[');
            for (size_t i = 0; i < a_.size(); ++i) {
                if (i) out += indent < 0 ? ", " : ",";
                newline(depth + 1);
                a_[i].write(out, indent, depth + 1);
            }
            if (!a_.empty()) newline(depth);
            out.push_back(']');
            break;
        case Object:
            out.push_back('{');
            for (size_t i = 0; i < o_.size(); ++i) {
                if (i) out += indent < 0 ? ", " : ",";
                newline(depth + 1);
                write_string(out, o_[i].first);
                out += ": ";
                o_[i].second.write(out, indent, depth + 1);
            }
            if (!o_.empty()) newline(depth);
            out.push_back('}');
            break;
    }
}

std::string Json::dump(int indent) const {
    std::string out;
    write(out, indent, 0);
    return out;
}

// ------------------------------------------------------------------------------------- parser
namespace {
struct Parser {
    const std::string& t;
    const std::string& where;
    size_t p = 0;

    [[noreturn]] void fail(const std::string& msg) const {
        throw std::runtime_error(where + ": not valid JSON: " + msg + " at byte " + std::to_string(p));
    }
    void ws() {
        while (p < t.size() && (t[p] == ' ' || t[p] == '\n' || t[p] == '\t' || t[p] == '\r')) ++p;
    }
    bool lit(const char* s) {
        size_t n = strlen(s);
        if (t.compare(p, n, s) == 0) { p += n; return true; }
        return false;
    }
    static void utf8(std::string& out, unsigned cp) {
        if (cp < 0x80) out.push_back((char)cp);
        else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
        else if (cp < 0x10000) {
            out.push_back((char)(0xE0 | (cp >> 12)));
            out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
            out.push_back((char)(0x80 | (cp & 0x3F)));
        } else {
            out.push_back((char)(0xF0 | (cp >> 18)));
            out.push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
            out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
            out.push_back((char)(0x80 | (cp & 0x3F)));
        }
    }
    unsigned hex4() {
        if (p + 4 > t.size()) fail("short \\u escape");
        unsigned v = 0;
        for (int i = 0; i < 4; ++i) {
            char c = t[p++];
            v <<= 4;
            if (c >= '0' && c <= '9') v |= (unsigned)(c - '0');
            else if (c >= 'a' && c <= 'f') v |= (unsigned)(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= (unsigned)(c - 'A' + 10);
            else fail("bad \\u escape");
        }
        return v;
    }
    std::string string() {
        ++p;  // opening quote
        std::string out;
        while (true) {
            if (p >= t.size()) fail("unterminated string");
            char c = t[p++];
            if (c == '"') return out;
            if (c != '\\') { out.push_back(c); continue; }
            if (p >= t.size()) fail("unterminated escape");
            char e = t[p++];
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
                    unsigned cp = hex4();
                    if (cp >= 0xD800 && cp < 0xDC00 && p + 1 < t.size() && t[p] == '\\' && t[p + 1] == 'u') {
                        p += 2;
                        unsigned lo = hex4();
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    utf8(out, cp);
                    break;
                }
                default: fail("unknown escape");
            }
        }
    }
    Json number() {
        size_t start = p;
        bool is_float = false;
        if (p < t.size() && (t[p] == '-' || t[p] == '+')) ++p;
        while (p < t.size()) {
            char c = t[p];
            if (c >= '0' && c <= '9') ++p;
            else if (c == '.' || c == 'e' || c == 'E' || c == '+' || c == '-') { is_float = true; ++p; }
            else break;
        }
        std::string s = t.substr(start, p - start);
        if (s.empty() || s == "-") fail("bad number");
        if (!is_float) {
            errno = 0;
            char* end = nullptr;
            long long v = strtoll(s.c_str(), &end, 10);
            if (errno == 0 && end && *end == 0) return Json((int64_t)v);
        }
        char* end = nullptr;
        double d = strtod(s.c_str(), &end);
        if (!end || *end != 0) fail("bad number '" + s + "'");
        return Json(d);
    }
    Json value(int depth) {
        if (depth > 200) fail("nested too deeply");
        ws();
        if (p >= t.size()) fail("unexpected end");
        char c = t[p];
        if (c == '{') {
            ++p;
            Json o = Json::object();
            ws();
            if (p < t.size() && t[p] == '}') { ++p; return o; }
            while (true) {
                ws();
                if (p >= t.size() || t[p] != '"') fail("expected a key");
                std::string k = string();
                ws();
                if (p >= t.size() || t[p] != ':') fail("expected ':'");
                ++p;
                o[k] = value(depth + 1);
                ws();
                if (p < t.size() && t[p] == ',') { ++p; continue; }
                if (p < t.size() && t[p] == '}') { ++p; return o; }
                fail("expected ',' or '}'");
            }
        }
        if (c == '[') {
            ++p;
            Json a = Json::array();
            ws();
            if (p < t.size() && t[p] == ']') { ++p; return a; }
            while (true) {
                a.push(value(depth + 1));
                ws();
                if (p < t.size() && t[p] == ',') { ++p; continue; }
                if (p < t.size() && t[p] == ']') { ++p; return a; }
                fail("expected ',' or ']'");
            }
        }
        if (c == '"') return Json(string());
        if (lit("true")) return Json(true);
        if (lit("false")) return Json(false);
        if (lit("null")) return Json();
        if (lit("NaN")) return Json(std::nan(""));
        if (lit("Infinity")) return Json(INFINITY);
        if (lit("-Infinity")) return Json(-INFINITY);
        if (c == '-' || (c >= '0' && c <= '9')) return number();
        fail(std::string("unexpected character '") + c + "'");
    }
};
}  // namespace

Json Json::parse(const std::string& text, const std::string& where) {
    Parser ps{text, where};
    Json v = ps.value(0);
    ps.ws();
    if (ps.p != text.size()) ps.fail("trailing characters");
    return v;
}

}  // namespace imp
