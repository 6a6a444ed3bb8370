#include "common/json.h"
#include <cctype>
#include <cstdlib>
namespace hcclb {
namespace {
struct P {
    const std::string &s;
    size_t i = 0;
    std::string err;
    void ws() { while (i < s.size() && isspace((unsigned char)s[i])) ++i; }
    bool fail(const char *m) { if (err.empty()) err = std::string(m) + " at offset " + std::to_string(i); return false; }
    bool str(std::string *o)
    {
        if (s[i] != '"') return fail("expected string");
        ++i;
        while (i < s.size() && s[i] != '"') {
            if (s[i] == '\\' && i + 1 < s.size()) {
                char c = s[i + 1];
                o->push_back(c == 'n' ? '\n' : c == 't' ? '\t' : c);
                i += 2;
            } else o->push_back(s[i++]);
        }
        if (i >= s.size()) return fail("unterminated string");
        ++i;
        return true;
    }
    bool val(JsonValue *v, int depth)
    {
        if (depth > 64) return fail("nesting too deep");
        ws();
        if (i >= s.size()) return fail("unexpected end");
        char c = s[i];
        if (c == '{') {
            v->type = JsonValue::OBJ;
            ++i; ws();
            if (i < s.size() && s[i] == '}') { ++i; return true; }
            for (;;) {
                ws();
                std::string k;
                if (i >= s.size() || !str(&k)) return fail("expected key");
                ws();
                if (i >= s.size() || s[i] != ':') return fail("expected ':'");
                ++i;
                if (!val(&v->obj[k], depth + 1)) return false;
                ws();
                if (i < s.size() && s[i] == ',') { ++i; continue; }
                if (i < s.size() && s[i] == '}') { ++i; return true; }
                return fail("expected ',' or '}'");
            }
        }
        if (c == '[') {
            v->type = JsonValue::ARR;
            ++i; ws();
            if (i < s.size() && s[i] == ']') { ++i; return true; }
            for (;;) {
                v->arr.emplace_back();
                if (!val(&v->arr.back(), depth + 1)) return false;
                ws();
                if (i < s.size() && s[i] == ',') { ++i; continue; }
                if (i < s.size() && s[i] == ']') { ++i; return true; }
                return fail("expected ',' or ']'");
            }
        }
        if (c == '"') { v->type = JsonValue::STR; return str(&v->str); }
        if (s.compare(i, 4, "true") == 0) { v->type = JsonValue::BOOL; v->b = true; i += 4; return true; }
        if (s.compare(i, 5, "false") == 0) { v->type = JsonValue::BOOL; v->b = false; i += 5; return true; }
        if (s.compare(i, 4, "null") == 0) { v->type = JsonValue::NUL; i += 4; return true; }
        char *end = nullptr;
        double d = strtod(s.c_str() + i, &end);
        if (end == s.c_str() + i) return fail("unexpected character");
        v->type = JsonValue::NUM;
        v->num = d;
        i = (size_t)(end - s.c_str());
        return true;
    }
};
}  // namespace
bool JsonValue::as_int(long *out) const
{
    if (type == NUM) { *out = (long)num; return true; }
    if (type == STR && !str.empty()) {
        char *end = nullptr;
        long v = strtol(str.c_str(), &end, 10);
        if (end && *end == 0) { *out = v; return true; }
    }
    return false;
}
bool json_parse(const std::string &text, JsonValue *out, std::string *err)
{
    P p{text};
    bool ok = p.val(out, 0);
    if (ok) {
        p.ws();
        if (p.i != text.size()) ok = p.fail("trailing characters");
    }
    if (!ok && err) *err = p.err;
    return ok;
}
}  // namespace hcclb
