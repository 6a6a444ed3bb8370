// Tiny JSON reader (objects, arrays, strings, numbers, true/false/null) for rank-table files.
#pragma once
#include <map>
#include <memory>
#include <string>
#include <vector>
namespace hcclb {
struct JsonValue {
    enum Type { NUL, BOOL, NUM, STR, ARR, OBJ } type = NUL;
    bool b = false;
    double num = 0;
    std::string str;
    std::vector<JsonValue> arr;
    std::map<std::string, JsonValue> obj;
    const JsonValue *get(const std::string &k) const
    {
        auto it = obj.find(k);
        return it == obj.end() ? nullptr : &it->second;
    }
    // numeric value of a number or of a string holding a number (rank tables quote their integers)
    bool as_int(long *out) const;
};
// Returns false and fills *err on malformed input.
bool json_parse(const std::string &text, JsonValue *out, std::string *err);
}  // namespace hcclb
