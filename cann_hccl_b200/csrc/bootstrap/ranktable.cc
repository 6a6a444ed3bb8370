#include "bootstrap/ranktable.h"
#include <algorithm>
#include <fstream>
#include <sstream>
#include "common/json.h"
#include "health/consistency.h"
namespace hcclb {
HcclResult parse_ranktable(const std::string &text, RankTable *out, std::string *err)
{
    JsonValue root;
    std::string perr;
    auto bad = [&](const std::string &m) { if (err) *err = m; return HCCL_E_PARA; };
    if (!json_parse(text, &root, &perr)) return bad("rank table is not valid JSON: " + perr);
    if (root.type != JsonValue::OBJ) return bad("rank table must be a JSON object");
    if (const JsonValue *st = root.get("status"))
        if (st->type == JsonValue::STR && st->str != "completed") return bad("rank table status is not 'completed'");
    const JsonValue *sl = root.get("server_list");
    if (!sl || sl->type != JsonValue::ARR || sl->arr.empty()) return bad("rank table has no server_list");
    if (sl->arr.size() != 1) return bad("rank table lists more than one server: a communicator spans one NVSwitch domain");
    if (const JsonValue *sc = root.get("server_count")) {
        long n;
        if (sc->as_int(&n) && n != (long)sl->arr.size()) return bad("server_count does not match server_list");
    }
    RankTable t;
    const JsonValue &srv = sl->arr[0];
    std::string sid;
    if (const JsonValue *v = srv.get("server_id")) sid = v->str;
    if (const JsonValue *v = srv.get("host_ip")) t.host_ip = v->str;
    if (const JsonValue *v = srv.get("host_port")) { long p; if (v->as_int(&p)) t.host_port = (int)p; }
    const JsonValue *dev = srv.get("device");
    if (!dev || dev->type != JsonValue::ARR || dev->arr.empty()) return bad("server entry has no device list");
    for (const JsonValue &d : dev->arr) {
        RankEntry e;
        long v;
        const JsonValue *di = d.get("device_id"), *ri = d.get("rank_id");
        if (!di || !di->as_int(&v) || v < 0) return bad("device entry without a valid device_id");
        e.device_id = (int)v;
        if (!ri || !ri->as_int(&v) || v < 0) return bad("device entry without a valid rank_id");
        e.rank_id = (int)v;
        e.server_id = sid;
        t.ranks.push_back(e);
    }
    std::sort(t.ranks.begin(), t.ranks.end(), [](const RankEntry &a, const RankEntry &b) { return a.rank_id < b.rank_id; });
    for (size_t i = 0; i < t.ranks.size(); ++i)
        if (t.ranks[i].rank_id != (int)i) return bad("rank ids must be unique and dense from 0");
    t.crc = crc32(text.data(), text.size(), 0);
    *out = t;
    return HCCL_SUCCESS;
}
HcclResult load_ranktable_file(const char *path, RankTable *out, std::string *err)
{
    std::ifstream f(path);
    if (!f) { if (err) *err = std::string("cannot open ") + path; return HCCL_E_OPEN_FILE_FAILURE; }
    std::stringstream ss;
    ss << f.rdbuf();
    return parse_ranktable(ss.str(), out, err);
}
HcclResult partition_ranktable(const RankTable &t, const std::vector<uint32_t> &ids, RankTable *out)
{
    RankTable s = t;
    s.ranks.clear();
    for (size_t i = 0; i < ids.size(); ++i) {
        if (ids[i] >= t.ranks.size()) return HCCL_E_PARA;
        for (size_t j = 0; j < i; ++j) if (ids[j] == ids[i]) return HCCL_E_PARA;
        RankEntry e = t.ranks[ids[i]];
        e.rank_id = (int)i;
        s.ranks.push_back(e);
    }
    *out = s;
    return HCCL_SUCCESS;
}
}  // namespace hcclb
