// Group-name front end (include/hccl/hcom.h): a process-wide table group name -> communicator, world-rank lists of the
// groups, and the gradient-fusion settings per group.  Role of the reference's framework/hcom/hcom_common.cc; the
// reference keeps the same three maps (group -> comm in HcomInfo, g_segmentIdxMap, g_segmentSizeMap).
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>
#include "common/log.h"
#include "hccl/hcom.h"

using namespace hcclb;

namespace {
struct Group {
    HcclComm comm = nullptr;          // null on ranks that are not members
    bool owned = false;               // destroyed by HcomDestroy / HcomDestroyGroup
    std::vector<uint32_t> world_ranks;  // position = group rank
};
struct HcomState {
    std::mutex mu;
    std::map<std::string, Group> groups;
    std::map<std::string, std::vector<uint32_t>> fusion_idx;
    std::map<std::string, std::vector<float>> fusion_size;
    uint64_t next_sub_id = 1;
};
HcomState &state()
{
    static HcomState s;
    return s;
}
HcclResult check_name(const char *group, std::string *out)
{
    *out = group ? group : HCCL_WORLD_GROUP;
    CHK_RET_LOG(out->empty() || out->size() > HCOM_GROUP_NAME_MAX_LENGTH, HCCL_E_PARA, "group name length %zu outside [1,%d]", out->size(),
                HCOM_GROUP_NAME_MAX_LENGTH);
    return HCCL_SUCCESS;
}
// FNV-1a: members derive the same sub-communicator id from the group name without talking to each other
uint64_t name_hash(const std::string &s)
{
    uint64_t h = 1469598103934665603ull;
    for (unsigned char ch : s) { h ^= ch; h *= 1099511628211ull; }
    return h & 0xffffffffffull;
}
HcclResult init_world(HcclComm comm, bool owned)
{
    HcomState &S = state();
    std::lock_guard<std::mutex> lk(S.mu);
    CHK_RET_LOG(S.groups.count(HCCL_WORLD_GROUP) != 0, HCCL_E_PARA, "hcom is already initialised");
    uint32_t n = 0;
    CHK_RET(HcclGetRankSize(comm, &n));
    Group g;
    g.comm = comm;
    g.owned = owned;
    for (uint32_t r = 0; r < n; ++r) g.world_ranks.push_back(r);
    S.groups[HCCL_WORLD_GROUP] = g;
    return HCCL_SUCCESS;
}
HcclResult find_group(const char *group, Group *out)
{
    std::string name;
    CHK_RET(check_name(group, &name));
    HcomState &S = state();
    std::lock_guard<std::mutex> lk(S.mu);
    auto it = S.groups.find(name);
    CHK_RET_LOG(it == S.groups.end(), HCCL_E_NOT_FOUND, "group %s does not exist", name.c_str());
    *out = it->second;
    return HCCL_SUCCESS;
}
}  // namespace

extern "C" {

HcclResult HcomInitByFile(const char *rankTablePath, const char *identify)
{
    CHK_RET_LOG(!rankTablePath || !identify, HCCL_E_PTR, "[EI0003] HcomInitByFile: null pointer");
    char *end = nullptr;
    long rank = strtol(identify, &end, 10);
    CHK_RET_LOG(end == identify || *end != '\0' || rank < 0, HCCL_E_PARA, "HcomInitByFile: identify '%s' is not a rank id", identify);
    HcclComm comm = nullptr;
    CHK_RET(HcclCommInitClusterInfo(rankTablePath, (uint32_t)rank, &comm));
    HcclResult rc = init_world(comm, true);
    if (rc != HCCL_SUCCESS) HcclCommDestroy(comm);
    return rc;
}

HcclResult HcomInitByComm(HcclComm worldComm)
{
    CHK_RET_LOG(!worldComm, HCCL_E_PTR, "[EI0003] HcomInitByComm: worldComm is null");
    return init_world(worldComm, false);
}

HcclResult HcomDestroy(void)
{
    HcomState &S = state();
    std::map<std::string, Group> groups;
    {
        std::lock_guard<std::mutex> lk(S.mu);
        groups.swap(S.groups);
        S.fusion_idx.clear();
        S.fusion_size.clear();
    }
    HcclResult first = HCCL_SUCCESS;
    // sub-groups before the world group they were cut from
    for (auto &kv : groups)
        if (kv.first != HCCL_WORLD_GROUP && kv.second.owned && kv.second.comm) {
            HcclResult rc = HcclCommDestroy(kv.second.comm);
            if (first == HCCL_SUCCESS) first = rc;
        }
    auto w = groups.find(HCCL_WORLD_GROUP);
    if (w != groups.end() && w->second.owned && w->second.comm) {
        HcclResult rc = HcclCommDestroy(w->second.comm);
        if (first == HCCL_SUCCESS) first = rc;
    }
    return first;
}

HcclResult HcomCreateGroup(const char *group, uint32_t rankNum, uint32_t *rankIds)
{
    CHK_RET_LOG(!group || !rankIds, HCCL_E_PTR, "[EI0003] HcomCreateGroup: null pointer");
    std::string name;
    CHK_RET(check_name(group, &name));
    CHK_RET_LOG(name == HCCL_WORLD_GROUP, HCCL_E_PARA, "HcomCreateGroup: %s is reserved", HCCL_WORLD_GROUP);
    Group world;
    CHK_RET(find_group(nullptr, &world));
    uint32_t wsize = (uint32_t)world.world_ranks.size(), me = 0;
    CHK_RET(HcclGetRankId(world.comm, &me));
    CHK_RET_LOG(rankNum == 0 || rankNum > wsize, HCCL_E_PARA, "HcomCreateGroup: rankNum %u outside [1,%u]", rankNum, wsize);
    Group g;
    uint32_t my_pos = 0xFFFFFFFFu;
    for (uint32_t i = 0; i < rankNum; ++i) {
        CHK_RET_LOG(rankIds[i] >= wsize, HCCL_E_PARA, "HcomCreateGroup: rank id %u outside the world group of %u", rankIds[i], wsize);
        for (uint32_t j = 0; j < i; ++j) CHK_RET_LOG(rankIds[j] == rankIds[i], HCCL_E_PARA, "HcomCreateGroup: rank id %u listed twice", rankIds[i]);
        if (rankIds[i] == me) my_pos = i;
        g.world_ranks.push_back(rankIds[i]);
    }
    {
        std::lock_guard<std::mutex> lk(state().mu);
        CHK_RET_LOG(state().groups.count(name) != 0, HCCL_E_PARA, "group %s already exists", name.c_str());
    }
    if (my_pos != 0xFFFFFFFFu) {
        HcclCommConfig cfg;
        HcclCommConfigInit(&cfg);
        snprintf(cfg.hcclCommName, sizeof(cfg.hcclCommName), "%s", name.c_str());
        HcclComm sub = nullptr;
        CHK_RET(HcclCreateSubCommConfig(&world.comm, rankNum, rankIds, name_hash(name), my_pos, &cfg, &sub));
        g.comm = sub;
        g.owned = true;
    }
    std::lock_guard<std::mutex> lk(state().mu);
    state().groups[name] = g;
    return HCCL_SUCCESS;
}

HcclResult HcomDestroyGroup(const char *group)
{
    CHK_RET_LOG(!group, HCCL_E_PTR, "[EI0003] HcomDestroyGroup: group is null");
    std::string name;
    CHK_RET(check_name(group, &name));
    CHK_RET_LOG(name == HCCL_WORLD_GROUP, HCCL_E_PARA, "HcomDestroyGroup: the world group goes with HcomDestroy");
    Group g;
    {
        std::lock_guard<std::mutex> lk(state().mu);
        auto it = state().groups.find(name);
        CHK_RET_LOG(it == state().groups.end(), HCCL_E_NOT_FOUND, "group %s does not exist", name.c_str());
        g = it->second;
        state().groups.erase(it);
        state().fusion_idx.erase(name);
        state().fusion_size.erase(name);
    }
    if (g.owned && g.comm) return HcclCommDestroy(g.comm);
    return HCCL_SUCCESS;
}

HcclResult HcomGetRankSize(const char *group, uint32_t *rankSize)
{
    CHK_RET_LOG(!rankSize, HCCL_E_PTR, "[EI0003] HcomGetRankSize: rankSize is null");
    Group g;
    CHK_RET(find_group(group, &g));
    *rankSize = (uint32_t)g.world_ranks.size();
    return HCCL_SUCCESS;
}

HcclResult HcomGetRankId(const char *group, uint32_t *rankId)
{
    CHK_RET_LOG(!rankId, HCCL_E_PTR, "[EI0003] HcomGetRankId: rankId is null");
    Group g;
    CHK_RET(find_group(group, &g));
    CHK_RET_LOG(!g.comm, HCCL_E_NOT_FOUND, "this rank is not a member of the group");
    return HcclGetRankId(g.comm, rankId);
}

HcclResult HcomGetWorldRankFromGroupRank(const char *group, uint32_t groupRank, uint32_t *worldRank)
{
    CHK_RET_LOG(!worldRank, HCCL_E_PTR, "[EI0003] HcomGetWorldRankFromGroupRank: worldRank is null");
    Group g;
    CHK_RET(find_group(group, &g));
    CHK_RET_LOG(groupRank >= g.world_ranks.size(), HCCL_E_PARA, "group rank %u outside the group of %zu", groupRank, g.world_ranks.size());
    *worldRank = g.world_ranks[groupRank];
    return HCCL_SUCCESS;
}

HcclResult HcomGetGroupRankFromWorldRank(uint32_t worldRank, const char *group, uint32_t *groupRank)
{
    CHK_RET_LOG(!groupRank, HCCL_E_PTR, "[EI0003] HcomGetGroupRankFromWorldRank: groupRank is null");
    Group g;
    CHK_RET(find_group(group, &g));
    for (size_t i = 0; i < g.world_ranks.size(); ++i)
        if (g.world_ranks[i] == worldRank) { *groupRank = (uint32_t)i; return HCCL_SUCCESS; }
    HLOG_ERROR("world rank %u is not in the group", worldRank);
    return HCCL_E_PARA;
}

HcclResult HcomGetCommHandleByGroup(const char *group, HcclComm *commHandle)
{
    CHK_RET_LOG(!commHandle, HCCL_E_PTR, "[EI0003] HcomGetCommHandleByGroup: commHandle is null");
    Group g;
    CHK_RET(find_group(group, &g));
    CHK_RET_LOG(!g.comm, HCCL_E_NOT_FOUND, "this rank is not a member of the group");
    *commHandle = g.comm;
    return HCCL_SUCCESS;
}

HcclResult HcomGetTopoDesc(const char *group, HcclTopoDescs *topoDescs, uint32_t topoSize)
{
    Group g;
    CHK_RET(find_group(group, &g));
    CHK_RET_LOG(!g.comm, HCCL_E_NOT_FOUND, "this rank is not a member of the group");
    return HcclGetTopoDesc(g.comm, topoDescs, topoSize);
}

HcclResult HcomSetGradFusionByIndex(const char *group, uint32_t segmentNum, const uint32_t *inputIdxList)
{
    CHK_RET_LOG(!inputIdxList, HCCL_E_PTR, "[EI0003] HcomSetGradFusionByIndex: inputIdxList is null");
    CHK_RET_LOG(segmentNum == 0, HCCL_E_PARA, "[EI0003] HcomSetGradFusionByIndex: segmentNum is 0");
    std::string name;
    CHK_RET(check_name(group, &name));
    std::vector<uint32_t> v(inputIdxList, inputIdxList + segmentNum);
    for (size_t i = 0; i + 1 < v.size(); ++i) CHK_RET_LOG(v[i] >= v[i + 1], HCCL_E_PARA, "HcomSetGradFusionByIndex: index list is not ascending");
    std::lock_guard<std::mutex> lk(state().mu);
    state().fusion_idx[name] = v;
    return HCCL_SUCCESS;
}

HcclResult HcomSetGradFusionBySize(const char *group, uint32_t segmentNum, const float *sizeList)
{
    CHK_RET_LOG(!sizeList, HCCL_E_PTR, "[EI0003] HcomSetGradFusionBySize: sizeList is null");
    CHK_RET_LOG(segmentNum == 0, HCCL_E_PARA, "[EI0003] HcomSetGradFusionBySize: segmentNum is 0");
    std::string name;
    CHK_RET(check_name(group, &name));
    std::vector<float> v(sizeList, sizeList + segmentNum);
    float total = 0;
    for (float f : v) {
        CHK_RET_LOG(f < 0, HCCL_E_PARA, "HcomSetGradFusionBySize: negative share");
        total += f;
    }
    CHK_RET_LOG(std::fabs(total - 100.0f) > 1e-4f, HCCL_E_PARA, "HcomSetGradFusionBySize: shares sum to %f, not 100", (double)total);
    std::lock_guard<std::mutex> lk(state().mu);
    state().fusion_size[name] = v;
    return HCCL_SUCCESS;
}

HcclResult HcomGetGradFusionByIndex(const char *group, uint32_t *segmentNum, uint32_t *inputIdxList)
{
    CHK_RET_LOG(!segmentNum || !inputIdxList, HCCL_E_PTR, "[EI0003] HcomGetGradFusionByIndex: null pointer");
    std::string name;
    CHK_RET(check_name(group, &name));
    std::lock_guard<std::mutex> lk(state().mu);
    auto it = state().fusion_idx.find(name);
    if (it == state().fusion_idx.end()) return HCCL_E_NOT_FOUND;
    CHK_RET_LOG(*segmentNum < it->second.size(), HCCL_E_MEMORY, "HcomGetGradFusionByIndex: %zu entries needed, %u given", it->second.size(), *segmentNum);
    memcpy(inputIdxList, it->second.data(), it->second.size() * sizeof(uint32_t));
    *segmentNum = (uint32_t)it->second.size();
    return HCCL_SUCCESS;
}

HcclResult HcomGetGradFusionBySize(const char *group, uint32_t *segmentNum, float *sizeList)
{
    CHK_RET_LOG(!segmentNum || !sizeList, HCCL_E_PTR, "[EI0003] HcomGetGradFusionBySize: null pointer");
    std::string name;
    CHK_RET(check_name(group, &name));
    std::lock_guard<std::mutex> lk(state().mu);
    auto it = state().fusion_size.find(name);
    if (it == state().fusion_size.end()) return HCCL_E_NOT_FOUND;
    CHK_RET_LOG(*segmentNum < it->second.size(), HCCL_E_MEMORY, "HcomGetGradFusionBySize: %zu entries needed, %u given", it->second.size(), *segmentNum);
    memcpy(sizeList, it->second.data(), it->second.size() * sizeof(float));
    *segmentNum = (uint32_t)it->second.size();
    return HCCL_SUCCESS;
}

}  // extern "C"
