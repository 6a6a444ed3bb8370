// C API: argument validation, early-outs and dispatch to the Communicator.  Validation order and result codes follow
// the reference's op_base layer (framework/op_base/src/op_base.cc: null pointers -> HCCL_E_PTR, count == 0 ->
// HCCL_SUCCESS, unsupported dtype/op -> HCCL_E_NOT_SUPPORT / HCCL_E_PARA, HcclCommDestroy while busy -> HCCL_E_AGAIN).
#include <arpa/inet.h>
#include <unistd.h>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <set>
#include <sstream>
#include <thread>
#include <cuda_runtime.h>
#include "bootstrap/ranktable.h"
#include "bootstrap/socket.h"
#include "common/dtype_host.h"
#include "common/env.h"
#include "common/log.h"
#include "core/communicator.h"
#include "hccl/hccl_b200.h"
#include "core/topo_probe.h"
#include "health/consistency.h"
#include "health/fault_inject.h"
#include "kernels/moe_a2a.h"

using namespace hcclb;

namespace {
// state of the framework allocator pool (HcclB200PoolBind, hcclb200_torch_malloc / _free)
std::mutex g_pool_mu;
Communicator *g_pool_comm = nullptr;
struct PoolBlock { void *ptr; size_t bytes; int handle; bool in_use; };
std::vector<PoolBlock> g_pool_blocks;
void pool_forget(Communicator *c)
{
    std::lock_guard<std::mutex> lk(g_pool_mu);
    if (g_pool_comm != c) return;
    g_pool_blocks.clear();  // the communicator releases its symmetric memory itself
    g_pool_comm = nullptr;
}
constexpr uint64_t kSysMaxCount = 0x7FFFFFFFFull;  // reference: SYS_MAX_COUNT
std::mutex g_comm_mu;
std::set<Communicator *> g_comms;
int g_deterministic = 0;  // HcclSetConfig value

Communicator *as_comm(HcclComm c)
{
    std::lock_guard<std::mutex> lk(g_comm_mu);
    auto *p = (Communicator *)c;
    return g_comms.count(p) ? p : nullptr;
}
void track(Communicator *c)
{
    std::lock_guard<std::mutex> lk(g_comm_mu);
    g_comms.insert(c);
}

bool dtype_valid(int dt) { return dtype_size(dt) != 0; }

HcclResult check_buf_count(const void *a, const void *b, uint64_t count, const char *api)
{
    CHK_RET_LOG(!a || !b, HCCL_E_PTR, "[EI0003] %s: buffer pointer is null", api);
    CHK_RET_LOG(count > kSysMaxCount, HCCL_E_PARA, "%s: count %llu above the supported maximum", api, (unsigned long long)count);
    return HCCL_SUCCESS;
}
HcclResult check_reduce(int dt, int op, const char *api)
{
    CHK_RET_LOG(!dtype_valid(dt), HCCL_E_PARA, "%s: unknown data type %d", api, dt);
    CHK_RET_LOG(op < HCCL_REDUCE_SUM || op > HCCL_REDUCE_MIN, HCCL_E_PARA, "%s: unknown reduce op %d", api, op);
    CHK_RET_LOG(!dtype_reducible(dt), HCCL_E_NOT_SUPPORT, "%s: data type %d cannot be reduced (transport only)", api, dt);
    return HCCL_SUCCESS;
}

CommSettings settings_from(const HcclCommConfig *cfg, HcclResult *rc)
{
    const EnvConfig &env = env_config();
    CommSettings st;
    *rc = HCCL_SUCCESS;
    st.stage_half_bytes = (uint64_t)env.buffsize_mb << 20;
    st.deterministic = g_deterministic != 0;
    st.expansion_mode = env.expansion_mode;
    if (cfg) {
        // layout check (reference: CommConfig::Load / CheckMagicWord, framework/communicator/comm_config.cc)
        struct Head { size_t size; uint32_t magic; uint32_t version; uint64_t rsv; } h;
        memcpy(&h, cfg, sizeof(h));
        if (h.magic != HCCL_COMM_CONFIG_MAGIC_WORD) {
            HLOG_ERROR("HcclCommConfig magic word 0x%x invalid: initialise it with HcclCommConfigInit", h.magic);
            *rc = HCCL_E_PARA;
            return st;
        }
        if (h.version > HCCL_COMM_CONFIG_VERSION) HLOG_WARN("HcclCommConfig version %u is newer than %u; extra fields ignored", h.version, HCCL_COMM_CONFIG_VERSION);
        if (h.version >= 1) {
            if (cfg->hcclBufferSize != HCCL_COMM_BUFFSIZE_CONFIG_NOT_SET) {
                if (cfg->hcclBufferSize < 1) { HLOG_ERROR("hcclBufferSize must be at least 1 MB"); *rc = HCCL_E_PARA; return st; }
                if (!env.buffsize_set) st.stage_half_bytes = (uint64_t)cfg->hcclBufferSize << 20;
            }
            if (cfg->hcclDeterministic != HCCL_COMM_DETERMINISTIC_CONFIG_NOT_SET) {
                if (cfg->hcclDeterministic > 1) { HLOG_ERROR("hcclDeterministic must be 0 or 1"); *rc = HCCL_E_PARA; return st; }
                st.deterministic = cfg->hcclDeterministic == 1;
            }
        }
        if (h.version >= 2 && cfg->hcclCommName[0]) st.name = std::string(cfg->hcclCommName, strnlen(cfg->hcclCommName, COMM_NAME_MAX_LENGTH));
        if (h.version >= 4) {
            if (cfg->hcclOpExpansionMode > 3) { HLOG_ERROR("hcclOpExpansionMode must be 0..3"); *rc = HCCL_E_PARA; return st; }
            if (cfg->hcclOpExpansionMode) st.expansion_mode = (int)cfg->hcclOpExpansionMode;
        }
        if (h.version >= 5) {
            if (cfg->hcclRdmaTrafficClass != HCCL_COMM_TRAFFIC_CLASS_CONFIG_NOT_SET && (cfg->hcclRdmaTrafficClass > 255 || cfg->hcclRdmaTrafficClass % 4)) {
                HLOG_ERROR("hcclRdmaTrafficClass must be in [0,255] and a multiple of 4"); *rc = HCCL_E_PARA; return st;
            }
            if (cfg->hcclRdmaServiceLevel != HCCL_COMM_SERVICE_LEVEL_CONFIG_NOT_SET && cfg->hcclRdmaServiceLevel > 7) {
                HLOG_ERROR("hcclRdmaServiceLevel must be in [0,7]"); *rc = HCCL_E_PARA; return st;
            }
        }
    }
    // transport: explicit env, else device when a GPU is usable
    int ndev = 0;
    bool have_gpu = cudaGetDeviceCount(&ndev) == cudaSuccess && ndev > 0;
    if (!have_gpu) (void)cudaGetLastError();
    st.transport = (env.transport == "host" || !have_gpu) ? TR_HOST : TR_DEVICE;
    if (st.transport == TR_DEVICE) {
        int dev = 0;
        cudaGetDevice(&dev);
        st.device = dev;
    }
    return st;
}

HcclResult start_hub(const std::string &ip, int port, const std::string &ident, RootHandle *h)
{
    const EnvConfig &env = env_config();
    std::string err;
    Hub *hub = Hub::start(ip, port, env.socket_family, &err);
    CHK_RET_LOG(!hub, HCCL_E_TCP_CONNECT, "cannot start the bootstrap hub: %s", err.c_str());
    memset(h, 0, sizeof(*h));
    h->magic = kRootMagic;
    h->version = 1;
    h->port = (uint32_t)hub->port();
    h->family = (uint32_t)env.socket_family;
    snprintf(h->ip, sizeof(h->ip), "%s", ip.c_str());
    std::string id = ident.empty() ? make_identifier(ip, hub->port()) : ident;
    snprintf(h->identifier, sizeof(h->identifier), "%s", id.c_str());
    register_hub(h->identifier, hub);
    return HCCL_SUCCESS;
}

OpRequest base_request(int coll, uint64_t count, int dt, int op, int root, void *stream)
{
    OpRequest rq;
    rq.coll = coll; rq.count = count; rq.dtype = dt; rq.redop = op; rq.root = root; rq.stream = stream;
    return rq;
}
HcclResult run_single(Communicator *c, OpRequest &rq, const void *in, void *out)
{
    CHK_RET_LOG(c->nlocal() != 1, HCCL_E_PARA, "this entry point needs one local rank per communicator; use HcclB200Collective");
    const void *ins[1] = {in};
    void *outs[1] = {out};
    rq.in = ins;
    rq.out = outs;
    return c->collective(rq);
}
}  // namespace

extern "C" {

const char *HcclGetErrorString(HcclResult code)
{
    static const char *names[] = {"no error", "parameter error", "empty pointer", "memory error", "internal error",
                                  "not support feature", "not found specific resource", "resource unavailable",
                                  "call system interface error", "timeout", "open file fail", "tcp connect fail",
                                  "roce connect fail", "tcp transfer fail", "roce transfer fail", "call runtime api fail",
                                  "call driver api fail", "call profiling api fail", "call cce api fail",
                                  "call network api fail", "try again", "error cqe", "error communicator suspending"};
    if ((int)code < 0 || (int)code >= (int)(sizeof(names) / sizeof(names[0]))) return "unknow error";
    return names[code];
}
const char *HcclB200GetLastError(void) { return last_error_message().c_str(); }
const char *HcclB200AlgoName(int32_t algo) { return algo_name(algo); }
HcclResult HcclB200ReloadEnv(void)
{
    const EnvConfig &e = env_config(true);
    fault::reload();
    return e.valid ? HCCL_SUCCESS : HCCL_E_PARA;
}

uint32_t HcclGetCommConfigCapability(void)
{
    // bit i set = HcclCommConfigCapability i is honoured
    return (1u << HCCL_COMM_CONFIG_BUFFER_SIZE) | (1u << HCCL_COMM_CONFIG_DETERMINISTIC) | (1u << HCCL_COMM_CONFIG_COMM_NAME) |
           (1u << HCCL_COMM_CONFIG_OP_EXPANSION_MODE) | (1u << HCCL_COMM_CONFIG_SUPPORT_INIT_BY_ENV);
}

HcclResult HcclSetConfig(HcclConfig config, union HcclConfigValue value)
{
    CHK_RET_LOG(config != HCCL_DETERMINISTIC, HCCL_E_NOT_SUPPORT, "HcclSetConfig: unknown config %d", (int)config);
    CHK_RET_LOG(value.value != 0 && value.value != 1, HCCL_E_PARA, "HCCL_DETERMINISTIC must be 0 or 1");
    if (env_config().deterministic >= 0) {
        HLOG_WARN("HCCL_DETERMINISTIC is set in the environment and takes precedence over HcclSetConfig");
        return HCCL_SUCCESS;
    }
    g_deterministic = value.value;
    std::lock_guard<std::mutex> lk(g_comm_mu);
    for (auto *c : g_comms) c->set_deterministic(value.value != 0);
    return HCCL_SUCCESS;
}
HcclResult HcclGetConfig(HcclConfig config, union HcclConfigValue *value)
{
    CHK_RET_LOG(!value, HCCL_E_PTR, "[EI0003] HcclGetConfig: value pointer is null");
    CHK_RET_LOG(config != HCCL_DETERMINISTIC, HCCL_E_NOT_SUPPORT, "HcclGetConfig: unknown config %d", (int)config);
    int e = env_config().deterministic;
    value->value = e >= 0 ? e : g_deterministic;
    return HCCL_SUCCESS;
}

HcclResult HcclGetRootInfo(HcclRootInfo *rootInfo)
{
    CHK_RET_LOG(!rootInfo, HCCL_E_PTR, "[EI0003] HcclGetRootInfo: rootInfo is null");
    const EnvConfig &env = env_config();
    CHK_RET_LOG(!env.valid, HCCL_E_PARA, "invalid environment: %s", env.error.c_str());
    std::string ip = env.if_ip.empty() ? (getenv("MASTER_ADDR") ? "127.0.0.1" : "127.0.0.1") : env.if_ip;
    RootHandle h;
    int port = 0;
    if (env.port_range_lo > 0) {  // HCCL_HOST_SOCKET_PORT_RANGE: first free port of the range
        HcclResult rc = HCCL_E_TCP_CONNECT;
        for (port = env.port_range_lo; port <= env.port_range_hi && rc != HCCL_SUCCESS; ++port) rc = start_hub(ip, port, "", &h);
        CHK_RET(rc);
    } else CHK_RET(start_hub(ip, 0, "", &h));
    memset(rootInfo, 0, sizeof(*rootInfo));
    static_assert(sizeof(RootHandle) <= HCCL_ROOT_INFO_BYTES, "root handle must fit the blob");
    memcpy(rootInfo->internal, &h, sizeof(h));
    return HCCL_SUCCESS;
}

HcclResult HcclCommInitRootInfoConfig(uint32_t nRanks, const HcclRootInfo *rootInfo, uint32_t rank, const HcclCommConfig *config,
                                      HcclComm *comm)
{
    CHK_RET_LOG(!rootInfo || !comm, HCCL_E_PTR, "[EI0003] HcclCommInitRootInfo: null pointer");
    const EnvConfig &env = env_config();
    CHK_RET_LOG(!env.valid, HCCL_E_PARA, "invalid environment: %s", env.error.c_str());
    RootHandle h;
    memcpy(&h, rootInfo->internal, sizeof(h));
    HcclResult rc;
    CommSettings st = settings_from(config, &rc);
    CHK_RET(rc);
    Communicator *c = nullptr;
    CHK_RET(Communicator::create(nRanks, h, rank, st, &c));
    track(c);
    *comm = c;
    return HCCL_SUCCESS;
}
HcclResult HcclCommInitRootInfo(uint32_t nRanks, const HcclRootInfo *rootInfo, uint32_t rank, HcclComm *comm)
{
    return HcclCommInitRootInfoConfig(nRanks, rootInfo, rank, nullptr, comm);
}

HcclResult HcclCommInitClusterInfoConfig(const char *clusterInfo, uint32_t rank, HcclCommConfig *config, HcclComm *comm)
{
    CHK_RET_LOG(!clusterInfo || !comm, HCCL_E_PTR, "[EI0003] HcclCommInitClusterInfo: null pointer");
    const EnvConfig &env = env_config();
    RankTable t;
    std::string err;
    HcclResult rc = load_ranktable_file(clusterInfo, &t, &err);
    CHK_RET_LOG(rc != HCCL_SUCCESS, rc, "rank table %s: %s", clusterInfo, err.c_str());
    CHK_RET_LOG(rank >= t.ranks.size(), HCCL_E_PARA, "rank %u not in the rank table (%zu ranks)", rank, t.ranks.size());
    int port = t.host_port ? t.host_port : env.if_base_port;
    char ident[96];
    snprintf(ident, sizeof(ident), "ranktable_%08x_%d", t.crc, port);
    RootHandle h;
    if (rank == 0) CHK_RET(start_hub(t.host_ip, port, ident, &h));
    else {
        memset(&h, 0, sizeof(h));
        h.magic = kRootMagic; h.version = 1; h.port = (uint32_t)port; h.family = (uint32_t)env.socket_family;
        snprintf(h.ip, sizeof(h.ip), "%s", t.host_ip.c_str());
        snprintf(h.identifier, sizeof(h.identifier), "%s", ident);
    }
    CommSettings st = settings_from(config, &rc);
    CHK_RET(rc);
    if (st.transport == TR_DEVICE) {
        st.device = t.ranks[rank].device_id;
        CHK_RET_LOG(cudaSetDevice(st.device) != cudaSuccess, HCCL_E_RUNTIME, "cudaSetDevice(%d) failed", st.device);
    }
    Communicator *c = nullptr;
    CHK_RET(Communicator::create((uint32_t)t.ranks.size(), h, rank, st, &c));
    track(c);
    *comm = c;
    return HCCL_SUCCESS;
}
HcclResult HcclCommInitClusterInfo(const char *clusterInfo, uint32_t rank, HcclComm *comm)
{
    return HcclCommInitClusterInfoConfig(clusterInfo, rank, nullptr, comm);
}

HcclResult HcclCommInitAll(uint32_t ndev, int32_t *devices, HcclComm *comms)
{
    CHK_RET_LOG(!devices || !comms, HCCL_E_PTR, "[EI0003] HcclCommInitAll: null pointer");
    CHK_RET_LOG(ndev == 0 || ndev > (uint32_t)kMaxRanks, HCCL_E_PARA, "HcclCommInitAll: ndev %u outside [1,%d]", ndev, kMaxRanks);
    for (uint32_t i = 0; i < ndev; ++i)
        for (uint32_t j = 0; j < i; ++j) CHK_RET_LOG(devices[i] == devices[j], HCCL_E_PARA, "HcclCommInitAll: device %d listed twice", devices[i]);
    HcclRootInfo info;
    CHK_RET(HcclGetRootInfo(&info));
    HcclResult rc0;
    CommSettings probe = settings_from(nullptr, &rc0);
    std::vector<HcclResult> rcs(ndev, HCCL_SUCCESS);
    std::vector<std::thread> th;
    // one thread per device, like the reference (op_base.cc:168-242)
    for (uint32_t i = 0; i < ndev; ++i)
        th.emplace_back([&, i] {
            if (probe.transport == TR_DEVICE && cudaSetDevice(devices[i]) != cudaSuccess) { rcs[i] = HCCL_E_RUNTIME; return; }
            rcs[i] = HcclCommInitRootInfo(ndev, &info, i, &comms[i]);
        });
    for (auto &t : th) t.join();
    for (auto r : rcs) CHK_RET(r);
    return HCCL_SUCCESS;
}

HcclResult HcclCreateSubCommConfig(HcclComm *comm, uint32_t rankNum, uint32_t *rankIds, uint64_t subCommId,
                                   uint32_t subCommRankId, HcclCommConfig *config, HcclComm *subComm)
{
    CHK_RET_LOG(!comm || !subComm, HCCL_E_PTR, "[EI0003] HcclCreateSubCommConfig: null pointer");
    Communicator *c = as_comm(*comm);
    CHK_RET_LOG(!c, HCCL_E_PARA, "HcclCreateSubCommConfig: unknown communicator");
    if (subCommRankId == 0xFFFFFFFFu || !rankIds) {  // not a member
        *subComm = nullptr;
        return HCCL_SUCCESS;
    }
    HcclResult rc;
    CommSettings st = settings_from(config, &rc);
    CHK_RET(rc);
    Communicator *s = nullptr;
    CHK_RET(c->create_sub(rankNum, rankIds, subCommId, subCommRankId, st, &s));
    track(s);
    *subComm = s;
    return HCCL_SUCCESS;
}

HcclResult HcclB200CommInitLocal(uint32_t nRanks, int transport, int device, const HcclCommConfig *config, HcclComm *comm)
{
    CHK_RET_LOG(!comm, HCCL_E_PTR, "[EI0003] HcclB200CommInitLocal: comm is null");
    HcclResult rc;
    CommSettings st = settings_from(config, &rc);
    CHK_RET(rc);
    st.transport = transport ? TR_DEVICE : TR_HOST;
    st.device = device;
    Communicator *c = nullptr;
    CHK_RET(Communicator::create_local(nRanks, st, &c));
    track(c);
    *comm = c;
    return HCCL_SUCCESS;
}

HcclResult HcclCommDestroy(HcclComm comm)
{
    CHK_RET_LOG(!comm, HCCL_E_PTR, "[EI0003] HcclCommDestroy: comm is null");
    Communicator *c = as_comm(comm);
    CHK_RET_LOG(!c, HCCL_E_PARA, "HcclCommDestroy: unknown communicator");
    {
        std::lock_guard<std::mutex> lk(g_comm_mu);
        g_comms.erase(c);
    }
    HcclResult rc = c->destroy();
    if (rc == HCCL_E_AGAIN) track(c);
    else pool_forget(c);
    return rc;
}

#define GET_COMM(api)                                                        \
    Communicator *c = as_comm(comm);                                         \
    CHK_RET_LOG(!comm, HCCL_E_PTR, "[EI0003] %s: comm is null", api);         \
    CHK_RET_LOG(!c, HCCL_E_PARA, "%s: unknown communicator", api)

HcclResult HcclGetCommName(HcclComm comm, char *commName)
{
    GET_COMM("HcclGetCommName");
    CHK_RET_LOG(!commName, HCCL_E_PTR, "[EI0003] HcclGetCommName: commName is null");
    snprintf(commName, COMM_NAME_MAX_LENGTH, "%s", c->name().c_str());
    return HCCL_SUCCESS;
}
HcclResult HcclGetRankSize(HcclComm comm, uint32_t *rankSize)
{
    GET_COMM("HcclGetRankSize");
    CHK_RET_LOG(!rankSize, HCCL_E_PTR, "[EI0003] HcclGetRankSize: rankSize is null");
    *rankSize = (uint32_t)c->nranks();
    return HCCL_SUCCESS;
}
HcclResult HcclGetRankId(HcclComm comm, uint32_t *rank)
{
    GET_COMM("HcclGetRankId");
    CHK_RET_LOG(!rank, HCCL_E_PTR, "[EI0003] HcclGetRankId: rank is null");
    *rank = (uint32_t)c->rank();
    return HCCL_SUCCESS;
}
HcclResult HcclB200GetLocalRankNum(HcclComm comm, uint32_t *n)
{
    GET_COMM("HcclB200GetLocalRankNum");
    *n = (uint32_t)c->nlocal();
    return HCCL_SUCCESS;
}
HcclResult HcclGetCommAsyncError(HcclComm comm, HcclResult *asyncError)
{
    GET_COMM("HcclGetCommAsyncError");
    CHK_RET_LOG(!asyncError, HCCL_E_PTR, "[EI0003] HcclGetCommAsyncError: asyncError is null");
    *asyncError = c->async_error();
    return HCCL_SUCCESS;
}

// ---------------------------------------------------------------------------------------------- collectives
HcclResult HcclAllReduce(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op, HcclComm comm,
                         aclrtStream stream)
{
    GET_COMM("HcclAllReduce");
    if (count == 0) { HLOG_WARN("HcclAllReduce: count is 0, nothing to do"); return HCCL_SUCCESS; }
    CHK_RET(check_buf_count(sendBuf, recvBuf, count, "HcclAllReduce"));
    CHK_RET(check_reduce(dataType, op, "HcclAllReduce"));
    OpRequest rq = base_request(COLL_ALLREDUCE, count, dataType, op, 0, stream);
    return run_single(c, rq, sendBuf, recvBuf);
}
HcclResult HcclBroadcast(void *buf, uint64_t count, HcclDataType dataType, uint32_t root, HcclComm comm, aclrtStream stream)
{
    GET_COMM("HcclBroadcast");
    if (count == 0) { HLOG_WARN("HcclBroadcast: count is 0, nothing to do"); return HCCL_SUCCESS; }
    CHK_RET(check_buf_count(buf, buf, count, "HcclBroadcast"));
    CHK_RET_LOG(!dtype_valid(dataType), HCCL_E_PARA, "HcclBroadcast: unknown data type %d", (int)dataType);
    CHK_RET_LOG(root >= (uint32_t)c->nranks(), HCCL_E_PARA, "HcclBroadcast: root %u outside the communicator", root);
    OpRequest rq = base_request(COLL_BROADCAST, count, dataType, 0, (int)root, stream);
    return run_single(c, rq, buf, buf);
}
HcclResult HcclReduceScatter(void *sendBuf, void *recvBuf, uint64_t recvCount, HcclDataType dataType, HcclReduceOp op,
                             HcclComm comm, aclrtStream stream)
{
    GET_COMM("HcclReduceScatter");
    if (recvCount == 0) { HLOG_WARN("HcclReduceScatter: recvCount is 0, nothing to do"); return HCCL_SUCCESS; }
    CHK_RET(check_buf_count(sendBuf, recvBuf, recvCount, "HcclReduceScatter"));
    CHK_RET(check_reduce(dataType, op, "HcclReduceScatter"));
    OpRequest rq = base_request(COLL_REDUCE_SCATTER, recvCount, dataType, op, 0, stream);
    return run_single(c, rq, sendBuf, recvBuf);
}
HcclResult HcclReduceScatterV(void *sendBuf, const void *sendCounts, const void *sendDispls, void *recvBuf, uint64_t recvCount,
                              HcclDataType dataType, HcclReduceOp op, HcclComm comm, aclrtStream stream)
{
    GET_COMM("HcclReduceScatterV");
    CHK_RET_LOG(!sendCounts || !sendDispls, HCCL_E_PTR, "[EI0003] HcclReduceScatterV: counts or displacements are null");
    const uint64_t *sc = (const uint64_t *)sendCounts;
    uint64_t total = 0;
    for (int i = 0; i < c->nranks(); ++i) {
        CHK_RET_LOG(sc[i] > kSysMaxCount, HCCL_E_PARA, "HcclReduceScatterV: sendCounts[%d] too large", i);
        total += sc[i];
    }
    CHK_RET_LOG(recvCount != sc[c->rank()], HCCL_E_PARA, "HcclReduceScatterV: recvCount %llu differs from sendCounts[rank] %llu",
                (unsigned long long)recvCount, (unsigned long long)sc[c->rank()]);
    if (total == 0) return HCCL_SUCCESS;
    CHK_RET_LOG(!sendBuf || (!recvBuf && recvCount), HCCL_E_PTR, "[EI0003] HcclReduceScatterV: buffer pointer is null");
    CHK_RET(check_reduce(dataType, op, "HcclReduceScatterV"));
    OpRequest rq = base_request(COLL_REDUCE_SCATTER_V, recvCount, dataType, op, 0, stream);
    rq.counts = sc;
    rq.displs = (const uint64_t *)sendDispls;
    return run_single(c, rq, sendBuf, recvBuf);
}
HcclResult HcclScatter(void *sendBuf, void *recvBuf, uint64_t recvCount, HcclDataType dataType, uint32_t root, HcclComm comm,
                       aclrtStream stream)
{
    GET_COMM("HcclScatter");
    if (recvCount == 0) { HLOG_WARN("HcclScatter: recvCount is 0, nothing to do"); return HCCL_SUCCESS; }
    CHK_RET_LOG(root >= (uint32_t)c->nranks(), HCCL_E_PARA, "HcclScatter: root %u outside the communicator", root);
    CHK_RET_LOG(!recvBuf || ((uint32_t)c->rank() == root && !sendBuf), HCCL_E_PTR, "[EI0003] HcclScatter: buffer pointer is null");
    CHK_RET_LOG(!dtype_valid(dataType), HCCL_E_PARA, "HcclScatter: unknown data type %d", (int)dataType);
    CHK_RET_LOG(recvCount > kSysMaxCount, HCCL_E_PARA, "HcclScatter: count too large");
    OpRequest rq = base_request(COLL_SCATTER, recvCount, dataType, 0, (int)root, stream);
    return run_single(c, rq, sendBuf, recvBuf);
}
HcclResult HcclGather(void *sendBuf, void *recvBuf, uint64_t sendCount, HcclDataType dataType, uint32_t root, HcclComm comm,
                      aclrtStream stream)
{
    GET_COMM("HcclGather");
    if (sendCount == 0) { HLOG_WARN("HcclGather: sendCount is 0, nothing to do"); return HCCL_SUCCESS; }
    CHK_RET_LOG(root >= (uint32_t)c->nranks(), HCCL_E_PARA, "HcclGather: root %u outside the communicator", root);
    CHK_RET_LOG(!sendBuf || ((uint32_t)c->rank() == root && !recvBuf), HCCL_E_PTR, "[EI0003] HcclGather: buffer pointer is null");
    CHK_RET_LOG(!dtype_valid(dataType), HCCL_E_PARA, "HcclGather: unknown data type %d", (int)dataType);
    CHK_RET_LOG(sendCount > kSysMaxCount, HCCL_E_PARA, "HcclGather: count too large");
    OpRequest rq = base_request(COLL_GATHER, sendCount, dataType, 0, (int)root, stream);
    return run_single(c, rq, sendBuf, recvBuf);
}
HcclResult HcclAllGather(void *sendBuf, void *recvBuf, uint64_t sendCount, HcclDataType dataType, HcclComm comm, aclrtStream stream)
{
    GET_COMM("HcclAllGather");
    if (sendCount == 0) { HLOG_WARN("HcclAllGather: sendCount is 0, nothing to do"); return HCCL_SUCCESS; }
    CHK_RET(check_buf_count(sendBuf, recvBuf, sendCount, "HcclAllGather"));
    CHK_RET_LOG(!dtype_valid(dataType), HCCL_E_PARA, "HcclAllGather: unknown data type %d", (int)dataType);
    OpRequest rq = base_request(COLL_ALLGATHER, sendCount, dataType, 0, 0, stream);
    return run_single(c, rq, sendBuf, recvBuf);
}
HcclResult HcclAllGatherV(void *sendBuf, uint64_t sendCount, void *recvBuf, const void *recvCounts, const void *recvDispls,
                          HcclDataType dataType, HcclComm comm, aclrtStream stream)
{
    GET_COMM("HcclAllGatherV");
    CHK_RET_LOG(!recvCounts || !recvDispls, HCCL_E_PTR, "[EI0003] HcclAllGatherV: counts or displacements are null");
    const uint64_t *rc = (const uint64_t *)recvCounts;
    uint64_t total = 0;
    for (int i = 0; i < c->nranks(); ++i) {
        CHK_RET_LOG(rc[i] > kSysMaxCount, HCCL_E_PARA, "HcclAllGatherV: recvCounts[%d] too large", i);
        total += rc[i];
    }
    CHK_RET_LOG(sendCount != rc[c->rank()], HCCL_E_PARA, "HcclAllGatherV: sendCount %llu differs from recvCounts[rank] %llu",
                (unsigned long long)sendCount, (unsigned long long)rc[c->rank()]);
    if (total == 0) return HCCL_SUCCESS;
    CHK_RET_LOG(!recvBuf || (!sendBuf && sendCount), HCCL_E_PTR, "[EI0003] HcclAllGatherV: buffer pointer is null");
    CHK_RET_LOG(!dtype_valid(dataType), HCCL_E_PARA, "HcclAllGatherV: unknown data type %d", (int)dataType);
    OpRequest rq = base_request(COLL_ALLGATHER_V, sendCount, dataType, 0, 0, stream);
    rq.counts = rc;
    rq.displs = (const uint64_t *)recvDispls;
    return run_single(c, rq, sendBuf, recvBuf);
}
HcclResult HcclBarrier(HcclComm comm, aclrtStream stream)
{
    GET_COMM("HcclBarrier");
    OpRequest rq = base_request(COLL_BARRIER, 0, HCCL_DATA_TYPE_FP32, 0, 0, stream);
    return run_single(c, rq, nullptr, nullptr);
}
HcclResult HcclReduce(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op, uint32_t root,
                      HcclComm comm, aclrtStream stream)
{
    GET_COMM("HcclReduce");
    if (count == 0) { HLOG_WARN("HcclReduce: count is 0, nothing to do"); return HCCL_SUCCESS; }
    CHK_RET_LOG(root >= (uint32_t)c->nranks(), HCCL_E_PARA, "HcclReduce: root %u outside the communicator", root);
    CHK_RET_LOG(!sendBuf || ((uint32_t)c->rank() == root && !recvBuf), HCCL_E_PTR, "[EI0003] HcclReduce: buffer pointer is null");
    CHK_RET_LOG(count > kSysMaxCount, HCCL_E_PARA, "HcclReduce: count too large");
    CHK_RET(check_reduce(dataType, op, "HcclReduce"));
    OpRequest rq = base_request(COLL_REDUCE, count, dataType, op, (int)root, stream);
    return run_single(c, rq, sendBuf, recvBuf);
}

HcclResult HcclAlltoAll(const void *sendBuf, uint64_t sendCount, HcclDataType sendType, const void *recvBuf, uint64_t recvCount,
                        HcclDataType recvType, HcclComm comm, aclrtStream stream)
{
    GET_COMM("HcclAlltoAll");
    if (sendCount == 0 && recvCount == 0) return HCCL_SUCCESS;
    CHK_RET(check_buf_count(sendBuf, recvBuf, sendCount, "HcclAlltoAll"));
    CHK_RET_LOG(sendCount != recvCount, HCCL_E_PARA, "HcclAlltoAll: sendCount %llu differs from recvCount %llu",
                (unsigned long long)sendCount, (unsigned long long)recvCount);
    CHK_RET_LOG(sendType != recvType, HCCL_E_PARA, "HcclAlltoAll: sendType and recvType differ");
    CHK_RET_LOG(sendBuf == recvBuf, HCCL_E_PARA, "HcclAlltoAll: sendBuf and recvBuf must be different buffers");
    CHK_RET_LOG(!dtype_valid(sendType), HCCL_E_PARA, "HcclAlltoAll: unknown data type %d", (int)sendType);
    OpRequest rq = base_request(COLL_ALLTOALL, sendCount, sendType, 0, 0, stream);
    return run_single(c, rq, sendBuf, const_cast<void *>(recvBuf));
}
HcclResult HcclAlltoAllV(const void *sendBuf, const void *sendCounts, const void *sdispls, HcclDataType sendType,
                         const void *recvBuf, const void *recvCounts, const void *rdispls, HcclDataType recvType, HcclComm comm,
                         aclrtStream stream)
{
    GET_COMM("HcclAlltoAllV");
    CHK_RET_LOG(!sendCounts || !sdispls || !recvCounts || !rdispls, HCCL_E_PTR, "[EI0003] HcclAlltoAllV: counts or displacements are null");
    CHK_RET_LOG(sendType != recvType, HCCL_E_PARA, "HcclAlltoAllV: sendType and recvType differ");
    CHK_RET_LOG(!dtype_valid(sendType), HCCL_E_PARA, "HcclAlltoAllV: unknown data type %d", (int)sendType);
    const uint64_t *sc = (const uint64_t *)sendCounts, *rc = (const uint64_t *)recvCounts;
    uint64_t ts = 0, tr = 0;
    for (int i = 0; i < c->nranks(); ++i) {
        CHK_RET_LOG(sc[i] > kSysMaxCount || rc[i] > kSysMaxCount, HCCL_E_PARA, "HcclAlltoAllV: count for rank %d too large", i);
        ts += sc[i]; tr += rc[i];
    }
    CHK_RET_LOG((ts && !sendBuf) || (tr && !recvBuf), HCCL_E_PTR, "[EI0003] HcclAlltoAllV: buffer pointer is null");
    CHK_RET_LOG(sendBuf && sendBuf == recvBuf, HCCL_E_PARA, "HcclAlltoAllV: sendBuf and recvBuf must be different buffers");
    CHK_RET_LOG(sc[c->rank()] != rc[c->rank()], HCCL_E_PARA, "HcclAlltoAllV: the block a rank sends to itself must match what it receives");
    OpRequest rq = base_request(COLL_ALLTOALLV, 0, sendType, 0, 0, stream);
    rq.send_counts = sc; rq.send_displs = (const uint64_t *)sdispls;
    rq.recv_counts = rc; rq.recv_displs = (const uint64_t *)rdispls;
    return run_single(c, rq, sendBuf, const_cast<void *>(recvBuf));
}
HcclResult HcclAlltoAllVC(const void *sendBuf, const void *sendCountMatrix, HcclDataType sendType, const void *recvBuf,
                          HcclDataType recvType, HcclComm comm, aclrtStream stream)
{
    GET_COMM("HcclAlltoAllVC");
    CHK_RET_LOG(!sendCountMatrix, HCCL_E_PTR, "[EI0003] HcclAlltoAllVC: count matrix is null");
    CHK_RET_LOG(sendType != recvType, HCCL_E_PARA, "HcclAlltoAllVC: sendType and recvType differ");
    CHK_RET_LOG(!dtype_valid(sendType), HCCL_E_PARA, "HcclAlltoAllVC: unknown data type %d", (int)sendType);
    CHK_RET_LOG(c->nlocal() != 1, HCCL_E_PARA, "HcclAlltoAllVC needs one local rank per communicator");
    const uint64_t *m = (const uint64_t *)sendCountMatrix;
    int p = c->nranks(), me = c->rank();
    // rows derived from the matrix; blocks are packed in rank order on both sides
    std::vector<uint64_t> sc(p), sd(p), rc(p), rd(p);
    uint64_t so = 0, ro = 0;
    for (int j = 0; j < p; ++j) {
        sc[j] = m[(size_t)me * p + j]; sd[j] = so; so += sc[j];
        rc[j] = m[(size_t)j * p + me]; rd[j] = ro; ro += rc[j];
    }
    CHK_RET_LOG((so && !sendBuf) || (ro && !recvBuf), HCCL_E_PTR, "[EI0003] HcclAlltoAllVC: buffer pointer is null");
    OpRequest rq = base_request(COLL_ALLTOALLVC, 0, sendType, 0, 0, stream);
    rq.send_counts = sc.data(); rq.send_displs = sd.data(); rq.recv_counts = rc.data(); rq.recv_displs = rd.data();
    return run_single(c, rq, sendBuf, const_cast<void *>(recvBuf));
}

HcclResult HcclSend(void *sendBuf, uint64_t count, HcclDataType dataType, uint32_t destRank, HcclComm comm, aclrtStream stream)
{
    GET_COMM("HcclSend");
    if (count == 0) return HCCL_SUCCESS;
    CHK_RET(check_buf_count(sendBuf, sendBuf, count, "HcclSend"));
    CHK_RET_LOG(!dtype_valid(dataType), HCCL_E_PARA, "HcclSend: unknown data type %d", (int)dataType);
    CHK_RET_LOG(destRank >= (uint32_t)c->nranks() || destRank == (uint32_t)c->rank(), HCCL_E_PARA, "HcclSend: bad destination rank %u", destRank);
    return c->send(sendBuf, count, dataType, (int)destRank, stream);
}
HcclResult HcclRecv(void *recvBuf, uint64_t count, HcclDataType dataType, uint32_t srcRank, HcclComm comm, aclrtStream stream)
{
    GET_COMM("HcclRecv");
    if (count == 0) return HCCL_SUCCESS;
    CHK_RET(check_buf_count(recvBuf, recvBuf, count, "HcclRecv"));
    CHK_RET_LOG(!dtype_valid(dataType), HCCL_E_PARA, "HcclRecv: unknown data type %d", (int)dataType);
    CHK_RET_LOG(srcRank >= (uint32_t)c->nranks() || srcRank == (uint32_t)c->rank(), HCCL_E_PARA, "HcclRecv: bad source rank %u", srcRank);
    return c->recv(recvBuf, count, dataType, (int)srcRank, stream);
}
HcclResult HcclBatchSendRecv(HcclSendRecvItem *items, uint32_t itemNum, HcclComm comm, aclrtStream stream)
{
    GET_COMM("HcclBatchSendRecv");
    if (itemNum == 0) { HLOG_WARN("HcclBatchSendRecv: itemNum is 0, nothing to do"); return HCCL_SUCCESS; }
    CHK_RET_LOG(!items, HCCL_E_PTR, "[EI0003] HcclBatchSendRecv: item list is null");
    for (uint32_t i = 0; i < itemNum; ++i) {
        CHK_RET_LOG(!items[i].buf, HCCL_E_PTR, "[EI0003] HcclBatchSendRecv: item %u has a null buffer", i);
        CHK_RET_LOG(items[i].sendRecvType != HCCL_SEND && items[i].sendRecvType != HCCL_RECV, HCCL_E_PARA, "HcclBatchSendRecv: item %u has no direction", i);
        CHK_RET_LOG(items[i].remoteRank >= (uint32_t)c->nranks(), HCCL_E_PARA, "HcclBatchSendRecv: item %u names rank %u", i, items[i].remoteRank);
        CHK_RET_LOG(!dtype_valid(items[i].dataType), HCCL_E_PARA, "HcclBatchSendRecv: item %u has an unknown data type", i);
        CHK_RET_LOG(items[i].count > kSysMaxCount, HCCL_E_PARA, "HcclBatchSendRecv: item %u count too large", i);
    }
    return c->batch_send_recv(items, itemNum, stream);
}

// ---------------------------------------------------------------------------------------------- extensions
HcclResult HcclB200Collective(HcclComm comm, const HcclB200Op *op, void *const *sendBufs, void *const *recvBufs, aclrtStream stream)
{
    GET_COMM("HcclB200Collective");
    CHK_RET_LOG(!op, HCCL_E_PTR, "[EI0003] HcclB200Collective: op is null");
    CHK_RET_LOG(op->coll < 0 || op->coll > COLL_GATHER, HCCL_E_PARA, "HcclB200Collective: unknown collective %d", op->coll);
    CHK_RET_LOG(!dtype_valid(op->dataType), HCCL_E_PARA, "HcclB200Collective: unknown data type %d", op->dataType);
    bool reducing = op->coll == COLL_ALLREDUCE || op->coll == COLL_REDUCE || op->coll == COLL_REDUCE_SCATTER || op->coll == COLL_REDUCE_SCATTER_V;
    if (reducing) CHK_RET(check_reduce(op->dataType, op->op, "HcclB200Collective"));
    CHK_RET_LOG(op->root < 0 || op->root >= c->nranks(), HCCL_E_PARA, "HcclB200Collective: root %d outside the communicator", op->root);
    if (op->coll != COLL_BARRIER) CHK_RET_LOG(!sendBufs || !recvBufs, HCCL_E_PTR, "[EI0003] HcclB200Collective: buffer lists are null");
    bool v = op->coll == COLL_ALLGATHER_V || op->coll == COLL_REDUCE_SCATTER_V;
    bool a2av = op->coll == COLL_ALLTOALLV || op->coll == COLL_ALLTOALLVC;
    if (v) CHK_RET_LOG(!op->counts || !op->displs, HCCL_E_PTR, "[EI0003] HcclB200Collective: counts/displs are null");
    if (a2av) CHK_RET_LOG(!op->sendCounts || !op->sdispls || !op->recvCounts || !op->rdispls, HCCL_E_PTR, "[EI0003] HcclB200Collective: AlltoAllV rows are null");
    if (!v && !a2av && op->coll != COLL_BARRIER && op->count == 0) return HCCL_SUCCESS;
    OpRequest rq = base_request(op->coll, op->count, op->dataType, op->op, op->root, stream);
    rq.algo = op->algo; rq.nchan = op->nchan;
    rq.counts = op->counts; rq.displs = op->displs;
    rq.send_counts = op->sendCounts; rq.send_displs = op->sdispls; rq.recv_counts = op->recvCounts; rq.recv_displs = op->rdispls;
    rq.in = (const void *const *)sendBufs;
    rq.out = recvBufs;
    return c->collective(rq);
}
HcclResult HcclB200Repeat(HcclComm comm, const HcclB200Op *op, void *const *sendBufs, void *const *recvBufs, uint32_t iters,
                          uint64_t strideBytes, uint32_t nwin, aclrtStream stream)
{
    // hccl_test-style loop in C: `iters` back-to-back calls; call i uses the buffers shifted by (i % nwin) * strideBytes
    GET_COMM("HcclB200Repeat");
    CHK_RET_LOG(!op || !sendBufs || !recvBufs, HCCL_E_PTR, "[EI0003] HcclB200Repeat: null pointer");
    int nl = c->nlocal();
    std::vector<void *> s(nl), r(nl);
    if (nwin == 0) nwin = 1;
    for (uint32_t i = 0; i < iters; ++i) {
        uint64_t off = (uint64_t)(i % nwin) * strideBytes;
        for (int l = 0; l < nl; ++l) { s[l] = (char *)sendBufs[l] + off; r[l] = (char *)recvBufs[l] + off; }
        CHK_RET(HcclB200Collective(comm, op, s.data(), r.data(), stream));
    }
    return HCCL_SUCCESS;
}
HcclResult HcclB200NcclAllReduceRepeat(HcclComm comm, void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op,
                                       uint32_t iters, uint64_t strideBytes, uint32_t nwin, aclrtStream stream)
{
    GET_COMM("HcclB200NcclAllReduceRepeat");
    if (nwin == 0) nwin = 1;
    for (uint32_t i = 0; i < iters; ++i) {
        uint64_t off = (uint64_t)(i % nwin) * strideBytes;
        CHK_RET(c->nccl_baseline_allreduce((char *)sendBuf + off, (char *)recvBuf + off, count, dataType, op, stream));
    }
    return HCCL_SUCCESS;
}
HcclResult HcclB200LocalSendRecv(HcclComm comm, uint32_t src, uint32_t dst, const void *sendBuf, void *recvBuf, uint64_t count,
                                 HcclDataType dataType, aclrtStream stream)
{
    GET_COMM("HcclB200LocalSendRecv");
    if (count == 0) return HCCL_SUCCESS;
    CHK_RET(check_buf_count(sendBuf, recvBuf, count, "HcclB200LocalSendRecv"));
    return c->local_send_recv((int)src, (int)dst, sendBuf, recvBuf, count, dataType, stream);
}
HcclResult HcclB200StreamSync(HcclComm comm, aclrtStream stream)
{
    GET_COMM("HcclB200StreamSync");
    return c->sync_stream(stream);
}
HcclResult HcclB200MoeCount(const int32_t *topkIdx, int64_t nPairs, int32_t nExperts, int32_t *hist, int32_t *pos, aclrtStream stream)
{
    CHK_RET_LOG(!topkIdx || !hist || !pos, HCCL_E_PTR, "[EI0003] HcclB200MoeCount: null pointer");
    return moe_count(topkIdx, nPairs, nExperts, hist, pos, stream);
}
HcclResult HcclB200MoeOffsets(const int32_t *counts, int32_t nRanks, int32_t nExperts, int32_t rank, int32_t *base, int32_t *expertOffsets,
                              int32_t *recvRows, int64_t capacityRows, int32_t *overflow, aclrtStream stream)
{
    CHK_RET_LOG(!counts || !base || !expertOffsets || !recvRows || !overflow, HCCL_E_PTR, "[EI0003] HcclB200MoeOffsets: null pointer");
    return moe_offsets(counts, nRanks, nExperts, rank, base, expertOffsets, recvRows, capacityRows, overflow, stream);
}
HcclResult HcclB200MoeDispatch(const void *x, const int32_t *topkIdx, const int32_t *pos, const int32_t *base, int64_t tokens, int32_t topk,
                               int32_t hidden, int32_t nExperts, int32_t nRanks, int32_t rank, int32_t pairwise, void *const *recvPeers,
                               int32_t *dstRow, int64_t capacityRows, aclrtStream stream)
{
    CHK_RET_LOG(!x || !topkIdx || !pos || !base || !recvPeers || !dstRow, HCCL_E_PTR, "[EI0003] HcclB200MoeDispatch: null pointer");
    return moe_dispatch(x, topkIdx, pos, base, tokens, topk, hidden, nExperts, nRanks, rank, pairwise, recvPeers, dstRow, capacityRows, stream);
}
HcclResult HcclB200MoeCombine(void *const *yPeers, const int32_t *topkIdx, const float *gates, const int32_t *dstRow, int64_t tokens,
                              int32_t topk, int32_t hidden, int32_t nExperts, int32_t nRanks, int32_t rank, int32_t pairwise, void *out,
                              int64_t capacityRows, aclrtStream stream)
{
    CHK_RET_LOG(!yPeers || !topkIdx || !gates || !dstRow || !out, HCCL_E_PTR, "[EI0003] HcclB200MoeCombine: null pointer");
    return moe_combine(yPeers, topkIdx, gates, dstRow, tokens, topk, hidden, nExperts, nRanks, rank, pairwise, out, capacityRows, stream);
}
HcclResult HcclB200GemmBf16(const void *A, const void *B, void *C, int32_t M, int32_t N, int32_t K, aclrtStream stream)
{
    CHK_RET_LOG(!A || !B || !C, HCCL_E_PTR, "[EI0003] HcclB200GemmBf16: null pointer");
    return gemm_bf16_plain(A, B, C, M, N, K, stream);
}
HcclResult HcclB200GemmLaunchCounts(uint64_t *single, uint64_t *pair)
{
    CHK_RET_LOG(!single || !pair, HCCL_E_PTR, "[EI0003] HcclB200GemmLaunchCounts: null pointer");
    tp_gemm_launch_counts(single, pair);
    return HCCL_SUCCESS;
}
HcclResult HcclB200AllGatherMatmul(HcclComm comm, void *const *xShards, void *const *weights, void *const *outs, int32_t M, int32_t N, int32_t K,
                                   aclrtStream stream)
{
    GET_COMM("HcclB200AllGatherMatmul");
    CHK_RET_LOG(!xShards || !weights || !outs, HCCL_E_PTR, "[EI0003] HcclB200AllGatherMatmul: null pointer");
    return c->tp_all_gather_matmul((const void *const *)xShards, (const void *const *)weights, outs, M, N, K, stream);
}
HcclResult HcclB200MatmulReduceScatter(HcclComm comm, void *const *inputs, void *const *weights, void *const *outs, int32_t M, int32_t N,
                                       int32_t K, aclrtStream stream)
{
    GET_COMM("HcclB200MatmulReduceScatter");
    CHK_RET_LOG(!inputs || !weights || !outs, HCCL_E_PTR, "[EI0003] HcclB200MatmulReduceScatter: null pointer");
    return c->tp_matmul_reduce_scatter((const void *const *)inputs, (const void *const *)weights, outs, M, N, K, stream);
}
HcclResult HcclB200GetKernelTrace(HcclComm comm, uint32_t localRank, uint64_t *out, size_t capWords, int32_t *nsteps)
{
    GET_COMM("HcclB200GetKernelTrace");
    CHK_RET_LOG(!out, HCCL_E_PTR, "[EI0003] HcclB200GetKernelTrace: out is null");
    int n = 0;
    CHK_RET(c->kernel_trace((int)localRank, out, capWords, &n));
    if (nsteps) *nsteps = n;
    return HCCL_SUCCESS;
}
HcclResult HcclB200WaitProbe(HcclComm comm, uint32_t localRank, double timeoutMs, aclrtStream stream)
{
    GET_COMM("HcclB200WaitProbe");
    return c->wait_probe((int)localRank, timeoutMs, stream);
}
HcclResult HcclB200GetStatus(HcclComm comm, uint32_t localRank, HcclB200Status *st)
{
    GET_COMM("HcclB200GetStatus");
    CHK_RET_LOG(!st || localRank >= (uint32_t)c->nlocal(), HCCL_E_PARA, "HcclB200GetStatus: bad arguments");
    DevStatus *d = c->status((int)localRank);
    st->code = d->code; st->step = d->step; st->peer = d->peer; st->chan = d->chan;
    st->expected = d->expected; st->seen = d->seen; st->seq = d->seq; st->head = d->head; st->tail = d->tail;
    return HCCL_SUCCESS;
}
HcclResult HcclB200DescribeStatus(HcclComm comm, uint32_t localRank, char *text, size_t cap)
{
    GET_COMM("HcclB200DescribeStatus");
    CHK_RET_LOG(!text || localRank >= (uint32_t)c->nlocal(), HCCL_E_PARA, "HcclB200DescribeStatus: bad arguments");
    DevStatus *d = c->status((int)localRank);
    if (d->code == 0) snprintf(text, cap, "rank %d of %s: no error (ops started %llu, completed %llu)", c->ctx((int)localRank).rank,
                               c->name().c_str(), (unsigned long long)d->head, (unsigned long long)d->tail);
    else
        snprintf(text, cap, "rank %d of %s: %s in op #%llu at step %d, channel %u, waiting for rank %d: flag expected >= 0x%llx "
                 "(op %llu, step value %llu) but saw 0x%llx (op %llu, step value %llu)",
                 c->ctx((int)localRank).rank, c->name().c_str(), HcclGetErrorString((HcclResult)d->code), (unsigned long long)d->seq,
                 (int)d->step, d->chan, d->peer, (unsigned long long)d->expected, (unsigned long long)(d->expected >> kSeqShift),
                 (unsigned long long)(d->expected & ((1u << kSeqShift) - 1)), (unsigned long long)d->seen,
                 (unsigned long long)(d->seen >> kSeqShift), (unsigned long long)(d->seen & ((1u << kSeqShift) - 1)));
    return HCCL_SUCCESS;
}
HcclResult HcclB200Select(HcclComm comm, int32_t coll, uint64_t count, HcclDataType dataType, HcclReduceOp op, int32_t *algo,
                          int32_t *nchan, double *estimateUs)
{
    GET_COMM("HcclB200Select");
    Selection s = c->select(coll, count, dataType, op);
    if (algo) *algo = s.algo;
    if (nchan) *nchan = s.nchan;
    if (estimateUs) *estimateUs = s.est_us;
    return HCCL_SUCCESS;
}
static HcclResult copy_out(const std::string &s, char *buf, size_t cap)
{
    CHK_RET_LOG(!buf || cap == 0, HCCL_E_PTR, "[EI0003] output buffer is null");
    CHK_RET_LOG(s.size() + 1 > cap, HCCL_E_MEMORY, "output buffer of %zu bytes too small for %zu", cap, s.size() + 1);
    memcpy(buf, s.c_str(), s.size() + 1);
    return HCCL_SUCCESS;
}
HcclResult HcclB200GetStatsJson(HcclComm comm, char *json, size_t cap)
{
    GET_COMM("HcclB200GetStatsJson");
    return copy_out(c->stats_json(), json, cap);
}
HcclResult HcclB200GetTraceJson(HcclComm comm, char *json, size_t cap)
{
    GET_COMM("HcclB200GetTraceJson");
    std::ostringstream o;
    o << "[";
    bool first = true;
    for (auto &t : c->trace_snapshot()) {
        o << (first ? "" : ",") << "{\"seq\":" << t.seq << ",\"op\":\"" << coll_name(t.coll) << "\",\"algo\":\"" << algo_name(t.algo)
          << "\",\"nchan\":" << t.nchan << ",\"count\":" << t.count << ",\"bytes\":" << t.bytes << ",\"dtype\":" << t.dtype
          << ",\"redop\":" << t.redop << ",\"root\":" << t.root << ",\"host_us\":" << t.host_us << "}";
        first = false;
    }
    o << "]";
    return copy_out(o.str(), json, cap);
}
HcclResult HcclB200Calibrate(HcclComm comm, aclrtStream stream)
{
    GET_COMM("HcclB200Calibrate");
    return c->calibrate(stream);
}
HcclResult HcclB200SetCostModel(HcclComm comm, double alphaUs, double betaGBps, double nvlsGBps, double gammaGBps, double launchUs)
{
    GET_COMM("HcclB200SetCostModel");
    CostModel &m = c->cost_model();
    if (alphaUs > 0) m.alpha_us = alphaUs;
    if (betaGBps > 0) m.beta_gbps = betaGBps;
    if (nvlsGBps > 0) m.nvls_gbps = nvlsGBps;
    if (gammaGBps > 0) m.gamma_gbps = gammaGBps;
    if (launchUs > 0) m.launch_us = launchUs;
    return HCCL_SUCCESS;
}
HcclResult HcclB200HasNvls(HcclComm comm, int32_t *has)
{
    GET_COMM("HcclB200HasNvls");
    *has = c->has_nvls() ? 1 : 0;
    return HCCL_SUCCESS;
}
HcclResult HcclB200MemAlloc(HcclComm comm, size_t bytes, void **localPtrs, int32_t *handle)
{
    GET_COMM("HcclB200MemAlloc");
    CHK_RET_LOG(!localPtrs || !handle || bytes == 0, HCCL_E_PARA, "HcclB200MemAlloc: bad arguments");
    int h = 0;
    CHK_RET(c->sym_alloc(bytes, localPtrs, &h));
    *handle = h;
    return HCCL_SUCCESS;
}
HcclResult HcclB200MemFree(HcclComm comm, int32_t handle)
{
    GET_COMM("HcclB200MemFree");
    return c->sym_free(handle);
}
// ---- allocator hooks for frameworks with pluggable device allocators (torch.cuda.memory.CUDAPluggableAllocator /
// torch.cuda.MemPool): tensors created inside such a pool live in registered symmetric memory, so collectives on them
// take the zero-copy paths without any call of this API by the user.  The pool is bound to ONE communicator with one local
// rank; an allocation is a collective (every rank's allocator has to ask for the same sizes in the same order, which
// same-program ranks do).  Blocks that the framework returns are kept and handed out again for the same size: releasing
// symmetric memory is collective as well, and a framework frees at moments of its own choosing; everything is released
// when the communicator is destroyed or the pool is unbound.
HcclResult HcclB200PoolBind(HcclComm comm)
{
    std::lock_guard<std::mutex> lk(g_pool_mu);
    if (!comm) {  // unbind: the blocks go back with a collective release each (all ranks unbind together)
        if (g_pool_comm && as_comm((HcclComm)g_pool_comm))
            for (auto &b : g_pool_blocks) g_pool_comm->sym_free(b.handle);
        g_pool_blocks.clear();
        g_pool_comm = nullptr;
        return HCCL_SUCCESS;
    }
    GET_COMM("HcclB200PoolBind");
    CHK_RET_LOG(c->nlocal() != 1 || c->transport() != TR_DEVICE, HCCL_E_NOT_SUPPORT, "the allocator pool needs a device communicator with one rank per process");
    CHK_RET_LOG(g_pool_comm && g_pool_comm != c, HCCL_E_PARA, "the allocator pool is bound to another communicator");
    g_pool_comm = c;
    return HCCL_SUCCESS;
}
void *hcclb200_torch_malloc(ssize_t size, int device, void *stream)
{
    (void)stream;
    std::lock_guard<std::mutex> lk(g_pool_mu);
    if (!g_pool_comm || !as_comm((HcclComm)g_pool_comm) || size <= 0 || device != g_pool_comm->device()) return nullptr;
    const size_t bytes = ((size_t)size + 255) / 256 * 256;
    for (auto &b : g_pool_blocks)
        if (!b.in_use && b.bytes == bytes) { b.in_use = true; return b.ptr; }
    void *ptr = nullptr;
    int h = 0;
    if (g_pool_comm->sym_alloc(bytes, &ptr, &h) != HCCL_SUCCESS) return nullptr;
    g_pool_blocks.push_back(PoolBlock{ptr, bytes, h, true});
    return ptr;
}
void hcclb200_torch_free(void *ptr, ssize_t size, int device, void *stream)
{
    (void)size; (void)device; (void)stream;
    std::lock_guard<std::mutex> lk(g_pool_mu);
    for (auto &b : g_pool_blocks)
        if (b.ptr == ptr) { b.in_use = false; return; }
}

HcclResult HcclB200MemQuery(HcclComm comm, int32_t handle, void **peerPtrs, void **mcPtrs, size_t *bytes)
{
    GET_COMM("HcclB200MemQuery");
    CHK_RET_LOG(!peerPtrs, HCCL_E_PTR, "[EI0003] HcclB200MemQuery: peerPtrs is null");
    return c->sym_query(handle, peerPtrs, mcPtrs, bytes);
}
HcclResult HcclB200Put(HcclComm comm, uint32_t localRank, int32_t handle, uint32_t peer, size_t offset, const void *src, size_t bytes,
                       aclrtStream stream)
{
    GET_COMM("HcclB200Put");
    CHK_RET_LOG(!src && bytes, HCCL_E_PTR, "[EI0003] HcclB200Put: src is null");
    return c->sym_put((int)localRank, handle, (int)peer, offset, src, bytes, stream);
}
HcclResult HcclB200Get(HcclComm comm, uint32_t localRank, int32_t handle, uint32_t peer, size_t offset, void *dst, size_t bytes,
                       aclrtStream stream)
{
    GET_COMM("HcclB200Get");
    CHK_RET_LOG(!dst && bytes, HCCL_E_PTR, "[EI0003] HcclB200Get: dst is null");
    return c->sym_get((int)localRank, handle, (int)peer, offset, dst, bytes, stream);
}
HcclResult HcclB200GetTopoJson(HcclComm comm, char *json, size_t cap)
{
    GET_COMM("HcclB200GetTopoJson");
    CHK_RET_LOG(!json || cap == 0, HCCL_E_PTR, "[EI0003] HcclB200GetTopoJson: json is null");
    std::string s = c->topo_json();
    CHK_RET_LOG(s.size() + 1 > cap, HCCL_E_MEMORY, "HcclB200GetTopoJson: %zu bytes needed, %zu given", s.size() + 1, cap);
    memcpy(json, s.c_str(), s.size() + 1);
    return HCCL_SUCCESS;
}
HcclResult HcclB200GetOverflowCount(HcclComm comm, uint64_t *count)
{
    GET_COMM("HcclB200GetOverflowCount");
    CHK_RET_LOG(!count, HCCL_E_PTR, "[EI0003] HcclB200GetOverflowCount: count is null");
    *count = c->overflow_count();
    return HCCL_SUCCESS;
}
HcclResult HcclGetTopoDesc(HcclComm comm, HcclTopoDescs *topoDescs, uint32_t topoSize)
{
    // reference: op_base.cc:3523 and hccl_communicator.cc:7236-7257 (L0 = the server's link type and rank count, L1 empty)
    GET_COMM("HcclGetTopoDesc");
    CHK_RET_LOG(!topoDescs, HCCL_E_PTR, "[EI0003] HcclGetTopoDesc: topoDescs is null");
    CHK_RET_LOG(topoSize < (uint32_t)HCCL_TOPO_MAX, HCCL_E_PARA, "HcclGetTopoDesc: topoSize %u is below %d", topoSize, (int)HCCL_TOPO_MAX);
    topoDescs[HCCL_TOPO_L0].algSets = HCCL_ALG_MESH | HCCL_ALG_RING | (c->has_nvls() ? HCCL_ALG_SWITCH : 0u);
    topoDescs[HCCL_TOPO_L0].rankSize = (uint32_t)c->nranks();
    topoDescs[HCCL_TOPO_L1].algSets = 0;
    topoDescs[HCCL_TOPO_L1].rankSize = 0;
    return HCCL_SUCCESS;
}
HcclResult HcclB200PlanCheck(int32_t coll, int32_t algo, uint32_t nRanks, uint64_t count, HcclDataType dataType, uint32_t nChannels,
                             uint64_t stageHalfBytes, int32_t skewStep, int64_t skewBytes, char *message, size_t cap)
{
    OpDesc d;
    d.coll = coll; d.algo = algo; d.nranks = (int)nRanks; d.dtype = dataType; d.nchan = (int)nChannels;
    d.count = count; d.chunk_off = 0; d.chunk_count = count;
    std::vector<int> local;
    for (uint32_t r = 0; r < nRanks; ++r) local.push_back((int)r);
    Plan plan;
    CHK_RET(build_plan(d, local, &plan));
    if (skewStep >= 0 && !plan.steps.empty() && skewStep < (int)plan.steps[0].size()) plan.steps[0][skewStep].d_off += (uint64_t)skewBytes;
    std::string why;
    HcclResult rc = verify_plan(d, local, plan, stageHalfBytes, &why);
    if (message && cap) snprintf(message, cap, "%s", rc == HCCL_SUCCESS ? plan.name.c_str() : why.c_str());
    return rc;
}
HcclResult HcclB200PlanRaceCheck(int32_t coll, int32_t algo, uint32_t nRanks, uint64_t count, HcclDataType dataType, uint32_t nChannels,
                                 uint32_t root, int32_t inPlace, int32_t dropWaitRank, int32_t dropWaitStep, char *message, size_t cap)
{
    OpDesc d;
    d.coll = coll; d.algo = algo; d.nranks = (int)nRanks; d.dtype = dataType; d.nchan = (int)nChannels; d.root = (int)root;
    d.count = count; d.chunk_off = 0; d.chunk_count = count;
    std::vector<int> local;
    for (uint32_t r = 0; r < nRanks; ++r) local.push_back((int)r);
    const int p = (int)nRanks;
    if (coll == COLL_ALLGATHER_V || coll == COLL_REDUCE_SCATTER_V) {
        // a non-uniform layout derived from `count`: rank j contributes count + 3 j elements (one rank nothing when count is 0 mod 5)
        uint64_t o = 0;
        for (int j = 0; j < p; ++j) {
            uint64_t c = (count % 5 == 0 && j == p / 2) ? 0 : count + 3 * (uint64_t)j;
            d.counts.push_back(c);
            d.displs.push_back(o);
            o += c;
        }
        uint64_t mx = 0;
        for (uint64_t c : d.counts) mx = std::max(mx, c);
        d.chunk_count = mx;
    } else if (coll == COLL_ALLTOALLV || coll == COLL_ALLTOALLVC) {
        // count matrix m[i][j] = count * ((i + 2 j) % 3 + 1) / 3 and slots of about a third of the largest block: several rounds
        // with acknowledgements per ordered pair
        std::vector<uint64_t> m((size_t)p * p);
        for (int i = 0; i < p; ++i)
            for (int j = 0; j < p; ++j) m[(size_t)i * p + j] = count * (uint64_t)((i + 2 * j) % 3 + 1) / 3;
        for (int i = 0; i < p; ++i) {
            uint64_t so = 0, ro = 0;
            for (int j = 0; j < p; ++j) {
                d.send_counts.push_back(m[(size_t)i * p + j]); d.send_displs.push_back(so); so += m[(size_t)i * p + j];
                d.recv_counts.push_back(m[(size_t)j * p + i]); d.recv_displs.push_back(ro); ro += m[(size_t)j * p + i];
            }
        }
        d.slot_bytes = std::max<uint64_t>(256, (count * (uint64_t)dtype_size(dataType) / 3 + 255) / 256 * 256);
    }
    Plan plan;
    CHK_RET(build_plan(d, local, &plan));
    // self-test of the checker: take one wait out of the plan and see the finding
    if (dropWaitRank >= 0 && dropWaitRank < (int)plan.steps.size() && dropWaitStep >= 0 && dropWaitStep < (int)plan.steps[dropWaitRank].size()) {
        Step &st = plan.steps[dropWaitRank][dropWaitStep];
        CHK_RET_LOG(st.wait_rank == RANK_NONE, HCCL_E_PARA, "step %d of rank %d has no wait to drop", dropWaitStep, dropWaitRank);
        st.wait_rank = RANK_NONE;
        st.flags &= (uint8_t)~SF_WAIT_ALLCH;
    }
    std::string why;
    HcclResult rc = race_check_plan(d, plan, inPlace != 0, &why);
    if (message && cap) snprintf(message, cap, "%s", rc == HCCL_SUCCESS ? plan.name.c_str() : why.c_str());
    return rc;
}
HcclResult HcclB200Exchange(HcclComm comm, const char *tag, const void *mine, size_t len, void *all)
{
    GET_COMM("HcclB200Exchange");
    CHK_RET_LOG(!tag || !mine || !all, HCCL_E_PTR, "[EI0003] HcclB200Exchange: null pointer");
    std::vector<std::string> out;
    CHK_RET(c->exchange(tag, std::string((const char *)mine, len), &out));
    for (size_t i = 0; i < out.size(); ++i) {
        CHK_RET_LOG(out[i].size() != len, HCCL_E_PARA, "HcclB200Exchange: rank %zu contributed %zu bytes, expected %zu", i, out[i].size(), len);
        memcpy((char *)all + i * len, out[i].data(), len);
    }
    return HCCL_SUCCESS;
}
HcclResult HcclB200GetDeviceContext(HcclComm comm, void **devCtxArray, uint64_t *nextSeq)
{
    GET_COMM("HcclB200GetDeviceContext");
    if (devCtxArray) *devCtxArray = c->device_ctx_array();
    if (nextSeq) *nextSeq = c->next_seq();
    return HCCL_SUCCESS;
}

// ---------------------------------------------------------------------------------------------- fault / memory
HcclResult HcclCommSuspend(HcclComm comm)
{
    GET_COMM("HcclCommSuspend");
    return c->suspend();
}
HcclResult HcclCommResume(HcclComm comm)
{
    GET_COMM("HcclCommResume");
    return c->resume();
}
// NVLink attributes of a GPU as JSON (no communicator needed; `device` is the NVML index when CUDA is absent).
HcclResult HcclB200ProbeLinks(int32_t device, char *json, size_t cap)
{
    CHK_RET_LOG(!json, HCCL_E_PTR, "HcclB200ProbeLinks: json is null");
    return copy_out(link_topo_json(probe_links(device, std::string())), json, cap);
}
// Process-wide abort handler (reference: ProcessTaskAbortHandleCallback, task_abort_handler.cc:28-128): runs one stage over
// every communicator of `device` (-1: all), each within `timeoutSec` (0 = no limit).  0 success, 1 failure, 2 time-out.
int32_t HcclB200TaskAbort(int32_t device, int32_t stage, uint32_t timeoutSec)
{
    std::vector<Communicator *> comms;
    {
        std::lock_guard<std::mutex> lk(g_comm_mu);
        for (auto *c : g_comms)
            if (device < 0 || c->transport() != TR_DEVICE || c->device() == device) comms.push_back(c);
    }
    const int budget_ms = (int)std::min<uint64_t>((uint64_t)timeoutSec * 1000, 0x7fffffff);
    for (auto *c : comms) {
        HcclResult rc = stage == 0 ? c->suspend_entry(budget_ms) : (stage == 1 ? c->stop_exec(budget_ms) : c->clean(budget_ms));
        if (rc == HCCL_E_TIMEOUT) { HLOG_ERROR("task abort stage %d timed out on communicator %s", stage, c->name().c_str()); return 2; }
        if (rc != HCCL_SUCCESS && rc != HCCL_E_SUSPENDING) { HLOG_ERROR("task abort stage %d failed on communicator %s (%d)", stage, c->name().c_str(), (int)rc); return 1; }
    }
    return 0;
}

// Zero-copy registration (reference: zero_copy_memory_agent.cc, request types SET_MEMORY_RANGE .. DEACTIVATE_COMM_MEMORY).
// HcclCommSetMemoryRange reserves an address range; HcclCommActivateCommMemory, called by every rank of the communicator
// in the same order, registers memory inside it as a symmetric allocation: peers map it, and collectives whose buffers lie
// in registered memory at the same offsets on all ranks take the zero-copy path.  With one rank per GPU `handle` is the
// driver allocation handle behind virPtr (created exportable as a POSIX file descriptor; the whole allocation, offset 0);
// a communicator that cannot map foreign memory (CPU ranks in separate processes) keeps the record and stages as before.
namespace {
struct Range { Communicator *c; void *base; size_t size; };
struct Activation { Communicator *c; void *ptr; size_t size; int handle; };
std::mutex g_range_mu;
std::vector<Range> g_ranges;
std::vector<Activation> g_acts;
}  // namespace
HcclResult HcclCommSetMemoryRange(HcclComm comm, void *baseVirPtr, size_t size, size_t alignment, uint64_t flags)
{
    GET_COMM("HcclCommSetMemoryRange");
    (void)alignment; (void)flags;
    CHK_RET_LOG(!baseVirPtr || size == 0, HCCL_E_PARA, "HcclCommSetMemoryRange: empty range");
    std::lock_guard<std::mutex> lk(g_range_mu);
    for (auto &r : g_ranges)
        CHK_RET_LOG(r.c == c && (char *)baseVirPtr < (char *)r.base + r.size && (char *)r.base < (char *)baseVirPtr + size, HCCL_E_PARA,
                    "HcclCommSetMemoryRange: range overlaps a registered range");
    g_ranges.push_back({c, baseVirPtr, size});
    return HCCL_SUCCESS;
}
HcclResult HcclCommUnsetMemoryRange(HcclComm comm, void *baseVirPtr)
{
    GET_COMM("HcclCommUnsetMemoryRange");
    std::lock_guard<std::mutex> lk(g_range_mu);
    for (size_t i = 0; i < g_ranges.size(); ++i)
        if (g_ranges[i].c == c && g_ranges[i].base == baseVirPtr) {
            for (auto &a : g_acts)
                CHK_RET_LOG(a.c == c && (char *)a.ptr >= (char *)g_ranges[i].base && (char *)a.ptr < (char *)g_ranges[i].base + g_ranges[i].size,
                            HCCL_E_PARA, "HcclCommUnsetMemoryRange: range still has activated memory");
            g_ranges.erase(g_ranges.begin() + i);
            return HCCL_SUCCESS;
        }
    return HCCL_E_NOT_FOUND;
}
HcclResult HcclCommActivateCommMemory(HcclComm comm, void *virPtr, size_t size, size_t offset, aclrtDrvMemHandle handle, uint64_t flags)
{
    GET_COMM("HcclCommActivateCommMemory");
    (void)flags;
    CHK_RET_LOG(!virPtr || size == 0, HCCL_E_PARA, "HcclCommActivateCommMemory: empty region");
    {
        std::lock_guard<std::mutex> lk(g_range_mu);
        bool inside = false;
        for (auto &r : g_ranges)
            inside |= r.c == c && (char *)virPtr >= (char *)r.base && (char *)virPtr + size <= (char *)r.base + r.size;
        CHK_RET_LOG(!inside, HCCL_E_PARA, "HcclCommActivateCommMemory: address not inside a range set with HcclCommSetMemoryRange");
        for (auto &a : g_acts)
            CHK_RET_LOG(a.c == c && (char *)virPtr < (char *)a.ptr + a.size && (char *)a.ptr < (char *)virPtr + size, HCCL_E_PARA,
                        "HcclCommActivateCommMemory: region overlaps activated memory");
    }
    int h = 0;
    if (c->nlocal() == 1) {
        void *ptrs[1] = {virPtr};
        unsigned long long dh[1] = {(unsigned long long)(uintptr_t)handle};
        HcclResult rc = c->sym_adopt(ptrs, size, handle ? dh : nullptr, offset, &h);
        if (rc == HCCL_E_NOT_SUPPORT) h = 0;  // recorded only: this transport cannot map foreign memory
        else CHK_RET(rc);
    }
    std::lock_guard<std::mutex> lk(g_range_mu);
    g_acts.push_back({c, virPtr, size, h});
    return HCCL_SUCCESS;
}
HcclResult HcclCommDeactivateCommMemory(HcclComm comm, void *virPtr)
{
    GET_COMM("HcclCommDeactivateCommMemory");
    Activation act{nullptr, nullptr, 0, 0};
    {
        std::lock_guard<std::mutex> lk(g_range_mu);
        for (size_t i = 0; i < g_acts.size(); ++i)
            if (g_acts[i].c == c && (char *)virPtr >= (char *)g_acts[i].ptr && (char *)virPtr < (char *)g_acts[i].ptr + g_acts[i].size) {
                act = g_acts[i];
                g_acts.erase(g_acts.begin() + i);
                break;
            }
    }
    if (!act.c) return HCCL_E_NOT_FOUND;
    if (act.handle) return c->sym_free(act.handle);
    return HCCL_SUCCESS;
}
HcclResult HcclB200MemAdopt(HcclComm comm, void *const *localPtrs, size_t bytes, const uint64_t *drvHandles, size_t handleOffset, int32_t *handle)
{
    GET_COMM("HcclB200MemAdopt");
    CHK_RET_LOG(!localPtrs || !handle, HCCL_E_PTR, "[EI0003] HcclB200MemAdopt: null pointer");
    CHK_RET_LOG(bytes == 0, HCCL_E_PARA, "HcclB200MemAdopt: empty region");
    for (int li = 0; li < c->nlocal(); ++li) CHK_RET_LOG(!localPtrs[li], HCCL_E_PTR, "[EI0003] HcclB200MemAdopt: localPtrs[%d] is null", li);
    std::vector<unsigned long long> dh;
    if (drvHandles) dh.assign(drvHandles, drvHandles + c->nlocal());
    int h = 0;
    CHK_RET(c->sym_adopt(localPtrs, bytes, drvHandles ? dh.data() : nullptr, handleOffset, &h));
    *handle = h;
    return HCCL_SUCCESS;
}

}  // extern "C"
