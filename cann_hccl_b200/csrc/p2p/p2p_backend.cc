#include "p2p/p2p_backend.h"
#include <dlfcn.h>
#include <cstring>
#include <mutex>
#include <cuda_runtime.h>
#include "common/base.h"
#include "common/env.h"
#include "common/log.h"
#include "core/communicator.h"

namespace hcclb {
namespace {
struct NcclUid { char internal[128]; };
struct NcclApi {
    int (*GetUniqueId)(NcclUid *);
    int (*CommInitRank)(void **, int, NcclUid, int);
    int (*CommDestroy)(void *);
    int (*CommAbort)(void *);
    int (*Send)(const void *, size_t, int, int, void *, void *);
    int (*Recv)(void *, size_t, int, int, void *, void *);
    int (*AllReduce)(const void *, void *, size_t, int, int, void *, void *);
    int (*GroupStart)();
    int (*GroupEnd)();
    const char *(*GetErrorString)(int);
    bool ok = false;
};
NcclApi &api()
{
    static NcclApi a;
    static std::once_flag once;
    std::call_once(once, [] {
        const EnvConfig &env = env_config();
        if (getenv("HCCL_P2P_BACKEND") && strcmp(getenv("HCCL_P2P_BACKEND"), "mailbox") == 0) return;
        void *h = nullptr;
        if (!env.ncc_lib.empty()) h = dlopen(env.ncc_lib.c_str(), RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return;
        auto sym = [&](const char *n) { return dlsym(h, n); };
        a.GetUniqueId = (decltype(a.GetUniqueId))sym("ncclGetUniqueId");
        a.CommInitRank = (decltype(a.CommInitRank))sym("ncclCommInitRank");
        a.CommDestroy = (decltype(a.CommDestroy))sym("ncclCommDestroy");
        a.CommAbort = (decltype(a.CommAbort))sym("ncclCommAbort");
        a.Send = (decltype(a.Send))sym("ncclSend");
        a.Recv = (decltype(a.Recv))sym("ncclRecv");
        a.AllReduce = (decltype(a.AllReduce))sym("ncclAllReduce");
        a.GroupStart = (decltype(a.GroupStart))sym("ncclGroupStart");
        a.GroupEnd = (decltype(a.GroupEnd))sym("ncclGroupEnd");
        a.GetErrorString = (decltype(a.GetErrorString))sym("ncclGetErrorString");
        a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.Send && a.Recv && a.GroupStart && a.GroupEnd;
    });
    return a;
}
constexpr int kNcclInt8 = 0;
}  // namespace

bool P2pBackend::available() { return api().ok; }

HcclResult P2pBackend::create(Communicator *comm, std::unique_ptr<P2pBackend> *out)
{
    if (!available()) return HCCL_E_UNAVAIL;
    std::unique_ptr<P2pBackend> b(new P2pBackend());
    b->device_ = comm->device();
    b->th_ = std::thread([p = b.get(), comm] { p->init_thread(comm); });
    *out = std::move(b);
    return HCCL_SUCCESS;
}

void P2pBackend::init_thread(Communicator *comm)
{
    cudaSetDevice(device_);
    NcclUid uid;
    memset(&uid, 0, sizeof(uid));
    if (comm->rank() == 0 && api().GetUniqueId(&uid) != 0) { ready_.store(-1); return; }
    std::vector<std::string> all;
    if (comm->exchange_p2p("nccl-uid", std::string((const char *)&uid, sizeof(uid)), &all) != HCCL_SUCCESS) { ready_.store(-1); return; }
    memcpy(&uid, all[0].data(), sizeof(uid));
    int rc = api().CommInitRank(&nccl_comm_, comm->nranks(), uid, comm->rank());
    if (rc != 0) {
        HLOG_ERROR("ncclCommInitRank failed: %s", api().GetErrorString ? api().GetErrorString(rc) : "?");
        ready_.store(-1);
        return;
    }
    ready_.store(1);
}

HcclResult P2pBackend::wait_ready()
{
    if (th_.joinable()) th_.join();
    return ready_.load() == 1 ? HCCL_SUCCESS : HCCL_E_UNAVAIL;
}

P2pBackend::~P2pBackend()
{
    if (th_.joinable()) th_.join();
    if (nccl_comm_) {
        cudaSetDevice(device_);
        api().CommDestroy(nccl_comm_);
    }
}

HcclResult P2pBackend::send(const void *buf, uint64_t count, int dtype, int peer, void *stream)
{
    CHK_RET(wait_ready());
    int rc = api().Send(buf, count * dtype_size(dtype), kNcclInt8, peer, nccl_comm_, stream);
    CHK_RET_LOG(rc != 0, HCCL_E_INTERNAL, "ncclSend failed: %s", api().GetErrorString(rc));
    return HCCL_SUCCESS;
}
HcclResult P2pBackend::recv(void *buf, uint64_t count, int dtype, int peer, void *stream)
{
    CHK_RET(wait_ready());
    int rc = api().Recv(buf, count * dtype_size(dtype), kNcclInt8, peer, nccl_comm_, stream);
    CHK_RET_LOG(rc != 0, HCCL_E_INTERNAL, "ncclRecv failed: %s", api().GetErrorString(rc));
    return HCCL_SUCCESS;
}
HcclResult P2pBackend::baseline_allreduce(const void *send, void *recv, uint64_t count, int dtype, int op, void *stream)
{
    CHK_RET(wait_ready());
    int nt;
    switch (dtype) {
        case HCCL_DATA_TYPE_INT8: nt = 0; break;
        case HCCL_DATA_TYPE_UINT8: nt = 1; break;
        case HCCL_DATA_TYPE_INT32: nt = 2; break;
        case HCCL_DATA_TYPE_UINT32: nt = 3; break;
        case HCCL_DATA_TYPE_INT64: nt = 4; break;
        case HCCL_DATA_TYPE_UINT64: nt = 5; break;
        case HCCL_DATA_TYPE_FP16: nt = 6; break;
        case HCCL_DATA_TYPE_FP32: nt = 7; break;
        case HCCL_DATA_TYPE_FP64: nt = 8; break;
        case HCCL_DATA_TYPE_BFP16: nt = 9; break;
        default: return HCCL_E_NOT_SUPPORT;
    }
    if (!api().AllReduce) return HCCL_E_UNAVAIL;
    int rc = api().AllReduce(send, recv, count, nt, op, nccl_comm_, stream);
    CHK_RET_LOG(rc != 0, HCCL_E_INTERNAL, "ncclAllReduce failed: %s", api().GetErrorString(rc));
    return HCCL_SUCCESS;
}

HcclResult P2pBackend::batch(const std::vector<HcclSendRecvItem *> &sends, const std::vector<HcclSendRecvItem *> &recvs, void *stream)
{
    CHK_RET(wait_ready());
    int rc = api().GroupStart();
    for (auto *s : sends)
        if (rc == 0) rc = api().Send(s->buf, s->count * dtype_size(s->dataType), kNcclInt8, (int)s->remoteRank, nccl_comm_, stream);
    for (auto *r : recvs)
        if (rc == 0) rc = api().Recv(r->buf, r->count * dtype_size(r->dataType), kNcclInt8, (int)r->remoteRank, nccl_comm_, stream);
    int rc2 = api().GroupEnd();
    if (rc == 0) rc = rc2;
    CHK_RET_LOG(rc != 0, HCCL_E_INTERNAL, "NCCL batched send/recv failed: %s", api().GetErrorString(rc));
    return HCCL_SUCCESS;
}
}  // namespace hcclb
