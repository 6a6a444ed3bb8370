/*
 * Public C API of the B200-native HCCL-compatible collective library.
 *
 * Names and argument order follow the Ascend HCCL header (reference:
 * inc/hccl/hccl.h:30-471).  `aclrtStream` is an alias of a CUDA stream
 * (cudaStream_t can be passed directly).  All collectives are asynchronous
 * with respect to the host: they enqueue one fused sm_100a kernel (or, on the
 * host-memory transport, run on the calling thread) and return.
 *
 * Buffer arguments are device pointers on the device transport and plain host
 * pointers on the host-memory transport (HCCL_TRANSPORT=host).
 * Counts / displacement arrays are host arrays of uint64_t, in elements.
 */
#ifndef HCCL_H_
#define HCCL_H_

#include "hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef void *aclrtStream;       /* == cudaStream_t */
typedef void *aclrtDrvMemHandle; /* == CUmemGenericAllocationHandle cast to a pointer */

/* ---- communicator lifetime -------------------------------------------- */

/* Rank-table (JSON file) initialisation; single-node concise table
 * {"server_list":[{"server_id":..,"device":[{"device_id":..,"rank_id":..}]}]}
 * plus optional "host_ip"/"port" of the rendezvous hub. */
extern HcclResult HcclCommInitClusterInfo(const char *clusterInfo, uint32_t rank, HcclComm *comm);
extern HcclResult HcclCommInitClusterInfoConfig(const char *clusterInfo, uint32_t rank,
                                                HcclCommConfig *config, HcclComm *comm);

/* Carve a sub-communicator out of *comm; ranks that are not members pass
 * subCommRankId = 0xFFFFFFFF and receive a null handle. */
extern HcclResult HcclCreateSubCommConfig(HcclComm *comm, uint32_t rankNum, uint32_t *rankIds,
                                          uint64_t subCommId, uint32_t subCommRankId,
                                          HcclCommConfig *config, HcclComm *subComm);

/* Root rank: start the TCP rendezvous hub and describe it in *rootInfo. */
extern HcclResult HcclGetRootInfo(HcclRootInfo *rootInfo);
/* Every rank: join the hub, exchange rank table and memory handles. */
extern HcclResult HcclCommInitRootInfo(uint32_t nRanks, const HcclRootInfo *rootInfo, uint32_t rank,
                                       HcclComm *comm);
extern HcclResult HcclCommInitRootInfoConfig(uint32_t nRanks, const HcclRootInfo *rootInfo, uint32_t rank,
                                             const HcclCommConfig *config, HcclComm *comm);
/* One process, ndev devices: a communicator per device (thread per device). */
extern HcclResult HcclCommInitAll(uint32_t ndev, int32_t *devices, HcclComm *comms);
extern HcclResult HcclCommDestroy(HcclComm comm);

/* ---- configuration / queries ------------------------------------------ */
extern HcclResult HcclSetConfig(HcclConfig config, union HcclConfigValue configValue);
extern HcclResult HcclGetConfig(HcclConfig config, union HcclConfigValue *configValue);
extern HcclResult HcclGetCommName(HcclComm comm, char *commName);
extern HcclResult HcclGetRankSize(HcclComm comm, uint32_t *rankSize);
extern HcclResult HcclGetRankId(HcclComm comm, uint32_t *rank);
extern HcclResult HcclGetCommAsyncError(HcclComm comm, HcclResult *asyncError);
extern const char *HcclGetErrorString(HcclResult code);
extern uint32_t HcclGetCommConfigCapability(void);

/* ---- collectives -------------------------------------------------------- */
extern HcclResult HcclAllReduce(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType,
                                HcclReduceOp op, HcclComm comm, aclrtStream stream);
extern HcclResult HcclBroadcast(void *buf, uint64_t count, HcclDataType dataType, uint32_t root,
                                HcclComm comm, aclrtStream stream);
extern HcclResult HcclReduceScatter(void *sendBuf, void *recvBuf, uint64_t recvCount, HcclDataType dataType,
                                    HcclReduceOp op, HcclComm comm, aclrtStream stream);
extern HcclResult HcclReduceScatterV(void *sendBuf, const void *sendCounts, const void *sendDispls,
                                     void *recvBuf, uint64_t recvCount, HcclDataType dataType,
                                     HcclReduceOp op, HcclComm comm, aclrtStream stream);
extern HcclResult HcclScatter(void *sendBuf, void *recvBuf, uint64_t recvCount, HcclDataType dataType,
                              uint32_t root, HcclComm comm, aclrtStream stream);
extern HcclResult HcclAllGather(void *sendBuf, void *recvBuf, uint64_t sendCount, HcclDataType dataType,
                                HcclComm comm, aclrtStream stream);
extern HcclResult HcclAllGatherV(void *sendBuf, uint64_t sendCount, void *recvBuf, const void *recvCounts,
                                 const void *recvDispls, HcclDataType dataType, HcclComm comm,
                                 aclrtStream stream);
extern HcclResult HcclBarrier(HcclComm comm, aclrtStream stream);
extern HcclResult HcclSend(void *sendBuf, uint64_t count, HcclDataType dataType, uint32_t destRank,
                           HcclComm comm, aclrtStream stream);
extern HcclResult HcclRecv(void *recvBuf, uint64_t count, HcclDataType dataType, uint32_t srcRank,
                           HcclComm comm, aclrtStream stream);
extern HcclResult HcclAlltoAllV(const void *sendBuf, const void *sendCounts, const void *sdispls,
                                HcclDataType sendType, const void *recvBuf, const void *recvCounts,
                                const void *rdispls, HcclDataType recvType, HcclComm comm,
                                aclrtStream stream);
extern HcclResult HcclAlltoAll(const void *sendBuf, uint64_t sendCount, HcclDataType sendType,
                               const void *recvBuf, uint64_t recvCount, HcclDataType recvType,
                               HcclComm comm, aclrtStream stream);
extern HcclResult HcclReduce(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType,
                             HcclReduceOp op, uint32_t root, HcclComm comm, aclrtStream stream);
extern HcclResult HcclBatchSendRecv(HcclSendRecvItem *sendRecvInfo, uint32_t itemNum, HcclComm comm,
                                    aclrtStream stream);

/* Fill *config with {size, magic, version} and "not set" defaults. */
static inline void HcclCommConfigInit(HcclCommConfig *config)
{
    struct HcclCfgHead { size_t size; uint32_t magic; uint32_t version; uint64_t rsv; };
    if (!config) return;
    struct HcclCfgHead *h = (struct HcclCfgHead *)(void *)config;
    h->size = sizeof(HcclCommConfig);
    h->magic = HCCL_COMM_CONFIG_MAGIC_WORD;
    h->version = HCCL_COMM_CONFIG_VERSION;
    h->rsv = 0;
    config->hcclBufferSize = HCCL_COMM_BUFFSIZE_CONFIG_NOT_SET;
    config->hcclDeterministic = HCCL_COMM_DETERMINISTIC_CONFIG_NOT_SET;
    config->hcclCommName[0] = 0;
    config->hcclUdi[0] = 0;
    config->hcclOpExpansionMode = HCCL_COMM_DEFAULT_OP_EXPANSION_MODE;
    config->hcclRdmaTrafficClass = HCCL_COMM_TRAFFIC_CLASS_CONFIG_NOT_SET;
    config->hcclRdmaServiceLevel = HCCL_COMM_SERVICE_LEVEL_CONFIG_NOT_SET;
}

/* ---- fault handling / memory registration ----------------------------- */
/* Suspend: raise the abort word that every device-side wait polls; running
 * kernels return with status HCCL_E_SUSPENDING, new ops are refused. */
extern HcclResult HcclCommSuspend(HcclComm comm);
/* Resume: all ranks rendezvous, flag pages and sequence numbers are re-armed. */
extern HcclResult HcclCommResume(HcclComm comm);
/* Reserve / release a peer-mappable virtual range for zero-copy collectives. */
extern HcclResult HcclCommSetMemoryRange(HcclComm comm, void *baseVirPtr, size_t size, size_t alignment,
                                         uint64_t flags);
extern HcclResult HcclCommUnsetMemoryRange(HcclComm comm, void *baseVirPtr);
extern HcclResult HcclCommActivateCommMemory(HcclComm comm, void *virPtr, size_t size, size_t offset,
                                             aclrtDrvMemHandle handle, uint64_t flags);
extern HcclResult HcclCommDeactivateCommMemory(HcclComm comm, void *virPtr);

/* ---- topology ----------------------------------------------------------- */
/* topoSize = entries in topoDescs, at least HCCL_TOPO_MAX. */
extern HcclResult HcclGetTopoDesc(HcclComm comm, HcclTopoDescs *topoDescs, uint32_t topoSize);

#ifdef __cplusplus
}
#endif
#endif /* HCCL_H_ */
