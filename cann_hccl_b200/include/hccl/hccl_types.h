/*
 * Public types of the B200-native HCCL-compatible collective library.
 *
 * Numeric values of every enum, the 4108-byte root-info blob and the
 * HcclCommConfig layout are kept binary compatible with the Ascend HCCL
 * public header (reference: inc/hccl/hccl_types.h:23-153) so that code
 * written against HCCL recompiles unchanged.  Everything behind these types
 * is a new implementation for NVLink 5 / NVSwitch.
 */
#ifndef HCCL_TYPES_H_
#define HCCL_TYPES_H_

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Result codes (reference: hccl_types.h:23-48). */
typedef enum {
    HCCL_SUCCESS = 0,
    HCCL_E_PARA = 1,
    HCCL_E_PTR = 2,
    HCCL_E_MEMORY = 3,
    HCCL_E_INTERNAL = 4,
    HCCL_E_NOT_SUPPORT = 5,
    HCCL_E_NOT_FOUND = 6,
    HCCL_E_UNAVAIL = 7,
    HCCL_E_SYSCALL = 8,
    HCCL_E_TIMEOUT = 9,
    HCCL_E_OPEN_FILE_FAILURE = 10,
    HCCL_E_TCP_CONNECT = 11,
    HCCL_E_ROCE_CONNECT = 12,
    HCCL_E_TCP_TRANSFER = 13,
    HCCL_E_ROCE_TRANSFER = 14,
    HCCL_E_RUNTIME = 15,
    HCCL_E_DRV = 16,
    HCCL_E_PROFILING = 17,
    HCCL_E_CCE = 18,
    HCCL_E_NETWORK = 19,
    HCCL_E_AGAIN = 20,
    HCCL_E_REMOTE = 21,
    HCCL_E_SUSPENDING = 22,
    HCCL_E_RESERVED
} HcclResult;

/* Opaque communicator handle. */
typedef void *HcclComm;

/* Reduction operators; all four are fused into the transfer kernels. */
typedef enum {
    HCCL_REDUCE_SUM = 0,
    HCCL_REDUCE_PROD = 1,
    HCCL_REDUCE_MAX = 2,
    HCCL_REDUCE_MIN = 3,
    HCCL_REDUCE_RESERVED = 255
} HcclReduceOp;

/* Element types (reference numbering, hccl_types.h:69-87).  Reductions are
 * implemented for the integer and floating types up to 64 bit; INT128, HIF8
 * and the FP8 types are transport-only (copy collectives). */
typedef enum {
    HCCL_DATA_TYPE_INT8 = 0,
    HCCL_DATA_TYPE_INT16 = 1,
    HCCL_DATA_TYPE_INT32 = 2,
    HCCL_DATA_TYPE_FP16 = 3,
    HCCL_DATA_TYPE_FP32 = 4,
    HCCL_DATA_TYPE_INT64 = 5,
    HCCL_DATA_TYPE_UINT64 = 6,
    HCCL_DATA_TYPE_UINT8 = 7,
    HCCL_DATA_TYPE_UINT16 = 8,
    HCCL_DATA_TYPE_UINT32 = 9,
    HCCL_DATA_TYPE_FP64 = 10,
    HCCL_DATA_TYPE_BFP16 = 11,
    HCCL_DATA_TYPE_INT128 = 12,
    HCCL_DATA_TYPE_HIF8 = 13,
    HCCL_DATA_TYPE_FP8E4M3 = 14,
    HCCL_DATA_TYPE_FP8E5M2 = 15,
    HCCL_DATA_TYPE_RESERVED = 255
} HcclDataType;

/* Process-wide knobs reachable through HcclSetConfig / HcclGetConfig. */
typedef enum {
    HCCL_DETERMINISTIC = 0,
    HCCL_CONFIG_RESERVED
} HcclConfig;

union HcclConfigValue {
    int32_t value;
};

#define HCCL_ROOT_INFO_BYTES 4108u
#define COMM_NAME_MAX_LENGTH 128u
#define UDI_MAX_LENGTH 128u

/* Opaque rendezvous blob produced by HcclGetRootInfo on one rank and shipped
 * out of band to all others.  Our payload: magic, address of the bootstrap
 * hub, port and a unique communicator identifier. */
typedef struct HcclRootInfoDef {
    char internal[HCCL_ROOT_INFO_BYTES];
} HcclRootInfo;

#define HCCL_COMM_CONFIG_INFO_BYTES 24u
#define HCCL_COMM_CONFIG_MAGIC_WORD 0xf0f0f0f0u
#define HCCL_COMM_CONFIG_VERSION 5u
#define HCCL_COMM_DEFAULT_BUFFSIZE 200u /* MB, per direction */
#define HCCL_COMM_BUFFSIZE_CONFIG_NOT_SET 0xffffffffu
#define HCCL_COMM_DEFAULT_DETERMINISTIC 0u
#define HCCL_COMM_DETERMINISTIC_CONFIG_NOT_SET 0xffffffffu
#define HCCL_COMM_DEFAULT_OP_EXPANSION_MODE 0u
#define HCCL_COMM_TRAFFIC_CLASS_CONFIG_NOT_SET 0xffffffffu
#define HCCL_COMM_SERVICE_LEVEL_CONFIG_NOT_SET 0xffffffffu

/* Per-communicator configuration.  `reserved` carries {size, magic, version}
 * written by HcclCommConfigInit.  hcclOpExpansionMode on this platform:
 * 0 = auto, 1 = host-orchestrated (plan executor only), 2 and 3 = device
 * kernels (one-shot / NVLS fast paths allowed). */
typedef struct HcclCommConfigDef {
    char reserved[HCCL_COMM_CONFIG_INFO_BYTES];
    uint32_t hcclBufferSize;
    uint32_t hcclDeterministic;
    char hcclCommName[COMM_NAME_MAX_LENGTH];
    char hcclUdi[UDI_MAX_LENGTH];
    uint32_t hcclOpExpansionMode;
    uint32_t hcclRdmaTrafficClass;
    uint32_t hcclRdmaServiceLevel;
} HcclCommConfig;

typedef enum {
    HCCL_COMM_CONFIG_BUFFER_SIZE = 0,
    HCCL_COMM_CONFIG_DETERMINISTIC = 1,
    HCCL_COMM_CONFIG_COMM_NAME = 2,
    HCCL_COMM_CONFIG_OP_EXPANSION_MODE = 3,
    HCCL_COMM_CONFIG_SUPPORT_INIT_BY_ENV = 4,
    HCCL_COMM_CONFIG_RESERVED
} HcclCommConfigCapability;

typedef enum {
    HCCL_SEND = 0,
    HCCL_RECV = 1,
    HCCL_SEND_RECV_RESERVED
} HcclSendRecvType;

typedef struct HcclSendRecvItemDef {
    HcclSendRecvType sendRecvType;
    void *buf;
    uint64_t count;
    HcclDataType dataType;
    uint32_t remoteRank;
} HcclSendRecvItem;

/* Topology description per level (HcclGetTopoDesc; the reference declares these in a closed header and fills them in
 * hccl_communicator.cc:7236-7257).  One NVSwitch domain is a single level: L0 holds every rank, L1 is empty. */
typedef enum {
    HCCL_TOPO_L0 = 0,
    HCCL_TOPO_L1 = 1,
    HCCL_TOPO_MAX
} HcclTopoLevel;

#define HCCL_ALG_MESH 0x1u   /* every rank reaches every peer directly */
#define HCCL_ALG_RING 0x2u
#define HCCL_ALG_SWITCH 0x4u /* in-switch reduction / multicast (NVLS) is available */

typedef struct HcclTopoDescsDef {
    uint64_t algSets;  /* HCCL_ALG_* bits usable at this level */
    uint32_t rankSize; /* ranks at this level */
} HcclTopoDescs;

#ifdef __cplusplus
}
#endif
#endif /* HCCL_TYPES_H_ */
