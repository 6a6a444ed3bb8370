"""ctypes binding of libhccl_b200.so (the C API of include/hccl/hccl.h and hccl_b200.h)."""
import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# HCCL_B200_LIB: another build of the library (a sanitizer build, for one)
LIB_PATH = os.environ.get("HCCL_B200_LIB") or os.path.join(_PKG, "lib", "libhccl_b200.so")

HCCL_ROOT_INFO_BYTES = 4108
COMM_NAME_MAX_LENGTH = 128

# result codes
SUCCESS, E_PARA, E_PTR, E_MEMORY, E_INTERNAL, E_NOT_SUPPORT, E_NOT_FOUND, E_UNAVAIL, E_SYSCALL, E_TIMEOUT = range(10)
E_OPEN_FILE_FAILURE, E_TCP_CONNECT, E_ROCE_CONNECT, E_TCP_TRANSFER, E_ROCE_TRANSFER, E_RUNTIME, E_DRV = range(10, 17)
E_PROFILING, E_CCE, E_NETWORK, E_AGAIN, E_REMOTE, E_SUSPENDING = range(17, 23)

# reduce ops
SUM, PROD, MAX, MIN = 0, 1, 2, 3
# data types (HcclDataType numbering)
INT8, INT16, INT32, FP16, FP32, INT64, UINT64, UINT8, UINT16, UINT32, FP64, BFP16, INT128, HIF8, FP8E4M3, FP8E5M2 = range(16)
DTYPE_SIZE = {INT8: 1, INT16: 2, INT32: 4, FP16: 2, FP32: 4, INT64: 8, UINT64: 8, UINT8: 1, UINT16: 2, UINT32: 4,
              FP64: 8, BFP16: 2, INT128: 16, HIF8: 1, FP8E4M3: 1, FP8E5M2: 1}

# collectives / algorithms of HcclB200Collective
(ALLREDUCE, BROADCAST, REDUCE_SCATTER, REDUCE_SCATTER_V, SCATTER, ALLGATHER, ALLGATHER_V, BARRIER, ALLTOALL,
 ALLTOALLV, ALLTOALLVC, REDUCE, GATHER) = range(13)
(ALGO_AUTO, ALGO_MESH, ALGO_MESH_ONESHOT, ALGO_RING, ALGO_RHD, ALGO_PAIRWISE, ALGO_STAR, ALGO_TREE, ALGO_NVLS,
 ALGO_NVLS_ONESHOT, ALGO_SINGLE, ALGO_MESH_PIPE, ALGO_NVLS_PIPE, ALGO_NVLS_ZC, ALGO_LL, ALGO_MESH_ZC, ALGO_DIRECT) = range(17)
ALGO_NAMES = ["auto", "mesh", "mesh_oneshot", "ring", "rhd", "pairwise", "star", "tree", "nvls", "nvls_oneshot", "single",
              "mesh_pipe", "nvls_pipe", "nvls_zerocopy", "ll", "mesh_zerocopy", "direct"]


class RootInfo(C.Structure):
    _fields_ = [("internal", C.c_char * HCCL_ROOT_INFO_BYTES)]


class TopoDescs(C.Structure):
    _fields_ = [("algSets", C.c_uint64), ("rankSize", C.c_uint32)]


ALG_MESH, ALG_RING, ALG_SWITCH = 1, 2, 4
TOPO_L0, TOPO_L1, TOPO_MAX = 0, 1, 2


class CommConfig(C.Structure):
    _fields_ = [("reserved", C.c_char * 24), ("hcclBufferSize", C.c_uint32), ("hcclDeterministic", C.c_uint32),
                ("hcclCommName", C.c_char * 128), ("hcclUdi", C.c_char * 128), ("hcclOpExpansionMode", C.c_uint32),
                ("hcclRdmaTrafficClass", C.c_uint32), ("hcclRdmaServiceLevel", C.c_uint32)]

    @classmethod
    def default(cls):
        """Python rendering of the inline HcclCommConfigInit."""
        cfg = cls()
        head = (C.c_uint64 * 1)(C.sizeof(cls))
        C.memmove(C.addressof(cfg), head, 8)
        mv = (C.c_uint32 * 2)(0xF0F0F0F0, 5)
        C.memmove(C.addressof(cfg) + 8, mv, 8)
        cfg.hcclBufferSize = 0xFFFFFFFF
        cfg.hcclDeterministic = 0xFFFFFFFF
        cfg.hcclOpExpansionMode = 0
        cfg.hcclRdmaTrafficClass = 0xFFFFFFFF
        cfg.hcclRdmaServiceLevel = 0xFFFFFFFF
        return cfg


class SendRecvItem(C.Structure):
    _fields_ = [("sendRecvType", C.c_int), ("buf", C.c_void_p), ("count", C.c_uint64), ("dataType", C.c_int),
                ("remoteRank", C.c_uint32)]


class B200Op(C.Structure):
    _fields_ = [("coll", C.c_int32), ("algo", C.c_int32), ("nchan", C.c_int32), ("dataType", C.c_int32),
                ("op", C.c_int32), ("root", C.c_int32), ("count", C.c_uint64),
                ("counts", C.c_void_p), ("displs", C.c_void_p),
                ("sendCounts", C.c_void_p), ("sdispls", C.c_void_p), ("recvCounts", C.c_void_p), ("rdispls", C.c_void_p)]


class B200Status(C.Structure):
    _fields_ = [("code", C.c_uint32), ("step", C.c_uint32), ("peer", C.c_int32), ("chan", C.c_uint32),
                ("expected", C.c_uint64), ("seen", C.c_uint64), ("seq", C.c_uint64), ("head", C.c_uint64),
                ("tail", C.c_uint64)]


_lib = None


def _nccl_path():
    try:
        import nvidia.nccl  # type: ignore
        for d in nvidia.nccl.__path__:
            p = os.path.join(d, "lib", "libnccl.so.2")
            if os.path.exists(p):
                return p
    except Exception:
        pass
    return None


def lib():
    """Load (building first when missing) the native library."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        from . import build as _build
        _build.build()
    if "HCCL_NCCL_LIB" not in os.environ:
        p = _nccl_path()
        if p:
            os.environ["HCCL_NCCL_LIB"] = p
    L = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    vp, u32, u64, i32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int32
    P = C.POINTER
    sigs = {
        "HcclGetRootInfo": [P(RootInfo)],
        "HcclCommInitRootInfo": [u32, P(RootInfo), u32, P(vp)],
        "HcclCommInitRootInfoConfig": [u32, P(RootInfo), u32, P(CommConfig), P(vp)],
        "HcclCommInitClusterInfo": [C.c_char_p, u32, P(vp)],
        "HcclCommInitClusterInfoConfig": [C.c_char_p, u32, P(CommConfig), P(vp)],
        "HcclCommInitAll": [u32, P(i32), P(vp)],
        "HcclCreateSubCommConfig": [P(vp), u32, P(u32), u64, u32, P(CommConfig), P(vp)],
        "HcclCommDestroy": [vp],
        "HcclSetConfig": [C.c_int, i32],
        "HcclGetConfig": [C.c_int, P(i32)],
        "HcclGetCommName": [vp, C.c_char_p],
        "HcclGetRankSize": [vp, P(u32)],
        "HcclGetRankId": [vp, P(u32)],
        "HcclGetCommAsyncError": [vp, P(C.c_int)],
        "HcclAllReduce": [vp, vp, u64, C.c_int, C.c_int, vp, vp],
        "HcclBroadcast": [vp, u64, C.c_int, u32, vp, vp],
        "HcclReduceScatter": [vp, vp, u64, C.c_int, C.c_int, vp, vp],
        "HcclReduceScatterV": [vp, vp, vp, vp, u64, C.c_int, C.c_int, vp, vp],
        "HcclScatter": [vp, vp, u64, C.c_int, u32, vp, vp],
        "HcclGather": [vp, vp, u64, C.c_int, u32, vp, vp],
        "HcclAllGather": [vp, vp, u64, C.c_int, vp, vp],
        "HcclAllGatherV": [vp, u64, vp, vp, vp, C.c_int, vp, vp],
        "HcclBarrier": [vp, vp],
        "HcclSend": [vp, u64, C.c_int, u32, vp, vp],
        "HcclRecv": [vp, u64, C.c_int, u32, vp, vp],
        "HcclAlltoAllV": [vp, vp, vp, C.c_int, vp, vp, vp, C.c_int, vp, vp],
        "HcclAlltoAllVC": [vp, vp, C.c_int, vp, C.c_int, vp, vp],
        "HcclAlltoAll": [vp, u64, C.c_int, vp, u64, C.c_int, vp, vp],
        "HcclReduce": [vp, vp, u64, C.c_int, C.c_int, u32, vp, vp],
        "HcclBatchSendRecv": [P(SendRecvItem), u32, vp, vp],
        "HcclCommSuspend": [vp],
        "HcclCommResume": [vp],
        "HcclCommSetMemoryRange": [vp, vp, C.c_size_t, C.c_size_t, u64],
        "HcclCommUnsetMemoryRange": [vp, vp],
        "HcclCommActivateCommMemory": [vp, vp, C.c_size_t, C.c_size_t, vp, u64],
        "HcclCommDeactivateCommMemory": [vp, vp],
        "HcclB200CommInitLocal": [u32, C.c_int, C.c_int, P(CommConfig), P(vp)],
        "HcclB200Collective": [vp, P(B200Op), P(vp), P(vp), vp],
        "HcclB200Repeat": [vp, P(B200Op), P(vp), P(vp), u32, u64, u32, vp],
        "HcclB200NcclAllReduceRepeat": [vp, vp, vp, u64, C.c_int, C.c_int, u32, u64, u32, vp],
        "HcclB200LocalSendRecv": [vp, u32, u32, vp, vp, u64, C.c_int, vp],
        "HcclB200StreamSync": [vp, vp],
        "HcclB200GetStatus": [vp, u32, P(B200Status)],
        "HcclB200MoeCount": [vp, C.c_int64, i32, vp, vp, vp],
        "HcclB200MoeOffsets": [vp, i32, i32, i32, vp, vp, vp, C.c_int64, vp, vp],
        "HcclB200MoeDispatch": [vp, vp, vp, vp, C.c_int64, i32, i32, i32, i32, i32, i32, P(vp), vp, C.c_int64, vp],
        "HcclB200MoeCombine": [P(vp), vp, vp, vp, C.c_int64, i32, i32, i32, i32, i32, i32, vp, C.c_int64, vp],
        "HcclB200GemmBf16": [vp, vp, vp, i32, i32, i32, vp],
        "HcclB200GemmLaunchCounts": [P(u64), P(u64)],
        "HcclB200AllGatherMatmul": [vp, P(vp), P(vp), P(vp), i32, i32, i32, vp],
        "HcclB200MatmulReduceScatter": [vp, P(vp), P(vp), P(vp), i32, i32, i32, vp],
        "HcclB200GetKernelTrace": [vp, u32, P(u64), C.c_size_t, P(i32)],
        "HcclB200WaitProbe": [vp, u32, C.c_double, vp],
        "HcclB200DescribeStatus": [vp, u32, C.c_char_p, C.c_size_t],
        "HcclB200Select": [vp, i32, u64, C.c_int, C.c_int, P(i32), P(i32), P(C.c_double)],
        "HcclB200GetStatsJson": [vp, C.c_char_p, C.c_size_t],
        "HcclB200GetTraceJson": [vp, C.c_char_p, C.c_size_t],
        "HcclB200Calibrate": [vp, vp],
        "HcclB200SetCostModel": [vp, C.c_double, C.c_double, C.c_double, C.c_double, C.c_double],
        "HcclB200HasNvls": [vp, P(i32)],
        "HcclB200GetLocalRankNum": [vp, P(u32)],
        "HcclB200MemAlloc": [vp, C.c_size_t, P(vp), P(i32)],
        "HcclB200MemAdopt": [vp, P(vp), C.c_size_t, P(u64), C.c_size_t, P(i32)],
        "HcclB200MemFree": [vp, i32],
        "HcclB200MemQuery": [vp, i32, P(vp), P(vp), P(C.c_size_t)],
        "HcclB200Exchange": [vp, C.c_char_p, vp, C.c_size_t, vp],
        "HcclB200GetDeviceContext": [vp, P(vp), P(u64)],
        "HcclB200ReloadEnv": [],
        "HcclB200PoolBind": [vp],
        "HcclB200PlanCheck": [i32, i32, u32, u64, C.c_int, u32, u64, i32, C.c_int64, C.c_char_p, C.c_size_t],
        "HcclB200PlanRaceCheck": [i32, i32, u32, u64, C.c_int, u32, u32, i32, i32, i32, C.c_char_p, C.c_size_t],
        "HcclB200Put": [vp, u32, i32, u32, C.c_size_t, vp, C.c_size_t, vp],
        "HcclB200Get": [vp, u32, i32, u32, C.c_size_t, vp, C.c_size_t, vp],
        "HcclB200GetTopoJson": [vp, C.c_char_p, C.c_size_t],
        "HcclB200GetOverflowCount": [vp, P(u64)],
        "HcclGetTopoDesc": [vp, P(TopoDescs), u32],
        "HcomInitByFile": [C.c_char_p, C.c_char_p],
        "HcomInitByComm": [vp],
        "HcomDestroy": [],
        "HcomCreateGroup": [C.c_char_p, u32, P(u32)],
        "HcomDestroyGroup": [C.c_char_p],
        "HcomGetRankSize": [C.c_char_p, P(u32)],
        "HcomGetRankId": [C.c_char_p, P(u32)],
        "HcomGetWorldRankFromGroupRank": [C.c_char_p, u32, P(u32)],
        "HcomGetGroupRankFromWorldRank": [u32, C.c_char_p, P(u32)],
        "HcomGetCommHandleByGroup": [C.c_char_p, P(vp)],
        "HcomGetTopoDesc": [C.c_char_p, P(TopoDescs), u32],
        "HcomSetGradFusionByIndex": [C.c_char_p, u32, P(u32)],
        "HcomSetGradFusionBySize": [C.c_char_p, u32, P(C.c_float)],
        "HcomGetGradFusionByIndex": [C.c_char_p, P(u32), P(u32)],
        "HcomGetGradFusionBySize": [C.c_char_p, P(u32), P(C.c_float)],
    }
    for name, args in sigs.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = C.c_int
    L.HcclGetErrorString.argtypes = [C.c_int]
    L.HcclGetErrorString.restype = C.c_char_p
    L.HcclB200GetLastError.argtypes = []
    L.HcclB200GetLastError.restype = C.c_char_p
    L.HcclB200AlgoName.argtypes = [i32]
    L.HcclB200AlgoName.restype = C.c_char_p
    L.HcclGetCommConfigCapability.argtypes = []
    L.HcclGetCommConfigCapability.restype = C.c_uint32
    _lib = L
    return L


class HcclError(RuntimeError):
    def __init__(self, code, where):
        L = lib()
        self.code = int(code)
        detail = L.HcclB200GetLastError().decode(errors="replace")
        super().__init__("%s failed: %s (%d)%s" % (where, L.HcclGetErrorString(code).decode(), code,
                                                   (": " + detail) if detail else ""))


def check(code, where):
    if code != SUCCESS:
        raise HcclError(code, where)
