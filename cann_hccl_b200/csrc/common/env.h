// Environment configuration, parsed once per process (reference tiers: closed InitExternalInput +
// framework/common/src/config/env_config.cc).  Every knob listed here is honoured somewhere in the
// library; the RDMA class/level and socket-port-range knobs are parsed and range-checked for API
// fidelity only (a single NVSwitch domain has no RoCE plane).
#pragma once
#include <map>
#include <string>
#include "hccl/hccl_types.h"
namespace hcclb {
struct EnvConfig {
    std::map<std::string, std::string> algo;  // HCCL_ALGO: "allreduce=ring;allgather=mesh" or a bare name for all ops
    uint32_t buffsize_mb = HCCL_COMM_DEFAULT_BUFFSIZE;  // HCCL_BUFFSIZE (MB per staging direction)
    bool buffsize_set = false;
    int deterministic = -1;        // HCCL_DETERMINISTIC: -1 unset, 0/1
    int expansion_mode = 0;        // HCCL_OP_EXPANSION_MODE: 0 auto, 1 HOST, 2 AI_CPU, 3 AIV(device kernels)
    int connect_timeout_s = 120;   // HCCL_CONNECT_TIMEOUT
    int exec_timeout_s = 1836;     // HCCL_EXEC_TIMEOUT (HCCL default 1836 s)
    double exec_timeout_ms = -1;   // HCCL_EXEC_TIMEOUT_MS overrides (tests use milliseconds)
    int if_base_port = 60000;      // HCCL_IF_BASE_PORT
    std::string if_ip;             // HCCL_IF_IP
    int socket_family = 4;         // HCCL_SOCKET_FAMILY: AF_INET / AF_INET6 -> 4 / 6
    bool retry_enable = false;     // HCCL_OP_RETRY_ENABLE ("L0:1" or "1")
    int retry_max = 3;             // HCCL_OP_RETRY_PARAMS MaxCnt
    int retry_hold_ms = 5000;      // ... HoldTime
    int retry_interval_ms = 1000;  // ... IntervalTime
    bool entry_log = false;        // HCCL_ENTRY_LOG_ENABLE
    bool op_counter = true;        // HCCL_OP_COUNTER
    int nvls_enable = -1;          // HCCL_NVLS_ENABLE: -1 auto, 0 off, 1 force
    std::string transport;         // HCCL_TRANSPORT: "", "host", "p2p"
    std::string fault_inject;      // HCCL_FAULT_INJECT (host side only)
    int rdma_tc = 132;             // HCCL_RDMA_TC (0..255, multiple of 4)
    int rdma_sl = 4;               // HCCL_RDMA_SL (0..7)
    int port_range_lo = 0, port_range_hi = 0;  // HCCL_HOST_SOCKET_PORT_RANGE "lo-hi"
    int heartbeat_ms = 50;         // HCCL_HEARTBEAT_INTERVAL_MS (reference BROADCAST_INTERVAL 50 ms)
    int stuck_ms = 300000;         // HCCL_STUCK_DETECT_TIME (seconds in env; reference STUCK_INTERVAL 300 s)
    int heartbeat_lost_ms = 3000;  // HCCL_HEARTBEAT_LOST_MS: silence after which a peer counts as lost
    bool plan_race_check = false;  // HCCL_PLAN_RACE_CHECK=1: every plan goes through the static race check (algo/racecheck.cc) when it is built
    int a2av_check = -1;           // HCCL_ALLTOALLV_CHECK: count-matrix cross-check of AlltoAllV/VC: 1 every call, 0 never, unset = the first 16 calls
    bool calibrate = true;         // HCCL_CALIBRATE=0: device communicators skip the measurement pass at creation
    int calibrate_max_mb = 0;      // HCCL_CALIBRATE_MAX_MB: largest message of the calibration ladder (0 = 64)
    int channels = 0;              // HCCL_CHANNELS: force CTAs per op (0 = selector decides)
    uint64_t pipe_chunk_bytes = 0; // HCCL_PIPE_CHUNK_KB: bytes a chunk of the pipelined large-message kernels moves over the links (0 = by message size)
    int pipe_slots = 0;            // HCCL_PIPE_SLOTS: ring depth of the pipelined kernels (0 = default, at most 16)
    int pipe_ctas[3] = {0, 0, 0};  // HCCL_PIPE_CTAS "a,b,c": CTAs of the copy-in / transfer / copy-out stage (0 = default)
    int pipe_groups[3] = {0, 0, 0};  // HCCL_PIPE_GROUPS "a,b,c": groups per stage that take chunks in turn (0 = default)
    bool tp_gemm_pair = true;      // HCCL_TP_GEMM_PAIR=0: fused GEMM kernels on single CTAs only (default: clusters of two CTAs on 256 x 256 tiles, tcgen05 cta_group::2, where the shape allows)
    std::string ncc_lib;           // HCCL_NCCL_LIB: path of libnccl.so.2 for Send/Recv
    bool whitelist_enable = false; // HCCL_WHITELIST_DISABLE=0 switches the connection whitelist on (HCCL convention: 1 = off, the default)
    std::string whitelist_file;    // HCCL_WHITELIST_FILE: JSON {"host_ip": ["a.b.c.d", ...]} of addresses that may connect to the bootstrap hub
    bool nvtx = false;             // HCCL_NVTX: NVTX range around every API-level operation
    bool overflow_check = false;   // HCCL_OVERFLOW_CHECK: scan the output of floating-point reductions for Inf / NaN
    std::string stats_dump;        // HCCL_STATS_DUMP: file that receives the statistics JSON when a communicator is destroyed
    bool valid = true;
    std::string error;             // first parse error, if any
};
// Parse (or re-parse when `force`) the environment.  Invalid values mark cfg.valid=false and keep defaults.
const EnvConfig &env_config(bool force = false);
// Parse helper exposed for tests: fills cfg from an explicit name->value map instead of getenv.
EnvConfig parse_env(const std::map<std::string, std::string> &vars);
}  // namespace hcclb
