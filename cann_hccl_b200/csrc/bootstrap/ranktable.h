// Rank-table file loader for HcclCommInitClusterInfo.  One concise format is supported
// (reference: framework/common/src/topo/topoinfo_ranktableConcise.cc:203-860; key names from
// framework/inc/topoinfo_struct.h:122-160):
//   {"version":"1.0","status":"completed","server_count":"1",
//    "server_list":[{"server_id":"10.0.0.1","host_ip":"10.0.0.1","host_port":"60000",
//                    "device":[{"device_id":"0","rank_id":"0"}, ...]}]}
// All ranks must live on one server (one NVSwitch domain).  host_ip/host_port name where rank 0 runs the hub.
#pragma once
#include <string>
#include <vector>
#include "hccl/hccl_types.h"
namespace hcclb {
struct RankEntry { int rank_id = -1; int device_id = -1; std::string server_id; };
struct RankTable {
    std::vector<RankEntry> ranks;  // sorted by rank_id, dense 0..n-1
    std::string host_ip = "127.0.0.1";
    int host_port = 0;             // 0: HCCL_IF_BASE_PORT
    uint32_t crc = 0;              // CRC32 of the file text: all ranks must load the same table
};
HcclResult parse_ranktable(const std::string &json_text, RankTable *out, std::string *err);
HcclResult load_ranktable_file(const char *path, RankTable *out, std::string *err);
// Sub-table with the listed ranks renumbered 0..k-1 (reference: topoinfo_ranktable_partition.cc).
HcclResult partition_ranktable(const RankTable &t, const std::vector<uint32_t> &rank_ids, RankTable *out);
}  // namespace hcclb
