// NVLink / NVSwitch attributes of a GPU, read from the management library (NVML, loaded with dlopen; HCCL_NVML_LIB names
// another library, which is how the tests substitute a fake).  Role of the reference's attribute collector
// (framework/communicator/impl/hccl_communicator_attrs.cc:1227-1262: device type, link kinds, mesh / switch layout).
// Nothing is changed on the device: every call is a query.
#pragma once
#include <string>
#include "common/base.h"
namespace hcclb {
struct LinkTopo {
    bool probed = false;        // false: the management library was not found or a query failed; the fields keep defaults
    int links_total = 0;        // NVLink ports the device reports
    int links_active = 0;
    int links_to_switch = 0;    // active links whose far end is an NVSwitch
    int nvlink_version = 0;     // NVML numbering: 6 = NVLink 4, 7 = NVLink 5
    double link_gbps = 0;       // per link and direction, from the version (and the speed field when the driver offers it)
    bool multicast = false;     // the driver can create multicast objects on this device (NVLS)
    std::string name;
    double egress_gbps() const { return links_active * link_gbps; }  // nominal per direction
};
// `device`: CUDA ordinal (its PCI bus id selects the NVML handle); pci_bus_id "" = use the ordinal as NVML index.
LinkTopo probe_links(int device, const std::string &pci_bus_id);
std::string link_topo_json(const LinkTopo &t);
}  // namespace hcclb
