#include "core/topo_probe.h"
#include <dlfcn.h>
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <sstream>
#include "common/log.h"

namespace hcclb {

namespace {
typedef void *nvmlDev;
constexpr int kMaxLinks = 32;
constexpr unsigned kFieldSpeedMbpsCommon = 90;  // NVML_FI_DEV_NVLINK_SPEED_MBPS_COMMON
constexpr unsigned kRemoteSwitch = 1;           // NVML_NVLINK_DEVICE_TYPE_SWITCH
struct FieldValue {   // nvmlFieldValue_t
    unsigned fieldId, scopeId;
    long long timestamp, latencyUsec;
    unsigned valueType, nvmlReturn;
    union { double d; unsigned ui; unsigned long ul; unsigned long long ull; long long sll; } value;
};
struct Nvml {
    void *lib = nullptr;
    int (*init)() = nullptr;
    int (*by_index)(unsigned, nvmlDev *) = nullptr;
    int (*by_pci)(const char *, nvmlDev *) = nullptr;
    int (*name)(nvmlDev, char *, unsigned) = nullptr;
    int (*link_state)(nvmlDev, unsigned, unsigned *) = nullptr;
    int (*link_version)(nvmlDev, unsigned, unsigned *) = nullptr;
    int (*link_remote)(nvmlDev, unsigned, unsigned *) = nullptr;
    int (*fields)(nvmlDev, int, FieldValue *) = nullptr;
};
bool load(Nvml &n)
{
    const char *path = getenv("HCCL_NVML_LIB");
    n.lib = dlopen(path && *path ? path : "libnvidia-ml.so.1", RTLD_NOW | RTLD_LOCAL);
    if (!n.lib) return false;
    auto sym = [&](const char *s) { return dlsym(n.lib, s); };
    n.init = (int (*)())sym("nvmlInit_v2");
    n.by_index = (int (*)(unsigned, nvmlDev *))sym("nvmlDeviceGetHandleByIndex_v2");
    n.by_pci = (int (*)(const char *, nvmlDev *))sym("nvmlDeviceGetHandleByPciBusId_v2");
    n.name = (int (*)(nvmlDev, char *, unsigned))sym("nvmlDeviceGetName");
    n.link_state = (int (*)(nvmlDev, unsigned, unsigned *))sym("nvmlDeviceGetNvLinkState");
    n.link_version = (int (*)(nvmlDev, unsigned, unsigned *))sym("nvmlDeviceGetNvLinkVersion");
    n.link_remote = (int (*)(nvmlDev, unsigned, unsigned *))sym("nvmlDeviceGetNvLinkRemoteDeviceType");
    n.fields = (int (*)(nvmlDev, int, FieldValue *))sym("nvmlDeviceGetFieldValues");
    return n.init && n.by_index && n.link_state;
}
double gbps_of_version(int v)
{
    if (v >= 7) return 50.0;   // NVLink 5: 18 links x 50 GB/s = 900 GB/s per direction
    if (v >= 4) return 25.0;   // NVLink 3 / 4
    return v > 0 ? 20.0 : 0.0;
}
}  // namespace

LinkTopo probe_links(int device, const std::string &pci_bus_id)
{
    LinkTopo t;
    Nvml n;
    if (!load(n)) return t;
    // the library stays loaded (NVML keeps process-wide state); nvmlShutdown is left to process exit
    if (n.init() != 0) return t;
    nvmlDev dev = nullptr;
    int rc = !pci_bus_id.empty() && n.by_pci ? n.by_pci(pci_bus_id.c_str(), &dev) : n.by_index((unsigned)device, &dev);
    if (rc != 0 || !dev) return t;
    char nm[96] = {0};
    if (n.name && n.name(dev, nm, sizeof(nm)) == 0) t.name = nm;
    for (unsigned l = 0; l < kMaxLinks; ++l) {
        unsigned active = 0;
        if (n.link_state(dev, l, &active) != 0) break;  // past the last port
        t.links_total++;
        if (!active) continue;
        t.links_active++;
        unsigned ver = 0, remote = 0;
        if (n.link_version && n.link_version(dev, l, &ver) == 0) t.nvlink_version = std::max(t.nvlink_version, (int)ver);
        if (n.link_remote && n.link_remote(dev, l, &remote) == 0 && remote == kRemoteSwitch) t.links_to_switch++;
    }
    t.link_gbps = gbps_of_version(t.nvlink_version);
    if (n.fields && t.links_active) {
        FieldValue fv;
        memset(&fv, 0, sizeof(fv));
        fv.fieldId = kFieldSpeedMbpsCommon;
        if (n.fields(dev, 1, &fv) == 0 && fv.nvmlReturn == 0 && fv.value.ui > 0) t.link_gbps = fv.value.ui / 1000.0;  // MB/s per direction
    }
    t.probed = true;
    return t;
}

std::string link_topo_json(const LinkTopo &t)
{
    std::ostringstream o;
    o << "{\"probed\":" << (t.probed ? "true" : "false") << ",\"name\":\"" << t.name << "\",\"links_total\":" << t.links_total
      << ",\"links_active\":" << t.links_active << ",\"links_to_switch\":" << t.links_to_switch << ",\"nvlink_version\":" << t.nvlink_version
      << ",\"link_gbps_per_direction\":" << t.link_gbps << ",\"egress_gbps\":" << t.egress_gbps() << ",\"nvswitch\":" << (t.links_to_switch > 0 ? "true" : "false")
      << ",\"multicast\":" << (t.multicast ? "true" : "false") << "}";
    return o.str();
}

}  // namespace hcclb
