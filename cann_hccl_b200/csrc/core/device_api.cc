#include "core/device_api.h"
#include <mutex>
#include "common/log.h"
namespace hcclb {
template <class F>
static bool load(const char *name, F *fn)
{
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
        (void)cudaGetLastError();
        return false;
    }
    *fn = (F)p;
    return true;
}
const DriverApi &driver_api()
{
    static DriverApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        int n = 0;
        if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
            (void)cudaGetLastError();
            return;
        }
        bool ok = true;
        ok &= load("cuMemCreate", &api.MemCreate);
        ok &= load("cuMemRelease", &api.MemRelease);
        ok &= load("cuMemAddressReserve", &api.MemAddressReserve);
        ok &= load("cuMemAddressFree", &api.MemAddressFree);
        ok &= load("cuMemMap", &api.MemMap);
        ok &= load("cuMemUnmap", &api.MemUnmap);
        ok &= load("cuMemSetAccess", &api.MemSetAccess);
        ok &= load("cuMemExportToShareableHandle", &api.MemExportToShareableHandle);
        ok &= load("cuMemImportFromShareableHandle", &api.MemImportFromShareableHandle);
        ok &= load("cuMemGetAllocationGranularity", &api.MemGetAllocationGranularity);
        ok &= load("cuDeviceGet", &api.DeviceGet);
        ok &= load("cuDeviceGetAttribute", &api.DeviceGetAttribute);
        ok &= load("cuGetErrorString", &api.GetErrorString);
        ok &= load("cuTensorMapEncodeTiled", &api.TensorMapEncodeTiled);
        // multicast entry points are optional (absent => no NVLS)
        if (!load("cuMulticastCreate", &api.MulticastCreate) || !load("cuMulticastAddDevice", &api.MulticastAddDevice) ||
            !load("cuMulticastBindMem", &api.MulticastBindMem) || !load("cuMulticastUnbind", &api.MulticastUnbind) ||
            !load("cuMulticastGetGranularity", &api.MulticastGetGranularity))
            api.MulticastCreate = nullptr;
        api.ok = ok;
        if (!ok) HLOG_WARN("CUDA driver entry points unavailable; device transport disabled");
    });
    return api;
}
const char *cu_err(CUresult r)
{
    const char *s = "unknown";
    if (driver_api().GetErrorString) driver_api().GetErrorString(r, &s);
    return s ? s : "unknown";
}
}  // namespace hcclb
