// Symmetric memory: an allocation of the same size on every rank with every peer's copy mapped into the local
// address space (and, on NVSwitch systems, one multicast mapping over all copies).  This is the B200 counterpart
// of the reference's TransportManager link set-up plus CCL buffer manager (framework/communicator/impl/
// resource_manager/transport_manager.cc:330-455, algorithm/impl/resource_manager/ccl_buffer_manager.cc):
// instead of per-link transports, kernels get a table of peer base pointers.
//
// Back ends:
//   host-local   : all ranks in one process, plain heap memory (emulated ranks, unit tests)
//   host-shm     : one rank per process / thread, POSIX shared memory named through the hub
//   device-local : all ranks are virtual ranks on one GPU (single-GPU emulation of the multi-rank kernels)
//   device-vmm   : one rank per GPU; cuMemCreate + POSIX fd export (SCM_RIGHTS over a unix socket) + cuMemMap of
//                  every peer, optional cuMulticast object bound over all copies; falls back to CUDA IPC handles
#pragma once
#include <string>
#include <vector>
#include "bootstrap/hub.h"
#include "common/base.h"

namespace hcclb {

struct SymSegment {
    size_t bytes = 0;
    uint8_t *peer[kMaxRanks] = {nullptr};  // peer[q] = rank q's copy as seen from this rank
    uint8_t *mc = nullptr;                 // multicast mapping or null
    // bookkeeping for release
    unsigned long long handles[kMaxRanks] = {0};
    unsigned long long mc_handle = 0;
    size_t map_bytes = 0;
    int kind = 0;                          // back-end specific; kSegAdopted* = caller-owned memory
    std::string shm_name;
};

constexpr int kSegAdoptedLocal = 9;  // caller-owned, peers in the same process: nothing to undo
constexpr int kSegAdoptedVmm = 3;    // caller-owned VMM allocation mapped by the peers

class SymAllocator {
public:
    virtual ~SymAllocator() {}
    // Collective over all ranks of the communicator.  out->size() == number of local ranks.
    virtual HcclResult alloc(size_t bytes, bool want_mc, std::vector<SymSegment> *out) = 0;
    // Registers memory that the caller owns and keeps (one pointer per local rank, `bytes` each) as a symmetric segment, so
    // that peers can reach it like memory from alloc().  Collective.  Back ends whose ranks share a process record the
    // pointers; the one-rank-per-GPU back end needs the driver allocation handle behind the pointer (created exportable as a
    // POSIX file descriptor; the registered memory is the whole allocation: `handle_offset` 0 and `bytes` its size, because the
    // driver maps allocations only as a whole) and maps it on every peer.  release() undoes the registration and leaves the memory alone.
    virtual HcclResult adopt(void *const *local_ptrs, size_t bytes, const unsigned long long *drv_handles, size_t handle_offset,
                             bool want_mc, std::vector<SymSegment> *out)
    {
        (void)local_ptrs; (void)bytes; (void)drv_handles; (void)handle_offset; (void)want_mc; (void)out;
        return HCCL_E_NOT_SUPPORT;
    }
    virtual void release(std::vector<SymSegment> *segs) = 0;
    virtual bool is_device() const = 0;
    virtual bool has_multicast() const { return false; }
};

SymAllocator *make_host_local_allocator(int nranks);
SymAllocator *make_host_shm_allocator(HubClient *hub, const std::string &ident, int rank, int nranks, int timeout_ms);
SymAllocator *make_device_local_allocator(int nranks, int device);
SymAllocator *make_device_vmm_allocator(HubClient *hub, const std::string &ident, int rank, int nranks, int device,
                                        bool want_nvls, int timeout_ms);

}  // namespace hcclb
