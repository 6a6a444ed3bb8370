#include "core/symmem.h"
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <thread>
#include "bootstrap/socket.h"
#include "common/log.h"
#include "core/device_api.h"

namespace hcclb {
namespace {

std::atomic<uint64_t> g_alloc_seq{0};

// ---------------------------------------------------------------- host, all ranks local
class HostLocal : public SymAllocator {
public:
    explicit HostLocal(int n) : n_(n) {}
    HcclResult alloc(size_t bytes, bool, std::vector<SymSegment> *out) override
    {
        std::vector<uint8_t *> mem(n_);
        for (int r = 0; r < n_; ++r) {
            void *p = nullptr;
            if (posix_memalign(&p, 4096, bytes) != 0) return HCCL_E_MEMORY;
            memset(p, 0, bytes);
            mem[r] = (uint8_t *)p;
        }
        out->assign(n_, SymSegment());
        for (int r = 0; r < n_; ++r) {
            (*out)[r].bytes = bytes;
            for (int q = 0; q < n_; ++q) (*out)[r].peer[q] = mem[q];
        }
        return HCCL_SUCCESS;
    }
    HcclResult adopt(void *const *local_ptrs, size_t bytes, const unsigned long long *, size_t, bool, std::vector<SymSegment> *out) override
    {
        out->assign(n_, SymSegment());
        for (int r = 0; r < n_; ++r) {
            (*out)[r].bytes = bytes;
            (*out)[r].kind = kSegAdoptedLocal;
            for (int q = 0; q < n_; ++q) (*out)[r].peer[q] = (uint8_t *)local_ptrs[q];
        }
        return HCCL_SUCCESS;
    }
    void release(std::vector<SymSegment> *segs) override
    {
        if (!segs->empty() && (*segs)[0].kind != kSegAdoptedLocal)
            for (int q = 0; q < n_; ++q) free((*segs)[0].peer[q]);
        segs->clear();
    }
    bool is_device() const override { return false; }

private:
    int n_;
};

// ---------------------------------------------------------------- host, POSIX shared memory
class HostShm : public SymAllocator {
public:
    HostShm(HubClient *hub, std::string ident, int rank, int n, int tmo) : hub_(hub), ident_(std::move(ident)), rank_(rank), n_(n), tmo_(tmo) {}
    HcclResult alloc(size_t bytes, bool, std::vector<SymSegment> *out) override
    {
        uint64_t seq = seq_++;
        auto name_of = [&](int r) { return "/hcclb-" + ident_ + "-" + std::to_string(seq) + "-" + std::to_string(r); };
        std::string mine = name_of(rank_);
        int fd = shm_open(mine.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
        if (fd < 0 || ftruncate(fd, (off_t)bytes) != 0) {
            HLOG_ERROR("shm_open/ftruncate %s (%zu bytes) failed", mine.c_str(), bytes);
            if (fd >= 0) close(fd);
            return HCCL_E_MEMORY;
        }
        void *p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
        close(fd);
        if (p == MAP_FAILED) return HCCL_E_MEMORY;
        memset(p, 0, bytes);
        SymSegment s;
        s.bytes = bytes;
        s.peer[rank_] = (uint8_t *)p;
        s.shm_name = mine;
        HcclResult rc = hub_->barrier(ident_ + "/shm-created/" + std::to_string(seq), n_, rank_, tmo_);
        if (rc == HCCL_SUCCESS) {
            for (int q = 0; q < n_ && rc == HCCL_SUCCESS; ++q) {
                if (q == rank_) continue;
                int pfd = shm_open(name_of(q).c_str(), O_RDWR, 0600);
                void *pp = pfd >= 0 ? mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, pfd, 0) : MAP_FAILED;
                if (pfd >= 0) close(pfd);
                if (pp == MAP_FAILED) {
                    HLOG_ERROR("cannot map shared segment of rank %d", q);
                    rc = HCCL_E_MEMORY;
                } else s.peer[q] = (uint8_t *)pp;
            }
        }
        HcclResult rc2 = hub_->barrier(ident_ + "/shm-mapped/" + std::to_string(seq), n_, rank_, tmo_);
        shm_unlink(mine.c_str());  // mappings stay valid; the name never outlives the communicator
        if (rc == HCCL_SUCCESS) rc = rc2;
        out->assign(1, s);
        if (rc != HCCL_SUCCESS) release(out);
        return rc;
    }
    void release(std::vector<SymSegment> *segs) override
    {
        for (auto &s : *segs)
            for (int q = 0; q < n_; ++q)
                if (s.peer[q]) munmap(s.peer[q], s.bytes);
        segs->clear();
    }
    bool is_device() const override { return false; }

private:
    HubClient *hub_;
    std::string ident_;
    int rank_, n_, tmo_;
    uint64_t seq_ = 0;
};

// ---------------------------------------------------------------- device, virtual ranks on one GPU
class DeviceLocal : public SymAllocator {
public:
    DeviceLocal(int n, int dev) : n_(n), dev_(dev) {}
    HcclResult alloc(size_t bytes, bool, std::vector<SymSegment> *out) override
    {
        if (cudaSetDevice(dev_) != cudaSuccess) return HCCL_E_RUNTIME;
        std::vector<uint8_t *> mem(n_);
        for (int r = 0; r < n_; ++r) {
            void *p = nullptr;
            if (cudaMalloc(&p, bytes) != cudaSuccess) {
                HLOG_ERROR("cudaMalloc of %zu bytes failed", bytes);
                return HCCL_E_MEMORY;
            }
            cudaMemset(p, 0, bytes);
            mem[r] = (uint8_t *)p;
        }
        cudaDeviceSynchronize();
        out->assign(n_, SymSegment());
        for (int r = 0; r < n_; ++r) {
            (*out)[r].bytes = bytes;
            for (int q = 0; q < n_; ++q) (*out)[r].peer[q] = mem[q];
        }
        return HCCL_SUCCESS;
    }
    HcclResult adopt(void *const *local_ptrs, size_t bytes, const unsigned long long *, size_t, bool, std::vector<SymSegment> *out) override
    {
        out->assign(n_, SymSegment());
        for (int r = 0; r < n_; ++r) {
            (*out)[r].bytes = bytes;
            (*out)[r].kind = kSegAdoptedLocal;
            for (int q = 0; q < n_; ++q) (*out)[r].peer[q] = (uint8_t *)local_ptrs[q];
        }
        return HCCL_SUCCESS;
    }
    void release(std::vector<SymSegment> *segs) override
    {
        if (!segs->empty() && (*segs)[0].kind != kSegAdoptedLocal)
            for (int q = 0; q < n_; ++q) cudaFree((*segs)[0].peer[q]);
        segs->clear();
    }
    bool is_device() const override { return true; }

private:
    int n_, dev_;
};

// ---------------------------------------------------------------- device, one rank per GPU
class DeviceVmm : public SymAllocator {
public:
    DeviceVmm(HubClient *hub, std::string ident, int rank, int n, int dev, bool nvls, int tmo)
        : hub_(hub), ident_(std::move(ident)), rank_(rank), n_(n), dev_(dev), want_nvls_(nvls), tmo_(tmo)
    {
        lsock_ = net::unix_listen(sock_name(rank_));
        const DriverApi &d = driver_api();
        if (d.ok) {
            CUdevice cd;
            int v = 0;
            if (d.DeviceGet(&cd, dev_) == CUDA_SUCCESS) {
                if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, cd) == CUDA_SUCCESS) vmm_ok_ = v != 0;
                v = 0;
                if (d.MulticastCreate && d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cd) == CUDA_SUCCESS) mc_ok_ = v != 0;
            }
        }
        if (lsock_ < 0) vmm_ok_ = false;
    }
    ~DeviceVmm() override { net::close_fd(lsock_); }
    bool is_device() const override { return true; }
    bool has_multicast() const override { return mc_live_; }

    HcclResult alloc(size_t bytes, bool want_mc, std::vector<SymSegment> *out) override
    {
        if (cudaSetDevice(dev_) != cudaSuccess) return HCCL_E_RUNTIME;
        uint64_t seq = seq_++;
        // agree on the path: every rank must be able to use fd-exported VMM memory, else all use CUDA IPC
        std::vector<std::string> caps;
        std::string cap(2, 0);
        cap[0] = vmm_ok_ ? 1 : 0;
        cap[1] = (mc_ok_ && want_nvls_ && want_mc) ? 1 : 0;
        CHK_RET(hub_->rendezvous(ident_ + "/symcaps/" + std::to_string(seq), n_, rank_, cap, &caps, tmo_));
        bool use_vmm = true, use_mc = n_ > 1;
        for (auto &c : caps) { use_vmm &= c[0] != 0; use_mc &= c[1] != 0; }
        out->assign(1, SymSegment());
        SymSegment &s = (*out)[0];
        HcclResult rc = use_vmm ? alloc_vmm(bytes, use_mc, seq, &s) : alloc_ipc(bytes, seq, &s);
        if (rc != HCCL_SUCCESS) out->clear();
        return rc;
    }

    HcclResult adopt(void *const *local_ptrs, size_t bytes, const unsigned long long *drv_handles, size_t handle_offset, bool want_mc,
                     std::vector<SymSegment> *out) override
    {
        if (cudaSetDevice(dev_) != cudaSuccess) return HCCL_E_RUNTIME;
        uint64_t seq = seq_++;
        // every rank states whether it can take part (exportable handle given, size on the allocation granularity) and its
        // size, so that all ranks return the same verdict instead of some waiting for a peer that gave up
        const DriverApi &d = driver_api();
        size_t gran = 2u << 20;
        if (d.ok) {
            CUmemAllocationProp prop;
            memset(&prop, 0, sizeof(prop));
            prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
            prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
            prop.location.id = dev_;
            prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
            d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM);
        }
        struct { uint32_t ok, mc; uint64_t bytes; } me_v{0, 0, bytes};
        me_v.ok = vmm_ok_ && drv_handles && drv_handles[0] && local_ptrs && local_ptrs[0] && bytes && bytes % gran == 0 && handle_offset == 0;
        me_v.mc = mc_ok_ && want_nvls_ && want_mc;
        std::vector<std::string> all;
        CHK_RET(hub_->rendezvous(ident_ + "/adoptcaps/" + std::to_string(seq), n_, rank_, std::string((const char *)&me_v, sizeof(me_v)), &all, tmo_));
        bool ok = true, use_mc = n_ > 1;
        for (auto &blob : all) {
            decltype(me_v) o;
            memcpy(&o, blob.data(), sizeof(o));
            ok &= o.ok != 0 && o.bytes == bytes;
            use_mc &= o.mc != 0;
        }
        CHK_RET_LOG(!ok, HCCL_E_PARA, "registering user memory needs, on every rank, a whole allocation (offset 0) whose handle is exportable as a file "
                    "descriptor, and one common size that is a multiple of %zu bytes", gran);
        out->assign(1, SymSegment());
        HcclResult rc = alloc_vmm(bytes, use_mc, seq, &(*out)[0], (CUmemGenericAllocationHandle)drv_handles[0], (uint8_t *)local_ptrs[0], handle_offset);
        if (rc != HCCL_SUCCESS) out->clear();
        return rc;
    }

    void release(std::vector<SymSegment> *segs) override
    {
        const DriverApi &d = driver_api();
        cudaSetDevice(dev_);
        cudaDeviceSynchronize();
        for (auto &s : *segs) {
            if (s.kind == 1 || s.kind == kSegAdoptedVmm) {
                if (s.mc) {
                    d.MemUnmap((CUdeviceptr)s.mc, s.map_bytes);
                    d.MemAddressFree((CUdeviceptr)s.mc, s.map_bytes);
                    CUdevice cd;
                    d.DeviceGet(&cd, dev_);
                    d.MulticastUnbind((CUmemGenericAllocationHandle)s.mc_handle, cd, 0, s.map_bytes);
                    d.MemRelease((CUmemGenericAllocationHandle)s.mc_handle);
                }
                for (int q = 0; q < n_; ++q) {
                    if (!s.peer[q]) continue;
                    if (s.kind == kSegAdoptedVmm && q == rank_) continue;  // the caller's own mapping and handle stay
                    d.MemUnmap((CUdeviceptr)s.peer[q], s.map_bytes);
                    d.MemAddressFree((CUdeviceptr)s.peer[q], s.map_bytes);
                    d.MemRelease((CUmemGenericAllocationHandle)s.handles[q]);
                }
            } else if (s.kind == 2) {
                for (int q = 0; q < n_; ++q) {
                    if (!s.peer[q]) continue;
                    if (q == rank_) cudaFree(s.peer[q]);
                    else cudaIpcCloseMemHandle(s.peer[q]);
                }
            }
        }
        segs->clear();
    }

private:
    std::string sock_name(int r) const { return "hcclb-" + ident_ + "-" + std::to_string(r); }

    // Send my fds to every peer and collect theirs: all[q] = fds of rank q.
    HcclResult exchange_fds(const std::vector<int> &mine, std::vector<std::vector<int>> *all)
    {
        all->assign(n_, std::vector<int>());
        (*all)[rank_] = mine;
        std::atomic<bool> send_ok{true};
        std::thread sender([&] {
            for (int i = 1; i < n_; ++i) {
                int q = (rank_ + i) % n_;
                int fd = net::unix_connect(sock_name(q), tmo_);
                if (fd < 0 || !net::send_fds(fd, rank_, mine.data(), (int)mine.size())) send_ok = false;
                // wait for the receiver's one-byte acknowledgement so that the fds are not closed in flight
                char ack;
                if (fd >= 0 && !net::recv_all(fd, &ack, 1, tmo_)) send_ok = false;
                net::close_fd(fd);
            }
        });
        bool ok = true;
        for (int i = 1; i < n_ && ok; ++i) {
            int cfd = net::accept_timeout(lsock_, tmo_);
            if (cfd < 0) { ok = false; break; }
            int src = -1;
            std::vector<int> fds;
            if (!net::recv_fds(cfd, &src, &fds, tmo_) || src < 0 || src >= n_) ok = false;
            else (*all)[src] = fds;
            char ack = 1;
            net::send_all(cfd, &ack, 1);
            net::close_fd(cfd);
        }
        sender.join();
        if (!ok || !send_ok) {
            HLOG_ERROR("file-descriptor exchange between ranks failed");
            return HCCL_E_NETWORK;
        }
        return HCCL_SUCCESS;
    }

    // ext_handle != 0: the memory is the caller's allocation `ext_handle` (from byte ext_off on), already mapped at ext_va;
    // nothing is created, cleared or mapped for this rank itself, only exported for the peers.
    HcclResult alloc_vmm(size_t bytes, bool use_mc, uint64_t seq, SymSegment *s, CUmemGenericAllocationHandle ext_handle = 0,
                         uint8_t *ext_va = nullptr, size_t ext_off = 0)
    {
        (void)ext_off;  // cuMemMap only maps whole allocations from offset 0; adopt() has checked that
        const DriverApi &d = driver_api();
        CUdevice cd;
        d.DeviceGet(&cd, dev_);
        CUmemAllocationProp prop;
        memset(&prop, 0, sizeof(prop));
        prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        prop.location.id = dev_;
        prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        size_t gran = 2u << 20;
        d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
        CUmulticastObjectProp mprop;
        memset(&mprop, 0, sizeof(mprop));
        if (use_mc) {
            mprop.numDevices = (unsigned)n_;
            mprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
            mprop.size = bytes;
            size_t mg = gran;
            if (d.MulticastGetGranularity(&mg, &mprop, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran) gran = mg;
        }
        size_t sz = ext_handle ? bytes : (bytes + gran - 1) / gran * gran;
        mprop.size = sz;
        CUmemGenericAllocationHandle mine = ext_handle, mch = 0;
        CUresult cr = CUDA_SUCCESS;
        if (!ext_handle) {
            cr = d.MemCreate(&mine, sz, &prop, 0);
            CHK_RET_LOG(cr != CUDA_SUCCESS, HCCL_E_MEMORY, "cuMemCreate(%zu) failed: %s", sz, cu_err(cr));
        }
        std::vector<int> myfds;
        int fd = -1;
        cr = d.MemExportToShareableHandle(&fd, mine, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
        CHK_RET_LOG(cr != CUDA_SUCCESS, HCCL_E_DRV, "cuMemExportToShareableHandle failed: %s", cu_err(cr));
        myfds.push_back(fd);
        bool mc_created = false;
        if (use_mc && rank_ == 0) {
            cr = d.MulticastCreate(&mch, &mprop);
            if (cr == CUDA_SUCCESS) {
                int mfd = -1;
                cr = d.MemExportToShareableHandle(&mfd, mch, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
                if (cr == CUDA_SUCCESS) { myfds.push_back(mfd); mc_created = true; }
            }
            if (!mc_created) HLOG_WARN("multicast object unavailable (%s); NVLS algorithms disabled", cu_err(cr));
        }
        CHK_RET(hub_->barrier(ident_ + "/vmm-listen/" + std::to_string(seq), n_, rank_, tmo_));
        std::vector<std::vector<int>> all;
        CHK_RET(exchange_fds(myfds, &all));
        bool mc_on = use_mc && all[0].size() >= 2;
        s->bytes = bytes;
        s->map_bytes = sz;
        s->kind = ext_handle ? kSegAdoptedVmm : 1;
        CUmemAccessDesc acc;
        memset(&acc, 0, sizeof(acc));
        acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        acc.location.id = dev_;
        acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        HcclResult rc = HCCL_SUCCESS;
        for (int q = 0; q < n_ && rc == HCCL_SUCCESS; ++q) {
            CUmemGenericAllocationHandle h = mine;
            if (q == rank_ && ext_handle) {  // the caller's own mapping serves
                s->peer[q] = ext_va;
                s->handles[q] = 0;
                continue;
            }
            if (q != rank_) {
                cr = d.MemImportFromShareableHandle(&h, (void *)(uintptr_t)all[q][0], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
                if (cr != CUDA_SUCCESS) { HLOG_ERROR("import of rank %d memory failed: %s", q, cu_err(cr)); rc = HCCL_E_DRV; break; }
            }
            CUdeviceptr va = 0;
            cr = d.MemAddressReserve(&va, sz, gran, 0, 0);
            if (cr == CUDA_SUCCESS) cr = d.MemMap(va, sz, 0, h, 0);
            if (cr == CUDA_SUCCESS) cr = d.MemSetAccess(va, sz, &acc, 1);
            if (cr != CUDA_SUCCESS) { HLOG_ERROR("mapping rank %d memory failed: %s", q, cu_err(cr)); rc = HCCL_E_DRV; break; }
            s->peer[q] = (uint8_t *)va;
            s->handles[q] = h;
        }
        if (rc == HCCL_SUCCESS && mc_on) {
            if (rank_ != 0) {
                cr = d.MemImportFromShareableHandle(&mch, (void *)(uintptr_t)all[0][1], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
                if (cr != CUDA_SUCCESS) { HLOG_WARN("multicast import failed: %s", cu_err(cr)); mc_on = false; }
            }
            if (mc_on) {
                cr = d.MulticastAddDevice(mch, cd);
                if (cr != CUDA_SUCCESS) { HLOG_WARN("cuMulticastAddDevice failed: %s", cu_err(cr)); mc_on = false; }
            }
        }
        // every rank must have added its device before anyone binds; also agree whether multicast is usable
        std::vector<std::string> flags;
        std::string f(1, (char)(mc_on ? 1 : 0));
        HcclResult rb = hub_->rendezvous(ident_ + "/vmm-added/" + std::to_string(seq), n_, rank_, f, &flags, tmo_);
        if (rc == HCCL_SUCCESS) rc = rb;
        if (rc == HCCL_SUCCESS) {
            bool all_on = use_mc;
            for (auto &x : flags) all_on &= x[0] != 0;
            if (all_on) {
                cr = d.MulticastBindMem(mch, 0, mine, 0, sz, 0);
                CUdeviceptr mva = 0;
                if (cr == CUDA_SUCCESS) cr = d.MemAddressReserve(&mva, sz, gran, 0, 0);
                if (cr == CUDA_SUCCESS) cr = d.MemMap(mva, sz, 0, mch, 0);
                if (cr == CUDA_SUCCESS) cr = d.MemSetAccess(mva, sz, &acc, 1);
                if (cr != CUDA_SUCCESS) {
                    HLOG_ERROR("multicast bind/map failed: %s", cu_err(cr));
                    rc = HCCL_E_DRV;
                } else {
                    s->mc = (uint8_t *)mva;
                    s->mc_handle = mch;
                    mc_live_ = true;
                }
            } else if (mch) {
                d.MemRelease(mch);
            }
        }
        for (auto &v : all)
            for (int x : v) close(x);
        if (rc == HCCL_SUCCESS) {
            if (!ext_handle) cudaMemset(s->peer[rank_], 0, bytes);
            cudaDeviceSynchronize();
        }
        HcclResult rb2 = hub_->barrier(ident_ + "/vmm-ready/" + std::to_string(seq), n_, rank_, tmo_);
        return rc == HCCL_SUCCESS ? rb2 : rc;
    }

    HcclResult alloc_ipc(size_t bytes, uint64_t seq, SymSegment *s)
    {
        void *p = nullptr;
        CHK_RET_LOG(cudaMalloc(&p, bytes) != cudaSuccess, HCCL_E_MEMORY, "cudaMalloc(%zu) failed", bytes);
        cudaMemset(p, 0, bytes);
        cudaDeviceSynchronize();
        cudaIpcMemHandle_t h;
        CHK_RET_LOG(cudaIpcGetMemHandle(&h, p) != cudaSuccess, HCCL_E_RUNTIME, "cudaIpcGetMemHandle failed");
        std::vector<std::string> all;
        CHK_RET(hub_->rendezvous(ident_ + "/ipc/" + std::to_string(seq), n_, rank_, std::string((const char *)&h, sizeof(h)), &all, tmo_));
        s->bytes = bytes;
        s->kind = 2;
        for (int q = 0; q < n_; ++q) {
            if (q == rank_) { s->peer[q] = (uint8_t *)p; continue; }
            cudaIpcMemHandle_t ph;
            memcpy(&ph, all[q].data(), sizeof(ph));
            void *pp = nullptr;
            cudaError_t e = cudaIpcOpenMemHandle(&pp, ph, cudaIpcMemLazyEnablePeerAccess);
            CHK_RET_LOG(e != cudaSuccess, HCCL_E_RUNTIME, "cudaIpcOpenMemHandle(rank %d) failed: %s", q, cudaGetErrorString(e));
            s->peer[q] = (uint8_t *)pp;
        }
        return hub_->barrier(ident_ + "/ipc-ready/" + std::to_string(seq), n_, rank_, tmo_);
    }

    HubClient *hub_;
    std::string ident_;
    int rank_, n_, dev_;
    bool want_nvls_;
    int tmo_;
    int lsock_ = -1;
    bool vmm_ok_ = false, mc_ok_ = false, mc_live_ = false;
    uint64_t seq_ = 0;
};

}  // namespace

SymAllocator *make_host_local_allocator(int nranks) { return new HostLocal(nranks); }
SymAllocator *make_host_shm_allocator(HubClient *hub, const std::string &ident, int rank, int nranks, int tmo)
{
    return new HostShm(hub, ident, rank, nranks, tmo);
}
SymAllocator *make_device_local_allocator(int nranks, int device) { return new DeviceLocal(nranks, device); }
SymAllocator *make_device_vmm_allocator(HubClient *hub, const std::string &ident, int rank, int nranks, int device,
                                        bool want_nvls, int tmo)
{
    return new DeviceVmm(hub, ident, rank, nranks, device, want_nvls, tmo);
}

}  // namespace hcclb
