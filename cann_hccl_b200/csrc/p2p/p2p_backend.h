// Point-to-point backend of the device transport: HcclSend / HcclRecv / HcclBatchSendRecv are carried by NCCL
// p2p (ncclSend / ncclRecv inside a group), stream ordered and overlappable with our own collective kernels.
// libnccl is loaded at run time (HCCL_NCCL_LIB, else the usual library names); without it the mailbox plans of
// the generic executor carry p2p traffic instead.  The NCCL communicator is initialised on a helper thread that
// starts when the HCCL communicator is created, so that initialisation (a collective over all ranks) can never
// deadlock against ranks that do not take part in a given Send/Recv.
#pragma once
#include <atomic>
#include <memory>
#include <thread>
#include <vector>
#include "hccl/hccl_types.h"
namespace hcclb {
class Communicator;
class P2pBackend {
public:
    static bool available();
    static HcclResult create(Communicator *comm, std::unique_ptr<P2pBackend> *out);
    ~P2pBackend();
    HcclResult send(const void *buf, uint64_t count, int dtype, int peer, void *stream);
    HcclResult recv(void *buf, uint64_t count, int dtype, int peer, void *stream);
    // NCCL all-reduce on the same communicator: the measured baseline next to our own kernels (never used by a collective).
    HcclResult baseline_allreduce(const void *send, void *recv, uint64_t count, int dtype, int op, void *stream);
    HcclResult batch(const std::vector<HcclSendRecvItem *> &sends, const std::vector<HcclSendRecvItem *> &recvs, void *stream);

private:
    P2pBackend() = default;
    HcclResult wait_ready();
    void init_thread(Communicator *comm);
    void *nccl_comm_ = nullptr;
    std::thread th_;
    std::atomic<int> ready_{0};  // 0 pending, 1 ok, -1 failed
    int device_ = 0;
};
}  // namespace hcclb
