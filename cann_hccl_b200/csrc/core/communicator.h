// Communicator: owns the symmetric memory of a rank (staging halves, flag page, mailbox), the plan cache, the
// op sequence and the health state; runs collectives by selecting an algorithm, lowering it to a Plan and handing
// the plan to the device executor kernel or the host executor.  Counterpart of the reference's hcclComm facade +
// HcclCommunicator core (framework/communicator/hccl_comm.cc, framework/communicator/impl/hccl_communicator.cc:
// Init :227-261, ExecOp :3959-4071, AllocAlgResource :5575-5713, Suspend/Resume :4383/:7757).
#pragma once
#include <atomic>
#include <condition_variable>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>
#include "algo/schedule.h"
#include "algo/selector.h"
#include "bootstrap/hub.h"
#include "core/symmem.h"
#include "core/topo_probe.h"

namespace hcclb {

constexpr uint32_t kRootMagic = 0x42323030u;  // "B200"
// Payload stored inside the 4108-byte HcclRootInfo blob.
struct RootHandle {
    uint32_t magic;
    uint32_t version;
    uint32_t port;
    uint32_t family;
    char ip[64];
    char identifier[128];
};

enum CommState : int { CS_IDLE = 0, CS_INUSE = 1, CS_BUILDING = 2, CS_SUSPENDED = 3 };
enum TransportKind : int { TR_HOST = 0, TR_DEVICE = 1 };

struct CommSettings {
    int transport = TR_DEVICE;
    int device = 0;
    uint64_t stage_half_bytes = (uint64_t)HCCL_COMM_DEFAULT_BUFFSIZE << 20;
    bool deterministic = false;
    int expansion_mode = 0;
    std::string name;
    bool heartbeat = true;
};

struct OpRequest {
    int coll = COLL_ALLREDUCE;
    int algo = ALGO_AUTO;
    int nchan = 0;
    uint64_t count = 0;
    int dtype = HCCL_DATA_TYPE_FP32;
    int redop = HCCL_REDUCE_SUM;
    int root = 0;
    const void *const *in = nullptr;  // one pointer per local rank
    void *const *out = nullptr;
    const uint64_t *counts = nullptr, *displs = nullptr;  // AllGatherV / ReduceScatterV (nranks entries)
    const uint64_t *send_counts = nullptr, *send_displs = nullptr, *recv_counts = nullptr, *recv_displs = nullptr;  // [nlocal][nranks]
    void *stream = nullptr;
};

struct CommStats {
    uint64_t ops[COLL_COUNT] = {0};
    uint64_t bytes[COLL_COUNT] = {0};
    uint64_t algo_hist[ALGO_COUNT] = {0};
    uint64_t launches = 0;       // executor kernel launches (device) or plan executions (host)
    uint64_t plans_built = 0;
    uint64_t retries = 0;
    uint64_t timeouts = 0;
};

struct TraceRecord {
    uint64_t seq;
    int coll, algo, nchan;
    uint64_t count, bytes;
    int dtype, redop, root;
    double host_us;  // time spent in the API call
};

class P2pBackend;  // NCCL point-to-point (device transport)

class Communicator {
public:
    ~Communicator();
    static HcclResult create(uint32_t nranks, const RootHandle &root, uint32_t rank, const CommSettings &st,
                             Communicator **out);
    // All ranks are local: virtual ranks on one GPU (device) or threads over heap memory (host).
    static HcclResult create_local(uint32_t nranks, const CommSettings &st, Communicator **out);
    HcclResult create_sub(uint32_t rank_num, const uint32_t *rank_ids, uint64_t sub_id, uint32_t sub_rank,
                          const CommSettings &st, Communicator **out);
    HcclResult destroy();  // HCCL_E_AGAIN while an op is in flight on another thread

    int nranks() const { return nranks_; }
    int rank() const { return local_ranks_[0]; }
    int nlocal() const { return (int)local_ranks_.size(); }
    const std::string &name() const { return name_; }
    const std::string &identifier() const { return ident_; }
    int transport() const { return settings_.transport; }
    bool has_nvls() const { return nvls_; }
    bool deterministic() const;
    void set_deterministic(bool d) { settings_.deterministic = d; }
    CostModel &cost_model() { return model_; }

    HcclResult collective(const OpRequest &rq);
    // Send/Recv between two ranks.  Exactly one side per call on ordinary communicators; on all-local communicators
    // both sides are given and run together.
    HcclResult send(const void *buf, uint64_t count, int dtype, int dest, void *stream);
    HcclResult recv(void *buf, uint64_t count, int dtype, int src, void *stream);
    HcclResult batch_send_recv(HcclSendRecvItem *items, uint32_t n, void *stream);
    HcclResult local_send_recv(int src, int dst, const void *sbuf, void *rbuf, uint64_t count, int dtype, void *stream);

    // NCCL all-reduce baseline on the p2p backend's communicator (benchmarks only).
    HcclResult nccl_baseline_allreduce(const void *send, void *recv, uint64_t count, int dtype, int op, void *stream);
    HcclResult suspend();
    // The three stages of an abort, each with a time budget in milliseconds (0 = none); HCCL_E_TIMEOUT when it runs out.
    HcclResult suspend_entry(int budget_ms);
    HcclResult stop_exec(int budget_ms);
    HcclResult clean(int budget_ms);
    HcclResult resume();
    HcclResult resume_locked();
    HcclResult async_error();  // first error seen by this rank or reported by a peer
    HcclResult sync_stream(void *stream);  // wait for enqueued device work and return its status
    // Diagnostic: make local rank `local` wait for a flag that no rank ever sets, with a bound of timeout_ms.
    // The wait must run out and leave HCCL_E_TIMEOUT in the status block; resume() re-arms the communicator.
    HcclResult wait_probe(int local, double timeout_ms, void *stream);

    // Symmetric user memory (zero-copy paths, fused kernels).  Collective over the communicator.
    HcclResult sym_alloc(size_t bytes, void **local_ptrs /*nlocal*/, int *handle);
    // Registers caller-owned memory (one pointer per local rank) as a symmetric allocation; sym_free() undoes it and leaves
    // the memory alone.  drv_handles: driver allocation handles behind the pointers (one rank per GPU only), else null.
    HcclResult sym_adopt(void *const *local_ptrs, size_t bytes, const unsigned long long *drv_handles, size_t handle_offset, int *handle);
    HcclResult sym_free(int handle);
    // Peer pointer table of a symmetric allocation: ptrs[local][rank]; mc[local]
    HcclResult sym_query(int handle, void **peer_ptrs, void **mc_ptrs, size_t *bytes);

    // One-sided copy between a local buffer and rank `peer`'s copy of a symmetric allocation (stream-ordered on the device
    // transport, immediate on the host transport).  Only the caller takes part.
    HcclResult sym_put(int local, int handle, int peer, size_t offset, const void *src, size_t bytes, void *stream);
    HcclResult sym_get(int local, int handle, int peer, size_t offset, void *dst, size_t bytes, void *stream);
    // Ranks (host, pid, device), transport, NVLS and the peer-access matrix of the local devices, as JSON.
    std::string topo_json();
    // Outputs of floating-point reductions that were Inf or NaN (counted only with HCCL_OVERFLOW_CHECK=1).
    uint64_t overflow_count();

    // Fused tensor-parallel operators (kernels/fused/tp_gemm_sm100.cu).  Pointers per local rank; bf16; weights [N, K].
    //   all_gather_matmul:     y[M,N]     = all_gather(x_shard[M/p,K]) * w[N,K]^T
    //   matmul_reduce_scatter: out[M/p,N] = reduce_scatter_rows(h[M,K] * w[N,K]^T)
    HcclResult tp_all_gather_matmul(const void *const *x_shard, const void *const *w, void *const *y, int M, int N, int K, void *stream);
    HcclResult tp_matmul_reduce_scatter(const void *const *h, const void *const *w, void *const *out, int M, int N, int K, void *stream);
    // Selection only (no execution).
    Selection select(int coll, uint64_t count, int dtype, int redop) const;
    const CommStats &stats() const { return stats_; }
    std::vector<TraceRecord> trace_snapshot();
    std::string stats_json();
    HcclResult calibrate(void *stream);
    // Internal rendezvous over the hub among all ranks (used by the Python layer to share small blobs).
    HcclResult exchange(const std::string &tag, const std::string &mine, std::vector<std::string> *all);
    // Same, over the dedicated connection of the p2p backend's helper thread.
    HcclResult exchange_p2p(const std::string &tag, const std::string &mine, std::vector<std::string> *all);
    // Timestamps of the newest executor launch of local rank `local` (ns): out[0] kernel start, then per step
    // {after wait, after data movement, after signal} as seen by the first channel of the step.  Needs HCCL_KERNEL_TRACE=1.
    HcclResult kernel_trace(int local, uint64_t *out, size_t cap_words, int *nsteps);
    DevStatus *status(int local) { return status_[local]; }
    const RankCtx &ctx(int local) const { return ctx_[local]; }
    void *device_ctx_array() const { return dev_ctx_; }
    uint64_t next_seq() { return seq_; }
    int device() const { return settings_.device; }
    void set_fault_hook(std::function<void(uint64_t)> f) { fault_hook_ = std::move(f); }

private:
    Communicator() = default;
    HcclResult init_common();
    HcclResult check_ready();
    HcclResult run_plan(const Plan &plan, const void *dev_steps_base, const OpRequest &rq, uint64_t seq, int dtype,
                        int redop, bool track_done, const std::vector<const void *> &in, const std::vector<void *> &out);
    struct CachedPlan {
        Plan plan;
        std::vector<Step *> dev_steps;  // per local rank (device transport)
    };
    HcclResult get_plan(const OpDesc &d, const std::string &key, CachedPlan **out);
    HcclResult run_collective_once(const OpRequest &rq);
    HcclResult run_ll_allreduce(const OpRequest &rq);
    HcclResult run_pipe(const OpRequest &rq, bool want_mc, int zc_handle = 0, size_t zc_off = 0);
    HcclResult run_a2av(const OpRequest &rq);
    int pipe_mode_for(int coll) const;  // PipeMode of a collective, -1 when it has no pipelined kernel
    HcclResult tp_workspace(const std::string &key, size_t data_bytes, int M, void **ws_out);
    void tp_release_workspaces();
    int overlap_kind(const OpRequest &rq, int li) const;
    HcclResult a2av_check(const OpRequest &rq);
    HcclResult consistency_check(const OpRequest &rq, int algo, uint64_t zc_in = 0, uint64_t zc_out = 0);
    HcclResult maybe_retry(const OpRequest &rq, HcclResult failure, uint64_t op_index);
    // Device transport: the newest collective as it was issued (deep copy), so that a failure its kernel reports later,
    // at the next call or at a synchronisation, can be answered by running it again.
    struct LastOp {
        bool valid = false, retriable = false;
        uint64_t op_index = 0, first_seq = 0;
        OpRequest rq;
        std::vector<const void *> in;
        std::vector<void *> out;
        std::vector<uint64_t> counts, displs, sc, sd, rc, rd;
    };
    LastOp last_op_;
    void remember_op(const OpRequest &rq);
    HcclResult retry_last_op(HcclResult failure);
    void heartbeat_loop();
    void record_trace(const OpRequest &rq, int algo, int nchan, uint64_t bytes, double us);
    HcclResult overflow_scan(const OpRequest &rq);
    HcclResult p2p_plan_exec(bool is_send, int peer, const void *sbuf, void *rbuf, uint64_t count, int dtype, void *stream);

    CommSettings settings_;
    int nranks_ = 1;
    std::vector<int> local_ranks_;
    std::string ident_, name_;
    bool all_local_ = false;
    bool nvls_ = false;

    std::unique_ptr<Hub> owned_hub_;       // only on the rank that started it and passed ownership
    std::shared_ptr<HubClient> hub_;       // control connection (shared with sub-communicators)
    std::unique_ptr<HubClient> hb_conn_;   // heartbeat connection
    std::unique_ptr<HubClient> p2p_conn_;  // connection used by the p2p backend's helper thread
    RootHandle root_{};
    std::string key_prefix_;               // hub key namespace of this communicator

    std::unique_ptr<SymAllocator> alloc_;
    std::vector<SymSegment> seg_;          // [local]
    std::vector<RankCtx> ctx_;             // host copies (pointers valid on the executing side)
    std::vector<DevStatus *> status_;      // host-visible status blocks
    std::vector<volatile uint32_t *> abort_;
    void *dev_ctx_ = nullptr;              // device array of RankCtx
    void *dev_exit_ = nullptr;
    void *dev_pipe_cnt_ = nullptr;         // arrival counters of the pipelined kernels (kPipeCounterWords per local rank)
    void *dev_trace_ = nullptr;            // in-kernel timestamp buffers (kTraceWords per local rank) when enabled
    void *pinned_ = nullptr;               // host-mapped block holding status + abort words
    uint64_t p2p_slot_ = 0;
    uint64_t ll_seq_ = 0;                  // number of LL operations issued (tag and mailbox parity)
    bool ll_ok_ = false;
    uint64_t ll_two_shot_min_ = 256u << 10;  // from this size on the LL path of three and more ranks goes two-shot
    uint64_t ll_max_bytes() const;            // largest message the LL path takes on this communicator

    std::mutex op_mu_;
    std::atomic<int> state_{CS_IDLE};
    uint64_t seq_ = 1;
    std::atomic<uint64_t> resume_gen_{0};
    std::map<std::string, CachedPlan> plans_;
    std::map<std::string, bool> checked_;
    std::map<std::pair<int, int>, uint32_t> p2p_rounds_;  // (src,dst) -> rounds exchanged
    CostModel model_;
    LinkTopo links_;                        // NVLink attributes of this rank's GPU (device transport)
    // Measured times per collective, (size bucket, algorithm), from calibrate(); empty until calibrated.  Where a table exists
    // the selector picks the fastest measured algorithm that is allowed for the (dtype, op) at hand instead of the model's guess.
    struct TunedTable {
        std::vector<uint64_t> sizes;            // bytes per rank in the sense of the API count
        std::vector<std::vector<double>> us;    // [bucket][algo], <= 0 = not measured
    };
    std::map<int, TunedTable> tuned_;           // by collective
    bool calibrating_ = false;                  // calibration traffic: no parameter exchange, no fault hooks
    CommStats stats_;
    std::vector<TraceRecord> trace_;
    size_t trace_pos_ = 0;
    std::mutex trace_mu_;

    std::map<int, std::vector<SymSegment>> user_segs_;
    std::map<int, std::vector<void *>> user_peer_tabs_;   // per allocation and local rank: array of nranks peer pointers (device or host memory)
    // Finds the registered allocation that holds [ptr, ptr+bytes) of local rank li; returns its handle or 0.
    int find_user_seg(int li, const void *ptr, size_t bytes, size_t *offset);
    HcclResult register_user_segs(std::vector<SymSegment> segs, int *handle);
    int next_handle_ = 1;
    struct ZcArgs { uint8_t *const *in_tab; uint8_t *const *out_tab; uint8_t *in_mc; uint8_t *out_mc; size_t oin, oout; };
    std::vector<ZcArgs> zc_args_;   // zero-copy pointers of the op being launched (per local rank)

    std::thread hb_thread_;
    std::atomic<bool> hb_stop_{false};
    std::atomic<uint32_t> remote_error_{0};  // HcclResult learned from heartbeat
    std::atomic<int> remote_bad_rank_{-1};
    std::mutex hb_mu_;
    std::condition_variable hb_cv_;
    uint64_t op_index_ = 0;                  // API-level op counter (one per collective call)
    uint64_t a2av_calls_ = 0;                // AlltoAllV / VC calls so far (which of them get their count matrix checked)
    std::function<void(uint64_t)> fault_hook_;
    std::unique_ptr<P2pBackend> p2p_;
    struct TopoEntry { int rank; uint32_t pid; int device; std::string host; };
    std::vector<TopoEntry> topo_;            // one entry per rank (filled at creation)
    unsigned long long *overflow_word_ = nullptr;  // host-mapped (device transport) or heap counter of non-finite outputs
    friend class P2pBackend;
};

// RAII: marks the communicator in use for the duration of an API call (reference: StateGuard, state_guard.h).
class StateGuard {
public:
    StateGuard(std::atomic<int> &s, int busy) : s_(s), prev_(s.exchange(busy)) {}
    ~StateGuard() { int busy = s_.load(); if (busy != CS_SUSPENDED) s_.store(prev_ == CS_SUSPENDED ? CS_SUSPENDED : CS_IDLE); }
private:
    std::atomic<int> &s_;
    int prev_;
};

// Plain tcgen05 GEMM C[M,N] = A[M,K] * B[N,K]^T in bf16 (no communicator needed).
HcclResult gemm_bf16_plain(const void *A, const void *B, void *C, int M, int N, int K, void *stream);
// Launches of the fused GEMM kernels in this process: one CTA per tile / clusters of two CTAs per 256 x 256 tile.
void tp_gemm_launch_counts(uint64_t *single, uint64_t *pair);
// Device executor entry (kernels/exec_plan.cu).
HcclResult launch_exec_plan(const RankCtx *dev_ctx, const ExecArgs *args, int nlocal, int nchan, void *stream, bool co_resident = false);
// Unique identifier helper used by HcclGetRootInfo.
std::string make_identifier(const std::string &ip, int port);
// Process-wide registry of hubs started by HcclGetRootInfo (the communicator created by the same process with the
// matching identifier adopts the hub and stops it on destroy).
void register_hub(const std::string &ident, Hub *hub);
Hub *adopt_hub(const std::string &ident);

}  // namespace hcclb
