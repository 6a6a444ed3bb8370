#include "core/communicator.h"
#include <sys/time.h>
#include <time.h>
#include <unistd.h>
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <sstream>
#include <cuda_runtime.h>
#include "bootstrap/socket.h"
#include "common/dtype_host.h"
#include "common/env.h"
#include "common/log.h"
#include "health/consistency.h"
#include "health/fault_inject.h"
#include "kernels/a2av.h"
#include "kernels/ar_ll.h"
#include "kernels/overflow.h"
#include "kernels/pipe_coll.h"
#include <nvtx3/nvToolsExt.h>
#include <fstream>
#include "core/topo_probe.h"
#include "p2p/p2p_backend.h"
#include "transport/host_exec.h"

namespace hcclb {

namespace {
std::mutex g_hub_mu;
std::map<std::string, Hub *> g_hubs;
double now_us()
{
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec * 1e6 + ts.tv_nsec * 1e-3;
}
constexpr size_t kTraceCap = 4096;
constexpr uint64_t kP2pSlot = 256u << 10;
size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
}  // namespace

void register_hub(const std::string &ident, Hub *hub)
{
    std::lock_guard<std::mutex> lk(g_hub_mu);
    g_hubs[ident] = hub;
}
Hub *adopt_hub(const std::string &ident)
{
    std::lock_guard<std::mutex> lk(g_hub_mu);
    auto it = g_hubs.find(ident);
    if (it == g_hubs.end()) return nullptr;
    Hub *h = it->second;
    g_hubs.erase(it);
    return h;
}
std::string make_identifier(const std::string &ip, int port)
{
    struct timeval tv;
    gettimeofday(&tv, nullptr);
    static std::atomic<uint32_t> ctr{0};
    char buf[128];
    snprintf(buf, sizeof(buf), "%s_%d_%d_%llu_%u", ip.c_str(), port, (int)getpid(),
             (unsigned long long)tv.tv_sec * 1000000ull + tv.tv_usec, ctr.fetch_add(1));
    return buf;
}

bool Communicator::deterministic() const
{
    const EnvConfig &e = env_config();
    if (e.deterministic >= 0) return e.deterministic != 0;  // the environment wins (reference: op_base.cc:1204)
    return settings_.deterministic;
}

// ------------------------------------------------------------------------------------------------ creation
HcclResult Communicator::create(uint32_t nranks, const RootHandle &root, uint32_t rank, const CommSettings &st,
                                Communicator **out)
{
    const EnvConfig &env = env_config();
    CHK_RET_LOG(nranks == 0 || nranks > (uint32_t)kMaxRanks, HCCL_E_PARA, "rank count %u outside [1,%d]", nranks, kMaxRanks);
    CHK_RET_LOG(rank >= nranks, HCCL_E_PARA, "rank %u not below rank count %u", rank, nranks);
    CHK_RET_LOG(root.magic != kRootMagic, HCCL_E_PARA, "root info was not produced by HcclGetRootInfo");
    std::unique_ptr<Communicator> c(new Communicator());
    c->settings_ = st;
    c->nranks_ = (int)nranks;
    c->local_ranks_ = {(int)rank};
    c->root_ = root;
    c->ident_ = root.identifier;
    c->name_ = st.name.empty() ? c->ident_ : st.name;
    c->key_prefix_ = c->ident_;
    if (Hub *h = adopt_hub(c->ident_)) c->owned_hub_.reset(h);
    int tmo = env.connect_timeout_s * 1000;
    c->hub_ = std::make_shared<HubClient>();
    CHK_RET(c->hub_->connect(root.ip, (int)root.port, (int)root.family, tmo));
    // rank table exchange: every rank publishes {rank, pid, host, device, transport}; the table is checked for
    // duplicates and mixed transports (reference: TopoInfoExchangeAgent::VerifyClusterInfo, exchange_agent.cc:376)
    struct Entry { uint32_t rank, pid, device, transport; char host[64]; } me;
    memset(&me, 0, sizeof(me));
    me.rank = rank; me.pid = (uint32_t)getpid(); me.device = (uint32_t)st.device; me.transport = (uint32_t)st.transport;
    gethostname(me.host, sizeof(me.host) - 1);
    std::vector<std::string> table;
    CHK_RET(c->hub_->rendezvous(c->key_prefix_ + "/ranktable", nranks, rank, std::string((const char *)&me, sizeof(me)), &table, tmo));
    for (uint32_t r = 0; r < nranks; ++r) {
        Entry e;
        CHK_RET_LOG(table[r].size() != sizeof(e), HCCL_E_INTERNAL, "malformed rank table entry %u", r);
        memcpy(&e, table[r].data(), sizeof(e));
        CHK_RET_LOG(e.rank != r, HCCL_E_PARA, "rank table entry %u carries rank %u", r, e.rank);
        CHK_RET_LOG(e.transport != me.transport, HCCL_E_PARA, "rank %u uses a different transport", r);
        CHK_RET_LOG(strcmp(e.host, me.host) != 0, HCCL_E_NOT_SUPPORT, "rank %u is on host %s: one NVSwitch domain per communicator", r, e.host);
        c->topo_.push_back(TopoEntry{(int)r, e.pid, (int)e.device, std::string(e.host)});
    }
    if (st.transport == TR_HOST) c->alloc_.reset(make_host_shm_allocator(c->hub_.get(), c->ident_, (int)rank, (int)nranks, tmo));
    else {
        CHK_RET_LOG(cudaSetDevice(st.device) != cudaSuccess, HCCL_E_RUNTIME, "cudaSetDevice(%d) failed", st.device);
        bool want_nvls = env.nvls_enable != 0 && nranks > 1;
        c->alloc_.reset(make_device_vmm_allocator(c->hub_.get(), c->ident_, (int)rank, (int)nranks, st.device, want_nvls, tmo));
    }
    CHK_RET(c->init_common());
    if (st.heartbeat && nranks > 1) {
        c->hb_conn_.reset(new HubClient());
        if (c->hb_conn_->connect(root.ip, (int)root.port, (int)root.family, tmo) == HCCL_SUCCESS)
            c->hb_thread_ = std::thread([p = c.get()] { p->heartbeat_loop(); });
    }
    if (st.transport == TR_DEVICE && nranks > 1 && P2pBackend::available()) {
        c->p2p_conn_.reset(new HubClient());
        if (c->p2p_conn_->connect(root.ip, (int)root.port, (int)root.family, tmo) == HCCL_SUCCESS) P2pBackend::create(c.get(), &c->p2p_);
    }
    if (st.transport == TR_DEVICE && nranks > 1 && env.calibrate) {
        // every rank runs it (the decision depends on the shared environment only); a failure leaves the default model
        HcclResult crc = c->calibrate(nullptr);
        if (crc != HCCL_SUCCESS) { HLOG_WARN("calibration failed (%d): selecting from the default cost model", (int)crc); CHK_RET(c->resume()); }
    }
    *out = c.release();
    return HCCL_SUCCESS;
}

HcclResult Communicator::create_local(uint32_t nranks, const CommSettings &st, Communicator **out)
{
    CHK_RET_LOG(nranks == 0 || nranks > (uint32_t)kMaxRanks, HCCL_E_PARA, "rank count %u outside [1,%d]", nranks, kMaxRanks);
    std::unique_ptr<Communicator> c(new Communicator());
    c->settings_ = st;
    c->nranks_ = (int)nranks;
    for (uint32_t r = 0; r < nranks; ++r) c->local_ranks_.push_back((int)r);
    c->all_local_ = true;
    c->ident_ = make_identifier("local", 0);
    c->name_ = st.name.empty() ? c->ident_ : st.name;
    if (st.transport == TR_HOST) c->alloc_.reset(make_host_local_allocator((int)nranks));
    else {
        CHK_RET_LOG(cudaSetDevice(st.device) != cudaSuccess, HCCL_E_RUNTIME, "cudaSetDevice(%d) failed", st.device);
        c->alloc_.reset(make_device_local_allocator((int)nranks, st.device));
    }
    CHK_RET(c->init_common());
    *out = c.release();
    return HCCL_SUCCESS;
}

HcclResult Communicator::create_sub(uint32_t rank_num, const uint32_t *rank_ids, uint64_t sub_id, uint32_t sub_rank,
                                    const CommSettings &st, Communicator **out)
{
    // Sub-communicator = new identifier "<parent>_sub_<id>" (reference: op_base.cc:650-790), same hub, own memory.
    CHK_RET_LOG(all_local_, HCCL_E_NOT_SUPPORT, "sub-communicators of all-local communicators are not supported");
    CHK_RET_LOG(rank_num == 0 || rank_num > (uint32_t)nranks_ || sub_rank >= rank_num, HCCL_E_PARA, "bad sub-communicator shape");
    CHK_RET_LOG(rank_ids[sub_rank] != (uint32_t)rank(), HCCL_E_PARA, "rankIds[%u] is %u but this rank is %d", sub_rank, rank_ids[sub_rank], rank());
    const EnvConfig &env = env_config();
    int tmo = env.connect_timeout_s * 1000;
    std::unique_ptr<Communicator> c(new Communicator());
    c->settings_ = st;
    c->settings_.transport = settings_.transport;
    c->settings_.device = settings_.device;
    c->nranks_ = (int)rank_num;
    c->local_ranks_ = {(int)sub_rank};
    c->root_ = root_;
    c->ident_ = ident_ + "_sub_" + std::to_string(sub_id);
    c->name_ = st.name.empty() ? c->ident_ : st.name;
    c->key_prefix_ = c->ident_;
    c->hub_ = std::make_shared<HubClient>();
    CHK_RET(c->hub_->connect(root_.ip, (int)root_.port, (int)root_.family, tmo));
    // members check that they agree on the member list
    std::string ids((const char *)rank_ids, rank_num * sizeof(uint32_t));
    std::vector<std::string> all;
    CHK_RET(c->hub_->rendezvous(c->key_prefix_ + "/members", rank_num, sub_rank, ids, &all, tmo));
    for (auto &a : all) CHK_RET_LOG(a != ids, HCCL_E_PARA, "sub-communicator members disagree on the rank list");
    if (settings_.transport == TR_HOST) c->alloc_.reset(make_host_shm_allocator(c->hub_.get(), c->ident_, (int)sub_rank, (int)rank_num, tmo));
    else c->alloc_.reset(make_device_vmm_allocator(c->hub_.get(), c->ident_, (int)sub_rank, (int)rank_num, settings_.device, env.nvls_enable != 0, tmo));
    CHK_RET(c->init_common());
    if (c->settings_.transport == TR_DEVICE && rank_num > 1 && env.calibrate) {
        HcclResult crc = c->calibrate(nullptr);
        if (crc != HCCL_SUCCESS) { HLOG_WARN("calibration failed (%d): selecting from the default cost model", (int)crc); CHK_RET(c->resume()); }
    }
    *out = c.release();
    return HCCL_SUCCESS;
}

HcclResult Communicator::init_common()
{
    const EnvConfig &env = env_config();
    int nl = nlocal();
    p2p_slot_ = kP2pSlot;
    size_t flags_bytes = kFlagPageBytes;
    size_t p2p_bytes = align_up((size_t)nranks_ * p2p_slot_, 4096);
    size_t half = align_up((size_t)settings_.stage_half_bytes, 4096);
    settings_.stage_half_bytes = half;
    bool dev0 = settings_.transport == TR_DEVICE;
    size_t ll_bytes = dev0 ? align_up((size_t)2 * nranks_ * kLlSlotBytes, 4096) : 0;
    ll_ok_ = dev0 && nranks_ > 1;
    size_t total = flags_bytes + p2p_bytes + ll_bytes + 2 * half;
    CHK_RET(alloc_->alloc(total, true, &seg_));
    CHK_RET_LOG((int)seg_.size() != nl, HCCL_E_INTERNAL, "allocator returned %zu segments for %d local ranks", seg_.size(), nl);
    nvls_ = seg_[0].mc != nullptr;
    bool dev = settings_.transport == TR_DEVICE;
    size_t blk = align_up(sizeof(DevStatus), 64) + 64;
    if (dev) {
        CHK_RET_LOG(cudaHostAlloc(&pinned_, blk * nl, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess, HCCL_E_MEMORY, "cudaHostAlloc failed");
    } else {
        pinned_ = calloc(nl, blk);
        CHK_RET_LOG(!pinned_, HCCL_E_MEMORY, "out of host memory");
    }
    memset(pinned_, 0, blk * nl);
    double tmo_ms = env.exec_timeout_ms > 0 ? env.exec_timeout_ms : (env.exec_timeout_s > 0 ? env.exec_timeout_s * 1000.0 : 3600e3);
    if (tmo_ms > 3600e3) tmo_ms = 3600e3;  // never unbounded: a wait always ends
    ctx_.assign(nl, RankCtx());
    status_.assign(nl, nullptr);
    abort_.assign(nl, nullptr);
    if (dev) {
        CHK_RET_LOG(cudaMalloc(&dev_exit_, sizeof(uint32_t) * 4 * nl) != cudaSuccess, HCCL_E_MEMORY, "cudaMalloc failed");
        cudaMemset(dev_exit_, 0, sizeof(uint32_t) * 4 * nl);
    }
    if (dev) {
        CHK_RET_LOG(cudaMalloc(&dev_pipe_cnt_, sizeof(uint32_t) * kPipeCounterWords * nl) != cudaSuccess, HCCL_E_MEMORY, "cudaMalloc failed");
        cudaMemset(dev_pipe_cnt_, 0, sizeof(uint32_t) * kPipeCounterWords * nl);
    }
    if (dev && getenv("HCCL_KERNEL_TRACE") && atoi(getenv("HCCL_KERNEL_TRACE")) > 0) {
        CHK_RET_LOG(cudaMalloc(&dev_trace_, sizeof(uint64_t) * kTraceWords * nl) != cudaSuccess, HCCL_E_MEMORY, "cudaMalloc failed");
        cudaMemset(dev_trace_, 0, sizeof(uint64_t) * kTraceWords * nl);
    }
    for (int li = 0; li < nl; ++li) {
        RankCtx &x = ctx_[li];
        memset(&x, 0, sizeof(x));
        x.rank = local_ranks_[li];
        x.nranks = nranks_;
        for (int q = 0; q < nranks_; ++q) {
            uint8_t *base = seg_[li].peer[q];
            x.flags[q] = (uint64_t *)base;
            x.p2p[q] = base + flags_bytes;
            x.ll[q] = base + flags_bytes + p2p_bytes;
            x.stage[q] = base + flags_bytes + p2p_bytes + ll_bytes;
        }
        x.mc_stage = seg_[li].mc ? seg_[li].mc + flags_bytes + p2p_bytes + ll_bytes : nullptr;
        uint8_t *pb = (uint8_t *)pinned_ + blk * li;
        status_[li] = (DevStatus *)pb;
        abort_[li] = (volatile uint32_t *)(pb + align_up(sizeof(DevStatus), 64));
        x.status = status_[li];
        x.abort = abort_[li];
        x.exit_counter = dev ? (uint32_t *)dev_exit_ + 4 * li : nullptr;
        // completion word of the op-execution counter: host-mapped, so that the heartbeat thread reads it without a CUDA call
        // (a CUDA call can wait for seconds behind an allocation or a mapping made by another thread of the process, and a
        // silent heartbeat makes the peers report this rank as lost)
        x.dev_tail = dev ? (uint64_t *)(pb + align_up(sizeof(DevStatus), 64) + 16) : nullptr;
        x.pipe_cnt = dev ? (uint32_t *)dev_pipe_cnt_ + (size_t)li * kPipeCounterWords : nullptr;
        x.stage_half = half;
        x.trace = dev_trace_ ? (uint64_t *)dev_trace_ + (size_t)li * kTraceWords : nullptr;
        x.timeout_ns = (uint64_t)(tmo_ms * 1e6);
    }
    if (dev) {
        CHK_RET_LOG(cudaMalloc(&dev_ctx_, sizeof(RankCtx) * nl) != cudaSuccess, HCCL_E_MEMORY, "cudaMalloc failed");
        CHK_RET_LOG(cudaMemcpy(dev_ctx_, ctx_.data(), sizeof(RankCtx) * nl, cudaMemcpyHostToDevice) != cudaSuccess, HCCL_E_RUNTIME, "cudaMemcpy failed");
        cudaDeviceSynchronize();
    }
    if (dev) {
        // link attributes of this GPU: the selector's default bandwidths come from what the device reports (a measured
        // calibration, when it runs, replaces them)
        char bus[32] = {0};
        std::string pci = cudaDeviceGetPCIBusId(bus, sizeof(bus), settings_.device) == cudaSuccess ? std::string(bus) : std::string();
        links_ = probe_links(settings_.device, pci);
        int mc = 0;
        cudaDeviceGetAttribute(&mc, (cudaDeviceAttr)132 /* cudaDevAttrMulticastSupported, not named by every runtime header */, settings_.device);
        cudaGetLastError();
        links_.multicast = nvls_ || mc != 0;
        if (links_.probed && links_.egress_gbps() > 0) {
            model_.beta_gbps = 0.72 * links_.egress_gbps();   // what peer loads / stores of one kernel reach of the nominal rate
            model_.nvls_gbps = 0.55 * links_.egress_gbps();   // in-switch reductions run at about half the link rate per GPU
        }
    }
    trace_.resize(kTraceCap);
    HLOG_INFO("communicator %s: %d ranks, %d local, transport %s, staging 2x%zu MB, nvls %d", name_.c_str(), nranks_, nl,
              dev ? "device" : "host", half >> 20, (int)nvls_);
    return HCCL_SUCCESS;
}

Communicator::~Communicator()
{
    hb_stop_.store(true);
    { std::lock_guard<std::mutex> lk(hb_mu_); hb_cv_.notify_all(); }
    if (hb_thread_.joinable()) hb_thread_.join();
    p2p_.reset();
    bool dev = settings_.transport == TR_DEVICE;
    if (dev) {
        cudaSetDevice(settings_.device);
        cudaDeviceSynchronize();
        for (auto &kv : plans_)
            for (Step *s : kv.second.dev_steps) cudaFree(s);
    }
    tp_release_workspaces();
    for (auto &kv : user_segs_) alloc_->release(&kv.second);
    if (alloc_) alloc_->release(&seg_);
    if (dev) {
        if (dev_ctx_) cudaFree(dev_ctx_);
        if (dev_exit_) cudaFree(dev_exit_);
        if (dev_pipe_cnt_) cudaFree(dev_pipe_cnt_);
        if (dev_trace_) cudaFree(dev_trace_);
        if (pinned_) cudaFreeHost(pinned_);
        if (overflow_word_) cudaFreeHost(overflow_word_);
    } else {
        free(pinned_);
        free(overflow_word_);
    }
    alloc_.reset();
    if (hb_conn_) hb_conn_->bye();
    if (p2p_conn_) p2p_conn_->bye();
    if (hub_) hub_->bye();
    owned_hub_.reset();
}

HcclResult Communicator::destroy()
{
    int st = state_.load();
    if (st == CS_INUSE || st == CS_BUILDING) return HCCL_E_AGAIN;  // reference: HcclCommDestroy while in use
    if (!all_local_ && nranks_ > 1 && hub_ && hub_->connected()) {
        // leave together so that no rank unmaps memory a peer's kernel may still touch; bounded wait
        if (settings_.transport == TR_DEVICE) { cudaSetDevice(settings_.device); cudaDeviceSynchronize(); }
        hub_->barrier(key_prefix_ + "/destroy", nranks_, rank(), 10000);
    }
    if (!env_config().stats_dump.empty()) {
        // one JSON object per line and communicator; ranks of a job append to the same file
        std::ofstream f(env_config().stats_dump, std::ios::app);
        if (f) f << stats_json() << "\n";
    }
    delete this;
    return HCCL_SUCCESS;
}

// ------------------------------------------------------------------------------------------------ plans
HcclResult Communicator::get_plan(const OpDesc &d, const std::string &key, CachedPlan **out)
{
    auto it = plans_.find(key);
    if (it != plans_.end()) { *out = &it->second; return HCCL_SUCCESS; }
    if (plans_.size() >= 2048) {  // bound memory: drop everything once nothing is in flight
        if (settings_.transport == TR_DEVICE) {
            cudaDeviceSynchronize();
            for (auto &kv : plans_)
                for (Step *s : kv.second.dev_steps) cudaFree(s);
        }
        plans_.clear();
    }
    CachedPlan cp;
    CHK_RET(build_plan(d, local_ranks_, &cp.plan));
    {
        std::string why;
        HcclResult vrc = verify_plan(d, local_ranks_, cp.plan, d.coll == COLL_SEND || d.coll == COLL_RECV ? 0 : settings_.stage_half_bytes, &why);
        CHK_RET_LOG(vrc != HCCL_SUCCESS, vrc, "plan verification failed: %s", why.c_str());
    }
    if (env_config().plan_race_check && d.coll != COLL_SEND && d.coll != COLL_RECV) {
        // debug aid: the happens-before check over the step lists of ALL ranks (built here once more when this process
        // runs only some of them; AlltoAllV plans need every rank's rows, which only a process with all ranks has)
        const bool rows_only = (d.coll == COLL_ALLTOALLV || d.coll == COLL_ALLTOALLVC) && (int)local_ranks_.size() != nranks_;
        if (!rows_only) {
            std::vector<int> all_ranks;
            for (int r = 0; r < nranks_; ++r) all_ranks.push_back(r);
            Plan whole;
            const Plan *pp = &cp.plan;
            if ((int)local_ranks_.size() != nranks_) { CHK_RET(build_plan(d, all_ranks, &whole)); pp = &whole; }
            std::string why;
            HcclResult rrc = race_check_plan(d, *pp, false, &why);
            if (rrc == HCCL_SUCCESS) rrc = race_check_plan(d, *pp, true, &why);
            CHK_RET_LOG(rrc != HCCL_SUCCESS, rrc, "plan race check failed: %s", why.c_str());
        }
    }
    if (settings_.transport == TR_DEVICE) {
        for (auto &steps : cp.plan.steps) {
            Step *ds = nullptr;
            size_t bytes = std::max<size_t>(steps.size(), 1) * sizeof(Step);
            CHK_RET_LOG(cudaMalloc(&ds, bytes) != cudaSuccess, HCCL_E_MEMORY, "cudaMalloc(plan) failed");
            if (!steps.empty()) cudaMemcpy(ds, steps.data(), steps.size() * sizeof(Step), cudaMemcpyHostToDevice);
            cp.dev_steps.push_back(ds);
        }
    }
    stats_.plans_built++;
    auto ins = plans_.emplace(key, std::move(cp));
    *out = &ins.first->second;
    return HCCL_SUCCESS;
}

HcclResult Communicator::run_plan(const Plan &plan, const void *dev_steps_base, const OpRequest &rq, uint64_t seq,
                                  int dtype, int redop, bool track_done, const std::vector<const void *> &in,
                                  const std::vector<void *> &out)
{
    int nl = (int)plan.steps.size();
    const Step *const *dsteps = (const Step *const *)dev_steps_base;
    std::vector<ExecArgs> args(nl);
    for (int li = 0; li < nl; ++li) {
        ExecArgs &a = args[li];
        memset(&a, 0, sizeof(a));
        a.steps = settings_.transport == TR_DEVICE ? dsteps[li] : plan.steps[li].data();
        a.nsteps = (int)plan.steps[li].size();
        a.nchan = plan.nchan;
        a.seq = seq;
        a.in = (const uint8_t *)in[li];
        a.out = (uint8_t *)out[li];
        a.dtype = dtype;
        a.redop = redop;
        a.track_done = track_done ? 1 : 0;
        if (li < (int)zc_args_.size()) {
            // the plan addresses the buffers relative to the caller's pointers: shift the segment bases by the buffer offsets
            a.z_in_peer = zc_args_[li].in_tab; a.z_out_peer = zc_args_[li].out_tab;
            a.z_in_mc = zc_args_[li].in_mc ? zc_args_[li].in_mc + zc_args_[li].oin : nullptr;
            a.z_out_mc = zc_args_[li].out_mc ? zc_args_[li].out_mc + zc_args_[li].oout : nullptr;
            a.z_in_off = zc_args_[li].oin; a.z_out_off = zc_args_[li].oout;
        }
        if (track_done && settings_.transport == TR_DEVICE) __atomic_store_n(&status_[li]->head, (uint64_t)seq, __ATOMIC_RELAXED);  // completion (tail) is a device word
    }
    stats_.launches++;
    if (settings_.transport == TR_DEVICE && dev_trace_) {
        for (int li = 0; li < nlocal(); ++li) {  // the last two words (end of this / of the previous launch) persist
            cudaMemsetAsync((uint64_t *)dev_trace_ + (size_t)li * kTraceWords, 0, sizeof(uint64_t) * (kTraceWords - 2), (cudaStream_t)rq.stream);
            cudaMemsetAsync((uint64_t *)dev_trace_ + (size_t)li * kTraceWords, 0xff, 8, (cudaStream_t)rq.stream);
        }
    }
    if (settings_.transport == TR_DEVICE) {
        // map local index -> context: the plan may cover a subset of the local ranks (local Send/Recv)
        return launch_exec_plan((const RankCtx *)dev_ctx_, args.data(), nl, plan.nchan, rq.stream, plan.intra_rank_waits);
    }
    if (nl == 1) return exec_plan_host(ctx_[0], args[0]);
    std::vector<HcclResult> rcs(nl, HCCL_SUCCESS);
    std::vector<std::thread> th;
    for (int li = 0; li < nl; ++li) th.emplace_back([&, li] { rcs[li] = exec_plan_host(ctx_[li], args[li]); });
    for (auto &t : th) t.join();
    for (auto r : rcs)
        if (r != HCCL_SUCCESS) return r;
    return HCCL_SUCCESS;
}

HcclResult Communicator::check_ready()
{
    if (state_.load() == CS_SUSPENDED) return HCCL_E_SUSPENDING;
    for (auto *s : status_)
        if (s && s->code != 0) return (HcclResult)s->code;
    uint32_t re = remote_error_.load();
    if (re) return (HcclResult)re;
    return HCCL_SUCCESS;
}

Selection Communicator::select(int coll, uint64_t count, int dtype, int redop) const
{
    const EnvConfig &env = env_config();
    SelectInput si;
    si.coll = coll;
    si.bytes = count * (uint64_t)dtype_size(dtype);
    si.nranks = nranks_;
    si.dtype = dtype;
    si.redop = redop;
    si.deterministic = deterministic();
    si.nvls = nvls_;
    si.device = settings_.transport == TR_DEVICE;
    si.expansion_mode = settings_.expansion_mode ? settings_.expansion_mode : env.expansion_mode;
    si.max_channels = si.device ? (nranks_ == 1 ? 128 : 64) : 2;  // a single rank never waits: all SMs may copy
    si.forced = forced_algo_for(env, coll);
    si.ll_max_bytes = !ll_ok_ ? 0 : (coll == COLL_ALLREDUCE ? ll_max_bytes() : ll_block_max());
    Selection s = select_algo(si, model_);
    const int table_coll = coll == COLL_ALLGATHER_V ? COLL_ALLGATHER : (coll == COLL_REDUCE_SCATTER_V ? COLL_REDUCE_SCATTER : coll);
    auto tt = tuned_.find(table_coll);
    if (tt != tuned_.end() && !tt->second.sizes.empty() && si.forced.empty() && nranks_ > 1 && si.device) {
        // nearest bucket on a log scale; candidates must be legal for this dtype / op / determinism setting
        const TunedTable &tb = tt->second;
        size_t best_b = 0;
        double best_d = 1e300;
        for (size_t b = 0; b < tb.sizes.size(); ++b) {
            double d = std::fabs(std::log2((double)std::max<uint64_t>(si.bytes, 1)) - std::log2((double)tb.sizes[b]));
            if (d < best_d) { best_d = d; best_b = b; }
        }
        const bool reducing = table_coll == COLL_ALLREDUCE || table_coll == COLL_REDUCE_SCATTER;
        const bool nvls_ok = nvls_ && !si.deterministic && si.expansion_mode != 1 &&
                             (reducing ? nvls_reduce_supported(dtype, redop, si.bytes) : si.bytes % 16 == 0);
        const bool is_v = coll != table_coll;  // the V variants have plain schedules only
        double bt = -1;
        for (int a = 0; a < ALGO_COUNT; ++a) {
            double t = tb.us[best_b][a];
            if (t <= 0) continue;
            if ((a == ALGO_NVLS || a == ALGO_NVLS_ONESHOT || a == ALGO_NVLS_PIPE) && !nvls_ok) continue;
            if (a == ALGO_LL && (si.bytes > si.ll_max_bytes || si.expansion_mode == 1 || is_v)) continue;
            if ((a == ALGO_MESH_PIPE || a == ALGO_NVLS_PIPE) && (is_v || si.expansion_mode == 1)) continue;
            if (is_v && (a == ALGO_RHD || a == ALGO_PAIRWISE) && coll == COLL_REDUCE_SCATTER_V) continue;
            if (bt < 0 || t < bt) { bt = t; s.algo = a; }
        }
        if (bt > 0) s.est_us = bt;
    }
    if (env.channels > 0) s.nchan = env.channels;
    if (all_local_ && si.device) {
        // virtual ranks share one GPU: all CTAs of all ranks must be resident together (cooperative launch)
        int cap = std::max(1, 128 / std::max(1, nranks_));
        s.nchan = std::min(s.nchan, cap);
    }
    return s;
}

void Communicator::record_trace(const OpRequest &rq, int algo, int nchan, uint64_t bytes, double us)
{
    std::lock_guard<std::mutex> lk(trace_mu_);
    TraceRecord &t = trace_[trace_pos_++ % kTraceCap];
    t.seq = seq_;
    t.coll = rq.coll; t.algo = algo; t.nchan = nchan;
    t.count = rq.count; t.bytes = bytes; t.dtype = rq.dtype; t.redop = rq.redop; t.root = rq.root;
    t.host_us = us;
}
std::vector<TraceRecord> Communicator::trace_snapshot()
{
    std::lock_guard<std::mutex> lk(trace_mu_);
    std::vector<TraceRecord> out;
    size_t n = std::min(trace_pos_, kTraceCap);
    for (size_t i = 0; i < n; ++i) out.push_back(trace_[(trace_pos_ - n + i) % kTraceCap]);
    return out;
}
std::string Communicator::stats_json()
{
    std::ostringstream o;
    o << "{\"name\":\"" << name_ << "\",\"ranks\":" << nranks_ << ",\"rank\":" << rank() << ",\"nvls\":" << (nvls_ ? 1 : 0)
      << ",\"launches\":" << stats_.launches << ",\"plans_built\":" << stats_.plans_built << ",\"retries\":" << stats_.retries
      << ",\"timeouts\":" << stats_.timeouts << ",\"ops\":{";
    bool first = true;
    for (int c = 0; c < COLL_COUNT; ++c) {
        if (!stats_.ops[c]) continue;
        o << (first ? "" : ",") << "\"" << coll_name(c) << "\":{\"calls\":" << stats_.ops[c] << ",\"bytes\":" << stats_.bytes[c] << "}";
        first = false;
    }
    o << "},\"algos\":{";
    first = true;
    for (int a = 0; a < ALGO_COUNT; ++a) {
        if (!stats_.algo_hist[a]) continue;
        o << (first ? "" : ",") << "\"" << algo_name(a) << "\":" << stats_.algo_hist[a];
        first = false;
    }
    o << "},\"model\":{\"alpha_us\":" << model_.alpha_us << ",\"beta_gbps\":" << model_.beta_gbps << ",\"nvls_gbps\":" << model_.nvls_gbps
      << ",\"gamma_gbps\":" << model_.gamma_gbps << ",\"launch_us\":" << model_.launch_us << ",\"measured\":" << (tuned_.empty() ? "false" : "true") << "}";
    // measured selection tables: per collective the size ladder and, per algorithm that was timed, microseconds per size
    o << ",\"tuned\":{";
    first = true;
    for (auto &kv : tuned_) {
        o << (first ? "" : ",") << "\"" << coll_name(kv.first) << "\":{\"sizes\":[";
        for (size_t b = 0; b < kv.second.sizes.size(); ++b) o << (b ? "," : "") << kv.second.sizes[b];
        o << "],\"us\":{";
        bool fa = true;
        for (int a = 0; a < ALGO_COUNT; ++a) {
            bool any = false;
            for (auto &row : kv.second.us) any = any || row[a] > 0;
            if (!any) continue;
            o << (fa ? "" : ",") << "\"" << algo_name(a) << "\":[";
            for (size_t b = 0; b < kv.second.us.size(); ++b) o << (b ? "," : "") << (double)((long long)(kv.second.us[b][a] * 10 + 0.5)) / 10.0;
            o << "]";
            fa = false;
        }
        o << "}}";
        first = false;
    }
    o << "}}";
    return o.str();
}

// ------------------------------------------------------------------------------------------------ buffer overlap
// Byte ranges that a collective reads and writes on one rank, from the semantics of its count argument (reference:
// IsHcclOpInplace, algorithm/impl/coll_alg_utils.cc:253-307: AllGather writes p * count, ReduceScatter reads p * count,
// rooted ops touch the large side on the root only).
static void op_byte_ranges(const OpRequest &rq, int p, int rank, uint64_t *in_bytes, uint64_t *out_bytes)
{
    const uint64_t n = rq.count * (uint64_t)dtype_size(rq.dtype);
    uint64_t vin = 0, vout = 0;
    auto span = [&](const uint64_t *counts, const uint64_t *displs) {
        uint64_t hi = 0;
        for (int j = 0; j < p; ++j) hi = std::max(hi, displs[j] + counts[j]);
        return hi * (uint64_t)dtype_size(rq.dtype);
    };
    switch (rq.coll) {
        case COLL_ALLREDUCE: vin = vout = n; break;
        case COLL_BROADCAST: vin = rank == rq.root ? n : 0; vout = rank == rq.root ? 0 : n; break;  // one buffer: never "overlapping"
        case COLL_REDUCE: vin = n; vout = rank == rq.root ? n : 0; break;
        case COLL_ALLGATHER: vin = n; vout = n * p; break;
        case COLL_REDUCE_SCATTER: vin = n * p; vout = n; break;
        case COLL_GATHER: vin = n; vout = rank == rq.root ? n * p : 0; break;
        case COLL_SCATTER: vin = rank == rq.root ? n * p : 0; vout = n; break;
        case COLL_ALLTOALL: vin = vout = n * p; break;
        case COLL_ALLGATHER_V: vin = rq.counts[rank] * (uint64_t)dtype_size(rq.dtype); vout = span(rq.counts, rq.displs); break;
        case COLL_REDUCE_SCATTER_V: vin = span(rq.counts, rq.displs); vout = rq.counts[rank] * (uint64_t)dtype_size(rq.dtype); break;
        default: break;  // AlltoAllV / VC: checked against their own displacement tables by the API layer
    }
    *in_bytes = vin;
    *out_bytes = vout;
}

// 0: the buffers of local rank li are disjoint; 1: they overlap in the one form the op defines as "in place" (same
// pointer, or the rank's own block at its position inside the larger buffer); 2: any other overlap.
int Communicator::overlap_kind(const OpRequest &rq, int li) const
{
    if (!rq.in || !rq.out || !rq.in[li] || !rq.out[li]) return 0;
    const int p = nranks_, r = local_ranks_[li];
    uint64_t ib = 0, ob = 0;
    op_byte_ranges(rq, p, r, &ib, &ob);
    if (ib == 0 || ob == 0) return 0;
    const uint8_t *a = (const uint8_t *)rq.in[li], *b = (const uint8_t *)rq.out[li];
    if (a + ib <= b || b + ob <= a) return 0;
    const uint64_t n = rq.count * (uint64_t)dtype_size(rq.dtype);
    switch (rq.coll) {
        case COLL_ALLREDUCE: case COLL_REDUCE: return a == b ? 1 : 2;
        case COLL_ALLGATHER: return a == b + (uint64_t)r * n ? 1 : 2;
        case COLL_REDUCE_SCATTER: return b == a + (uint64_t)r * n ? 1 : 2;
        case COLL_GATHER: return a == b + (uint64_t)r * n ? 1 : 2;
        case COLL_SCATTER: return b == a + (uint64_t)r * n ? 1 : 2;
        case COLL_ALLGATHER_V: return a == b + rq.displs[r] * (uint64_t)dtype_size(rq.dtype) ? 1 : 2;
        case COLL_REDUCE_SCATTER_V: return b == a + rq.displs[r] * (uint64_t)dtype_size(rq.dtype) ? 1 : 2;
        default: return 2;
    }
}

// ------------------------------------------------------------------------------------------------ collectives
HcclResult Communicator::collective(const OpRequest &rq)
{
    std::lock_guard<std::mutex> lk(op_mu_);
    double t0 = now_us();
    ++op_index_;
    if (!calibrating_) {
        fault::before_op(rank(), op_index_);
        if (fault_hook_) fault_hook_(op_index_);
    }
    HcclResult ready = check_ready();
    const bool dev = settings_.transport == TR_DEVICE;
    const bool can_retry = env_config().retry_enable && !all_local_ && nranks_ > 1 && (ready == HCCL_E_TIMEOUT || ready == HCCL_E_REMOTE);
    bool own_fail = false;
    for (auto *st : status_) own_fail = own_fail || (st && st->code != 0);
    if (ready != HCCL_SUCCESS && can_retry && dev && own_fail) {
        // device transport: a kernel reports its failure after the call that launched it has returned, so the op to run
        // again is the previous one; the current op follows once that one has gone through
        HcclResult rr = retry_last_op(ready);
        if (rr != HCCL_SUCCESS) return rr;
        ready = HCCL_SUCCESS;
    }
    // a failure reported by a peer while this rank was between ops (its own kernels all finished) is a failure of the op it
    // is about to start, which the peer has launched already: with operator retry enabled the rank joins the peers' retry
    // round for this op instead of giving up
    bool peer_failed = ready != HCCL_SUCCESS && remote_error_.load() == (uint32_t)ready && can_retry;
    if (ready != HCCL_SUCCESS && !peer_failed) return ready;
    for (int li = 0; li < nlocal(); ++li)
        CHK_RET_LOG(overlap_kind(rq, li) == 2, HCCL_E_PARA,
                    "%s: send and receive buffers of rank %d overlap in a way the operation does not define (in place means the same "
                    "pointer, or the rank's own block at its position of the larger buffer)", coll_name(rq.coll), local_ranks_[li]);
    StateGuard guard(state_, CS_INUSE);
    const bool nvtx = env_config().nvtx;
    if (nvtx) nvtxRangePushA(coll_name(rq.coll));
    if (dev && !calibrating_) remember_op(rq);
    HcclResult rc = peer_failed ? ready : run_collective_once(rq);
    if (rc != HCCL_SUCCESS && (rc == HCCL_E_TIMEOUT || rc == HCCL_E_REMOTE)) {
        stats_.timeouts++;
        rc = maybe_retry(rq, rc, op_index_);
    }
    if (rc == HCCL_SUCCESS && env_config().overflow_check) rc = overflow_scan(rq);
    if (nvtx) nvtxRangePop();
    if (env_config().entry_log)
        HLOG_RUN("%s count=%llu dtype=%d op=%d root=%d -> %d, took %.1f us", coll_name(rq.coll), (unsigned long long)rq.count,
                 rq.dtype, rq.redop, rq.root, (int)rc, now_us() - t0);
    return rc;
}

HcclResult Communicator::run_collective_once(const OpRequest &rq)
{
    const int p = nranks_, nl = nlocal();
    const int es = dtype_size(rq.dtype);
    double t0 = now_us();
    bool is_v = rq.coll == COLL_ALLGATHER_V || rq.coll == COLL_REDUCE_SCATTER_V;
    bool is_a2av = rq.coll == COLL_ALLTOALLV || rq.coll == COLL_ALLTOALLVC;
    // total window over which the staging loop iterates (elements)
    uint64_t window = rq.count;
    if (is_v) {
        window = 0;
        for (int j = 0; j < p; ++j) window = std::max(window, rq.counts[j]);
    }
    uint64_t sel_count = rq.count;
    if (rq.coll == COLL_ALLTOALL) sel_count = rq.count * p;
    if (is_a2av) {
        sel_count = 0;
        for (int j = 0; j < p; ++j) sel_count += rq.send_counts[j];
    }
    if (is_v) sel_count = window;
    Selection sel = select(rq.coll, sel_count, rq.dtype, rq.redop);
    if (rq.algo != ALGO_AUTO) sel.algo = rq.algo;
    if (rq.nchan > 0) sel.nchan = rq.nchan;
    if (p == 1) sel.algo = ALGO_SINGLE;
    if (rq.coll == COLL_BARRIER) { sel.algo = p == 1 ? ALGO_SINGLE : ALGO_MESH; sel.nchan = 1; }
    // zero-copy: both buffers of every local rank inside registered symmetric memory with a multicast mapping.  The decision
    // is made from this rank's own lookup and nothing else: registration is collective, and a collective whose buffers lie in
    // registered memory has to be called with the same (allocation, offset) pair on every rank (the contract of symmetric
    // memory).  No agreement round per call, so no rank can wait alone in one; a caller that breaks the contract is caught
    // by the consistency check below, whose frame carries the algorithm and the offsets.
    struct ZcInfo { int hin = 0, hout = 0; size_t oin = 0, oout = 0; };
    std::vector<ZcInfo> zc(nl);
    bool use_zc = false;
    const bool host_tr = settings_.transport == TR_HOST;  // the host executor emulates the multicast accesses rank by rank
    // (two ranks: the in-switch reduction gains nothing over reading the one peer directly, which the peer-mapping form below does)
    if (rq.coll == COLL_ALLREDUCE && (p > 2 || (p == 2 && (rq.algo == ALGO_NVLS_ZC || host_tr))) && (nvls_ || host_tr) && !user_segs_.empty() &&
        (rq.algo == ALGO_AUTO || rq.algo == ALGO_NVLS_ZC) &&
        // (below 4 MiB the LL kernels are faster than the in-switch round trip even on registered buffers: measured on 4 GPUs)
        (rq.algo == ALGO_NVLS_ZC || rq.count * es >= (ll_ok_ && !host_tr ? (4u << 20) : (512u << 10))) && !deterministic() &&
        nvls_reduce_supported(rq.dtype, rq.redop, rq.count * es) && forced_algo_for(env_config(), rq.coll).empty()) {
        bool mine = true;
        for (int li = 0; li < nl && mine; ++li) {
            zc[li].hin = find_user_seg(li, rq.in[li], rq.count * es, &zc[li].oin);
            zc[li].hout = find_user_seg(li, rq.out[li], rq.count * es, &zc[li].oout);
            mine = zc[li].hin && zc[li].hout && (host_tr || (user_segs_[zc[li].hin][li].mc && user_segs_[zc[li].hout][li].mc)) &&
                   ((zc[li].oin | zc[li].oout) & 15) == 0;
            // virtual ranks of one process: the same pair on every local rank
            mine = mine && zc[li].hin == zc[0].hin && zc[li].hout == zc[0].hout && zc[li].oin == zc[0].oin && zc[li].oout == zc[0].oout;
        }
        use_zc = mine;
        CHK_RET_LOG(rq.algo == ALGO_NVLS_ZC && !use_zc, HCCL_E_PARA, "zero-copy AllReduce needs both buffers in registered symmetric memory at the same offsets on every rank");
        if (use_zc) {
            sel.algo = ALGO_NVLS_ZC;
            // nothing but the switch is busy in this path: more CTAs keep more multimem requests in flight
            int zch = all_local_ ? sel.nchan : 64;
            if (const char *e = getenv("HCCL_ZC_CHANNELS")) zch = std::max(1, std::min(atoi(e), kMaxChannels));
            if (rq.nchan <= 0 && rq.count * es >= (8u << 20)) sel.nchan = zch;
        }
    } else {
        CHK_RET_LOG(rq.algo == ALGO_NVLS_ZC, HCCL_E_NOT_SUPPORT, "zero-copy AllReduce needs NVLS, registered buffers, a reducible dtype/op pair and a multiple of 16 bytes");
    }
    if ((sel.algo == ALGO_NVLS || sel.algo == ALGO_NVLS_ONESHOT || sel.algo == ALGO_NVLS_PIPE) && !nvls_) {
        HLOG_ERROR("NVLS algorithm requested but no multicast mapping exists on this communicator");
        return HCCL_E_NOT_SUPPORT;
    }
    if (is_a2av) CHK_RET(a2av_check(rq));
    CHK_RET(consistency_check(rq, sel.algo, use_zc ? ((uint64_t)zc[0].hin << 48) ^ zc[0].oin : 0, use_zc ? ((uint64_t)zc[0].hout << 48) ^ zc[0].oout : 0));
    if (sel.algo == ALGO_LL) {
        const bool blocked = rq.coll == COLL_REDUCE_SCATTER || rq.coll == COLL_ALLGATHER;  // count = one rank's block
        bool fits = ll_ok_ && ((rq.coll == COLL_ALLREDUCE && rq.count * es <= ll_max_bytes()) || (blocked && rq.count * es <= ll_block_max()));
        if (fits) {
            HcclResult lrc = run_ll_allreduce(rq);
            stats_.ops[rq.coll]++;
            stats_.bytes[rq.coll] += rq.count * es;
            stats_.algo_hist[ALGO_LL]++;
            record_trace(rq, ALGO_LL, 0, rq.count * es, now_us() - t0);
            return lrc;
        }
        CHK_RET_LOG(rq.algo == ALGO_LL && !ll_ok_, HCCL_E_NOT_SUPPORT, "the LL kernels need the device transport and more than one rank");
        CHK_RET_LOG(rq.algo == ALGO_LL && !blocked && rq.coll != COLL_ALLREDUCE, HCCL_E_NOT_SUPPORT, "the LL protocol exists for AllReduce, ReduceScatter and AllGather");
        sel.algo = blocked ? ALGO_MESH : ALGO_MESH_ONESHOT;  // oversized (a decision every rank makes alike: it depends on the count only)
    }

    // registered send buffer (the same allocation and offset on every rank, by the contract of symmetric memory): two-rank
    // AllReduce, ReduceScatter and AllGather let the peers read it where it is
    if (!use_zc && settings_.transport == TR_DEVICE && p > 1 && !user_segs_.empty() && (rq.algo == ALGO_AUTO || rq.algo == ALGO_MESH_ZC) &&
        ((rq.coll == COLL_ALLREDUCE && p == 2) || rq.coll == COLL_REDUCE_SCATTER || rq.coll == COLL_ALLGATHER) &&
        (rq.algo == ALGO_MESH_ZC || rq.count * es >= (1u << 20)) && forced_algo_for(env_config(), rq.coll).empty()) {
        const size_t in_bytes = (size_t)rq.count * es * (rq.coll == COLL_REDUCE_SCATTER ? p : 1);
        int h0 = 0;
        size_t o0 = 0;
        bool mine = true;
        for (int li = 0; li < nl && mine; ++li) {
            size_t o = 0;
            int h = find_user_seg(li, rq.in[li], in_bytes, &o);
            if (li == 0) { h0 = h; o0 = o; }
            mine = h != 0 && h == h0 && o == o0 && (o & 15) == 0;
            // AllReduce in place would overwrite what the peer is still reading: that form stays on the staged paths
            if (rq.coll == COLL_ALLREDUCE && overlap_kind(rq, li) != 0) mine = false;
        }
        if (mine) {
            CHK_RET(consistency_check(rq, ALGO_MESH_ZC, ((uint64_t)h0 << 48) ^ o0, 0));
            HcclResult zrc = run_pipe(rq, false, h0, o0);
            uint64_t zbytes = sel_count * es;
            stats_.ops[rq.coll]++;
            stats_.bytes[rq.coll] += zbytes;
            stats_.algo_hist[ALGO_MESH_ZC]++;
            record_trace(rq, ALGO_MESH_ZC, 0, zbytes, now_us() - t0);
            return zrc;
        }
        CHK_RET_LOG(rq.algo == ALGO_MESH_ZC, HCCL_E_PARA, "zero-copy needs the send buffer in registered symmetric memory at the same offset on every rank");
    }
    CHK_RET_LOG(rq.algo == ALGO_MESH_ZC, HCCL_E_NOT_SUPPORT, "zero-copy over peer mappings exists for two-rank AllReduce, ReduceScatter and AllGather on the device transport");
    if ((is_a2av || rq.coll == COLL_ALLTOALL) && settings_.transport == TR_DEVICE && p > 1 && (rq.algo == ALGO_AUTO || rq.algo == ALGO_DIRECT) &&
        forced_algo_for(env_config(), rq.coll).empty()) {
        HcclResult arc = run_a2av(rq);
        uint64_t abytes = sel_count * es;
        stats_.ops[rq.coll]++;
        stats_.bytes[rq.coll] += abytes;
        stats_.algo_hist[ALGO_DIRECT]++;
        record_trace(rq, ALGO_DIRECT, 0, abytes, now_us() - t0);
        return arc;
    }
    CHK_RET_LOG(rq.algo == ALGO_DIRECT || sel.algo == ALGO_DIRECT, HCCL_E_NOT_SUPPORT, "the parametric AlltoAll kernel needs the device transport and more than one rank");
    if (sel.algo == ALGO_MESH_PIPE || sel.algo == ALGO_NVLS_PIPE) {
        if (settings_.transport == TR_DEVICE && pipe_mode_for(rq.coll) >= 0) {
            HcclResult prc = run_pipe(rq, sel.algo == ALGO_NVLS_PIPE);
            uint64_t pbytes = sel_count * es;
            stats_.ops[rq.coll]++;
            stats_.bytes[rq.coll] += pbytes;
            stats_.algo_hist[sel.algo]++;
            record_trace(rq, sel.algo, 0, pbytes, now_us() - t0);
            return prc;
        }
        // CPU ranks have no pipelined executor: the plain schedule of the same family moves the same bytes
        const bool mc = sel.algo == ALGO_NVLS_PIPE;
        sel.algo = rq.coll == COLL_REDUCE ? ALGO_TREE : rq.coll == COLL_BROADCAST ? (mc ? ALGO_NVLS : ALGO_RING) : (mc ? ALGO_NVLS : ALGO_MESH);
    }

    OpDesc d;
    d.coll = rq.coll; d.algo = sel.algo; d.nranks = p; d.root = rq.root; d.dtype = rq.dtype; d.redop = rq.redop;
    d.nchan = sel.nchan; d.count = rq.count;
    if (is_v) { d.counts.assign(rq.counts, rq.counts + p); d.displs.assign(rq.displs, rq.displs + p); }
    if (is_a2av) {
        d.send_counts.assign(rq.send_counts, rq.send_counts + (size_t)nl * p);
        d.send_displs.assign(rq.send_displs, rq.send_displs + (size_t)nl * p);
        d.recv_counts.assign(rq.recv_counts, rq.recv_counts + (size_t)nl * p);
        d.recv_displs.assign(rq.recv_displs, rq.recv_displs + (size_t)nl * p);
        d.slot_bytes = (settings_.stage_half_bytes / p) / 256 * 256;
        CHK_RET_LOG(d.slot_bytes < 256, HCCL_E_MEMORY, "staging buffer too small for AlltoAllV over %d ranks", p);
    }
    std::vector<const void *> in(nl);
    std::vector<void *> out(nl);
    for (int li = 0; li < nl; ++li) { in[li] = rq.in ? rq.in[li] : nullptr; out[li] = rq.out ? rq.out[li] : nullptr; }

    // staging loop (reference: CollAllReduceExecutor::RunLoop, coll_all_reduce_executor.cc:160-211)
    uint64_t max_chunk = window;
    if (!is_a2av && rq.coll != COLL_BARRIER && p > 1) {
        d.chunk_off = 0; d.chunk_count = window;
        if (plan_stage_bytes(d) > settings_.stage_half_bytes) {
            uint64_t lo = 1, hi = window;
            while (lo < hi) {
                uint64_t mid = lo + (hi - lo + 1) / 2;
                d.chunk_count = mid;
                if (plan_stage_bytes(d) <= settings_.stage_half_bytes) lo = mid; else hi = mid - 1;
            }
            uint64_t vec = es >= 16 ? 1 : 16 / es;
            max_chunk = lo > vec ? lo / vec * vec : lo;
            d.chunk_count = max_chunk;
            CHK_RET_LOG(plan_stage_bytes(d) > settings_.stage_half_bytes, HCCL_E_MEMORY, "staging buffer too small for one element per rank");
        }
    }
    HcclResult rc = HCCL_SUCCESS;
    uint64_t off = 0;
    do {
        uint64_t n = std::min(max_chunk, window - off);
        d.chunk_off = off; d.chunk_count = n;
        std::ostringstream key;
        key << rq.coll << ':' << d.algo << ':' << d.nchan << ':' << rq.dtype << ':' << rq.root << ':' << rq.count << ':' << off << ':' << n;
        if (is_v) for (int j = 0; j < p; ++j) key << ',' << d.counts[j] << '@' << d.displs[j];
        if (is_a2av) {
            uint32_t crc = crc32(d.send_counts.data(), d.send_counts.size() * 8, 0);
            crc = crc32(d.send_displs.data(), d.send_displs.size() * 8, crc);
            crc = crc32(d.recv_counts.data(), d.recv_counts.size() * 8, crc);
            crc = crc32(d.recv_displs.data(), d.recv_displs.size() * 8, crc);
            key << ",a2av" << crc << '/' << d.send_counts.size();
            for (size_t i = 0; i < std::min<size_t>(d.send_counts.size(), 4); ++i) key << '.' << d.send_counts[i];
        }
        CachedPlan *cp = nullptr;
        CHK_RET(get_plan(d, key.str(), &cp));
        zc_args_.clear();
        if (use_zc)
            for (int li = 0; li < nl; ++li)
                zc_args_.push_back({(uint8_t *const *)user_peer_tabs_[zc[li].hin][li], (uint8_t *const *)user_peer_tabs_[zc[li].hout][li],
                                    user_segs_[zc[li].hin][li].mc, user_segs_[zc[li].hout][li].mc, zc[li].oin, zc[li].oout});
        rc = run_plan(cp->plan, cp->dev_steps.data(), rq, seq_, rq.dtype, rq.redop, true, in, out);
        zc_args_.clear();
        ++seq_;
        if (rc != HCCL_SUCCESS) break;
        off += n;
    } while (off < window);
    uint64_t bytes = sel_count * es;
    stats_.ops[rq.coll]++;
    stats_.bytes[rq.coll] += bytes;
    stats_.algo_hist[sel.algo]++;
    record_trace(rq, sel.algo, sel.nchan, bytes, now_us() - t0);
    return rc;
}

int Communicator::pipe_mode_for(int coll) const
{
    switch (coll) {
        case COLL_ALLREDUCE: return nranks_ == 2 ? PM_AR1_PUSH : PM_AR2_PUSH;  // two ranks: one-shot moves the same bytes and saves a stage
        case COLL_REDUCE_SCATTER: return PM_RS_PUSH;
        case COLL_ALLGATHER: return PM_AG_PULL;
        case COLL_BROADCAST: return PM_BC_PUSH;
        case COLL_REDUCE: return PM_RD_PUSH;
        default: return -1;
    }
}

// Pipelined large-message path: one launch for a message of any size (the ring of staging slots replaces the staging
// loop).  Geometry: a chunk moves 8 MiB over the links (half the message below 16 MiB): a stage's per-chunk bookkeeping
// (completion of the bulk copies, fence, flag hop: several microseconds) has to stay small against the chunk's transfer
// time.  (Shorter chunks at both ends of the message, to fill and drain the pipeline sooner, measured slower: the flag
// hops of the extra chunks cost more than the fill saves.)  Every choice below depends only on facts that all ranks share (sizes, type, operator,
// environment), never on a rank's own pointers: the kernels take unaligned buffers on slower paths instead.
HcclResult Communicator::run_pipe(const OpRequest &rq, bool want_mc, int zc_handle, size_t zc_off)
{
    const EnvConfig &env = env_config();
    const int p = nranks_, nl = nlocal(), es = dtype_size(rq.dtype);
    int mode = pipe_mode_for(rq.coll);
    if (zc_handle) {
        // the send buffers are registered: one round, no staging; one gate CTA plus as many readers as 64 KiB pieces justify
        mode = rq.coll == COLL_ALLREDUCE ? PM_AR1_ZC : (rq.coll == COLL_REDUCE_SCATTER ? PM_RS_ZC : PM_AG_ZC);
        const uint64_t bytes = rq.count * (uint64_t)es * (mode == PM_AG_ZC ? (uint64_t)(p - 1) : 1);
        const int budget = all_local_ ? std::max(2, 128 / nl) : 128;
        const int readers = (int)std::max<uint64_t>(1, std::min<uint64_t>((uint64_t)budget - 1, bytes / (64u << 10)));
        std::vector<PipeArgs> zargs(nl);
        for (int li = 0; li < nl; ++li) {
            PipeArgs &a = zargs[li];
            memset(&a, 0, sizeof(a));
            a.in = (const uint8_t *)rq.in[li];
            a.out = (uint8_t *)rq.out[li];
            a.count = rq.count; a.chunk_elems = std::max<uint64_t>(1, rq.count); a.seq = seq_;
            a.mode = mode; a.dtype = rq.dtype; a.root = rq.root; a.nslots = 1;
            a.n1 = 1; a.n2 = readers; a.n3 = 0; a.g1 = a.g2 = a.g3 = 1;
            a.z_in_peer = (const uint8_t *const *)user_peer_tabs_[zc_handle][li];
            a.z_in_off = zc_off;
            __atomic_store_n(&status_[li]->head, (uint64_t)seq_, __ATOMIC_RELAXED);
        }
        stats_.launches++;
        HcclResult zrc = launch_pipe_coll((const RankCtx *)dev_ctx_, zargs.data(), nl, rq.redop, rq.stream);
        ++seq_;
        return zrc;
    }
    const uint64_t block_bytes = rq.count * (uint64_t)es;
    const bool reducing = rq.coll == COLL_ALLREDUCE || rq.coll == COLL_REDUCE_SCATTER;
    const bool use_mc = want_mc && nvls_ && block_bytes % 16 == 0 && (!reducing || nvls_reduce_supported(rq.dtype, rq.redop, block_bytes)) && !deterministic();
    if (use_mc) {
        if (mode == PM_AR2_PUSH) mode = PM_AR2_MC;
        else if (mode == PM_AR1_PUSH) mode = PM_AR1_MC;
        else if (mode == PM_RS_PUSH) mode = PM_RS_MC;
        else if (mode == PM_BC_PUSH) mode = PM_BC_MC;
    }
    // a chunk of ce elements per block moves about fan * ce elements over a rank's links
    const uint64_t fan = (pipe_mode_has_copy_out(mode) || pipe_mode_is_bcast(mode)) ? 1 : (uint64_t)(p - 1);
    uint64_t link_total = block_bytes * fan;
    uint64_t lc = env.pipe_chunk_bytes ? env.pipe_chunk_bytes : std::min<uint64_t>(8u << 20, std::max<uint64_t>(1u << 20, link_total / 2));
    int nslots = env.pipe_slots > 0 ? std::min(env.pipe_slots, kPipeMaxSlots) : kPipeMaxSlots;
    // elements: slices of a chunk stay 256-byte aligned (Reduce cuts a chunk into p - 1 slices and a slot into p - 1 source areas)
    const uint64_t unit = (mode == PM_RD_PUSH ? (uint64_t)p * std::max(1, p - 1) : (uint64_t)p) * (256 / es);
    auto slot_of = [&](uint64_t ce) { return pipe_slot_bytes(mode, ce, es, p); };
    uint64_t ce = std::max<uint64_t>(unit, lc / fan / es / unit * unit);
    while (nslots > 4 && slot_of(ce) * nslots > settings_.stage_half_bytes) --nslots;
    while (ce > unit && slot_of(ce) * nslots > settings_.stage_half_bytes) ce = std::max<uint64_t>(unit, ce / 2 / unit * unit);
    while (nslots > 1 && slot_of(ce) * nslots > settings_.stage_half_bytes) --nslots;
    CHK_RET_LOG(slot_of(ce) * nslots > settings_.stage_half_bytes, HCCL_E_MEMORY, "staging buffer too small for the pipelined kernels");
    while (ceil_div_u64(rq.count, ce) >= (1ull << kSeqShift) - 1) ce *= 2;  // chunk index travels in the low flag bits
    CHK_RET_LOG(slot_of(ce) * nslots > settings_.stage_half_bytes, HCCL_E_MEMORY, "message needs more pipeline chunks than a flag can count");
    // CTAs per stage.  A copy-engine driven CTA moves about 45 GB/s whatever the direction, so a stage that has to carry
    // the full link rate needs 16 to 32 of them; the reduce stage gets what is left of the 128.  No more CTAs than 16 KiB
    // pieces justify.
    const int budget = all_local_ ? std::max(3, 128 / nl) : 128;
    const bool three = pipe_mode_has_copy_out(mode), bc = pipe_mode_is_bcast(mode);
    int n[3] = {0, 0, 0}, g[3] = {1, 1, 1};
    if (three) { n[0] = std::max(1, budget / 4); n[2] = std::max(1, budget / 4); n[1] = budget - n[0] - n[2]; }
    else if (bc) { n[0] = std::max(1, budget / 4); }
    else if (mode == PM_AG_PULL) { n[0] = std::max(1, budget / 8); n[1] = std::max(1, budget / 2); }
    else { n[0] = std::max(1, budget / 4); n[1] = budget - n[0]; }
    if (env.pipe_ctas[0] > 0) { n[0] = env.pipe_ctas[0]; n[1] = env.pipe_ctas[1]; n[2] = env.pipe_ctas[2]; }
    if (bc) n[1] = n[2] = 0;
    if (!three) n[2] = 0;
    const uint64_t chunk_bytes = std::min(ce, rq.count) * (uint64_t)es;
    auto cap = [&](int v, uint64_t bytes) { return (int)std::max<uint64_t>(1, std::min<uint64_t>((uint64_t)std::max(1, v), bytes / (16u << 10))); };
    const bool rs = mode == PM_RS_MC || mode == PM_RS_PUSH;
    n[0] = cap(n[0], chunk_bytes * (rs ? p : 1));
    if (three) { n[1] = cap(n[1], chunk_bytes / p); n[2] = cap(n[2], chunk_bytes); }
    else if (!bc) n[1] = cap(n[1], chunk_bytes * (mode == PM_AG_PULL ? p - 1 : 1));
    // groups: two or three chunks in flight per stage hide a stage's flag traffic behind its transfers
    const uint64_t nchunks = ceil_div_u64(rq.count, ce);
    for (int i = 0; i < 3; ++i) {
        int want = env.pipe_groups[i] > 0 ? env.pipe_groups[i] : (i == 1 && !bc ? 4 : 2);
        while (want > 1 && (n[i] % want != 0 || (uint64_t)want > nchunks)) --want;
        g[i] = std::max(1, want);
    }
    std::vector<PipeArgs> args(nl);
    for (int li = 0; li < nl; ++li) {
        PipeArgs &a = args[li];
        memset(&a, 0, sizeof(a));
        a.in = (const uint8_t *)rq.in[li];
        a.out = (uint8_t *)rq.out[li];
        a.count = rq.count; a.chunk_elems = ce; a.seq = seq_;
        a.mode = mode; a.dtype = rq.dtype; a.root = rq.root; a.nslots = nslots;
        a.n1 = n[0]; a.n2 = n[1]; a.n3 = n[2]; a.g1 = g[0]; a.g2 = g[1]; a.g3 = g[2];
        __atomic_store_n(&status_[li]->head, (uint64_t)seq_, __ATOMIC_RELAXED);
    }
    stats_.launches++;
    if (dev_trace_)
        for (int li = 0; li < nl; ++li) {
            cudaMemsetAsync((uint64_t *)dev_trace_ + (size_t)li * kTraceWords, 0, sizeof(uint64_t) * (kTraceWords - 2), (cudaStream_t)rq.stream);
            cudaMemsetAsync((uint64_t *)dev_trace_ + (size_t)li * kTraceWords, 0xff, 8, (cudaStream_t)rq.stream);
        }
    HcclResult rc = launch_pipe_coll((const RankCtx *)dev_ctx_, args.data(), nl, rq.redop, rq.stream);
    ++seq_;
    return rc;
}

// AlltoAll / AlltoAllV / AlltoAllVC on the device transport: the parametric kernel (kernels/a2av.cu).  Counts and
// displacements go into the launch arguments; nothing is built, allocated or copied to the device for a new count matrix.
HcclResult Communicator::run_a2av(const OpRequest &rq)
{
    const int p = nranks_, nl = nlocal(), es = dtype_size(rq.dtype);
    // lanes per ordered pair: all CTAs of a launch must fit the GPU at once when virtual ranks share it
    // (a copy-engine driven CTA moves about 45 GB/s: 16 to 32 sending CTAs per rank carry the link rate; the lane count is
    // part of the slot layout on the receiver, so it depends on the rank count only, never on a rank's own counts)
    int lanes = std::max(1, std::min(kA2avMaxLanes, 128 / (2 * p * nl)));
    uint64_t sub = std::min<uint64_t>(2u << 20, settings_.stage_half_bytes / ((uint64_t)p * lanes * 2)) / 256 * 256;
    while (sub < 4096 && lanes > 1) { --lanes; sub = std::min<uint64_t>(2u << 20, settings_.stage_half_bytes / ((uint64_t)p * lanes * 2)) / 256 * 256; }
    CHK_RET_LOG(sub < 256, HCCL_E_MEMORY, "staging buffer too small for AlltoAllV over %d ranks", p);
    std::vector<A2avArgs> args(nl);
    for (int li = 0; li < nl; ++li) {
        A2avArgs &a = args[li];
        memset(&a, 0, sizeof(a));
        a.in = (const uint8_t *)rq.in[li];
        a.out = (uint8_t *)rq.out[li];
        for (int j = 0; j < p; ++j) {
            if (rq.coll == COLL_ALLTOALL) {
                a.send_counts[j] = a.recv_counts[j] = rq.count;
                a.send_displs[j] = a.recv_displs[j] = (uint64_t)j * rq.count;
            } else {
                a.send_counts[j] = rq.send_counts[(size_t)li * p + j]; a.send_displs[j] = rq.send_displs[(size_t)li * p + j];
                a.recv_counts[j] = rq.recv_counts[(size_t)li * p + j]; a.recv_displs[j] = rq.recv_displs[(size_t)li * p + j];
            }
        }
        a.seq = seq_; a.sub_bytes = sub; a.dtype = rq.dtype; a.lanes = lanes;
        (void)es;
        __atomic_store_n(&status_[li]->head, (uint64_t)seq_, __ATOMIC_RELAXED);
    }
    stats_.launches++;
    HcclResult rc = launch_a2av((const RankCtx *)dev_ctx_, args.data(), nl, p, rq.stream);
    ++seq_;
    return rc;
}

uint64_t Communicator::ll_max_bytes() const
{
    return nranks_ >= 3 ? std::max<uint64_t>(kLlMaxPayload, ll_two_shot_max(nranks_)) : kLlMaxPayload;
}

HcclResult Communicator::run_ll_allreduce(const OpRequest &rq)
{
    int nl = nlocal();
    // two-shot from three ranks on once the message is large enough for the saved link bytes to pay for the second hop
    const uint64_t bytes = rq.count * (uint64_t)dtype_size(rq.dtype);
    uint32_t kind = nranks_ >= 3 && bytes >= ll_two_shot_min_ && bytes <= ll_two_shot_max(nranks_) ? LL_AR_TWOSHOT : LL_AR_ONESHOT;
    if (rq.coll == COLL_REDUCE_SCATTER) kind = LL_REDUCE_SCATTER;
    else if (rq.coll == COLL_ALLGATHER) kind = LL_ALLGATHER;
    ++ll_seq_;
    uint32_t tag = (uint32_t)(ll_seq_ & 0xffffffffu);
    if (tag == 0) { ++ll_seq_; tag = 1; }
    std::vector<LlArgs> args(nl);
    for (int li = 0; li < nl; ++li) {
        LlArgs &a = args[li];
        memset(&a, 0, sizeof(a));
        for (int q = 0; q < nranks_; ++q) a.ll[q] = ctx_[li].ll[q];
        a.in = rq.in[li];
        a.out = rq.out[li];
        a.count = rq.count;
        a.slot_bytes = kLlSlotBytes;
        a.timeout_ns = ctx_[li].timeout_ns;
        a.seq = seq_;
        a.status = status_[li];
        a.abort = abort_[li];
        a.local_fail = ctx_[li].exit_counter + 1;
        a.rank = ctx_[li].rank;
        a.nranks = nranks_;
        a.tag = tag;
        a.parity = (uint32_t)(ll_seq_ & 1);
        a.two_shot = kind;
        // the LL path does not consume a plan sequence number: its op-execution id lives in a range of its own
        a.exit_counter = ctx_[li].exit_counter;
        a.dev_tail = ctx_[li].dev_tail;
        a.exe_id = (1ull << 62) | ll_seq_;
        __atomic_store_n(&status_[li]->head, (uint64_t)a.exe_id, __ATOMIC_RELAXED);
    }
    stats_.launches++;
    return launch_ar_ll(args.data(), nl, rq.dtype, rq.redop, rq.stream);
}

HcclResult Communicator::consistency_check(const OpRequest &rq, int algo, uint64_t zc_in, uint64_t zc_out)
{
    if (all_local_ || nranks_ == 1 || calibrating_ || !consistency_enabled()) return HCCL_SUCCESS;
    // one check per distinct op shape: the parameter frame of every rank must hash identically
    // (reference: RankConsistentcyChecker, common/health/rank_consistentcy_checker.cc)
    OpFrame f;
    memset(&f, 0, sizeof(f));
    f.coll = rq.coll; f.dtype = rq.dtype; f.redop = rq.redop; f.root = rq.root; f.algo = algo;
    bool uniform = !(rq.coll == COLL_ALLTOALLV || rq.coll == COLL_ALLTOALLVC);
    f.count = uniform ? rq.count : 0;
    f.stage_half = settings_.stage_half_bytes;
    f.zc_in = zc_in; f.zc_out = zc_out;
    if (rq.counts) f.counts_crc = crc32(rq.counts, 8 * (size_t)nranks_, 0);
    if (rq.displs) f.displs_crc = crc32(rq.displs, 8 * (size_t)nranks_, 0);
    std::string key((const char *)&f, sizeof(f));
    if (checked_.count(key)) return HCCL_SUCCESS;
    std::vector<std::string> all;
    int tmo = env_config().connect_timeout_s * 1000;
    uint32_t mine = crc32(&f, sizeof(f), 0);
    char tag[64];
    snprintf(tag, sizeof(tag), "/check/%llu", (unsigned long long)checked_.size());
    CHK_RET(hub_->rendezvous(key_prefix_ + tag, nranks_, rank(), std::string((const char *)&f, sizeof(f)), &all, tmo));
    for (int r = 0; r < nranks_; ++r) {
        if (all[r].size() != sizeof(f) || crc32(all[r].data(), sizeof(f), 0) != mine) {
            OpFrame o;
            memset(&o, 0, sizeof(o));
            if (all[r].size() == sizeof(o)) memcpy(&o, all[r].data(), sizeof(o));
            HLOG_ERROR("op parameters differ between rank %d and rank %d: %s count %llu dtype %d op %d root %d vs %s count %llu dtype %d op %d root %d",
                       rank(), r, coll_name(f.coll), (unsigned long long)f.count, f.dtype, f.redop, f.root, coll_name(o.coll),
                       (unsigned long long)o.count, o.dtype, o.redop, o.root);
            return HCCL_E_PARA;
        }
    }
    checked_[key] = true;
    return HCCL_SUCCESS;
}

// AlltoAllV / VC: what rank i sends to rank j must be what j expects from i (reference: alltoall_operator.cc:49-72 checks
// the exchanged count matrix).  Virtual ranks hold the whole matrix; processes publish their two rows over the hub.  The
// exchange costs a control-plane round trip, so by default only the first calls of a communicator are checked (the call
// count is the same on every rank, so all ranks agree on which calls those are); HCCL_ALLTOALLV_CHECK=1 checks every
// call, =0 none.
HcclResult Communicator::a2av_check(const OpRequest &rq)
{
    const int p = nranks_, nl = nlocal();
    const EnvConfig &env = env_config();
    if (p == 1 || calibrating_ || env.a2av_check == 0) return HCCL_SUCCESS;
    const uint64_t call = a2av_calls_++;
    if (env.a2av_check < 0 && call >= 16) return HCCL_SUCCESS;
    if (all_local_) {
        for (int i = 0; i < nl; ++i)
            for (int j = 0; j < nl; ++j) {
                const uint64_t sij = rq.send_counts[(size_t)i * p + j], rji = rq.recv_counts[(size_t)j * p + i];
                CHK_RET_LOG(sij != rji, HCCL_E_PARA, "%s: rank %d sends %llu elements to rank %d, which expects %llu", coll_name(rq.coll), i,
                            (unsigned long long)sij, j, (unsigned long long)rji);
            }
        return HCCL_SUCCESS;
    }
    std::string mine((const char *)rq.send_counts, (size_t)p * 8);
    mine.append((const char *)rq.recv_counts, (size_t)p * 8);
    std::vector<std::string> all;
    CHK_RET(hub_->rendezvous(key_prefix_ + "/a2av/" + std::to_string(call), nranks_, rank(), mine, &all, env.connect_timeout_s * 1000));
    const int me = rank();
    HcclResult rc = HCCL_SUCCESS;
    for (int j = 0; j < p; ++j) {
        if (all[j].size() != (size_t)p * 16) return HCCL_E_INTERNAL;
        const uint64_t *sj = (const uint64_t *)all[j].data(), *rj = sj + p;
        // every rank checks the whole matrix, so that all of them return the same verdict
        for (int i = 0; i < p; ++i) {
            const uint64_t *ri = (const uint64_t *)all[i].data() + p;
            if (sj[i] != ri[j]) {
                if (i == me || j == me)
                    HLOG_ERROR("%s: rank %d sends %llu elements to rank %d, which expects %llu", coll_name(rq.coll), j, (unsigned long long)sj[i], i,
                               (unsigned long long)ri[j]);
                rc = HCCL_E_PARA;
            }
        }
        (void)rj;
    }
    return rc;
}

// ------------------------------------------------------------------------------------------------ p2p
HcclResult Communicator::p2p_plan_exec(bool is_send, int peer, const void *sbuf, void *rbuf, uint64_t count, int dtype, void *stream)
{
    int me = rank();
    OpDesc d;
    d.coll = is_send ? COLL_SEND : COLL_RECV;
    d.algo = ALGO_MESH; d.nranks = nranks_; d.dtype = dtype; d.nchan = 2; d.count = count; d.peer = peer;
    d.p2p_slot = p2p_slot_;
    auto pr = is_send ? std::make_pair(me, peer) : std::make_pair(peer, me);
    d.p2p_round0 = p2p_rounds_[pr];
    int es = dtype_size(dtype);
    uint64_t slotE = (p2p_slot_ / es) / (es >= 16 ? 1 : 16 / es) * (es >= 16 ? 1 : 16 / es);
    uint32_t rounds = (uint32_t)ceil_div_u64(count, slotE);
    std::ostringstream key;
    key << "p2p:" << is_send << ':' << peer << ':' << dtype << ':' << count << ':' << d.p2p_round0;
    CachedPlan *cp = nullptr;
    CHK_RET(get_plan(d, key.str(), &cp));
    p2p_rounds_[pr] += rounds;
    OpRequest rq;
    rq.stream = stream;
    std::vector<const void *> in{sbuf};
    std::vector<void *> out{rbuf};
    return run_plan(cp->plan, cp->dev_steps.data(), rq, 0, dtype, HCCL_REDUCE_SUM, false, in, out);
}

HcclResult Communicator::send(const void *buf, uint64_t count, int dtype, int dest, void *stream)
{
    std::lock_guard<std::mutex> lk(op_mu_);
    CHK_RET(check_ready());
    CHK_RET_LOG(all_local_, HCCL_E_NOT_SUPPORT, "use the local send/recv entry on all-local communicators");
    StateGuard guard(state_, CS_INUSE);
    stats_.ops[COLL_SEND]++;
    stats_.bytes[COLL_SEND] += count * dtype_size(dtype);
    if (p2p_) return p2p_->send(buf, count, dtype, dest, stream);
    return p2p_plan_exec(true, dest, buf, nullptr, count, dtype, stream);
}
HcclResult Communicator::recv(void *buf, uint64_t count, int dtype, int src, void *stream)
{
    std::lock_guard<std::mutex> lk(op_mu_);
    CHK_RET(check_ready());
    CHK_RET_LOG(all_local_, HCCL_E_NOT_SUPPORT, "use the local send/recv entry on all-local communicators");
    StateGuard guard(state_, CS_INUSE);
    stats_.ops[COLL_RECV]++;
    stats_.bytes[COLL_RECV] += count * dtype_size(dtype);
    if (p2p_) return p2p_->recv(buf, count, dtype, src, stream);
    return p2p_plan_exec(false, src, nullptr, buf, count, dtype, stream);
}

HcclResult Communicator::nccl_baseline_allreduce(const void *send, void *recv, uint64_t count, int dtype, int op, void *stream)
{
    if (!p2p_) return HCCL_E_UNAVAIL;
    return p2p_->baseline_allreduce(send, recv, count, dtype, op, stream);
}

HcclResult Communicator::batch_send_recv(HcclSendRecvItem *items, uint32_t n, void *stream)
{
    std::lock_guard<std::mutex> lk(op_mu_);
    CHK_RET(check_ready());
    CHK_RET_LOG(all_local_, HCCL_E_NOT_SUPPORT, "use the local send/recv entry on all-local communicators");
    StateGuard guard(state_, CS_INUSE);
    stats_.ops[COLL_BATCH_SENDRECV]++;
    int me = rank(), p = nranks_;
    // Pairwise ordering relative to this rank (reference: coll_batch_send_recv_executor.cc): sends ordered by
    // (dest - me) mod p, receives by (me - src) mod p, so that matching pairs meet in the same round everywhere.
    std::vector<HcclSendRecvItem *> sends, recvs;
    for (uint32_t i = 0; i < n; ++i) (items[i].sendRecvType == HCCL_SEND ? sends : recvs).push_back(&items[i]);
    std::stable_sort(sends.begin(), sends.end(), [&](auto *a, auto *b) { return (a->remoteRank + p - me) % p < (b->remoteRank + p - me) % p; });
    std::stable_sort(recvs.begin(), recvs.end(), [&](auto *a, auto *b) { return (me + p - a->remoteRank) % p < (me + p - b->remoteRank) % p; });
    // a send to self paired with a receive from self is a local copy
    for (auto si = sends.begin(); si != sends.end();) {
        if ((int)(*si)->remoteRank != me) { ++si; continue; }
        auto ri = std::find_if(recvs.begin(), recvs.end(), [&](auto *r) { return (int)r->remoteRank == me; });
        CHK_RET_LOG(ri == recvs.end(), HCCL_E_PARA, "send to self without a matching receive from self");
        size_t bytes = std::min((*si)->count, (*ri)->count) * dtype_size((*si)->dataType);
        if (settings_.transport == TR_DEVICE) cudaMemcpyAsync((*ri)->buf, (*si)->buf, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
        else memmove((*ri)->buf, (*si)->buf, bytes);
        recvs.erase(ri);
        si = sends.erase(si);
    }
    if (p2p_) return p2p_->batch(sends, recvs, stream);
    if (settings_.transport == TR_DEVICE) {
        // mailbox path on the device: interleave in pairwise rounds, each a pair of executor launches on two streams
        // is unnecessary because every plan launch is asynchronous and short messages fit a mailbox slot
        HcclResult rc = HCCL_SUCCESS;
        size_t m = std::max(sends.size(), recvs.size());
        for (size_t i = 0; i < m && rc == HCCL_SUCCESS; ++i) {
            if (i < sends.size()) {
                CHK_RET_LOG(sends[i]->count * dtype_size(sends[i]->dataType) > p2p_slot_, HCCL_E_NOT_SUPPORT,
                            "BatchSendRecv items above %llu bytes need the NCCL p2p backend", (unsigned long long)p2p_slot_);
                rc = p2p_plan_exec(true, sends[i]->remoteRank, sends[i]->buf, nullptr, sends[i]->count, sends[i]->dataType, stream);
            }
            if (i < recvs.size() && rc == HCCL_SUCCESS)
                rc = p2p_plan_exec(false, recvs[i]->remoteRank, nullptr, recvs[i]->buf, recvs[i]->count, recvs[i]->dataType, stream);
        }
        return rc;
    }
    // host transport: sends on a helper thread, receives on the caller (reference: sends on the main stream,
    // receives on a slave stream), so multi-round transfers in both directions cannot block each other
    HcclResult src = HCCL_SUCCESS, rrc = HCCL_SUCCESS;
    std::vector<std::pair<CachedPlan *, HcclSendRecvItem *>> splans;
    // plans are built on this thread (the cache is not thread safe); execution of the sends moves to the helper
    for (auto *s : sends) {
        OpDesc d;
        d.coll = COLL_SEND; d.algo = ALGO_MESH; d.nranks = p; d.dtype = s->dataType; d.nchan = 2; d.count = s->count;
        d.peer = (int)s->remoteRank; d.p2p_slot = p2p_slot_;
        auto pr = std::make_pair(me, (int)s->remoteRank);
        d.p2p_round0 = p2p_rounds_[pr];
        int es = dtype_size(s->dataType);
        uint64_t vec = es >= 16 ? 1 : 16 / es, slotE = (p2p_slot_ / es) / vec * vec;
        p2p_rounds_[pr] += (uint32_t)ceil_div_u64(s->count, slotE);
        std::ostringstream key;
        key << "p2p:1:" << s->remoteRank << ':' << s->dataType << ':' << s->count << ':' << d.p2p_round0;
        CachedPlan *cp = nullptr;
        CHK_RET(get_plan(d, key.str(), &cp));
        splans.push_back({cp, s});
    }
    std::thread sender([&] {
        for (auto &ps : splans) {
            OpRequest rq;
            std::vector<const void *> in{ps.second->buf};
            std::vector<void *> out{nullptr};
            ExecArgs a;
            memset(&a, 0, sizeof(a));
            a.steps = ps.first->plan.steps[0].data(); a.nsteps = (int)ps.first->plan.steps[0].size(); a.nchan = ps.first->plan.nchan;
            a.in = (const uint8_t *)ps.second->buf; a.dtype = ps.second->dataType;
            HcclResult r = exec_plan_host(ctx_[0], a);
            if (r != HCCL_SUCCESS) { src = r; break; }
        }
    });
    for (auto *r : recvs) {
        rrc = p2p_plan_exec(false, (int)r->remoteRank, nullptr, r->buf, r->count, r->dataType, stream);
        if (rrc != HCCL_SUCCESS) break;
    }
    sender.join();
    return src != HCCL_SUCCESS ? src : rrc;
}

HcclResult Communicator::local_send_recv(int src, int dst, const void *sbuf, void *rbuf, uint64_t count, int dtype, void *stream)
{
    std::lock_guard<std::mutex> lk(op_mu_);
    CHK_RET(check_ready());
    CHK_RET_LOG(!all_local_, HCCL_E_NOT_SUPPORT, "local send/recv needs an all-local communicator");
    CHK_RET_LOG(src < 0 || dst < 0 || src >= nranks_ || dst >= nranks_ || src == dst, HCCL_E_PARA, "bad rank pair %d -> %d", src, dst);
    StateGuard guard(state_, CS_INUSE);
    int es = dtype_size(dtype);
    uint64_t vec = es >= 16 ? 1 : 16 / es, slotE = (p2p_slot_ / es) / vec * vec;
    auto pr = std::make_pair(src, dst);
    OpDesc d;
    d.algo = ALGO_MESH; d.nranks = nranks_; d.dtype = dtype; d.nchan = 2; d.count = count; d.p2p_slot = p2p_slot_;
    d.p2p_round0 = p2p_rounds_[pr];
    p2p_rounds_[pr] += (uint32_t)ceil_div_u64(count, slotE);
    Plan ps, prv;
    d.coll = COLL_SEND; d.peer = dst;
    CHK_RET(build_plan(d, {src}, &ps));
    d.coll = COLL_RECV; d.peer = src;
    CHK_RET(build_plan(d, {dst}, &prv));
    stats_.launches++;
    ExecArgs a[2];
    memset(a, 0, sizeof(a));
    Step *dsteps[2] = {nullptr, nullptr};
    const Plan *pl[2] = {&ps, &prv};
    int ranks[2] = {src, dst};
    bool dev = settings_.transport == TR_DEVICE;
    for (int i = 0; i < 2; ++i) {
        const auto &steps = pl[i]->steps[0];
        if (dev) {
            cudaMalloc(&dsteps[i], std::max<size_t>(1, steps.size()) * sizeof(Step));
            cudaMemcpy(dsteps[i], steps.data(), steps.size() * sizeof(Step), cudaMemcpyHostToDevice);
        }
        a[i].steps = dev ? dsteps[i] : steps.data();
        a[i].nsteps = (int)steps.size();
        a[i].nchan = 2;
        a[i].dtype = dtype;
        a[i].in = (const uint8_t *)(i == 0 ? sbuf : nullptr);
        a[i].out = (uint8_t *)(i == 1 ? rbuf : nullptr);
    }
    if (dev) {
        // the executor indexes contexts by blockIdx.y, so pass a two-entry context array for (src, dst)
        RankCtx two[2] = {ctx_[src], ctx_[dst]};
        RankCtx *dtwo = nullptr;
        cudaMalloc(&dtwo, sizeof(two));
        cudaMemcpy(dtwo, two, sizeof(two), cudaMemcpyHostToDevice);
        HcclResult rc = launch_exec_plan(dtwo, a, 2, 2, stream);
        cudaStreamSynchronize((cudaStream_t)stream);
        cudaFree(dtwo); cudaFree(dsteps[0]); cudaFree(dsteps[1]);
        return rc != HCCL_SUCCESS ? rc : check_ready();
    }
    HcclResult rcs[2];
    std::thread t([&] { rcs[0] = exec_plan_host(ctx_[ranks[0]], a[0]); });
    rcs[1] = exec_plan_host(ctx_[ranks[1]], a[1]);
    t.join();
    return rcs[0] != HCCL_SUCCESS ? rcs[0] : rcs[1];
}

// ------------------------------------------------------------------------------------------------ health
// Staged abort (reference: TaskAbortHandler stages 0 / 1 / 2 = Suspend / StopExec / Clean, each with its own time budget,
// framework/communicator/impl/task_abort_handler.cc:28-128; HcclCommunicator::Suspend / StopExec / Clean).
//   stage 0  suspend_entry: the communicator takes no new operation (HCCL_E_SUSPENDING) and the abort word is raised, which
//            ends the waits of CPU ranks and of kernels alike; an API call that is inside the library is given the budget
//            to leave it.
//   stage 1  stop_exec: the budget covers the exit of the kernels in flight, observed through an event recorded behind
//            the newest launch (never a blocking synchronisation).
//   stage 2  clean: status blocks, arrival counters and failure words are cleared locally.  The flags are re-armed under a
//            new common sequence by resume(), which is collective.
// Each stage returns HCCL_E_TIMEOUT when its budget runs out (0 = no limit) and can be called again.
HcclResult Communicator::suspend_entry(int budget_ms)
{
    for (auto *a : abort_) *a = 1;
    state_.store(CS_SUSPENDED);
    const double t0 = now_us();
    while (!op_mu_.try_lock()) {
        if (budget_ms > 0 && now_us() - t0 > budget_ms * 1e3) return HCCL_E_TIMEOUT;
        usleep(200);
    }
    op_mu_.unlock();
    return HCCL_SUCCESS;
}

HcclResult Communicator::stop_exec(int budget_ms)
{
    for (auto *a : abort_) *a = 1;
    state_.store(CS_SUSPENDED);
    if (settings_.transport != TR_DEVICE) return HCCL_SUCCESS;  // CPU ranks run inside the API call that stage 0 waited for
    cudaSetDevice(settings_.device);
    cudaEvent_t ev = nullptr;
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) return HCCL_E_RUNTIME;
    // the legacy default stream waits for every blocking stream of the context; streams created non-blocking are covered by
    // the bounded device waits themselves (the abort word ends them within microseconds)
    cudaEventRecord(ev, 0);
    const double t0 = now_us();
    HcclResult rc = HCCL_SUCCESS;
    for (;;) {
        cudaError_t q = cudaEventQuery(ev);
        if (q == cudaSuccess) break;
        if (q != cudaErrorNotReady) { rc = HCCL_E_RUNTIME; break; }
        if (budget_ms > 0 && now_us() - t0 > budget_ms * 1e3) { rc = HCCL_E_TIMEOUT; break; }
        usleep(200);
    }
    cudaEventDestroy(ev);
    return rc;
}

HcclResult Communicator::clean(int budget_ms)
{
    const double t0 = now_us();
    std::unique_lock<std::mutex> lk(op_mu_, std::defer_lock);
    while (!lk.try_lock()) {
        if (budget_ms > 0 && now_us() - t0 > budget_ms * 1e3) return HCCL_E_TIMEOUT;
        usleep(200);
    }
    const bool dev = settings_.transport == TR_DEVICE;
    if (dev) cudaSetDevice(settings_.device);
    for (int li = 0; li < nlocal(); ++li) memset(status_[li], 0, sizeof(DevStatus));
    if (dev && dev_exit_)
        for (int li = 0; li < nlocal(); ++li) cudaMemsetAsync((uint32_t *)dev_exit_ + 4 * li, 0, sizeof(uint32_t) * 2, 0);
    if (dev && dev_pipe_cnt_) cudaMemsetAsync(dev_pipe_cnt_, 0, sizeof(uint32_t) * kPipeCounterWords * nlocal(), 0);
    last_op_.valid = false;
    return HCCL_SUCCESS;
}

HcclResult Communicator::suspend()
{
    // HcclCommSuspend = stages 0 and 1 without a budget (reference: Suspend/StopExec, hccl_communicator.cc:4383-4500).
    HcclResult rc = suspend_entry(0);
    if (rc != HCCL_SUCCESS) return rc;
    return stop_exec(0);
}

HcclResult Communicator::resume()
{
    std::lock_guard<std::mutex> lk(op_mu_);
    return resume_locked();
}

HcclResult Communicator::resume_locked()
{
    bool dev = settings_.transport == TR_DEVICE;
    if (dev) { cudaSetDevice(settings_.device); cudaDeviceSynchronize(); }
    int tmo = env_config().connect_timeout_s * 1000;
    // every rank must have stopped before flags are re-armed, and re-armed before anyone runs again
    uint64_t gen = resume_gen_.load() + 1;
    std::string tag = key_prefix_ + "/resume/" + std::to_string(gen);
    std::vector<std::string> seqs;
    if (!all_local_ && nranks_ > 1) {
        CHK_RET(hub_->rendezvous(tag + "/a", nranks_, rank(), std::string((const char *)&seq_, 8), &seqs, tmo));
        uint64_t mx = seq_;
        for (auto &s : seqs) { uint64_t v; memcpy(&v, s.data(), 8); mx = std::max(mx, v); }
        seq_ = mx + 2;  // a fresh, common sequence: flags of abandoned ops are all smaller
    } else seq_ += 2;
    for (int li = 0; li < nlocal(); ++li) {
        memset(status_[li], 0, sizeof(DevStatus));
        // done words restart at the new sequence so the first ops after resume do not wait for abandoned ones
        std::vector<uint64_t> done(kMaxRanks, seq_);
        uint8_t *dst = (uint8_t *)(ctx_[li].flags[ctx_[li].rank] + done_index(0));
        if (dev) cudaMemcpy(dst, done.data(), kMaxRanks * 8, cudaMemcpyHostToDevice);
        else memcpy(dst, done.data(), kMaxRanks * 8);
    }
    if (dev && dev_exit_)
        for (int li = 0; li < nlocal(); ++li) cudaMemset((uint32_t *)dev_exit_ + 4 * li, 0, sizeof(uint32_t) * 2);  // counter + failure code
    if (dev && dev_pipe_cnt_) cudaMemset(dev_pipe_cnt_, 0, sizeof(uint32_t) * kPipeCounterWords * nlocal());  // an abandoned pipelined op leaves arrivals behind
    // order matters for the heartbeat thread: own status is clean, then the epoch moves (peers' older error reports
    // become stale), then what it may have recorded from those reports is dropped
    resume_gen_.store(gen);
    remote_error_.store(0);
    remote_bad_rank_.store(-1);
    for (int li = 0; li < nlocal(); ++li) *abort_[li] = 0;
    if (!all_local_ && nranks_ > 1) CHK_RET(hub_->barrier(tag + "/b", nranks_, rank(), tmo));
    state_.store(CS_IDLE);
    return HCCL_SUCCESS;
}

HcclResult Communicator::async_error()
{
    for (auto *s : status_)
        if (s && s->code != 0) return (HcclResult)s->code;
    uint32_t re = remote_error_.load();
    return (HcclResult)re;
}

HcclResult Communicator::sync_stream(void *stream)
{
    if (settings_.transport == TR_DEVICE) {
        cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
        CHK_RET_LOG(e != cudaSuccess, HCCL_E_RUNTIME, "stream synchronize failed: %s", cudaGetErrorString(e));
        HcclResult err = async_error();
        if ((err == HCCL_E_TIMEOUT || err == HCCL_E_REMOTE) && env_config().retry_enable && !all_local_ && nranks_ > 1) {
            std::lock_guard<std::mutex> lk(op_mu_);
            err = async_error();  // another thread's call may have dealt with it meanwhile
            if (err == HCCL_E_TIMEOUT || err == HCCL_E_REMOTE) return retry_last_op(err);
        }
        return err;
    }
    return async_error();
}

HcclResult Communicator::kernel_trace(int local, uint64_t *out, size_t cap_words, int *nsteps)
{
    if (!dev_trace_) return HCCL_E_UNAVAIL;
    if (local < 0 || local >= nlocal() || cap_words < 1) return HCCL_E_PARA;
    size_t n = std::min(cap_words, kTraceWords);
    cudaDeviceSynchronize();
    CHK_RET_LOG(cudaMemcpy(out, (uint64_t *)dev_trace_ + (size_t)local * kTraceWords, n * 8, cudaMemcpyDeviceToHost) != cudaSuccess, HCCL_E_RUNTIME, "cudaMemcpy failed");
    if (nsteps) *nsteps = (int)((n - 1) / 3);
    return HCCL_SUCCESS;
}

HcclResult Communicator::wait_probe(int local, double timeout_ms, void *stream)
{
    std::lock_guard<std::mutex> lk(op_mu_);
    CHK_RET_LOG(local < 0 || local >= nlocal() || nranks_ < 2, HCCL_E_PARA, "wait probe needs a valid local rank and at least two ranks");
    Step s;
    memset(&s, 0, sizeof(s));
    s.op = ST_NOP;
    s.a_buf = s.b_buf = s.d_buf = s.d2_buf = BUF_NONE;
    s.a_rank = s.b_rank = s.d_rank = RANK_SELF;
    s.sig_rank = RANK_NONE;
    s.wait_rank = (int16_t)((ctx_[local].rank + 1) % nranks_);
    s.wait_val = 0xFFFFFu;  // a step value no plan ever signals
    s.chan_lo = 0; s.chan_n = 1;
    ExecArgs a;
    memset(&a, 0, sizeof(a));
    a.nsteps = 1; a.nchan = 1; a.seq = seq_ + 1000000; a.dtype = HCCL_DATA_TYPE_FP32;
    RankCtx x = ctx_[local];
    x.timeout_ns = (uint64_t)(timeout_ms * 1e6);
    if (settings_.transport != TR_DEVICE) {
        a.steps = &s;
        return exec_plan_host(x, a);
    }
    Step *ds = nullptr;
    RankCtx *dx = nullptr;
    CHK_RET_LOG(cudaMalloc(&ds, sizeof(s)) != cudaSuccess || cudaMalloc(&dx, sizeof(x)) != cudaSuccess, HCCL_E_MEMORY, "cudaMalloc failed");
    cudaMemcpy(ds, &s, sizeof(s), cudaMemcpyHostToDevice);
    cudaMemcpy(dx, &x, sizeof(x), cudaMemcpyHostToDevice);
    a.steps = ds;
    HcclResult rc = launch_exec_plan(dx, &a, 1, 1, stream);
    cudaStreamSynchronize((cudaStream_t)stream);
    cudaFree(ds);
    cudaFree(dx);
    if (rc != HCCL_SUCCESS) return rc;
    return (HcclResult)status_[local]->code;
}

void Communicator::heartbeat_loop()
{
    const EnvConfig &env = env_config();
    uint64_t last_head = 0, last_tail = 0;
    double stuck_since = 0;
    while (!hb_stop_.load()) {
        HeartbeatMsg m;
        memset(&m, 0, sizeof(m));
        m.rank = (uint32_t)rank(); m.nranks = (uint32_t)nranks_;
        m.lost_ms = (uint32_t)env.heartbeat_lost_ms;
        m.epoch = (uint32_t)resume_gen_.load();
        DevStatus *s = status_[0];
        if (settings_.transport == TR_DEVICE && ctx_[0].dev_tail) {
            s->tail = __atomic_load_n((volatile uint64_t *)ctx_[0].dev_tail, __ATOMIC_RELAXED);
        }
        // the executing thread (or the GPU) writes these words while this thread reads them
        m.head = __atomic_load_n(&s->head, __ATOMIC_RELAXED); m.tail = __atomic_load_n(&s->tail, __ATOMIC_RELAXED);
        m.status = PEER_OK;
        const uint32_t code_now = __atomic_load_n(&s->code, __ATOMIC_ACQUIRE);
        if (code_now != 0) { m.status = PEER_ERROR; m.error_code = code_now; }
        // stuck: an op started (head) and its completion (tail) has not followed for the configured time
        // (reference: Heartbeat::StuckDetection, heartbeat.cc:1073-1104, comparing OpExeCounter head/tail)
        if (m.head != m.tail && m.head == last_head && m.tail == last_tail) {
            if (stuck_since == 0) stuck_since = now_us();
            else if (now_us() - stuck_since > env.stuck_ms * 1e3 && m.status == PEER_OK) m.status = PEER_STUCK;
        } else stuck_since = 0;
        last_head = m.head; last_tail = m.tail;
        if (!fault::drop_heartbeat(rank())) {
            HeartbeatSummary sum;
            HcclResult rc = hb_conn_->heartbeat(key_prefix_ + "/hb", m, &sum, std::max(1000, env.heartbeat_lost_ms));
            if (rc != HCCL_SUCCESS) {
                // the hub lives in the root rank's process: losing it means the root is gone
                if (!hb_stop_.load() && remote_error_.load() == 0) {
                    remote_bad_rank_.store(0);
                    remote_error_.store(HCCL_E_REMOTE);
                    for (auto *a : abort_) if (*a == 0) *a = 2;
                    HLOG_ERROR("heartbeat: bootstrap hub (rank 0) unreachable");
                }
            } else {
                // first peer whose bad report is current (reports from before this rank's last resume are stale)
                int bad = -1;
                for (int q = 0; q < nranks_ && bad < 0; ++q)
                    if (q != rank() && sum.status[q] != PEER_OK && (sum.status[q] == PEER_LOST || sum.epoch[q] >= m.epoch)) bad = q;
                if (bad >= 0 && remote_error_.load() == 0 && m.epoch == (uint32_t)resume_gen_.load()) {
                    sum.first_bad_rank = (uint32_t)bad;
                    uint32_t st = sum.status[sum.first_bad_rank];
                    uint32_t code = st == PEER_STUCK ? HCCL_E_TIMEOUT : HCCL_E_REMOTE;
                    remote_bad_rank_.store((int)sum.first_bad_rank);
                    remote_error_.store(code);
                    for (auto *a : abort_) {  // in-flight waits give up instead of running into their bound
                        uint32_t zero = 0;
                        __atomic_compare_exchange_n(a, &zero, 2u, false, __ATOMIC_RELEASE, __ATOMIC_RELAXED);
                    }
                    HLOG_ERROR("heartbeat: rank %u reported %s", sum.first_bad_rank, st == PEER_LOST ? "lost" : st == PEER_STUCK ? "stuck" : "error");
                }
            }
        }
        std::unique_lock<std::mutex> lk(hb_mu_);
        hb_cv_.wait_for(lk, std::chrono::milliseconds(env.heartbeat_ms), [&] { return hb_stop_.load(); });
    }
}

void Communicator::remember_op(const OpRequest &rq)
{
    LastOp &l = last_op_;
    const int nl = nlocal(), p = nranks_;
    l.valid = true;
    l.op_index = op_index_;
    l.first_seq = seq_;
    l.rq = rq;
    l.in.assign(nl, nullptr);
    l.out.assign(nl, nullptr);
    for (int li = 0; li < nl; ++li) { l.in[li] = rq.in ? rq.in[li] : nullptr; l.out[li] = rq.out ? rq.out[li] : nullptr; }
    l.rq.in = rq.in ? l.in.data() : nullptr;
    l.rq.out = rq.out ? l.out.data() : nullptr;
    auto keep = [&](const uint64_t *&field, std::vector<uint64_t> &store, size_t n) {
        if (!field) return;
        store.assign(field, field + n);
        field = store.data();
    };
    keep(l.rq.counts, l.counts, p); keep(l.rq.displs, l.displs, p);
    keep(l.rq.send_counts, l.sc, (size_t)nl * p); keep(l.rq.send_displs, l.sd, (size_t)nl * p);
    keep(l.rq.recv_counts, l.rc, (size_t)nl * p); keep(l.rq.recv_displs, l.rd, (size_t)nl * p);
    l.retriable = true;
    for (int li = 0; li < nl; ++li)
        if (overlap_kind(rq, li) != 0) l.retriable = false;  // its output overwrote what a second run would read
}

// Device transport: a kernel of the newest collective gave up (bounded wait, or a peer's failure learnt from the heartbeat).
// All ranks meet at the hub, agree to run that op again, re-arm the flags under a common new sequence and re-launch it;
// the attempt is awaited on its stream so that its outcome is known before anything else is launched.
HcclResult Communicator::retry_last_op(HcclResult failure)
{
    if (!last_op_.valid) return failure;
    uint64_t failed_seq = 0;
    for (auto *st : status_)
        if (st && st->code) failed_seq = std::max<uint64_t>(failed_seq, st->seq);
    if (failed_seq && failed_seq < last_op_.first_seq) {
        HLOG_ERROR("operator retry: the failure belongs to an op older than the newest one (sequence %llu < %llu); only the newest op can be re-run",
                   (unsigned long long)failed_seq, (unsigned long long)last_op_.first_seq);
        return failure;
    }
    stats_.timeouts++;
    StateGuard guard(state_, CS_INUSE);
    return maybe_retry(last_op_.rq, failure, last_op_.op_index);
}

HcclResult Communicator::maybe_retry(const OpRequest &rq, HcclResult failure, uint64_t op_index)
{
    // Operator retry (reference: cluster_maintenance/recovery/operator_retry, max 3 attempts): every rank that
    // failed meets at the hub, agrees that all members failed the same op and can re-run it (input untouched),
    // re-arms flags under a common new sequence and executes the op again.
    const EnvConfig &env = env_config();
    if (!env.retry_enable || all_local_ || nranks_ == 1) return failure;
    const bool dev = settings_.transport == TR_DEVICE;
    // an op whose output overlaps its input has destroyed what a second run would need (reference: retry-inplace rule,
    // coll_alg_operator.cc:588, decided from the byte ranges of IsHcclOpInplace)
    bool inplace = false;
    for (int li = 0; li < nlocal(); ++li)
        if (overlap_kind(rq, li) != 0) inplace = true;
    HcclResult rc = failure;
    for (int attempt = 1; attempt <= env.retry_max && rc != HCCL_SUCCESS; ++attempt) {
        struct Vote { uint64_t op_index; uint32_t can_retry; uint32_t code; } v{op_index, inplace ? 0u : 1u, (uint32_t)rc};
        std::vector<std::string> votes;
        char tag[96];
        snprintf(tag, sizeof(tag), "/retry/%llu/%d", (unsigned long long)op_index, attempt);
        int tmo = env.retry_hold_ms + (int)(ctx_[0].timeout_ns / 1000000) + 2000;
        HcclResult rr = hub_->rendezvous(key_prefix_ + tag, nranks_, rank(), std::string((const char *)&v, sizeof(v)), &votes, tmo);
        if (rr != HCCL_SUCCESS) return failure;  // not everyone arrived: some rank did not fail this op or is gone
        bool ok = true;
        for (auto &s : votes) {
            Vote o;
            memcpy(&o, s.data(), sizeof(o));
            ok &= o.op_index == op_index && o.can_retry;
        }
        if (!ok) { HLOG_ERROR("op %llu cannot be retried (in-place input or ranks out of step)", (unsigned long long)op_index); return failure; }
        usleep((useconds_t)env.retry_interval_ms * 1000);
        state_.store(CS_SUSPENDED);
        HcclResult rs = resume_locked();
        if (rs != HCCL_SUCCESS) return failure;
        state_.store(CS_INUSE);
        stats_.retries++;
        HLOG_WARN("retrying %s (attempt %d of %d)", coll_name(rq.coll), attempt, env.retry_max);
        fault::before_attempt(rank(), op_index, attempt);
        if (dev) last_op_.first_seq = seq_;
        rc = run_collective_once(rq);
        if (dev && rc == HCCL_SUCCESS) {
            // the launch is asynchronous: its outcome is in the status block once the stream has drained
            cudaError_t e = cudaStreamSynchronize((cudaStream_t)rq.stream);
            if (e != cudaSuccess) return HCCL_E_RUNTIME;
            rc = async_error();
            if (rc != HCCL_SUCCESS && rc != HCCL_E_TIMEOUT && rc != HCCL_E_REMOTE) return rc;
        }
    }
    return rc;
}

// ------------------------------------------------------------------------------------------------ overflow check, topology
static bool float_dtype(int dt)
{
    return dt == HCCL_DATA_TYPE_FP32 || dt == HCCL_DATA_TYPE_FP64 || dt == HCCL_DATA_TYPE_FP16 || dt == HCCL_DATA_TYPE_BFP16;
}

HcclResult Communicator::overflow_scan(const OpRequest &rq)
{
    const bool reduces = rq.coll == COLL_ALLREDUCE || rq.coll == COLL_REDUCE || rq.coll == COLL_REDUCE_SCATTER || rq.coll == COLL_REDUCE_SCATTER_V;
    if (!reduces || !float_dtype(rq.dtype)) return HCCL_SUCCESS;
    const bool dev = settings_.transport == TR_DEVICE;
    if (!overflow_word_) {
        if (dev) {
            CHK_RET_LOG(cudaHostAlloc((void **)&overflow_word_, 64, cudaHostAllocMapped) != cudaSuccess, HCCL_E_MEMORY, "cudaHostAlloc(overflow word) failed");
        } else {
            overflow_word_ = (unsigned long long *)malloc(64);
            CHK_RET_LOG(!overflow_word_, HCCL_E_MEMORY, "malloc failed");
        }
        *overflow_word_ = 0;
    }
    for (int li = 0; li < nlocal(); ++li) {
        const int r = local_ranks_[li];
        uint64_t n = rq.count;  // AllReduce: count; ReduceScatter: recvCount
        if (rq.coll == COLL_REDUCE && r != rq.root) continue;  // only the root holds a result
        if (rq.coll == COLL_REDUCE_SCATTER_V) n = rq.counts[r];
        if (dev) {
            unsigned long long *dptr = nullptr;
            CHK_RET_LOG(cudaHostGetDevicePointer((void **)&dptr, overflow_word_, 0) != cudaSuccess, HCCL_E_RUNTIME, "cudaHostGetDevicePointer failed");
            CHK_RET(launch_overflow_scan(rq.out[li], n, rq.dtype, dptr, rq.stream));
        } else {
            unsigned long long bad = 0;
            for (uint64_t i = 0; i < n; ++i) {
                double v = 0;
                switch (rq.dtype) {
                    case HCCL_DATA_TYPE_FP32: v = ((const float *)rq.out[li])[i]; break;
                    case HCCL_DATA_TYPE_FP64: v = ((const double *)rq.out[li])[i]; break;
                    case HCCL_DATA_TYPE_FP16: v = fp16_to_float(((const uint16_t *)rq.out[li])[i]); break;
                    default: v = bf16_to_float(((const uint16_t *)rq.out[li])[i]); break;
                }
                bad += std::isfinite(v) ? 0 : 1;
            }
            __atomic_fetch_add(overflow_word_, bad, __ATOMIC_RELAXED);
        }
    }
    return HCCL_SUCCESS;
}

uint64_t Communicator::overflow_count()
{
    if (!overflow_word_) return 0;
    return __atomic_load_n(overflow_word_, __ATOMIC_RELAXED);
}

std::string Communicator::topo_json()
{
    std::ostringstream o;
    const bool dev = settings_.transport == TR_DEVICE;
    o << "{\"identifier\":\"" << ident_ << "\",\"ranks\":" << nranks_ << ",\"transport\":\"" << (dev ? "device" : "host") << "\""
      << ",\"fabric\":\"" << (dev ? (nranks_ > 1 ? "nvlink-nvswitch" : "local") : "shared-memory") << "\",\"nvls\":" << (nvls_ ? "true" : "false")
      << ",\"levels\":[{\"level\":0,\"ranks\":" << nranks_ << ",\"algorithms\":[\"mesh\",\"ring\"" << (nvls_ ? ",\"switch\"" : "") << "]},{\"level\":1,\"ranks\":0,\"algorithms\":[]}]"
      << ",\"all_local\":" << (all_local_ ? "true" : "false") << ",\"rank_table\":[";
    char host[64] = {0};
    gethostname(host, sizeof(host) - 1);
    for (int r = 0; r < nranks_; ++r) {
        TopoEntry e{r, (uint32_t)getpid(), settings_.device, host};
        if (r < (int)topo_.size()) e = topo_[r];
        o << (r ? "," : "") << "{\"rank\":" << e.rank << ",\"host\":\"" << e.host << "\",\"pid\":" << e.pid << ",\"device\":" << (dev ? e.device : -1) << "}";
    }
    o << "]";
    if (dev) o << ",\"links\":" << link_topo_json(links_);
    if (dev) {
        // peer-access matrix over the devices that appear in the rank table (1 = this pair can map each other's memory)
        std::vector<int> devs;
        for (int r = 0; r < nranks_; ++r) {
            int d = r < (int)topo_.size() ? topo_[r].device : settings_.device;
            if (std::find(devs.begin(), devs.end(), d) == devs.end()) devs.push_back(d);
        }
        int ndev = 0;
        cudaGetDeviceCount(&ndev);
        o << ",\"devices\":[";
        for (size_t i = 0; i < devs.size(); ++i) o << (i ? "," : "") << devs[i];
        o << "],\"peer_access\":[";
        for (size_t i = 0; i < devs.size(); ++i) {
            o << (i ? "," : "") << "[";
            for (size_t j = 0; j < devs.size(); ++j) {
                int can = devs[i] == devs[j] ? 1 : 0;
                if (!can && devs[i] < ndev && devs[j] < ndev) cudaDeviceCanAccessPeer(&can, devs[i], devs[j]);
                o << (j ? "," : "") << can;
            }
            o << "]";
        }
        o << "]";
    }
    o << "}";
    return o.str();
}

// ------------------------------------------------------------------------------------------------ one-sided put / get
HcclResult Communicator::sym_put(int local, int handle, int peer, size_t offset, const void *src, size_t bytes, void *stream)
{
    std::lock_guard<std::mutex> lk(op_mu_);
    CHK_RET(check_ready());
    auto it = user_segs_.find(handle);
    CHK_RET_LOG(it == user_segs_.end(), HCCL_E_NOT_FOUND, "put: unknown symmetric allocation %d", handle);
    CHK_RET_LOG(local < 0 || local >= nlocal() || peer < 0 || peer >= nranks_, HCCL_E_PARA, "put: bad rank (local %d, peer %d)", local, peer);
    const SymSegment &sg = it->second[local];
    CHK_RET_LOG(offset > sg.bytes || bytes > sg.bytes - offset, HCCL_E_PARA, "put: [%zu, %zu) outside the allocation of %zu bytes", offset, offset + bytes, sg.bytes);
    if (bytes == 0) return HCCL_SUCCESS;
    StateGuard guard(state_, CS_INUSE);
    if (settings_.transport == TR_DEVICE) {
        CHK_RET_LOG(cudaMemcpyAsync(sg.peer[peer] + offset, src, bytes, cudaMemcpyDefault, (cudaStream_t)stream) != cudaSuccess, HCCL_E_RUNTIME, "put: cudaMemcpyAsync failed");
    } else {
        memcpy(sg.peer[peer] + offset, src, bytes);
        __atomic_thread_fence(__ATOMIC_SEQ_CST);
    }
    return HCCL_SUCCESS;
}

HcclResult Communicator::sym_get(int local, int handle, int peer, size_t offset, void *dst, size_t bytes, void *stream)
{
    std::lock_guard<std::mutex> lk(op_mu_);
    CHK_RET(check_ready());
    auto it = user_segs_.find(handle);
    CHK_RET_LOG(it == user_segs_.end(), HCCL_E_NOT_FOUND, "get: unknown symmetric allocation %d", handle);
    CHK_RET_LOG(local < 0 || local >= nlocal() || peer < 0 || peer >= nranks_, HCCL_E_PARA, "get: bad rank (local %d, peer %d)", local, peer);
    const SymSegment &sg = it->second[local];
    CHK_RET_LOG(offset > sg.bytes || bytes > sg.bytes - offset, HCCL_E_PARA, "get: [%zu, %zu) outside the allocation of %zu bytes", offset, offset + bytes, sg.bytes);
    if (bytes == 0) return HCCL_SUCCESS;
    StateGuard guard(state_, CS_INUSE);
    if (settings_.transport == TR_DEVICE) {
        CHK_RET_LOG(cudaMemcpyAsync(dst, sg.peer[peer] + offset, bytes, cudaMemcpyDefault, (cudaStream_t)stream) != cudaSuccess, HCCL_E_RUNTIME, "get: cudaMemcpyAsync failed");
    } else {
        __atomic_thread_fence(__ATOMIC_SEQ_CST);
        memcpy(dst, sg.peer[peer] + offset, bytes);
    }
    return HCCL_SUCCESS;
}

// ------------------------------------------------------------------------------------------------ symmetric user memory
HcclResult Communicator::sym_alloc(size_t bytes, void **local_ptrs, int *handle)
{
    std::lock_guard<std::mutex> lk(op_mu_);
    StateGuard guard(state_, CS_BUILDING);
    std::vector<SymSegment> segs;
    CHK_RET(alloc_->alloc(bytes, true, &segs));
    for (int li = 0; li < nlocal(); ++li) local_ptrs[li] = segs[li].peer[local_ranks_[li]];
    return register_user_segs(std::move(segs), handle);
}

HcclResult Communicator::sym_adopt(void *const *local_ptrs, size_t bytes, const unsigned long long *drv_handles, size_t handle_offset, int *handle)
{
    std::lock_guard<std::mutex> lk(op_mu_);
    StateGuard guard(state_, CS_BUILDING);
    std::vector<SymSegment> segs;
    CHK_RET(alloc_->adopt(local_ptrs, bytes, drv_handles, handle_offset, true, &segs));
    CHK_RET_LOG((int)segs.size() != nlocal(), HCCL_E_INTERNAL, "allocator returned %zu segments for %d local ranks", segs.size(), nlocal());
    return register_user_segs(std::move(segs), handle);
}

HcclResult Communicator::register_user_segs(std::vector<SymSegment> segs, int *handle)
{
    *handle = next_handle_++;
    std::vector<void *> tabs(nlocal(), nullptr);
    for (int li = 0; li < nlocal(); ++li) {
        std::vector<uint8_t *> tab(kMaxRanks, nullptr);
        for (int q = 0; q < nranks_; ++q) tab[q] = segs[li].peer[q];
        if (settings_.transport == TR_DEVICE) {
            CHK_RET_LOG(cudaMalloc(&tabs[li], sizeof(uint8_t *) * kMaxRanks) != cudaSuccess, HCCL_E_MEMORY, "cudaMalloc failed");
            cudaMemcpy(tabs[li], tab.data(), sizeof(uint8_t *) * kMaxRanks, cudaMemcpyHostToDevice);
        } else {
            tabs[li] = malloc(sizeof(uint8_t *) * kMaxRanks);
            memcpy(tabs[li], tab.data(), sizeof(uint8_t *) * kMaxRanks);
        }
    }
    user_peer_tabs_[*handle] = tabs;
    user_segs_[*handle] = std::move(segs);
    return HCCL_SUCCESS;
}
HcclResult Communicator::sym_free(int handle)
{
    std::lock_guard<std::mutex> lk(op_mu_);
    auto it = user_segs_.find(handle);
    if (it == user_segs_.end()) return HCCL_E_NOT_FOUND;
    if (!all_local_ && nranks_ > 1) hub_->barrier(key_prefix_ + "/symfree/" + std::to_string(handle), nranks_, rank(), 10000);
    alloc_->release(&it->second);
    user_segs_.erase(it);
    for (void *t : user_peer_tabs_[handle]) { if (settings_.transport == TR_DEVICE) cudaFree(t); else free(t); }
    user_peer_tabs_.erase(handle);
    return HCCL_SUCCESS;
}
int Communicator::find_user_seg(int li, const void *ptr, size_t bytes, size_t *offset)
{
    for (auto &kv : user_segs_) {
        const SymSegment &sg = kv.second[li];
        const uint8_t *base = sg.peer[local_ranks_[li]];
        if ((const uint8_t *)ptr >= base && (const uint8_t *)ptr + bytes <= base + sg.bytes) {
            if (offset) *offset = (size_t)((const uint8_t *)ptr - base);
            return kv.first;
        }
    }
    return 0;
}

HcclResult Communicator::sym_query(int handle, void **peer_ptrs, void **mc_ptrs, size_t *bytes)
{
    auto it = user_segs_.find(handle);
    if (it == user_segs_.end()) return HCCL_E_NOT_FOUND;
    for (int li = 0; li < nlocal(); ++li) {
        for (int q = 0; q < nranks_; ++q) peer_ptrs[li * nranks_ + q] = it->second[li].peer[q];
        if (mc_ptrs) mc_ptrs[li] = it->second[li].mc;
    }
    if (bytes) *bytes = it->second[0].bytes;
    return HCCL_SUCCESS;
}

HcclResult Communicator::exchange_p2p(const std::string &tag, const std::string &mine, std::vector<std::string> *all)
{
    if (!p2p_conn_) return HCCL_E_UNAVAIL;
    return p2p_conn_->rendezvous(key_prefix_ + "/p2p/" + tag, nranks_, rank(), mine, all, env_config().connect_timeout_s * 1000);
}

HcclResult Communicator::exchange(const std::string &tag, const std::string &mine, std::vector<std::string> *all)
{
    if (all_local_ || nranks_ == 1) { all->assign(1, mine); return HCCL_SUCCESS; }
    return hub_->rendezvous(key_prefix_ + "/x/" + tag, nranks_, rank(), mine, all, env_config().connect_timeout_s * 1000);
}

}  // namespace hcclb
