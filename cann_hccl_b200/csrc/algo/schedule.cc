#include "algo/schedule.h"
#include <algorithm>
#include <cstring>
#include "common/log.h"

namespace hcclb {

const char *coll_name(int c)
{
    static const char *n[] = {"AllReduce", "Broadcast", "ReduceScatter", "ReduceScatterV", "Scatter", "AllGather",
                              "AllGatherV", "Barrier", "AlltoAll", "AlltoAllV", "AlltoAllVC", "Reduce", "Gather",
                              "Send", "Recv", "BatchSendRecv"};
    return (c >= 0 && c < COLL_COUNT) ? n[c] : "Unknown";
}
const char *algo_name(int a)
{
    static const char *n[] = {"auto", "mesh", "mesh_oneshot", "ring", "rhd", "pairwise", "star", "tree", "nvls",
                              "nvls_oneshot", "single", "mesh_pipe", "nvls_pipe", "nvls_zerocopy", "ll", "mesh_zerocopy", "direct"};
    return (a >= 0 && a < ALGO_COUNT) ? n[a] : "unknown";
}
int algo_from_name(const std::string &s)
{
    for (int a = 0; a < ALGO_COUNT; ++a)
        if (s == algo_name(a)) return a;
    if (s == "hd" || s == "nhr" || s == "nb") return ALGO_RHD;  // reference names of log-step algorithms
    if (s == "fullmesh" || s == "twoshot") return ALGO_MESH;
    if (s == "oneshot") return ALGO_MESH_ONESHOT;
    return ALGO_AUTO;
}

namespace {

// Program under construction for all ranks.  sig_val of a step is its index + 1 unless set explicitly,
// so a consumer names a producer step by (rank, index).
struct Prog {
    int p, nchan, es;
    uint64_t vec;  // elements per 16 bytes
    std::vector<std::vector<Step>> s;
    Prog(int p_, int nchan_, int es_) : p(p_), nchan(nchan_), es(es_), vec(es_ >= 16 ? 1 : 16 / es_), s(p_) {}

    Step mk(uint8_t op) const
    {
        Step st;
        memset(&st, 0, sizeof(st));
        st.op = op;
        st.a_buf = st.b_buf = st.d_buf = st.d2_buf = BUF_NONE;
        st.a_rank = st.b_rank = st.d_rank = RANK_SELF;
        st.wait_rank = st.sig_rank = RANK_NONE;
        st.chan_lo = 0;
        st.chan_n = (uint16_t)nchan;
        return st;
    }
    int add(int r, Step st, bool explicit_sig = false)
    {
        int idx = (int)s[r].size();
        if (!explicit_sig) st.sig_val = (uint32_t)idx + 1;
        s[r].push_back(st);
        return idx;
    }
    int last(int r) const { return (int)s[r].size() - 1; }
    void wait_lane(Step &st, int q, int idx) const
    {
        st.wait_rank = (int16_t)q;
        st.wait_val = (uint32_t)idx + 1;
    }
    void wait_allch(Step &st, int q, int idx) const
    {
        wait_lane(st, q, idx);
        st.flags |= SF_WAIT_ALLCH;
        st.wait_clo = 0;
        st.wait_cn = (uint16_t)nchan;
    }
    // Every channel of rank r stops here until all of the rank's own channels have arrived.  Needed where later steps write
    // the caller's receive buffer in pieces that do not line up with the pieces in which earlier steps read the send buffer:
    // when both are the same memory (in place), one channel would otherwise overwrite input that a slower channel of the same
    // rank has yet to read.  Two steps: signal my own flag words, then wait for all of them (and tell the peers).
    void own_channels_barrier(int r)
    {
        Step sig = mk(ST_NOP);
        sig.sig_rank = (int16_t)r;
        sig.flags |= SF_INCLUDE_SELF;
        int i = add(r, sig);
        Step w = mk(ST_NOP);
        wait_allch(w, r, i);
        w.flags |= SF_INCLUDE_SELF;
        w.sig_rank = RANK_ALL;  // generators chain on "the last step of rank r": it has to be one that peers can wait for
        add(r, w);
    }
    Step copy(uint8_t ab, int ar, uint64_t aoff, uint8_t db, int dr, uint64_t doff, uint64_t count) const
    {
        Step st = mk(ST_COPY);
        st.a_buf = ab; st.a_rank = (int16_t)ar; st.a_off = aoff;
        st.d_buf = db; st.d_rank = (int16_t)dr; st.d_off = doff;
        st.count = count;
        return st;
    }
    Step reduce2(uint8_t ab, int ar, uint64_t aoff, uint8_t bb, uint64_t boff, uint8_t db, uint64_t doff,
                 uint64_t count) const
    {
        Step st = mk(ST_REDUCE2);
        st.a_buf = ab; st.a_rank = (int16_t)ar; st.a_off = aoff;
        st.b_buf = bb; st.b_rank = RANK_SELF; st.b_off = boff;
        st.d_buf = db; st.d_off = doff;
        st.count = count;
        return st;
    }
};

// Equal slicing of n elements into m pieces whose boundaries are multiples of 16 bytes.
struct Slices {
    uint64_t sl;  // slice length (elements), multiple of vec
    uint64_t n;
    uint64_t off(int j) const { return std::min(n, sl * (uint64_t)j); }
    uint64_t len(int j) const { return off(j + 1) - off(j); }
};
Slices make_slices(uint64_t n, int m, uint64_t vec)
{
    Slices s;
    s.n = n;
    s.sl = round_up_u64(ceil_div_u64(n, (uint64_t)m), vec);
    if (s.sl == 0) s.sl = vec;
    return s;
}

// ---- block structure of recursive halving-doubling with non-power-of-two fold --------------------
// (pattern: algorithm/base/alg_template/component/recursive_halvingdoubling_base.cc:22-60)
struct HdBlock {
    int p, B, part1;
    int block_of(int r) const { return r < part1 ? ((r & 1) ? -1 : r / 2) : r - part1 / 2; }
    int rank_of(int b) const { return b < part1 / 2 ? 2 * b : b + part1 / 2; }
    // ranks [lo, hi) whose slots belong to block rank b
    void ranks_of(int b, int &lo, int &hi) const
    {
        if (b < part1 / 2) { lo = 2 * b; hi = 2 * b + 2; }
        else { lo = b + part1 / 2; hi = lo + 1; }
    }
};
HdBlock make_block(int p)
{
    HdBlock h;
    h.p = p;
    h.B = 1;
    while (h.B * 2 <= p) h.B *= 2;
    h.part1 = 2 * (p - h.B);
    return h;
}

// ------------------------------------------------------------------------------------------------
// AllReduce
// ------------------------------------------------------------------------------------------------
void ar_mesh_oneshot(Prog &P, const OpDesc &d, bool nvls)
{
    uint64_t n = d.chunk_count, uoff = d.chunk_off * P.es;
    for (int r = 0; r < P.p; ++r) {
        Step c = P.copy(BUF_IN, RANK_SELF, uoff, BUF_STAGE, RANK_SELF, 0, n);
        c.sig_rank = RANK_ALL;
        int i0 = P.add(r, c);
        Step red = P.mk(nvls ? ST_MC_REDUCE : ST_REDUCE_ALL);
        red.a_buf = BUF_STAGE; red.a_rank = RANK_ALL; red.a_off = 0;
        red.d_buf = BUF_OUT; red.d_off = uoff; red.count = n;
        red.wait_rank = RANK_ALL; red.wait_val = (uint32_t)i0 + 1;
        P.add(r, red);
    }
}

void ar_mesh_twoshot(Prog &P, const OpDesc &d, bool nvls)
{
    uint64_t n = d.chunk_count, uoff = d.chunk_off * P.es;
    Slices S = make_slices(n, P.p, P.vec);
    // NVLS: the reduced slice is multicast over the raw slice in place: only its owner ever reads the raw slice, and it
    // writes an element after having read it
    uint64_t region2 = 0;
    for (int r = 0; r < P.p; ++r) {
        // one step copies all p slices, each split over the channels on its own: channel c of every rank stages piece c of
        // every slice, so the consumers' lanes line up with the producers' (a gather from this rank's own input)
        Step cin = P.mk(ST_GATHER_ALL);
        cin.a_buf = BUF_IN; cin.a_rank = RANK_SELF; cin.a_off = uoff; cin.a_stride = S.sl * P.es;
        cin.d_buf = BUF_STAGE; cin.d_off = 0; cin.d_stride = S.sl * P.es;
        cin.count = S.sl; cin.limit = n;
        cin.sig_rank = RANK_ALL;
        int last = P.add(r, cin);
        Step red = P.mk(nvls ? ST_MC_REDUCE : ST_REDUCE_ALL);
        red.a_buf = BUF_STAGE; red.a_rank = RANK_ALL; red.a_off = S.off(r) * P.es;
        red.count = S.len(r);
        red.d_buf = BUF_STAGE;
        if (nvls) { red.d_rank = RANK_ALL; red.d_off = region2 + S.off(r) * P.es; }
        else { red.d_rank = RANK_SELF; red.d_off = S.off(r) * P.es; }
        red.d2_buf = BUF_OUT; red.d2_off = uoff + S.off(r) * P.es;
        red.wait_rank = RANK_ALL; red.wait_val = (uint32_t)last + 1;
        red.sig_rank = RANK_ALL;
        int ri = P.add(r, red);
        Step g = P.mk(ST_GATHER_ALL);
        g.a_buf = BUF_STAGE; g.a_rank = nvls ? RANK_SELF : RANK_ALL; g.a_off = nvls ? region2 : 0;
        g.a_stride = S.sl * P.es;
        g.d_buf = BUF_OUT; g.d_off = uoff; g.d_stride = S.sl * P.es;
        g.count = S.sl; g.limit = n; g.flags |= SF_SKIP_SELF;
        g.wait_rank = RANK_ALL; g.wait_val = (uint32_t)ri + 1;
        P.add(r, g);
    }
}

// Ring reduce-scatter over p slices described by callbacks; rank r ends holding slice (r+c+2) mod p ... see notes
// in the body.  `fin_out(r, slice)` gives the BUF_OUT byte offset of the final slice (or ~0 to keep it in staging only).
struct SliceIo {
    std::vector<uint64_t> in_off, st_off, out_off, len;  // per slice; byte offsets, element lengths
};
// Step k (0..p-2): rank r reduces slice x = (r - k + c) mod p from its left neighbour's staging with its own input.
// Pre-step: rank r stages slice (r + 1 + c) mod p, which its right neighbour reads at k = 0.
// After the loop rank r holds slice (r + c + 2) mod p fully reduced: c = -1 -> r+1 (AllReduce), c = -2 -> r (ReduceScatter).
void ring_rs(Prog &P, const SliceIo &io, int c, bool final_to_out_only)
{
    int p = P.p;
    auto md = [&](int v) { return ((v % p) + p) % p; };
    for (int r = 0; r < p; ++r) {
        int x = md(r + 1 + c);
        Step pre = P.copy(BUF_IN, RANK_SELF, io.in_off[x], BUF_STAGE, RANK_SELF, io.st_off[x], io.len[x]);
        pre.sig_rank = (int16_t)md(r + 1);
        P.add(r, pre);
    }
    for (int k = 0; k <= p - 2; ++k) {
        for (int r = 0; r < p; ++r) {
            int x = md(r - k + c), left = md(r - 1);
            bool fin = (k == p - 2);
            Step st = P.reduce2(BUF_STAGE, left, io.st_off[x], BUF_IN, io.in_off[x],
                                (fin && final_to_out_only) ? BUF_OUT : BUF_STAGE,
                                (fin && final_to_out_only) ? io.out_off[x] : io.st_off[x], io.len[x]);
            if (fin && !final_to_out_only) { st.d2_buf = BUF_OUT; st.d2_off = io.out_off[x]; }
            P.wait_lane(st, left, k);  // left's step k-1 of the loop has index k (pre-step is index 0)
            st.sig_rank = (int16_t)md(r + 1);
            P.add(r, st);
        }
    }
}
// Ring all-gather: at step j rank r copies slice y = (r - 1 + h - j) mod p from its left neighbour, where left
// initially holds slice (left + h).  `first_idx` = index of the step on every rank that produced the initial slice.
void ring_ag(Prog &P, const SliceIo &io, int h, int first_idx)
{
    int p = P.p;
    auto md = [&](int v) { return ((v % p) + p) % p; };
    for (int j = 0; j <= p - 2; ++j) {
        for (int r = 0; r < p; ++r) {
            int y = md(r - 1 + h - j), left = md(r - 1);
            Step st = P.copy(BUF_STAGE, left, io.st_off[y], BUF_STAGE, RANK_SELF, io.st_off[y], io.len[y]);
            st.d2_buf = BUF_OUT; st.d2_off = io.out_off[y];
            P.wait_lane(st, left, first_idx + j);
            st.sig_rank = (int16_t)md(r + 1);
            P.add(r, st);
        }
    }
}

// Zero-copy NVLS AllReduce: both user buffers live in registered symmetric memory with a multicast mapping, so the
// switch reduces straight from the send buffers and multicasts straight into the receive buffers
// (role of the reference's zero-copy path for registered memory, hccl_communicator.cc:400-423 PrepareZeroCopy).
void ar_nvls_zerocopy(Prog &P, const OpDesc &d)
{
    uint64_t n = d.chunk_count, uoff = d.chunk_off * P.es;
    Slices S = make_slices(n, P.p, P.vec);
    for (int r = 0; r < P.p; ++r) {
        Step enter = P.mk(ST_NOP);  // my send buffer is final and my receive buffer may be written
        enter.sig_rank = RANK_ALL;
        int i0 = P.add(r, enter);
        Step red = P.mk(ST_MC_REDUCE);
        red.a_buf = BUF_ZIN; red.a_rank = RANK_ALL; red.a_off = uoff + S.off(r) * P.es;
        red.d_buf = BUF_ZOUT; red.d_rank = RANK_ALL; red.d_off = uoff + S.off(r) * P.es;
        red.count = S.len(r);
        red.wait_rank = RANK_ALL; red.wait_val = (uint32_t)i0 + 1;
        red.sig_rank = RANK_ALL;
        int i1 = P.add(r, red);
        Step fin = P.mk(ST_NOP);    // every slice has landed in my receive buffer and nobody reads my send buffer any more
        fin.wait_rank = RANK_ALL; fin.wait_val = (uint32_t)i1 + 1;
        P.add(r, fin);
    }
}

void ar_ring(Prog &P, const OpDesc &d)
{
    uint64_t n = d.chunk_count, uoff = d.chunk_off * P.es;
    Slices S = make_slices(n, P.p, P.vec);
    SliceIo io;
    for (int j = 0; j < P.p; ++j) {
        io.in_off.push_back(uoff + S.off(j) * P.es);
        io.out_off.push_back(uoff + S.off(j) * P.es);
        io.st_off.push_back(S.off(j) * P.es);
        io.len.push_back(S.len(j));
    }
    ring_rs(P, io, -1, false);
    ring_ag(P, io, 1, P.last(0));
}

// Halving (reduce-scatter) inside the power-of-two block.  range_off(b) = staging byte offset of the start of block
// slice b (b in 0..B), elements between two boundaries are contiguous in staging.  On return lastidx[r] is each
// rank's newest step.  When out_of(b) != ~0 the final step of block rank b also writes its slice to BUF_OUT there.
// Every halving step reduces into the rank's own staging range, split among its channels by the length of THAT step's
// range: the lane of a channel in one step overlaps the lanes of other channels in the step before.  So the channels of a
// rank meet before every step (`barrier_first`: also before the first one, when the caller has not just done so); the
// partner then waits for that meeting point, which lies behind all of the rank's channels.
template <class OffFn, class OutFn>
void hd_reduce_scatter(Prog &P, const HdBlock &H, OffFn range_off, OutFn out_of, bool barrier_first)
{
    int B = H.B;
    std::vector<int> lo(B, 0), hi(B, B);
    for (int width = B; width > 1; width /= 2) {
        if (width != B || barrier_first)
            for (int b = 0; b < B; ++b) P.own_channels_barrier(H.rank_of(b));
        std::vector<int> prev(P.p);
        for (int r = 0; r < P.p; ++r) prev[r] = P.last(r);
        for (int b = 0; b < B; ++b) {
            int half = width / 2, mid = lo[b] + half, partner, klo, khi;
            if (b < mid) { klo = lo[b]; khi = mid; partner = b + half; }
            else { klo = mid; khi = hi[b]; partner = b - half; }
            int r = H.rank_of(b), pr = H.rank_of(partner);
            uint64_t o0 = range_off(klo), o1 = range_off(khi);
            Step st = P.reduce2(BUF_STAGE, pr, o0, BUF_STAGE, o0, BUF_STAGE, o0, (o1 - o0) / P.es);
            if (half == 1) {
                uint64_t oo = out_of(b);
                if (oo != ~0ull) { st.d2_buf = BUF_OUT; st.d2_off = oo; }
            }
            P.wait_allch(st, pr, prev[pr]);
            st.sig_rank = RANK_ALL;
            P.add(r, st);
            lo[b] = klo; hi[b] = khi;
        }
    }
}

void ar_rhd(Prog &P, const OpDesc &d)
{
    uint64_t n = d.chunk_count, uoff = d.chunk_off * P.es;
    HdBlock H = make_block(P.p);
    Slices S = make_slices(n, H.B, P.vec);
    // fold: odd ranks of part one hand their whole input to the even neighbour
    for (int r = 0; r < P.p; ++r) {
        bool odd_p1 = r < H.part1 && (r & 1);
        bool even_p1 = r < H.part1 && !(r & 1);
        if (!even_p1) {
            Step c = P.copy(BUF_IN, RANK_SELF, uoff, BUF_STAGE, RANK_SELF, 0, n);
            c.sig_rank = RANK_ALL;
            P.add(r, c);
        }
        (void)odd_p1;
    }
    for (int r = 0; r < H.part1; r += 2) {
        Step st = P.reduce2(BUF_STAGE, r + 1, 0, BUF_IN, uoff, BUF_STAGE, 0, n);
        P.wait_lane(st, r + 1, 0);
        st.sig_rank = RANK_ALL;
        P.add(r, st);
    }
    // the halving steps write the receive buffer in ranges unrelated to the lanes of the input reads above
    for (int r = 0; r < P.p; ++r) P.own_channels_barrier(r);
    auto off = [&](int b) { return S.off(b) * P.es; };
    hd_reduce_scatter(P, H, off, [&](int b) { return uoff + S.off(b) * P.es; }, false);
    // doubling (all-gather) inside the block
    {
        int B = H.B;
        for (int size = 1; size < B; size *= 2) {
            std::vector<int> prev(P.p);
            for (int r = 0; r < P.p; ++r) prev[r] = P.last(r);
            for (int b = 0; b < B; ++b) {
                int partner = b ^ size;
                int mylo = b & ~(size - 1);
                int slo = (b & size) ? mylo - size : mylo + size;
                int r = H.rank_of(b), pr = H.rank_of(partner);
                uint64_t o0 = off(slo), o1 = off(slo + size);
                Step st = P.copy(BUF_STAGE, pr, o0, BUF_STAGE, RANK_SELF, o0, (o1 - o0) / P.es);
                st.d2_buf = BUF_OUT; st.d2_off = uoff + o0;
                P.wait_allch(st, pr, prev[pr]);
                st.sig_rank = RANK_ALL;
                P.add(r, st);
            }
        }
    }
    // unfold: odd ranks fetch the finished result from their even neighbour
    for (int r = 1; r < H.part1; r += 2) {
        Step st = P.copy(BUF_STAGE, r - 1, 0, BUF_OUT, RANK_SELF, uoff, n);
        P.wait_allch(st, r - 1, P.last(r - 1));
        P.add(r, st);
    }
}

// ------------------------------------------------------------------------------------------------
// ReduceScatter / ReduceScatterV.  slot j of staging (byte offset st[j]) holds the contribution to rank j.
// ------------------------------------------------------------------------------------------------
struct Slots {
    std::vector<uint64_t> in_off, out_off, st_off, len;  // per rank slot
    uint64_t total_stage = 0;
};
// Uniform slots: `n` elements of each rank's block, block j in the user buffer at element j*count + coff.
Slots uniform_slots(const Prog &P, uint64_t n, uint64_t count, uint64_t coff, bool user_is_in)
{
    Slots s;
    uint64_t nA = round_up_u64(std::max<uint64_t>(n, 1), P.vec);
    for (int j = 0; j < P.p; ++j) {
        uint64_t u = ((uint64_t)j * count + coff) * P.es;
        s.in_off.push_back(user_is_in ? u : 0);
        s.out_off.push_back(user_is_in ? 0 : u);
        s.st_off.push_back((uint64_t)j * nA * P.es);
        s.len.push_back(n);
    }
    s.total_stage = (uint64_t)P.p * nA * P.es;
    return s;
}
// V slots: windows [coff, coff+n) of every rank's block (clamped to its count).
Slots v_slots(const Prog &P, const std::vector<uint64_t> &counts, const std::vector<uint64_t> &displs, uint64_t coff,
              uint64_t n, bool user_is_in)
{
    Slots s;
    uint64_t o = 0;
    for (int j = 0; j < P.p; ++j) {
        uint64_t c = counts[j] > coff ? std::min(n, counts[j] - coff) : 0;
        uint64_t u = (displs[j] + coff) * P.es;
        s.in_off.push_back(user_is_in ? u : 0);
        s.out_off.push_back(user_is_in ? 0 : u);
        s.st_off.push_back(o);
        s.len.push_back(c);
        o += round_up_u64(std::max<uint64_t>(c, 1), P.vec) * P.es;
    }
    s.total_stage = o;
    return s;
}

void rs_mesh(Prog &P, const Slots &S, uint64_t out_off, bool nvls)
{
    for (int r = 0; r < P.p; ++r) {
        int last = 0;
        for (int j = 0; j < P.p; ++j) {
            Step c = P.copy(BUF_IN, RANK_SELF, S.in_off[j], BUF_STAGE, RANK_SELF, S.st_off[j], S.len[j]);
            if (j == P.p - 1) c.sig_rank = RANK_ALL;
            last = P.add(r, c);
        }
        Step red = P.mk(nvls ? ST_MC_REDUCE : ST_REDUCE_ALL);
        red.a_buf = BUF_STAGE; red.a_rank = RANK_ALL; red.a_off = S.st_off[r];
        red.d_buf = BUF_OUT; red.d_off = out_off; red.count = S.len[r];
        red.wait_rank = RANK_ALL; red.wait_val = (uint32_t)last + 1;
        P.add(r, red);
    }
}
void rs_ring(Prog &P, const Slots &S, uint64_t out_off)
{
    SliceIo io;
    io.in_off = S.in_off; io.st_off = S.st_off; io.len = S.len;
    io.out_off.assign(P.p, out_off);
    ring_rs(P, io, -2, true);
}
void rs_rhd(Prog &P, const Slots &S, uint64_t out_off)
{
    HdBlock H = make_block(P.p);
    int p = P.p;
    // every rank except the even ranks of part one stages its p contributions
    for (int r = 0; r < p; ++r) {
        bool even_p1 = r < H.part1 && !(r & 1);
        if (even_p1) continue;
        for (int j = 0; j < p; ++j) {
            Step c = P.copy(BUF_IN, RANK_SELF, S.in_off[j], BUF_STAGE, RANK_SELF, S.st_off[j], S.len[j]);
            c.sig_rank = RANK_ALL;
            P.add(r, c);
        }
    }
    for (int r = 0; r < H.part1; r += 2) {
        for (int j = 0; j < p; ++j) {
            Step st = P.reduce2(BUF_STAGE, r + 1, S.st_off[j], BUF_IN, S.in_off[j], BUF_STAGE, S.st_off[j], S.len[j]);
            P.wait_lane(st, r + 1, j);
            st.sig_rank = RANK_ALL;
            P.add(r, st);
        }
    }
    for (int r = 0; r < p; ++r) P.own_channels_barrier(r);  // in place: all input reads before the first output write
    auto off = [&](int b) -> uint64_t {
        if (b >= H.B) return S.total_stage;
        int lo, hi;
        H.ranks_of(b, lo, hi);
        return S.st_off[lo];
    };
    hd_reduce_scatter(P, H, off, [](int) { return ~0ull; }, false);
    // a folded pair's block spans two slots, so the lanes of the last halving step are not the lanes of the copy-out below:
    // the channels of such a rank meet once more (power-of-two rank counts: same range, same lanes, nothing to do)
    for (int r = 0; r < H.part1; r += 2) P.own_channels_barrier(r);
    std::vector<int> lastidx(p);
    for (int r = 0; r < p; ++r) lastidx[r] = P.last(r);
    for (int r = 0; r < p; ++r) {
        bool odd_p1 = r < H.part1 && (r & 1);
        int owner = odd_p1 ? r - 1 : r;
        Step st = P.copy(BUF_STAGE, owner == r ? RANK_SELF : owner, S.st_off[r], BUF_OUT, RANK_SELF, out_off, S.len[r]);
        if (owner != r) P.wait_allch(st, owner, lastidx[owner]);
        P.add(r, st);
    }
}

// ------------------------------------------------------------------------------------------------
// AllGather / AllGatherV.  slot j = block contributed by rank j.
// ------------------------------------------------------------------------------------------------
void ag_mesh(Prog &P, const Slots &S, uint64_t in_off, bool uniform, uint64_t d_stride, bool nvls)
{
    for (int r = 0; r < P.p; ++r) {
        if (nvls) {
            Step c = P.copy(BUF_IN, RANK_SELF, in_off, BUF_STAGE, RANK_ALL, S.st_off[r], S.len[r]);
            c.sig_rank = RANK_ALL;
            P.add(r, c);
        } else {
            Step c = P.copy(BUF_IN, RANK_SELF, in_off, BUF_STAGE, RANK_SELF, 0, S.len[r]);
            c.sig_rank = RANK_ALL;
            P.add(r, c);
        }
        if (uniform) {
            Step g = P.mk(ST_GATHER_ALL);
            g.a_buf = BUF_STAGE;
            g.a_rank = nvls ? RANK_SELF : RANK_ALL;
            g.a_off = 0;
            g.a_stride = nvls ? (S.st_off.size() > 1 ? S.st_off[1] - S.st_off[0] : 0) : 0;
            g.d_buf = BUF_OUT; g.d_off = S.out_off[0]; g.d_stride = d_stride;
            g.count = S.len[0];
            g.wait_rank = RANK_ALL; g.wait_val = 1;
            P.add(r, g);
        } else {
            for (int i = 0; i < P.p; ++i) {
                int q = (r + i) % P.p;
                Step c = nvls ? P.copy(BUF_STAGE, RANK_SELF, S.st_off[q], BUF_OUT, RANK_SELF, S.out_off[q], S.len[q])
                              : P.copy(BUF_STAGE, q == r ? RANK_SELF : q, 0, BUF_OUT, RANK_SELF, S.out_off[q], S.len[q]);
                if (q != r) P.wait_lane(c, q, 0);
                P.add(r, c);
            }
        }
    }
}
// Push variant of the mesh AllGather (role of the reference's AllGatherMeshDirect, all_gather_mesh_direct.cc, and of its
// AIV all-to-all push kernels): step i of rank r stores r's block straight into the staging slot r of rank (r+i)%p and
// signals that one rank; receivers copy each slot out as its flag arrives.  One remote store pass instead of a local staging
// copy followed by remote loads: the sender's input is read once and nothing waits for a round trip.
void ag_push(Prog &P, const Slots &S, uint64_t in_off)
{
    const int p = P.p;
    for (int r = 0; r < p; ++r) {
        P.add(r, P.copy(BUF_IN, RANK_SELF, in_off, BUF_OUT, RANK_SELF, S.out_off[r], S.len[r]));  // step 0: own block
        for (int i = 1; i < p; ++i) {  // step i: push to the i-th rank after me
            int q = (r + i) % p;
            Step c = P.copy(BUF_IN, RANK_SELF, in_off, BUF_STAGE, q, S.st_off[r], S.len[r]);
            c.sig_rank = (int16_t)q;
            P.add(r, c);
        }
        for (int i = 1; i < p; ++i) {  // the i-th rank before me pushed its block in its step i
            int src = (r - i + p) % p;
            Step c = P.copy(BUF_STAGE, RANK_SELF, S.st_off[src], BUF_OUT, RANK_SELF, S.out_off[src], S.len[src]);
            P.wait_lane(c, src, i);
            P.add(r, c);
        }
    }
}
void ag_ring(Prog &P, const Slots &S, uint64_t in_off)
{
    for (int r = 0; r < P.p; ++r) {
        Step c = P.copy(BUF_IN, RANK_SELF, in_off, BUF_STAGE, RANK_SELF, S.st_off[r], S.len[r]);
        c.d2_buf = BUF_OUT; c.d2_off = S.out_off[r];
        c.sig_rank = (int16_t)((r + 1) % P.p);
        P.add(r, c);
    }
    SliceIo io;
    io.st_off = S.st_off; io.out_off = S.out_off; io.len = S.len; io.in_off = S.in_off;
    ring_ag(P, io, 0, 0);
}
void ag_rhd(Prog &P, const Slots &S, uint64_t in_off)
{
    HdBlock H = make_block(P.p);
    int p = P.p;
    for (int r = 0; r < p; ++r) {
        Step c = P.copy(BUF_IN, RANK_SELF, in_off, BUF_STAGE, RANK_SELF, S.st_off[r], S.len[r]);
        c.d2_buf = BUF_OUT; c.d2_off = S.out_off[r];
        c.sig_rank = RANK_ALL;
        P.add(r, c);
    }
    for (int r = 0; r < H.part1; r += 2) {  // fold: even rank adopts the odd neighbour's block
        Step c = P.copy(BUF_STAGE, r + 1, S.st_off[r + 1], BUF_STAGE, RANK_SELF, S.st_off[r + 1], S.len[r + 1]);
        c.d2_buf = BUF_OUT; c.d2_off = S.out_off[r + 1];
        P.wait_lane(c, r + 1, 0);
        c.sig_rank = RANK_ALL;
        P.add(r, c);
    }
    for (int size = 1; size < H.B; size *= 2) {
        std::vector<int> prev(p);
        for (int r = 0; r < p; ++r) prev[r] = P.last(r);
        for (int b = 0; b < H.B; ++b) {
            int partner = b ^ size, mylo = b & ~(size - 1);
            int slo = (b & size) ? mylo - size : mylo + size;
            int r = H.rank_of(b), pr = H.rank_of(partner);
            for (int sb = slo; sb < slo + size; ++sb) {
                int lo, hi;
                H.ranks_of(sb, lo, hi);
                for (int j = lo; j < hi; ++j) {
                    Step c = P.copy(BUF_STAGE, pr, S.st_off[j], BUF_STAGE, RANK_SELF, S.st_off[j], S.len[j]);
                    c.d2_buf = BUF_OUT; c.d2_off = S.out_off[j];
                    P.wait_allch(c, pr, prev[pr]);
                    c.sig_rank = RANK_ALL;
                    P.add(r, c);
                }
            }
        }
    }
    for (int r = 1; r < H.part1; r += 2) {  // unfold
        int ev = r - 1, lastev = P.last(ev);
        for (int j = 0; j < p; ++j) {
            if (j == r) continue;
            Step c = P.copy(BUF_STAGE, ev, S.st_off[j], BUF_OUT, RANK_SELF, S.out_off[j], S.len[j]);
            P.wait_allch(c, ev, lastev);
            P.add(r, c);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Rooted collectives
// ------------------------------------------------------------------------------------------------
constexpr int kPipeSub = 4;  // sub-chunks used to pipeline chains

void bcast_star(Prog &P, const OpDesc &d, bool nvls)
{
    uint64_t n = d.chunk_count, uoff = d.chunk_off * P.es;
    for (int r = 0; r < P.p; ++r) {
        if (r == d.root) {
            Step c = P.copy(BUF_IN, RANK_SELF, uoff, BUF_STAGE, nvls ? RANK_ALL : RANK_SELF, 0, n);
            c.sig_rank = RANK_ALL;
            P.add(r, c);
        } else {
            Step c = P.copy(BUF_STAGE, nvls ? RANK_SELF : d.root, 0, BUF_OUT, RANK_SELF, uoff, n);
            P.wait_lane(c, d.root, 0);
            P.add(r, c);
        }
    }
}
void bcast_ring(Prog &P, const OpDesc &d)
{
    uint64_t n = d.chunk_count, uoff = d.chunk_off * P.es;
    Slices S = make_slices(n, kPipeSub, P.vec);
    int p = P.p;
    for (int t = 0; t < kPipeSub; ++t) {
        for (int r = 0; r < p; ++r) {
            int dist = (r - d.root + p) % p, left = (r - 1 + p) % p, right = (r + 1) % p;
            Step c;
            if (dist == 0) c = P.copy(BUF_IN, RANK_SELF, uoff + S.off(t) * P.es, BUF_STAGE, RANK_SELF, S.off(t) * P.es, S.len(t));
            else {
                c = P.copy(BUF_STAGE, left, S.off(t) * P.es, BUF_STAGE, RANK_SELF, S.off(t) * P.es, S.len(t));
                c.d2_buf = BUF_OUT; c.d2_off = uoff + S.off(t) * P.es;
                P.wait_lane(c, left, t);
            }
            if (dist != p - 1) c.sig_rank = (int16_t)right;
            P.add(r, c);
        }
    }
}
void bcast_tree(Prog &P, const OpDesc &d)
{
    uint64_t n = d.chunk_count, uoff = d.chunk_off * P.es;
    int p = P.p;
    for (int r = 0; r < p; ++r) {
        int v = (r - d.root + p) % p;
        Step c;
        if (v == 0) c = P.copy(BUF_IN, RANK_SELF, uoff, BUF_STAGE, RANK_SELF, 0, n);
        else {
            int pv = v & (v - 1), parent = (pv + d.root) % p;
            c = P.copy(BUF_STAGE, parent, 0, BUF_STAGE, RANK_SELF, 0, n);
            c.d2_buf = BUF_OUT; c.d2_off = uoff;
            P.wait_lane(c, parent, 0);
        }
        c.sig_rank = RANK_ALL;
        P.add(r, c);
    }
}

void reduce_star(Prog &P, const OpDesc &d)
{
    uint64_t n = d.chunk_count, uoff = d.chunk_off * P.es;
    for (int r = 0; r < P.p; ++r) {
        Step c = P.copy(BUF_IN, RANK_SELF, uoff, BUF_STAGE, RANK_SELF, 0, n);
        if (r != d.root) c.sig_rank = (int16_t)d.root;
        P.add(r, c);
        if (r == d.root) {
            Step red = P.mk(ST_REDUCE_ALL);
            red.a_buf = BUF_STAGE; red.a_rank = RANK_ALL; red.a_off = 0;
            red.d_buf = BUF_OUT; red.d_off = uoff; red.count = n;
            red.wait_rank = RANK_ALL; red.wait_val = 1;
            P.add(r, red);
        }
    }
}
void reduce_ring(Prog &P, const OpDesc &d)
{
    uint64_t n = d.chunk_count, uoff = d.chunk_off * P.es;
    Slices S = make_slices(n, kPipeSub, P.vec);
    int p = P.p;
    for (int t = 0; t < kPipeSub; ++t) {
        for (int r = 0; r < p; ++r) {
            int v = (r - d.root + p) % p, left = (r - 1 + p) % p, right = (r + 1) % p;
            uint64_t so = S.off(t) * P.es;
            Step c;
            if (v == 1) c = P.copy(BUF_IN, RANK_SELF, uoff + so, BUF_STAGE, RANK_SELF, so, S.len(t));
            else {
                c = P.reduce2(BUF_STAGE, left, so, BUF_IN, uoff + so, v == 0 ? BUF_OUT : BUF_STAGE,
                              v == 0 ? uoff + so : so, S.len(t));
                P.wait_lane(c, left, t);
            }
            if (v != 0) c.sig_rank = (int16_t)right;
            P.add(r, c);
        }
    }
}
void reduce_tree(Prog &P, const OpDesc &d)
{
    uint64_t n = d.chunk_count, uoff = d.chunk_off * P.es;
    int p = P.p;
    for (int r = 0; r < p; ++r) {
        Step c = P.copy(BUF_IN, RANK_SELF, uoff, BUF_STAGE, RANK_SELF, 0, n);
        c.sig_rank = RANK_ALL;
        P.add(r, c);
    }
    std::vector<bool> done(p, false);
    for (int mask = 1; mask < p; mask <<= 1) {
        std::vector<int> prev(p);
        for (int r = 0; r < p; ++r) prev[r] = P.last(r);
        for (int v = 0; v < p; ++v) {
            if (done[v]) continue;
            if (v & mask) { done[v] = true; continue; }
            int cv = v + mask;
            if (cv >= p) continue;
            int r = (v + d.root) % p, child = (cv + d.root) % p;
            Step st = P.reduce2(BUF_STAGE, child, 0, BUF_STAGE, 0, BUF_STAGE, 0, n);
            P.wait_lane(st, child, prev[child]);
            st.sig_rank = RANK_ALL;
            P.add(r, st);
        }
    }
    P.add(d.root, P.copy(BUF_STAGE, RANK_SELF, 0, BUF_OUT, RANK_SELF, uoff, n));
}
// Bandwidth-optimal rooted reduce: fold + halving inside the block, then the root collects the block slices.
void reduce_rhd(Prog &P, const OpDesc &d)
{
    uint64_t n = d.chunk_count, uoff = d.chunk_off * P.es;
    HdBlock H = make_block(P.p);
    Slices S = make_slices(n, H.B, P.vec);
    for (int r = 0; r < P.p; ++r) {
        bool even_p1 = r < H.part1 && !(r & 1);
        if (even_p1) continue;
        Step c = P.copy(BUF_IN, RANK_SELF, uoff, BUF_STAGE, RANK_SELF, 0, n);
        c.sig_rank = RANK_ALL;
        P.add(r, c);
    }
    for (int r = 0; r < H.part1; r += 2) {
        Step st = P.reduce2(BUF_STAGE, r + 1, 0, BUF_IN, uoff, BUF_STAGE, 0, n);
        P.wait_lane(st, r + 1, 0);
        st.sig_rank = RANK_ALL;
        P.add(r, st);
    }
    // in place at the root: all of its input reads before its first output write (block ranks meet in the halving steps anyway)
    if (H.block_of(d.root) < 0) P.own_channels_barrier(d.root);
    auto off = [&](int b) { return S.off(b) * P.es; };
    hd_reduce_scatter(P, H, off, [](int) { return ~0ull; }, true);
    std::vector<int> lastidx(P.p);
    for (int r = 0; r < P.p; ++r) lastidx[r] = P.last(r);
    for (int b = 0; b < H.B; ++b) {
        int owner = H.rank_of(b);
        Step c = P.copy(BUF_STAGE, owner == d.root ? RANK_SELF : owner, off(b), BUF_OUT, RANK_SELF, uoff + off(b), S.len(b));
        if (owner != d.root) P.wait_allch(c, owner, lastidx[owner]);
        P.add(d.root, c);
    }
}

void scatter_star(Prog &P, const OpDesc &d, const Slots &S, uint64_t out_off)
{
    int p = P.p;
    for (int j = 0; j < p; ++j) {
        Step c = P.copy(BUF_IN, RANK_SELF, S.in_off[j], BUF_STAGE, RANK_SELF, S.st_off[j], S.len[j]);
        if (j == p - 1) c.sig_rank = RANK_ALL;
        P.add(d.root, c);
    }
    for (int r = 0; r < p; ++r) {
        Step c = P.copy(BUF_STAGE, r == d.root ? RANK_SELF : d.root, S.st_off[r], BUF_OUT, RANK_SELF, out_off, S.len[r]);
        if (r != d.root) P.wait_lane(c, d.root, p - 1);
        P.add(r, c);
    }
}
void scatter_ring(Prog &P, const OpDesc &d, const Slots &S, uint64_t out_off)
{
    int p = P.p;
    // root stages the blocks in order of ring distance; rank at distance v forwards blocks of distance >= v
    for (int dist = 0; dist < p; ++dist) {
        int j = (d.root + dist) % p;
        Step c = P.copy(BUF_IN, RANK_SELF, S.in_off[j], BUF_STAGE, RANK_SELF, S.st_off[j], S.len[j]);
        if (dist == 0) { c.d2_buf = BUF_OUT; c.d2_off = out_off; }
        c.sig_rank = (int16_t)((d.root + 1) % p);
        P.add(d.root, c);
    }
    for (int v = 1; v < p; ++v) {
        int r = (d.root + v) % p, left = (r - 1 + p) % p;
        for (int dist = v; dist < p; ++dist) {
            int j = (d.root + dist) % p;
            Step c = P.copy(BUF_STAGE, left, S.st_off[j], dist == v ? BUF_OUT : BUF_STAGE, RANK_SELF,
                            dist == v ? out_off : S.st_off[j], S.len[j]);
            P.wait_lane(c, left, dist - (v - 1));
            if (v != p - 1) c.sig_rank = (int16_t)((r + 1) % p);
            P.add(r, c);
        }
    }
}
void gather_star(Prog &P, const OpDesc &d, const Slots &S, uint64_t in_off, uint64_t d_stride)
{
    for (int r = 0; r < P.p; ++r) {
        Step c = P.copy(BUF_IN, RANK_SELF, in_off, BUF_STAGE, RANK_SELF, 0, S.len[0]);
        if (r != d.root) c.sig_rank = (int16_t)d.root;
        P.add(r, c);
        if (r == d.root) {
            Step g = P.mk(ST_GATHER_ALL);
            g.a_buf = BUF_STAGE; g.a_rank = RANK_ALL; g.a_off = 0; g.a_stride = 0;
            g.d_buf = BUF_OUT; g.d_off = S.out_off[0]; g.d_stride = d_stride; g.count = S.len[0];
            g.wait_rank = RANK_ALL; g.wait_val = 1;
            P.add(r, g);
        }
    }
}
void gather_ring(Prog &P, const OpDesc &d, const Slots &S, uint64_t in_off)
{
    int p = P.p;
    // blocks flow towards the root against ring distance: rank at distance v holds blocks of distance v..p-1
    for (int v = p - 1; v >= 0; --v) {
        int r = (d.root + v) % p, from = (d.root + v + 1) % p, to = (d.root + v - 1 + p) % p;
        Step c = P.copy(BUF_IN, RANK_SELF, in_off, v == 0 ? BUF_OUT : BUF_STAGE, RANK_SELF,
                        v == 0 ? S.out_off[r] : S.st_off[r], S.len[r]);
        if (v != 0) c.sig_rank = (int16_t)to;
        P.add(r, c);
        for (int dist = v + 1; dist < p; ++dist) {
            int j = (d.root + dist) % p;
            Step f = P.copy(BUF_STAGE, from, S.st_off[j], v == 0 ? BUF_OUT : BUF_STAGE, RANK_SELF,
                            v == 0 ? S.out_off[j] : S.st_off[j], S.len[j]);
            P.wait_lane(f, from, dist - (v + 1));
            if (v != 0) f.sig_rank = (int16_t)to;
            P.add(r, f);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// AlltoAll (uniform)
// ------------------------------------------------------------------------------------------------
void a2a_uniform(Prog &P, const OpDesc &d, bool pairwise)
{
    uint64_t n = d.chunk_count;
    int p = P.p;
    uint64_t nA = round_up_u64(std::max<uint64_t>(n, 1), P.vec) * P.es;
    for (int r = 0; r < p; ++r) {
        int last = 0;
        for (int j = 0; j < p; ++j) {
            Step c = P.copy(BUF_IN, RANK_SELF, ((uint64_t)j * d.count + d.chunk_off) * P.es, BUF_STAGE, RANK_SELF,
                            (uint64_t)j * nA, n);
            if (j == p - 1) c.sig_rank = RANK_ALL;
            last = P.add(r, c);
        }
        if (!pairwise) {
            Step g = P.mk(ST_GATHER_ALL);
            g.a_buf = BUF_STAGE; g.a_rank = RANK_ALL; g.a_off = (uint64_t)r * nA; g.a_stride = 0;
            g.d_buf = BUF_OUT; g.d_off = d.chunk_off * P.es; g.d_stride = d.count * P.es; g.count = n;
            g.wait_rank = RANK_ALL; g.wait_val = (uint32_t)last + 1;
            P.add(r, g);
        } else {
            for (int i = 0; i < p; ++i) {
                int prev = (r - i + p) % p;
                Step c = P.copy(BUF_STAGE, prev == r ? RANK_SELF : prev, (uint64_t)r * nA, BUF_OUT, RANK_SELF,
                                ((uint64_t)prev * d.count + d.chunk_off) * P.es, n);
                if (prev != r) P.wait_lane(c, prev, last);
                P.add(r, c);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// AlltoAllV / AlltoAllVC: push into per-sender slots of the receiver's staging, rounds with acknowledgements
// (role of the BCopy mode of algorithm/base/alg_template/temp_alltoallv/alltoallv_pairwise.cc).
// Built per rank from that rank's own rows only; flag values count rounds per ordered pair.
// ------------------------------------------------------------------------------------------------
void a2av_rank(Prog &P, const OpDesc &d, int r, const uint64_t *sc, const uint64_t *sd, const uint64_t *rc,
               const uint64_t *rd, bool pairwise)
{
    int p = P.p;
    uint64_t slotE = (d.slot_bytes / P.es) / P.vec * P.vec;
    auto rounds = [&](uint64_t c) { return (uint32_t)ceil_div_u64(c, slotE); };
    auto push = [&](int to, uint32_t k) {
        uint64_t cnt = std::min(slotE, sc[to] - (uint64_t)k * slotE);
        Step c = P.copy(BUF_IN, RANK_SELF, (sd[to] + (uint64_t)k * slotE) * P.es, BUF_STAGE, to, (uint64_t)r * d.slot_bytes, cnt);
        if (k >= 1) {
            c.wait_rank = (int16_t)to; c.wait_bank = 1; c.wait_val = k;
            c.flags |= SF_WAIT_ALLCH; c.wait_clo = 0; c.wait_cn = (uint16_t)P.nchan;
        }
        c.sig_rank = (int16_t)to; c.sig_bank = 0; c.sig_val = k + 1;
        P.add(r, c, true);
    };
    auto pull = [&](int from, uint32_t k) {
        uint64_t cnt = std::min(slotE, rc[from] - (uint64_t)k * slotE);
        Step c = P.copy(BUF_STAGE, RANK_SELF, (uint64_t)from * d.slot_bytes, BUF_OUT, RANK_SELF,
                        (rd[from] + (uint64_t)k * slotE) * P.es, cnt);
        c.wait_rank = (int16_t)from; c.wait_bank = 0; c.wait_val = k + 1;
        c.sig_rank = (int16_t)from; c.sig_bank = 1; c.sig_val = k + 1;
        P.add(r, c, true);
    };
    P.add(r, P.copy(BUF_IN, RANK_SELF, sd[r] * P.es, BUF_OUT, RANK_SELF, rd[r] * P.es, std::min(sc[r], rc[r])), true);
    if (pairwise) {
        for (int i = 1; i < p; ++i) {
            int nx = (r + i) % p, pv = (r - i + p) % p;
            uint32_t Rs = rounds(sc[nx]), Rr = rounds(rc[pv]);
            for (uint32_t k = 0; k < std::max(Rs, Rr); ++k) {
                if (k < Rs) push(nx, k);
                if (k < Rr) pull(pv, k);
            }
        }
    } else {
        uint32_t R = 0;
        for (int q = 0; q < p; ++q)
            if (q != r) R = std::max(R, std::max(rounds(sc[q]), rounds(rc[q])));
        for (uint32_t k = 0; k < R; ++k) {
            for (int i = 1; i < p; ++i) { int q = (r + i) % p; if (k < rounds(sc[q])) push(q, k); }
            for (int i = 1; i < p; ++i) { int q = (r - i + p) % p; if (k < rounds(rc[q])) pull(q, k); }
        }
    }
}

// Send / Recv over the mailbox area (host and emulated transports; the device transport uses NCCL p2p).
void p2p_rank(Prog &P, const OpDesc &d, int r, bool is_send)
{
    uint64_t slotE = (d.p2p_slot / P.es) / P.vec * P.vec;
    uint32_t R = (uint32_t)ceil_div_u64(d.count, slotE);
    for (uint32_t k = 0; k < R; ++k) {
        uint32_t g = d.p2p_round0 + k + 1;  // 1-based round number on this ordered pair, since communicator creation
        uint64_t cnt = std::min(slotE, d.count - (uint64_t)k * slotE);
        Step c;
        if (is_send) {
            c = P.copy(BUF_IN, RANK_SELF, (uint64_t)k * slotE * P.es, BUF_P2P, d.peer, (uint64_t)r * d.p2p_slot, cnt);
            if (g > 1) {
                c.wait_rank = (int16_t)d.peer; c.wait_bank = 3; c.wait_val = g - 1;
                c.flags |= SF_WAIT_ALLCH; c.wait_clo = 0; c.wait_cn = (uint16_t)P.nchan;
            }
            c.sig_rank = (int16_t)d.peer; c.sig_bank = 2; c.sig_val = g;
        } else {
            c = P.copy(BUF_P2P, RANK_SELF, (uint64_t)d.peer * d.p2p_slot, BUF_OUT, RANK_SELF, (uint64_t)k * slotE * P.es, cnt);
            c.wait_rank = (int16_t)d.peer; c.wait_bank = 2; c.wait_val = g;
            c.sig_rank = (int16_t)d.peer; c.sig_bank = 3; c.sig_val = g;
        }
        c.flags |= SF_ABS_VALS;
        P.add(r, c, true);
    }
}

}  // namespace

uint64_t plan_stage_bytes(const OpDesc &d)
{
    int es = dtype_size(d.dtype);
    uint64_t vec = es >= 16 ? 1 : 16 / es;
    uint64_t n = d.chunk_count, p = (uint64_t)d.nranks;
    uint64_t nA = round_up_u64(std::max<uint64_t>(n, 1), vec) * es;
    switch (d.coll) {
        case COLL_ALLREDUCE: {
            int m = d.algo == ALGO_RHD ? make_block(d.nranks).B : d.nranks;
            uint64_t sl = std::max<uint64_t>(round_up_u64(ceil_div_u64(n, (uint64_t)m), vec), vec);
            uint64_t region = round_up_u64(sl * m * es, 256);
            if (d.algo == ALGO_NVLS_ZC) return 0;
            return std::max<uint64_t>(region, nA);
        }
        case COLL_REDUCE_SCATTER: case COLL_ALLGATHER: case COLL_SCATTER: case COLL_GATHER: case COLL_ALLTOALL:
            return p * nA;
        case COLL_REDUCE_SCATTER_V: case COLL_ALLGATHER_V: {
            uint64_t o = 0;
            for (uint64_t j = 0; j < p && j < d.counts.size(); ++j) {
                uint64_t c = d.counts[j] > d.chunk_off ? std::min(n, d.counts[j] - d.chunk_off) : 0;
                o += round_up_u64(std::max<uint64_t>(c, 1), vec) * es;
            }
            return o;
        }
        case COLL_ALLTOALLV: case COLL_ALLTOALLVC: return p * d.slot_bytes;
        case COLL_BARRIER: case COLL_SEND: case COLL_RECV: return 0;
        default: return nA + 256;  // Broadcast, Reduce
    }
}

HcclResult build_plan(const OpDesc &d, const std::vector<int> &local, Plan *plan)
{
    int es = dtype_size(d.dtype);
    if (es == 0 || d.nranks < 1 || d.nranks > kMaxRanks || d.nchan < 1 || d.nchan > kMaxChannels) return HCCL_E_PARA;
    Prog P(d.nranks, d.nchan, es);
    int p = d.nranks;
    uint64_t n = d.chunk_count, coff = d.chunk_off;
    bool ok = true;
    if (p == 1 || d.algo == ALGO_SINGLE) {
        // single rank: every collective degenerates to a local copy of the caller's block
        switch (d.coll) {
            case COLL_BARRIER: P.add(0, P.mk(ST_NOP)); break;
            case COLL_BROADCAST: P.add(0, P.mk(ST_NOP)); break;
            case COLL_ALLTOALLV: case COLL_ALLTOALLVC:
                P.add(0, P.copy(BUF_IN, RANK_SELF, d.send_displs[0] * es, BUF_OUT, RANK_SELF, d.recv_displs[0] * es, d.send_counts[0]));
                break;
            case COLL_ALLGATHER_V:
                P.add(0, P.copy(BUF_IN, RANK_SELF, coff * es, BUF_OUT, RANK_SELF, (d.displs[0] + coff) * es, n));
                break;
            case COLL_REDUCE_SCATTER_V:
                P.add(0, P.copy(BUF_IN, RANK_SELF, (d.displs[0] + coff) * es, BUF_OUT, RANK_SELF, coff * es, n));
                break;
            default: P.add(0, P.copy(BUF_IN, RANK_SELF, coff * es, BUF_OUT, RANK_SELF, coff * es, n)); break;
        }
    } else {
        switch (d.coll) {
            case COLL_ALLREDUCE:
                if (d.algo == ALGO_MESH_ONESHOT) ar_mesh_oneshot(P, d, false);
                else if (d.algo == ALGO_NVLS_ONESHOT) ar_mesh_oneshot(P, d, true);
                else if (d.algo == ALGO_MESH) ar_mesh_twoshot(P, d, false);
                else if (d.algo == ALGO_NVLS) ar_mesh_twoshot(P, d, true);
                else if (d.algo == ALGO_NVLS_ZC) ar_nvls_zerocopy(P, d);
                else if (d.algo == ALGO_RING) ar_ring(P, d);
                else if (d.algo == ALGO_RHD) ar_rhd(P, d);
                else ok = false;
                break;
            case COLL_REDUCE_SCATTER: case COLL_REDUCE_SCATTER_V: {
                Slots S = d.coll == COLL_REDUCE_SCATTER ? uniform_slots(P, n, d.count, coff, true)
                                                        : v_slots(P, d.counts, d.displs, coff, n, true);
                uint64_t oo = coff * es;
                if (d.algo == ALGO_MESH) rs_mesh(P, S, oo, false);
                else if (d.algo == ALGO_NVLS) rs_mesh(P, S, oo, true);
                else if (d.algo == ALGO_RING) rs_ring(P, S, oo);
                else if (d.algo == ALGO_RHD) rs_rhd(P, S, oo);
                else ok = false;
                break;
            }
            case COLL_ALLGATHER: case COLL_ALLGATHER_V: {
                bool uni = d.coll == COLL_ALLGATHER;
                Slots S = uni ? uniform_slots(P, n, d.count, coff, false) : v_slots(P, d.counts, d.displs, coff, n, false);
                uint64_t io = coff * es;
                if (d.algo == ALGO_MESH) ag_mesh(P, S, io, uni, d.count * es, false);
                else if (d.algo == ALGO_NVLS) ag_mesh(P, S, io, uni, d.count * es, true);
                else if (d.algo == ALGO_RING) ag_ring(P, S, io);
                else if (d.algo == ALGO_PAIRWISE) ag_push(P, S, io);
                else if (d.algo == ALGO_RHD) ag_rhd(P, S, io);
                else ok = false;
                break;
            }
            case COLL_BROADCAST:
                if (d.algo == ALGO_STAR || d.algo == ALGO_MESH) bcast_star(P, d, false);
                else if (d.algo == ALGO_NVLS) bcast_star(P, d, true);
                else if (d.algo == ALGO_RING) bcast_ring(P, d);
                else if (d.algo == ALGO_TREE || d.algo == ALGO_RHD) bcast_tree(P, d);
                else ok = false;
                break;
            case COLL_REDUCE:
                if (d.algo == ALGO_STAR || d.algo == ALGO_MESH) reduce_star(P, d);
                else if (d.algo == ALGO_RING) reduce_ring(P, d);
                else if (d.algo == ALGO_TREE) reduce_tree(P, d);
                else if (d.algo == ALGO_RHD) reduce_rhd(P, d);
                else ok = false;
                break;
            case COLL_SCATTER: {
                Slots S = uniform_slots(P, n, d.count, coff, true);
                if (d.algo == ALGO_STAR || d.algo == ALGO_MESH) scatter_star(P, d, S, coff * es);
                else if (d.algo == ALGO_RING) scatter_ring(P, d, S, coff * es);
                else ok = false;
                break;
            }
            case COLL_GATHER: {
                Slots S = uniform_slots(P, n, d.count, coff, false);
                if (d.algo == ALGO_STAR || d.algo == ALGO_MESH) gather_star(P, d, S, coff * es, d.count * es);
                else if (d.algo == ALGO_RING) gather_ring(P, d, S, coff * es);
                else ok = false;
                break;
            }
            case COLL_ALLTOALL:
                if (d.algo == ALGO_MESH) a2a_uniform(P, d, false);
                else if (d.algo == ALGO_PAIRWISE) a2a_uniform(P, d, true);
                else ok = false;
                break;
            case COLL_ALLTOALLV: case COLL_ALLTOALLVC: {
                if (d.algo != ALGO_MESH && d.algo != ALGO_PAIRWISE) { ok = false; break; }
                if (d.slot_bytes < 16 || d.send_counts.size() != local.size() * (size_t)p) return HCCL_E_PARA;
                for (size_t li = 0; li < local.size(); ++li)
                    a2av_rank(P, d, local[li], &d.send_counts[li * p], &d.send_displs[li * p], &d.recv_counts[li * p],
                              &d.recv_displs[li * p], d.algo == ALGO_PAIRWISE);
                break;
            }
            case COLL_BARRIER:
                for (int r = 0; r < p; ++r) {
                    Step a = P.mk(ST_NOP);
                    a.sig_rank = RANK_ALL;
                    P.add(r, a);
                    Step b = P.mk(ST_NOP);
                    b.wait_rank = RANK_ALL; b.wait_val = 1;
                    P.add(r, b);
                }
                break;
            case COLL_SEND: case COLL_RECV:
                if (d.peer < 0 || d.peer >= p || d.p2p_slot < 16 || local.size() != 1) return HCCL_E_PARA;
                p2p_rank(P, d, local[0], d.coll == COLL_SEND);
                break;
            default: ok = false;
        }
    }
    if (!ok) return HCCL_E_NOT_SUPPORT;
    plan->steps.clear();
    plan->intra_rank_waits = false;
    for (int r : local) {
        // a wait that covers the executing rank itself is a dependency between that rank's own CTAs
        for (const Step &st : P.s[r])
            if (st.wait_rank != RANK_NONE && (st.flags & SF_INCLUDE_SELF)) plan->intra_rank_waits = true;
        plan->steps.push_back(std::move(P.s[r]));
    }
    plan->nchan = d.nchan;
    plan->stage_bytes = plan_stage_bytes(d);
    plan->name = std::string(coll_name(d.coll)) + "/" + algo_name(d.algo);
    return HCCL_SUCCESS;
}

}  // namespace hcclb
