"""MoE expert-parallel exchange on symmetric memory: dispatch (push rows to the expert owners) and combine (pull the
expert outputs and form the gate-weighted sum while receiving).

    ex = MoEExchange(comm, tokens, hidden, n_experts, topk)
    recv, expert_offsets, recv_rows = ex.dispatch(x, topk_idx)          # recv rows grouped by local expert
    ... run the local experts on recv[expert_offsets[e]:expert_offsets[e+1]] and write into ex.expert_out ...
    out = ex.combine(gates)                                              # [tokens, hidden]

Counts travel over the device (all-gather of the per-expert histogram); nothing synchronises with the host.  On an
all-local communicator every tensor argument is a list with one entry per virtual rank.
"""
import ctypes as C

import torch

from .. import _lib as L
from ..ops.comm import _raw_stream


class _DevPtr:
    """Exposes a raw device pointer to torch through the CUDA array interface (int16 elements)."""

    def __init__(self, ptr, nelem):
        self.__cuda_array_interface__ = {"shape": (nelem,), "typestr": "<i2", "data": (int(ptr), False), "version": 3}


def tensor_from_ptr(ptr, rows, cols, device):
    """bf16 [rows, cols] torch view of symmetric memory."""
    t = torch.as_tensor(_DevPtr(ptr, rows * cols), device=device)
    return t.view(torch.bfloat16).view(rows, cols)


class MoEExchange:
    def __init__(self, comm, tokens, hidden, n_experts, topk, capacity_factor=1.5, device="cuda"):
        assert n_experts % comm.nranks == 0 and hidden % 8 == 0
        self.comm, self.T, self.H, self.E, self.k = comm, tokens, hidden, n_experts, topk
        self.p, self.nl = comm.nranks, comm.nlocal
        self.El = n_experts // self.p
        self.cap = int(tokens * topk * capacity_factor + 127) // 128 * 128
        nbytes = self.cap * hidden * 2
        self.h_recv, recv_local = comm.mem_alloc(nbytes)
        self.h_out, out_local = comm.mem_alloc(nbytes)
        self.recv_tab, _, _ = comm.mem_query(self.h_recv)   # [local][rank]
        self.out_tab, _, _ = comm.mem_query(self.h_out)
        self.recv = [tensor_from_ptr(recv_local[l], self.cap, hidden, device) for l in range(self.nl)]
        self.expert_out = [tensor_from_ptr(out_local[l], self.cap, hidden, device) for l in range(self.nl)]
        mk = lambda n, dt=torch.int32: [torch.zeros(n, device=device, dtype=dt) for _ in range(self.nl)]
        self.hist, self.pos, self.counts = mk(n_experts), mk(tokens * topk), mk(self.p * n_experts)
        self.base, self.expert_offsets, self.recv_rows, self.overflow = mk(n_experts), mk(self.El + 1), mk(1), mk(1)
        self.dst_row = mk(tokens * topk)
        self._topk = None
        self.ranks = list(range(self.p)) if self.nl > 1 else [comm.rank]

    def _l(self, x):
        return list(x) if isinstance(x, (list, tuple)) else [x]

    def dispatch(self, x, topk_idx, variant="mesh"):
        lib, st = L.lib(), C.c_void_p(_raw_stream())
        xs, idx = self._l(x), self._l(topk_idx)
        pw = 1 if variant == "pairwise" else 0
        for l in range(self.nl):
            assert idx[l].dtype == torch.int32 and idx[l].is_contiguous() and xs[l].dtype == torch.bfloat16 and xs[l].is_contiguous()
            L.check(lib.HcclB200MoeCount(idx[l].data_ptr(), self.T * self.k, self.E, self.hist[l].data_ptr(), self.pos[l].data_ptr(), st), "HcclB200MoeCount")
        # device-side count exchange: all-gather of the histograms
        self.comm.all_gather(self.hist if self.nl > 1 else self.hist[0], self.counts if self.nl > 1 else self.counts[0])
        for l in range(self.nl):
            L.check(lib.HcclB200MoeOffsets(self.counts[l].data_ptr(), self.p, self.E, self.ranks[l], self.base[l].data_ptr(),
                                           self.expert_offsets[l].data_ptr(), self.recv_rows[l].data_ptr(), self.cap,
                                           self.overflow[l].data_ptr(), st), "HcclB200MoeOffsets")
        self.comm.barrier()  # every rank is done with the previous round's buffers
        for l in range(self.nl):
            peers = (C.c_void_p * self.p)(*self.recv_tab[l])
            L.check(lib.HcclB200MoeDispatch(xs[l].data_ptr(), idx[l].data_ptr(), self.pos[l].data_ptr(), self.base[l].data_ptr(), self.T, self.k,
                                            self.H, self.E, self.p, self.ranks[l], pw, peers, self.dst_row[l].data_ptr(), self.cap, st),
                    "HcclB200MoeDispatch")
        self.comm.barrier()  # all rows have landed everywhere
        self._topk = idx
        one = self.nl == 1
        return (self.recv[0] if one else self.recv, self.expert_offsets[0] if one else self.expert_offsets,
                self.recv_rows[0] if one else self.recv_rows)

    def combine(self, gates, variant="mesh", source="expert_out", out=None):
        """gates: fp32 [tokens, topk].  source: 'expert_out' (after the experts ran) or 'recv' (identity experts)."""
        lib, st = L.lib(), C.c_void_p(_raw_stream())
        gs = self._l(gates)
        tab = self.out_tab if source == "expert_out" else self.recv_tab
        outs = self._l(out) if out is not None else [torch.empty(self.T, self.H, device=gs[0].device, dtype=torch.bfloat16) for _ in range(self.nl)]
        pw = 1 if variant == "pairwise" else 0
        self.comm.barrier()  # the expert outputs of every rank are complete
        for l in range(self.nl):
            assert gs[l].dtype == torch.float32 and gs[l].is_contiguous()
            peers = (C.c_void_p * self.p)(*tab[l])
            L.check(lib.HcclB200MoeCombine(peers, self._topk[l].data_ptr(), gs[l].data_ptr(), self.dst_row[l].data_ptr(), self.T, self.k, self.H,
                                           self.E, self.p, self.ranks[l], pw, outs[l].data_ptr(), self.cap, st), "HcclB200MoeCombine")
        return outs[0] if self.nl == 1 else outs

    def close(self):
        self.recv = self.expert_out = None
        self.comm.mem_free(self.h_recv)
        self.comm.mem_free(self.h_out)


def route(tokens, n_experts, topk, seed, rank, device="cuda"):
    """Synthetic router of the benchmark config: N(0,1) logits, softmax, top-k; returns (int32 experts, fp32 gates)."""
    g = torch.Generator(device=device).manual_seed(seed * 1000 + rank)
    logits = torch.randn(tokens, n_experts, device=device, generator=g)
    probs = torch.softmax(logits, dim=-1)
    gates, idx = torch.topk(probs, topk, dim=-1)
    gates = gates / gates.sum(dim=-1, keepdim=True)
    return idx.to(torch.int32).contiguous(), gates.to(torch.float32).contiguous()


def bench(comm, world, rank, dist, max_over_ranks, sync, tokens=8192, hidden=7168, n_experts=256, topk=8, iters=5):
    """Dispatch + combine (identity experts) of the benchmark config, both variants, next to NCCL all-to-all."""
    if n_experts % world:
        return {"skipped": "experts do not divide over ranks"}
    out = {"config": {"tokens_per_rank": tokens, "hidden": hidden, "experts": n_experts, "topk": topk, "dtype": "bf16", "seed": 7}}
    g = torch.Generator(device="cuda").manual_seed(70 + rank)
    x = torch.randn(tokens, hidden, device="cuda", generator=g).to(torch.bfloat16)
    idx, gates = route(tokens, n_experts, topk, 7, rank)
    ex = MoEExchange(comm, tokens, hidden, n_experts, topk)
    res = torch.empty(tokens, hidden, device="cuda", dtype=torch.bfloat16)

    def timed(fn):
        for _ in range(2):
            fn()
        sync()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / iters
        sync()
        return max_over_ranks(ms)

    for variant in ("mesh", "pairwise"):
        def ours():
            ex.dispatch(x, idx, variant=variant)
            ex.combine(gates, variant=variant, source="recv", out=res)
        out[variant + "_ms"] = round(timed(ours), 4)
    assert comm.sync() == 0, comm.describe_status()
    assert int(ex.overflow[0].item()) == 0, "receive buffer overflow"
    # identity experts: combine returns sum_k gate * x = x (gates are normalised)
    err = float((res.float() - x.float()).abs().max())
    out["check_max_abs_err"] = round(err, 4)
    send_rows = tokens * topk
    out["bytes_per_rank_each_way"] = send_rows * hidden * 2
    # what crosses the links: a rank keeps 1/world of its rows; dispatch and combine each move the rest once per direction
    crossing = out["bytes_per_rank_each_way"] * (world - 1) / max(1, world)
    best = min(out["mesh_ms"], out["pairwise_ms"])
    out["link_GBps_per_direction"] = round(2 * crossing / best / 1e6, 1)
    out["fraction_of_900GBps"] = round(2 * crossing / best / 1e6 / 900.0, 3)
    # ---- baseline: NCCL all_to_all_single with the split lists, buffers and permutations prepared once outside the timed
    # loop (no host synchronisation and no allocation per step), combine as one gather and one batched product
    if dist is not None:
        El = n_experts // world
        flat = idx.flatten().long()
        order = torch.argsort(flat, stable=True)
        inv = torch.argsort(order)
        tok_of = order // topk
        send_counts = torch.bincount(flat // El, minlength=world)
        rc = torch.empty_like(send_counts)
        dist.all_to_all_single(rc, send_counts)
        s_l, r_l = send_counts.tolist(), rc.tolist()
        sbuf = torch.empty(send_rows, hidden, device="cuda", dtype=torch.bfloat16)
        rbuf = torch.empty(sum(r_l), hidden, device="cuda", dtype=torch.bfloat16)
        back = torch.empty_like(sbuf)
        perm = torch.empty_like(sbuf)
        gates_b = gates.to(torch.bfloat16).unsqueeze(1).contiguous()      # [tokens, 1, topk]
        res3 = res.view(tokens, 1, hidden)

        def base():
            torch.index_select(x, 0, tok_of, out=sbuf)                    # rows in destination order
            dist.all_to_all_single(rbuf, sbuf, r_l, s_l)                  # dispatch
            dist.all_to_all_single(back, rbuf, s_l, r_l)                  # combine transport (identity experts)
            torch.index_select(back, 0, inv, out=perm)                    # back to (token, k) order
            torch.bmm(gates_b, perm.view(tokens, topk, hidden), out=res3)  # gate-weighted sum over k
        out["nccl_a2a_ms"] = round(timed(base), 4)
        out["nccl_check_max_abs_err"] = round(float((res.float() - x.float()).abs().max()), 4)
        out["speedup_vs_nccl"] = round(out["nccl_a2a_ms"] / best, 3)
        # ---- the same schedule with this library's HcclAlltoAllV (parametric kernel: counts are launch arguments) as transport
        sc = [c * hidden for c in s_l]
        rcv = [c * hidden for c in r_l]
        sd = [sum(sc[:i]) for i in range(world)]
        rd = [sum(rcv[:i]) for i in range(world)]
        sflat, rflat, bflat = sbuf.view(-1), rbuf.view(-1), back.view(-1)

        def through_api():
            torch.index_select(x, 0, tok_of, out=sbuf)
            comm.all_to_all_v(sflat, sc, sd, rflat, rcv, rd)              # dispatch
            comm.all_to_all_v(rflat, rcv, rd, bflat, sc, sd)              # combine transport (identity experts)
            torch.index_select(back, 0, inv, out=perm)
            torch.bmm(gates_b, perm.view(tokens, topk, hidden), out=res3)
        res.zero_()
        out["alltoallv_api_ms"] = round(timed(through_api), 4)
        assert comm.sync() == 0, comm.describe_status()
        out["alltoallv_api_check_max_abs_err"] = round(float((res.float() - x.float()).abs().max()), 4)
        out["alltoallv_api_speedup_vs_nccl"] = round(out["nccl_a2a_ms"] / out["alltoallv_api_ms"], 3)
    ex.close()
    return out
