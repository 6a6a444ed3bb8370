"""Communicator object: thin Python face of the C API.

Buffers may be numpy arrays (host-memory transport) or CUDA torch tensors (device transport).  On an all-local
communicator (`init_local`) every collective takes a list with one buffer per rank.
"""
import ctypes as C
import json

import numpy as np

from .. import _lib as L
from ..utils.dtypes import data_ptr, hccl_dtype, numel


def _u64(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.uint64))


class Communicator:
    def __init__(self, handle, device):
        self._h = C.c_void_p(handle)
        self.device = bool(device)
        lib = L.lib()
        n, r, nl = C.c_uint32(), C.c_uint32(), C.c_uint32()
        L.check(lib.HcclGetRankSize(self._h, C.byref(n)), "HcclGetRankSize")
        L.check(lib.HcclGetRankId(self._h, C.byref(r)), "HcclGetRankId")
        L.check(lib.HcclB200GetLocalRankNum(self._h, C.byref(nl)), "HcclB200GetLocalRankNum")
        self.nranks, self.rank, self.nlocal = n.value, r.value, nl.value
        self._keep = []

    # ------------------------------------------------------------------ creation
    @staticmethod
    def get_root_info():
        info = L.RootInfo()
        L.check(L.lib().HcclGetRootInfo(C.byref(info)), "HcclGetRootInfo")
        return C.string_at(C.addressof(info), L.HCCL_ROOT_INFO_BYTES)

    @classmethod
    def init_root(cls, nranks, root_info, rank, config=None, device=None):
        info = L.RootInfo()
        C.memmove(C.addressof(info), root_info, L.HCCL_ROOT_INFO_BYTES)
        h = C.c_void_p()
        lib = L.lib()
        if config is None:
            L.check(lib.HcclCommInitRootInfo(nranks, C.byref(info), rank, C.byref(h)), "HcclCommInitRootInfo")
        else:
            L.check(lib.HcclCommInitRootInfoConfig(nranks, C.byref(info), rank, C.byref(config), C.byref(h)),
                    "HcclCommInitRootInfoConfig")
        if device is None:
            import os
            device = _have_gpu() and os.environ.get("HCCL_TRANSPORT", "") != "host"
        return cls(h.value, device)

    @classmethod
    def init_cluster_info(cls, path, rank, config=None, device=None):
        h = C.c_void_p()
        lib = L.lib()
        if config is None:
            L.check(lib.HcclCommInitClusterInfo(path.encode(), rank, C.byref(h)), "HcclCommInitClusterInfo")
        else:
            L.check(lib.HcclCommInitClusterInfoConfig(path.encode(), rank, C.byref(config), C.byref(h)),
                    "HcclCommInitClusterInfoConfig")
        if device is None:
            import os
            device = _have_gpu() and os.environ.get("HCCL_TRANSPORT", "") != "host"
        return cls(h.value, device)

    @classmethod
    def init_local(cls, nranks, device=False, device_id=0, config=None):
        h = C.c_void_p()
        cfg = C.byref(config) if config is not None else None
        L.check(L.lib().HcclB200CommInitLocal(nranks, 1 if device else 0, device_id, cfg, C.byref(h)), "HcclB200CommInitLocal")
        return cls(h.value, device)

    def create_sub(self, rank_ids, sub_id, sub_rank, config=None):
        ids = (C.c_uint32 * len(rank_ids))(*rank_ids)
        sub = C.c_void_p()
        parent = C.c_void_p(self._h.value)
        cfg = C.byref(config) if config is not None else None
        L.check(L.lib().HcclCreateSubCommConfig(C.byref(parent), len(rank_ids), ids, sub_id,
                                                0xFFFFFFFF if sub_rank is None else sub_rank, cfg, C.byref(sub)),
                "HcclCreateSubCommConfig")
        return Communicator(sub.value, self.device) if sub.value else None

    @classmethod
    def from_handle(cls, handle, device=None, owned=True):
        """Wrap an HcclComm made elsewhere (for instance by the group-name front end).  With owned=False destroy() only
        forgets the handle."""
        if device is None:
            import os
            device = _have_gpu() and os.environ.get("HCCL_TRANSPORT", "") != "host"
        c = cls(handle, device)
        c._owned = owned
        return c

    def destroy(self):
        if not getattr(self, "_owned", True):
            self._h = C.c_void_p()
            return L.SUCCESS
        if self._h and self._h.value:
            code = L.lib().HcclCommDestroy(self._h)
            if code == L.SUCCESS:
                self._h = C.c_void_p()
            return code
        return L.SUCCESS

    # ------------------------------------------------------------------ helpers
    def _stream(self, stream):
        if not self.device:
            return None
        if stream is not None:
            return C.c_void_p(stream if isinstance(stream, int) else stream.cuda_stream)
        return C.c_void_p(_raw_stream())

    def _bufs(self, x):
        """one pointer per local rank"""
        if self.nlocal == 1 and not isinstance(x, (list, tuple)):
            x = [x]
        assert len(x) == self.nlocal, "need one buffer per local rank"
        arr = (C.c_void_p * self.nlocal)(*[data_ptr(b) for b in x])
        return arr, x

    def collective(self, coll, send, recv, count, dtype, op=L.SUM, root=0, algo=L.ALGO_AUTO, nchan=0, counts=None,
                   displs=None, rows=None, stream=None):
        o = L.B200Op()
        o.coll, o.algo, o.nchan, o.dataType, o.op, o.root, o.count = coll, algo, nchan, dtype, op, root, int(count)
        keep = []
        if counts is not None:
            c, d = _u64(counts), _u64(displs)
            keep += [c, d]
            o.counts, o.displs = c.ctypes.data, d.ctypes.data
        if rows is not None:
            sc, sd, rc, rd = [_u64(r) for r in rows]
            keep += [sc, sd, rc, rd]
            o.sendCounts, o.sdispls, o.recvCounts, o.rdispls = sc.ctypes.data, sd.ctypes.data, rc.ctypes.data, rd.ctypes.data
        if coll == L.BARRIER:
            sa = ra = None
        else:
            sa, _ = self._bufs(send)
            ra, _ = self._bufs(recv)
        code = L.lib().HcclB200Collective(self._h, C.byref(o), sa, ra, self._stream(stream))
        L.check(code, "HcclB200Collective(%d)" % coll)

    def repeat(self, coll, send, recv, count, dtype, iters, stride_bytes=0, nwin=1, op=L.SUM, root=0, algo=L.ALGO_AUTO, nchan=0,
               stream=None):
        """hccl_test-style loop issued from C (no per-call Python cost): `iters` calls, buffers shifted per call."""
        o = L.B200Op()
        o.coll, o.algo, o.nchan, o.dataType, o.op, o.root, o.count = coll, algo, nchan, dtype, op, root, int(count)
        sa, _ = self._bufs(send)
        ra, _ = self._bufs(recv)
        L.check(L.lib().HcclB200Repeat(self._h, C.byref(o), sa, ra, iters, stride_bytes, nwin, self._stream(stream)), "HcclB200Repeat")

    def nccl_allreduce_repeat(self, send, recv, count, dtype, iters, stride_bytes=0, nwin=1, op=L.SUM, stream=None):
        """The NCCL baseline issued the same way (needs the NCCL p2p backend, i.e. a multi-GPU communicator)."""
        return L.lib().HcclB200NcclAllReduceRepeat(self._h, data_ptr(send), data_ptr(recv), int(count), dtype, op, iters, stride_bytes,
                                                   nwin, self._stream(stream))

    # ------------------------------------------------------------------ collectives (HCCL semantics)
    def _first(self, x):
        return x[0] if isinstance(x, (list, tuple)) else x

    def all_reduce(self, send, recv, op=L.SUM, algo=L.ALGO_AUTO, nchan=0, stream=None):
        f = self._first(send)
        self.collective(L.ALLREDUCE, send, recv, numel(f), hccl_dtype(f), op=op, algo=algo, nchan=nchan, stream=stream)

    def broadcast(self, buf, root, algo=L.ALGO_AUTO, nchan=0, stream=None):
        f = self._first(buf)
        self.collective(L.BROADCAST, buf, buf, numel(f), hccl_dtype(f), root=root, algo=algo, nchan=nchan, stream=stream)

    def reduce_scatter(self, send, recv, op=L.SUM, algo=L.ALGO_AUTO, nchan=0, stream=None):
        f = self._first(recv)
        self.collective(L.REDUCE_SCATTER, send, recv, numel(f), hccl_dtype(f), op=op, algo=algo, nchan=nchan, stream=stream)

    def reduce_scatter_v(self, send, recv, counts, displs, op=L.SUM, algo=L.ALGO_AUTO, nchan=0, stream=None):
        f = self._first(send)
        self.collective(L.REDUCE_SCATTER_V, send, recv, 0, hccl_dtype(f), op=op, algo=algo, nchan=nchan, counts=counts,
                        displs=displs, stream=stream)

    def all_gather(self, send, recv, algo=L.ALGO_AUTO, nchan=0, stream=None):
        f = self._first(send)
        self.collective(L.ALLGATHER, send, recv, numel(f), hccl_dtype(f), algo=algo, nchan=nchan, stream=stream)

    def all_gather_v(self, send, recv, counts, displs, algo=L.ALGO_AUTO, nchan=0, stream=None):
        f = self._first(recv)
        self.collective(L.ALLGATHER_V, send, recv, 0, hccl_dtype(f), algo=algo, nchan=nchan, counts=counts, displs=displs,
                        stream=stream)

    def reduce(self, send, recv, root, op=L.SUM, algo=L.ALGO_AUTO, nchan=0, stream=None):
        f = self._first(send)
        self.collective(L.REDUCE, send, recv, numel(f), hccl_dtype(f), op=op, root=root, algo=algo, nchan=nchan, stream=stream)

    def scatter(self, send, recv, root, algo=L.ALGO_AUTO, nchan=0, stream=None):
        f = self._first(recv)
        self.collective(L.SCATTER, send, recv, numel(f), hccl_dtype(f), root=root, algo=algo, nchan=nchan, stream=stream)

    def gather(self, send, recv, root, algo=L.ALGO_AUTO, nchan=0, stream=None):
        f = self._first(send)
        self.collective(L.GATHER, send, recv, numel(f), hccl_dtype(f), root=root, algo=algo, nchan=nchan, stream=stream)

    def all_to_all(self, send, recv, algo=L.ALGO_AUTO, nchan=0, stream=None):
        f = self._first(send)
        self.collective(L.ALLTOALL, send, recv, numel(f) // self.nranks, hccl_dtype(f), algo=algo, nchan=nchan, stream=stream)

    def all_to_all_v(self, send, send_counts, sdispls, recv, recv_counts, rdispls, algo=L.ALGO_AUTO, nchan=0, stream=None):
        f = self._first(send)
        self.collective(L.ALLTOALLV, send, recv, 0, hccl_dtype(f), algo=algo, nchan=nchan,
                        rows=(send_counts, sdispls, recv_counts, rdispls), stream=stream)

    def barrier(self, stream=None):
        self.collective(L.BARRIER, None, None, 0, L.FP32, stream=stream)

    # plain C API entry points (one local rank), used to exercise the HCCL signatures themselves
    def send(self, buf, dest, stream=None):
        L.check(L.lib().HcclSend(data_ptr(buf), numel(buf), hccl_dtype(buf), dest, self._h, self._stream(stream)), "HcclSend")

    def recv(self, buf, src, stream=None):
        L.check(L.lib().HcclRecv(data_ptr(buf), numel(buf), hccl_dtype(buf), src, self._h, self._stream(stream)), "HcclRecv")

    def batch_send_recv(self, items, stream=None):
        """items: list of ('send'|'recv', buffer, remote_rank)"""
        arr = (L.SendRecvItem * len(items))()
        for i, (kind, buf, peer) in enumerate(items):
            arr[i].sendRecvType = 0 if kind == "send" else 1
            arr[i].buf = data_ptr(buf)
            arr[i].count = numel(buf)
            arr[i].dataType = hccl_dtype(buf)
            arr[i].remoteRank = peer
        L.check(L.lib().HcclBatchSendRecv(arr, len(items), self._h, self._stream(stream)), "HcclBatchSendRecv")

    def local_send_recv(self, src, dst, sbuf, rbuf, stream=None):
        L.check(L.lib().HcclB200LocalSendRecv(self._h, src, dst, data_ptr(sbuf), data_ptr(rbuf), numel(sbuf),
                                              hccl_dtype(sbuf), self._stream(stream)), "HcclB200LocalSendRecv")

    # ------------------------------------------------------------------ status / observability
    def sync(self, stream=None):
        return L.lib().HcclB200StreamSync(self._h, self._stream(stream))

    def kernel_trace(self, local=0, max_steps=64):
        """Per-step timestamps (us since kernel start) of the newest executor launch: list of (wait_done, moved, signalled)."""
        n = 1 + 3 * 340
        buf = (C.c_uint64 * n)()
        ns = C.c_int32()
        rc = L.lib().HcclB200GetKernelTrace(self._h, local, buf, n, C.byref(ns))
        if rc != L.SUCCESS:
            return None
        t0 = buf[0]
        out = []
        for i in range(ns.value):
            w, m, s = buf[1 + 3 * i], buf[2 + 3 * i], buf[3 + 3 * i]
            if w == 0 and m == 0:
                continue
            out.append((i, (w - t0) / 1e3, (m - t0) / 1e3, (s - t0) / 1e3 if s else None))
        self.last_launch = {"gap_before_us": (t0 - buf[n - 2]) / 1e3 if buf[n - 2] else None, "kernel_us": (buf[n - 1] - t0) / 1e3}
        return out[:max_steps]

    def wait_probe(self, local=0, timeout_ms=200.0, stream=None):
        """Starve one bounded wait on purpose; returns the result code the wait ended with."""
        return L.lib().HcclB200WaitProbe(self._h, local, float(timeout_ms), self._stream(stream))

    def async_error(self):
        e = C.c_int()
        L.check(L.lib().HcclGetCommAsyncError(self._h, C.byref(e)), "HcclGetCommAsyncError")
        return e.value

    def status(self, local=0):
        s = L.B200Status()
        L.check(L.lib().HcclB200GetStatus(self._h, local, C.byref(s)), "HcclB200GetStatus")
        return s

    def describe_status(self, local=0):
        buf = C.create_string_buffer(1024)
        L.check(L.lib().HcclB200DescribeStatus(self._h, local, buf, 1024), "HcclB200DescribeStatus")
        return buf.value.decode()

    def suspend(self):
        L.check(L.lib().HcclCommSuspend(self._h), "HcclCommSuspend")

    def resume(self):
        L.check(L.lib().HcclCommResume(self._h), "HcclCommResume")

    def select(self, coll, count, dtype, op=L.SUM):
        a, n, t = C.c_int32(), C.c_int32(), C.c_double()
        L.check(L.lib().HcclB200Select(self._h, coll, int(count), dtype, op, C.byref(a), C.byref(n), C.byref(t)), "HcclB200Select")
        return L.ALGO_NAMES[a.value], n.value, t.value

    def stats(self):
        buf = C.create_string_buffer(1 << 16)
        L.check(L.lib().HcclB200GetStatsJson(self._h, buf, 1 << 16), "HcclB200GetStatsJson")
        return json.loads(buf.value.decode())

    def trace(self):
        buf = C.create_string_buffer(1 << 22)
        L.check(L.lib().HcclB200GetTraceJson(self._h, buf, 1 << 22), "HcclB200GetTraceJson")
        return json.loads(buf.value.decode())

    def calibrate(self, stream=None):
        L.check(L.lib().HcclB200Calibrate(self._h, self._stream(stream)), "HcclB200Calibrate")

    def set_cost_model(self, alpha_us=0, beta_gbps=0, nvls_gbps=0, gamma_gbps=0, launch_us=0):
        L.check(L.lib().HcclB200SetCostModel(self._h, alpha_us, beta_gbps, nvls_gbps, gamma_gbps, launch_us), "HcclB200SetCostModel")

    def has_nvls(self):
        v = C.c_int32()
        L.check(L.lib().HcclB200HasNvls(self._h, C.byref(v)), "HcclB200HasNvls")
        return bool(v.value)

    def name(self):
        buf = C.create_string_buffer(L.COMM_NAME_MAX_LENGTH)
        L.check(L.lib().HcclGetCommName(self._h, buf), "HcclGetCommName")
        return buf.value.decode()

    def exchange(self, tag, payload):
        """All-gather a small bytes object over the control plane; returns the list of all ranks' payloads."""
        n = len(payload)
        out = C.create_string_buffer(n * self.nranks)
        L.check(L.lib().HcclB200Exchange(self._h, tag.encode(), payload, n, out), "HcclB200Exchange")
        return [out.raw[i * n:(i + 1) * n] for i in range(self.nranks if self.nlocal == 1 else 1)]

    # ------------------------------------------------------------------ symmetric memory
    def mem_alloc(self, nbytes):
        """Returns (handle, [local pointers])."""
        ptrs = (C.c_void_p * self.nlocal)()
        h = C.c_int32()
        L.check(L.lib().HcclB200MemAlloc(self._h, nbytes, ptrs, C.byref(h)), "HcclB200MemAlloc")
        return h.value, [ptrs[i] for i in range(self.nlocal)]

    def symmetric_empty(self, numel, dtype):
        """Buffer(s) of `numel` elements in registered symmetric memory (zero-copy collectives, fused kernels).
        Device transport: torch tensor(s) of torch dtype `dtype`; host transport: numpy array(s).  Returns (handle, buffers),
        one buffer per local rank; free with mem_free(handle) after dropping the buffers."""
        import numpy as np
        if self.device:
            import torch
            itemsize = torch.empty(0, dtype=dtype).element_size()
        else:
            itemsize = np.dtype(dtype).itemsize
        nbytes = (numel * itemsize + 255) // 256 * 256
        handle, ptrs = self.mem_alloc(nbytes)
        bufs = []
        for ptr in ptrs:
            if self.device:
                import torch

                class _P:
                    pass
                o = _P()
                o.__cuda_array_interface__ = {"shape": (numel * itemsize,), "typestr": "|u1", "data": (int(ptr), False), "version": 3}
                bufs.append(torch.as_tensor(o, device="cuda").view(dtype))
            else:
                raw = (C.c_uint8 * (numel * itemsize)).from_address(ptr)
                bufs.append(np.frombuffer(raw, dtype=dtype, count=numel))
        return handle, bufs

    def symmetric_pool(self):
        """A torch.cuda.MemPool whose blocks are registered symmetric memory of this communicator.  Tensors created under
        `with torch.cuda.use_mem_pool(pool):` are ordinary torch tensors, and collectives on them take the zero-copy paths
        (peers read and write them in place, no staging copy) without further calls.  Every rank has to create its tensors
        in the same order and with the same sizes inside the pool (allocation is collective).  One pool per process; call
        release_symmetric_pool() on every rank (or destroy the communicator) to give the memory back."""
        import torch
        L.check(L.lib().HcclB200PoolBind(self._h), "HcclB200PoolBind")
        if getattr(self, "_pool", None) is None:
            alloc = torch.cuda.memory.CUDAPluggableAllocator(L.LIB_PATH, "hcclb200_torch_malloc", "hcclb200_torch_free")
            self._pool_alloc = alloc
            self._pool = torch.cuda.MemPool(alloc.allocator())
        return self._pool

    def release_symmetric_pool(self):
        """Collective: drops the pool (its tensors must be gone) and releases its symmetric memory on every rank."""
        self._pool = None
        self._pool_alloc = None
        L.check(L.lib().HcclB200PoolBind(None), "HcclB200PoolBind")

    def mem_adopt(self, bufs, drv_handles=None):
        """Register caller-owned buffers (one per local rank; numpy arrays or torch tensors of equal byte size) as a symmetric
        allocation.  drv_handles: driver allocation handles behind the buffers (one rank per GPU).  Returns the handle for
        mem_free(), which leaves the memory alone."""
        bufs = list(bufs) if isinstance(bufs, (list, tuple)) else [bufs]
        assert len(bufs) == self.nlocal
        ptrs = (C.c_void_p * self.nlocal)(*[b.data_ptr() if hasattr(b, "data_ptr") else b.ctypes.data for b in bufs])
        b0 = bufs[0]
        nbytes = b0.numel() * b0.element_size() if hasattr(b0, "data_ptr") else b0.nbytes
        dh = None
        if drv_handles is not None:
            dh = (C.c_uint64 * self.nlocal)(*[int(h) for h in drv_handles])
        h = C.c_int32()
        L.check(L.lib().HcclB200MemAdopt(self._h, ptrs, nbytes, dh, 0, C.byref(h)), "HcclB200MemAdopt")
        self._keep.append(bufs)
        return h.value

    def mem_query(self, handle):
        """Returns (peer pointer table [local][rank], multicast pointers [local], bytes)."""
        peers = (C.c_void_p * (self.nlocal * self.nranks))()
        mcs = (C.c_void_p * self.nlocal)()
        nb = C.c_size_t()
        L.check(L.lib().HcclB200MemQuery(self._h, handle, peers, mcs, C.byref(nb)), "HcclB200MemQuery")
        table = [[peers[l * self.nranks + q] for q in range(self.nranks)] for l in range(self.nlocal)]
        return table, [mcs[i] for i in range(self.nlocal)], nb.value

    def mem_free(self, handle):
        L.check(L.lib().HcclB200MemFree(self._h, handle), "HcclB200MemFree")

    def put(self, handle, peer, offset, src_ptr, nbytes, local=0, stream=None):
        """One-sided: copy nbytes from src_ptr into rank `peer`'s copy of allocation `handle` at byte `offset`."""
        L.check(L.lib().HcclB200Put(self._h, local, handle, peer, offset, src_ptr, nbytes, self._stream(stream)), "HcclB200Put")

    def get(self, handle, peer, offset, dst_ptr, nbytes, local=0, stream=None):
        """One-sided: copy nbytes at byte `offset` of rank `peer`'s copy of allocation `handle` to dst_ptr."""
        L.check(L.lib().HcclB200Get(self._h, local, handle, peer, offset, dst_ptr, nbytes, self._stream(stream)), "HcclB200Get")

    def topology(self):
        """Ranks, transport, NVLS and peer-access matrix as a dict."""
        buf = C.create_string_buffer(1 << 16)
        L.check(L.lib().HcclB200GetTopoJson(self._h, buf, 1 << 16), "HcclB200GetTopoJson")
        return json.loads(buf.value.decode())

    def topo_desc(self):
        """HcclGetTopoDesc: [(algSets, rankSize)] per level."""
        d = (L.TopoDescs * L.TOPO_MAX)()
        L.check(L.lib().HcclGetTopoDesc(self._h, d, L.TOPO_MAX), "HcclGetTopoDesc")
        return [(int(x.algSets), int(x.rankSize)) for x in d]

    def overflow_count(self):
        v = C.c_uint64()
        L.check(L.lib().HcclB200GetOverflowCount(self._h, C.byref(v)), "HcclB200GetOverflowCount")
        return v.value

    def device_context(self):
        p, s = C.c_void_p(), C.c_uint64()
        L.check(L.lib().HcclB200GetDeviceContext(self._h, C.byref(p), C.byref(s)), "HcclB200GetDeviceContext")
        return p.value, s.value

    @property
    def handle(self):
        return self._h


_RAW = None


def _raw_stream():
    """Raw handle of torch's current CUDA stream (the cheap private accessor when it exists)."""
    global _RAW
    import torch
    if _RAW is None:
        _RAW = getattr(torch._C, "_cuda_getCurrentRawStream", False)
    if _RAW:
        return _RAW(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _have_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False
