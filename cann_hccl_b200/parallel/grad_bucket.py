"""Data-parallel gradient synchronisation in fused segments.

The reference lets a front end cut the gradient list of a group into segments that are all-reduced as one buffer each
(HcomSetGradFusionByIndex / HcomSetGradFusionBySize, framework/hcom/hcom_common.cc:1014-1122).  This module is that
consumer: it reads the group's setting (or falls back to one segment per `bucket_mb`), packs each segment's gradients into
one flat buffer, runs one AllReduce per segment and scatters the averaged values back.

Works with numpy arrays on the host transport and with torch tensors on the device transport.
"""
from .. import _lib as L
from ..ops import hcom as _hcom


def plan_segments(sizes, group=None, bucket_mb=25.0, itemsize=4):
    """Returns the list of (first, last_exclusive) gradient-index ranges.

    Priority: by-index setting of the group (ascending indices of each segment's last gradient; a tail after the final index
    forms its own segment), then by-size setting (percentages of the total element count), then buckets of bucket_mb."""
    n = len(sizes)
    if n == 0:
        return []
    idx = _hcom.grad_fusion_by_index(group)
    if idx:
        cuts, first = [], 0
        for last in idx:
            last = min(int(last), n - 1)
            if last + 1 > first:
                cuts.append((first, last + 1))
                first = last + 1
        if first < n:
            cuts.append((first, n))
        return cuts
    shares = _hcom.grad_fusion_by_size(group)
    total = float(sum(sizes))
    cuts, first, acc = [], 0, 0.0
    if shares:
        bounds, run = [], 0.0
        for s in shares:
            run += s
            bounds.append(run / 100.0 * total)
        b = 0
        for i, sz in enumerate(sizes):
            acc += sz
            while b < len(bounds) - 1 and acc >= bounds[b] - 1e-6:
                if i + 1 > first:
                    cuts.append((first, i + 1))
                    first = i + 1
                b += 1
        if first < n:
            cuts.append((first, n))
        return cuts
    limit = bucket_mb * (1 << 20) / itemsize
    for i, sz in enumerate(sizes):
        acc += sz
        if acc >= limit:
            cuts.append((first, i + 1))
            first, acc = i + 1, 0.0
    if first < n:
        cuts.append((first, n))
    return cuts


def all_reduce_gradients(comm, grads, group=None, average=True, bucket_mb=25.0):
    """In place: every array / tensor of `grads` becomes the sum (or mean) over the ranks of `comm`.  One AllReduce per
    fused segment.  All gradients must share one dtype."""
    if not grads:
        return []
    is_torch = hasattr(grads[0], "data_ptr")
    sizes = [int(g.numel()) if is_torch else int(g.size) for g in grads]
    itemsize = grads[0].element_size() if is_torch else grads[0].dtype.itemsize
    segs = plan_segments(sizes, group=group, bucket_mb=bucket_mb, itemsize=itemsize)
    for first, last in segs:
        part = grads[first:last]
        if is_torch:
            import torch
            flat = torch.cat([g.reshape(-1) for g in part])
            comm.all_reduce(flat, flat, op=L.SUM)
            if average:
                flat /= comm.nranks
            off = 0
            for g, sz in zip(part, sizes[first:last]):
                g.copy_(flat[off:off + sz].view_as(g))
                off += sz
        else:
            import numpy as np
            flat = np.concatenate([g.reshape(-1) for g in part])
            out = np.empty_like(flat)
            comm.all_reduce(flat, out, op=L.SUM)
            if average:
                out = (out / comm.nranks).astype(flat.dtype)
            off = 0
            for g, sz in zip(part, sizes[first:last]):
                g[...] = out[off:off + sz].reshape(g.shape)
                off += sz
    return segs
