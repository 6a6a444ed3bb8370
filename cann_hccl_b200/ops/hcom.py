"""Group-name front end (hccl/hcom.h): communicators addressed by a group string, and the gradient-fusion settings.

    hcom.init_by_comm(world)                 adopt an existing Communicator as "hccl_world_group"
    hcom.create_group("tp0", [0, 1])         collective over the listed world ranks
    comm = hcom.group_comm("tp0")            Communicator view of the group (None on non-members)
    hcom.set_grad_fusion_by_size(None, [30, 70])
"""
import ctypes as C

from .. import _lib as L
from .comm import Communicator

WORLD = "hccl_world_group"
_views = {}


def _g(group):
    return None if group is None else group.encode()


def init_by_comm(comm):
    L.check(L.lib().HcomInitByComm(comm.handle), "HcomInitByComm")
    _views[WORLD] = comm


def init_by_file(ranktable_path, rank):
    L.check(L.lib().HcomInitByFile(ranktable_path.encode(), str(rank).encode()), "HcomInitByFile")


def destroy():
    _views.clear()
    L.check(L.lib().HcomDestroy(), "HcomDestroy")


def create_group(group, world_ranks):
    arr = (C.c_uint32 * len(world_ranks))(*world_ranks)
    L.check(L.lib().HcomCreateGroup(group.encode(), len(world_ranks), arr), "HcomCreateGroup")


def destroy_group(group):
    _views.pop(group, None)
    L.check(L.lib().HcomDestroyGroup(group.encode()), "HcomDestroyGroup")


def rank_size(group=None):
    v = C.c_uint32()
    L.check(L.lib().HcomGetRankSize(_g(group), C.byref(v)), "HcomGetRankSize")
    return v.value


def rank_id(group=None):
    v = C.c_uint32()
    L.check(L.lib().HcomGetRankId(_g(group), C.byref(v)), "HcomGetRankId")
    return v.value


def world_rank_from_group_rank(group, group_rank):
    v = C.c_uint32()
    L.check(L.lib().HcomGetWorldRankFromGroupRank(_g(group), group_rank, C.byref(v)), "HcomGetWorldRankFromGroupRank")
    return v.value


def group_rank_from_world_rank(world_rank, group):
    v = C.c_uint32()
    L.check(L.lib().HcomGetGroupRankFromWorldRank(world_rank, _g(group), C.byref(v)), "HcomGetGroupRankFromWorldRank")
    return v.value


def group_comm(group=None):
    """Communicator object over the group's handle (not owning: destroy the group through this module)."""
    name = group or WORLD
    if name in _views:
        return _views[name]
    h = C.c_void_p()
    rc = L.lib().HcomGetCommHandleByGroup(_g(group), C.byref(h))
    if rc == L.E_NOT_FOUND:
        return None
    L.check(rc, "HcomGetCommHandleByGroup")
    world = _views.get(WORLD)
    view = Communicator.from_handle(h.value, device=world.device if world is not None else None, owned=False)
    _views[name] = view
    return view


def set_grad_fusion_by_index(group, last_indices):
    arr = (C.c_uint32 * len(last_indices))(*last_indices)
    L.check(L.lib().HcomSetGradFusionByIndex(_g(group), len(last_indices), arr), "HcomSetGradFusionByIndex")


def set_grad_fusion_by_size(group, percentages):
    arr = (C.c_float * len(percentages))(*percentages)
    L.check(L.lib().HcomSetGradFusionBySize(_g(group), len(percentages), arr), "HcomSetGradFusionBySize")


def grad_fusion_by_index(group=None, cap=1024):
    n = C.c_uint32(cap)
    arr = (C.c_uint32 * cap)()
    rc = L.lib().HcomGetGradFusionByIndex(_g(group), C.byref(n), arr)
    if rc == L.E_NOT_FOUND:
        return None
    L.check(rc, "HcomGetGradFusionByIndex")
    return [arr[i] for i in range(n.value)]


def grad_fusion_by_size(group=None, cap=1024):
    n = C.c_uint32(cap)
    arr = (C.c_float * cap)()
    rc = L.lib().HcomGetGradFusionBySize(_g(group), C.byref(n), arr)
    if rc == L.E_NOT_FOUND:
        return None
    L.check(rc, "HcomGetGradFusionBySize")
    return [arr[i] for i in range(n.value)]
