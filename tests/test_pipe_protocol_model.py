"""Happens-before model of the pipelined kernels' hand-shakes (cann_hccl_b200/csrc/kernels/pipe_coll.cuh).

The kernels run a message through a ring of K staging slots: the CTAs of a rank form up to three stages, the groups of a stage
take chunks in turn, and per (stage, source rank, slot) progress words order the stages of all ranks.  This file restates, mode
by mode, what a stage waits for, what it publishes and which memory it reads and writes for a chunk (the tables of
`pipe_coll_kernel`: the `switch (mode)` that fills ww0 / wm0 / sw0 / ... and the `role == 0 / 1 / 2` work sections), builds
the happens-before relation (chunks of one group in order; publish -> wait) and checks three things for every mode, rank
count, ring depth, group count, message length, root and in-place form:

  * every wait is satisfied by some publish, and the waits form no cycle;
  * the publishes of one progress word happen in chunk order (a word only ever grows, so a later chunk's value must not be
    overwritten by an earlier chunk's);
  * any two accesses to the same memory, one of them a write, are ordered: a slot is not refilled while a stage of any rank
    still reads the chunk before, and in place no stage overwrites input that another stage has yet to read.

It is a model of the design, kept next to the kernel by hand; the GPU tests check the code."""
import itertools

import pytest

READY, DONE, OUT = 0, 1, 2  # progress words (kPipeWordReady / Done / Out)
PUBLISHER_ROLE = {READY: 0, DONE: 1, OUT: 2}

MODES = ("AR2_MC", "AR2_PUSH", "AR1_MC", "AR1_PUSH", "RS_MC", "RS_PUSH", "AG_PULL", "BC_MC", "BC_PUSH", "RD_PUSH")


def stages(mode):
    return 3 if mode in ("AR2_MC", "AR2_PUSH", "RD_PUSH") else 2


def roles_of(mode, me, root):
    """Roles that exist on a rank."""
    if mode in ("BC_MC", "BC_PUSH"):
        return (0,) if me == root else (1,)
    if mode == "RD_PUSH":
        return (0, 1, 2) if me == root else (0, 1)
    return tuple(range(stages(mode)))


def flags(mode, role, me, p, root):
    """(waits, signals): waits = [(word, ranks, at_old)], signals = [(word, ranks)] — the kernel's wait / signal table."""
    allr, others = list(range(p)), [q for q in range(p) if q != me]
    succ, pred = (me + 1) % p, (me - 1) % p
    chain_last = succ == root
    if mode == "AR2_MC":
        return {0: ([(OUT, [me], True)], [(READY, allr)]), 1: ([(READY, allr, False)], [(DONE, allr)]), 2: ([(DONE, allr, False)], [(OUT, [me])])}[role]
    if mode == "AR2_PUSH":
        return {0: ([(DONE, allr, True)], [(READY, allr)]), 1: ([(READY, allr, False), (OUT, allr, True)], [(DONE, allr)]),
                2: ([(DONE, allr, False)], [(OUT, allr)])}[role]
    if mode == "RD_PUSH":
        return {0: ([(DONE, allr, True)], [(READY, allr)]), 1: ([(READY, allr, False), (OUT, [root], True)], [(DONE, allr)]),
                2: ([(DONE, allr, False)], [(OUT, allr)])}[role]
    if mode in ("AR1_MC", "AR1_PUSH", "RS_MC", "RS_PUSH"):
        return {0: ([(DONE, allr, True)], [(READY, allr)]), 1: ([(READY, allr, False)], [(DONE, allr)])}[role]
    if mode == "AG_PULL":
        return {0: ([(DONE, others, True)], [(READY, others)]), 1: ([(READY, others, False)], [(DONE, others)])}[role]
    if mode == "BC_MC":
        return {0: ([(DONE, others, True)], [(READY, others)]), 1: ([(READY, [root], False)], [(DONE, [root])])}[role]
    if mode == "BC_PUSH":
        if role == 0:
            return ([(DONE, [succ], True)], [(READY, [succ])])
        waits, sigs = [(READY, [pred], False)], [(DONE, [pred])]
        if not chain_last:
            waits.append((DONE, [succ], True))
            sigs.append((READY, [succ]))
        return waits, sigs
    raise ValueError(mode)


def publisher_role(mode, word, q, root):
    """Which stage of rank q publishes `word` (the broadcast chain's middle ranks publish Ready from their only stage)."""
    if mode in ("BC_MC", "BC_PUSH"):
        return 0 if q == root else 1
    return PUBLISHER_ROLE[word]


def rd_owners(p, root):
    return [root] if p == 2 else [(root + 1 + k) % p for k in range(p - 1)]


def accesses(mode, role, me, p, root, ch, slot, in_place):
    """[(region, is_write)] of one stage of one rank for one chunk.  Regions: ('u', rank, which, block, chunk, part) for the caller's
    buffers ('which' = 'in' / 'out', folded when in place; part None = the whole chunk) and ('s', rank, slot, area, part) for slots."""
    A = []
    others = [q for q in range(p) if q != me]
    succ = (me + 1) % p
    chain_last = succ == root

    def user(which, rank, block, part):
        if in_place:
            if mode in ("AR2_MC", "AR2_PUSH", "AR1_MC", "AR1_PUSH", "RD_PUSH"):
                which = "in"
            elif mode in ("RS_MC", "RS_PUSH") and which == "out":   # the receive buffer is block `rank` of the send buffer
                which, block = "in", rank
            elif mode == "AG_PULL" and which == "in":               # the send buffer is block `rank` of the receive buffer
                which, block = "out", rank
        return ("u", rank, which, block, ch, part)

    def rd(x): A.append((x, False))
    def wr(x): A.append((x, True))
    if mode == "AR2_MC":
        if role == 0: rd(user("in", me, 0, None)); wr(("s", me, slot, "A", None))
        elif role == 1:
            for q in range(p): rd(("s", q, slot, "A", me))
            for q in range(p): wr(("s", q, slot, "A", me))
        else: rd(("s", me, slot, "A", None)); wr(user("out", me, 0, None))
    elif mode == "AR2_PUSH":
        if role == 0:
            for q in others: rd(user("in", me, 0, q)); wr(("s", q, slot, "P", me))
        elif role == 1:
            rd(user("in", me, 0, me))
            for q in others: rd(("s", me, slot, "P", q))
            wr(user("out", me, 0, me))
            for q in others: wr(("s", q, slot, "R", me))
        else:
            for q in others: rd(("s", me, slot, "R", q)); wr(user("out", me, 0, q))
    elif mode == "RD_PUSH":
        owners = rd_owners(p, root)
        if role == 0:
            for o in owners:
                if o != me: rd(user("in", me, 0, o)); wr(("s", o, slot, "P", me))
        elif role == 1:
            if me in owners:
                rd(user("in", me, 0, me))
                for q in others: rd(("s", me, slot, "P", q))
                if me == root: wr(user("out", me, 0, me))
                else: wr(("s", root, slot, "R", me))
        else:
            for o in owners:
                if o != root: rd(("s", root, slot, "R", o)); wr(user("out", root, 0, o))
    elif mode == "AR1_MC":
        if role == 0: rd(user("in", me, 0, None)); wr(("s", me, slot, "A", None))
        else:
            for q in range(p): rd(("s", q, slot, "A", None))
            wr(user("out", me, 0, None))
    elif mode == "AR1_PUSH":
        if role == 0:
            rd(user("in", me, 0, None))
            for q in others: wr(("s", q, slot, "P", me))
        else:
            rd(user("in", me, 0, None))
            for q in others: rd(("s", me, slot, "P", q))
            wr(user("out", me, 0, None))
    elif mode == "RS_MC":
        if role == 0:
            for q in range(p): rd(user("in", me, q, None)); wr(("s", me, slot, "B", q))
        else:
            for q in range(p): rd(("s", q, slot, "B", me))
            wr(user("out", me, 0, None))
    elif mode == "RS_PUSH":
        if role == 0:
            for q in others: rd(user("in", me, q, None)); wr(("s", q, slot, "P", me))
        else:
            rd(user("in", me, me, None))
            for q in others: rd(("s", me, slot, "P", q))
            wr(user("out", me, 0, None))
    elif mode == "AG_PULL":
        if role == 0:
            rd(user("in", me, 0, None)); wr(("s", me, slot, "A", None))
            if not in_place: wr(user("out", me, me, None))
        else:
            for q in others: rd(("s", q, slot, "A", None)); wr(user("out", me, q, None))
    elif mode == "BC_MC":
        if role == 0:
            rd(("u", me, "buf", 0, ch, None))
            for q in range(p): wr(("s", q, slot, "A", None))
        else: rd(("s", me, slot, "A", None)); wr(("u", me, "buf", 0, ch, None))
    elif mode == "BC_PUSH":
        if role == 0: rd(("u", me, "buf", 0, ch, None)); wr(("s", succ, slot, "A", None))
        else:
            rd(("s", me, slot, "A", None)); wr(("u", me, "buf", 0, ch, None))
            if not chain_last: wr(("s", succ, slot, "A", None))
    return A


def overlap(a, b):
    return a[:-1] == b[:-1] and (a[-1] is None or b[-1] is None or a[-1] == b[-1])


def check(mode, p, K, groups, nchunks, root, in_place):
    nodes, index = [], {}
    for r in range(p):
        for role in roles_of(mode, r, root):
            for ch in range(nchunks):
                index[(r, role, ch)] = len(nodes)
                nodes.append((r, role, ch))
    N = len(nodes)
    preds = [[] for _ in range(N)]
    for (r, role, ch), n in index.items():
        G = groups[role]
        if ch - G >= 0:
            preds[n].append(index[(r, role, ch - G)])  # the same group takes chunk ch - G before chunk ch
    publishes = {}  # (word, src, dst, slot) -> [chunks]
    for (r, role, ch), n in index.items():
        waits, sigs = flags(mode, role, r, p, root)
        for word, ranks in sigs:
            for q in ranks:
                publishes.setdefault((word, r, q, ch % K), []).append(ch)
        for word, ranks, at_old in waits:
            want = (ch - K + 1 if ch >= K else 0) if at_old else ch + 1
            if want == 0:
                continue
            for q in ranks:
                src = (q, publisher_role(mode, word, q, root), want - 1)
                assert src in index, "%s: rank %d stage %d chunk %d waits for word %d of rank %d, which has no stage to publish it" % (mode, r, role, ch, word, q)
                _, sig_of_src = flags(mode, src[1], q, p, root)
                assert any(w == word and r in rk for w, rk in sig_of_src), "%s: rank %d stage %d waits for word %d from rank %d, which never sends it there" % (mode, r, role, word, q)
                preds[n].append(index[src])
    # ancestors (a cycle of waits is a deadlock)
    indeg = [len(x) for x in preds]
    succs = [[] for _ in range(N)]
    for n, ps in enumerate(preds):
        for q in ps:
            succs[q].append(n)
    anc = [0] * N
    order = [n for n in range(N) if indeg[n] == 0]
    i = 0
    while i < len(order):
        n = order[i]; i += 1
        for m in succs[n]:
            anc[m] |= anc[n] | (1 << n)
            indeg[m] -= 1
            if indeg[m] == 0:
                order.append(m)
    assert len(order) == N, "%s: the waits form a cycle" % mode
    before = lambda a, b: (anc[b] >> a) & 1
    # a progress word only grows: its publishes come in chunk order
    for (word, src, dst, slot), chunks in publishes.items():
        role = publisher_role(mode, word, src, root)
        for c0, c1 in zip(sorted(chunks), sorted(chunks)[1:]):
            assert before(index[(src, role, c0)], index[(src, role, c1)]), "%s: word %d of rank %d for rank %d, slot %d: chunk %d may be published after chunk %d" % (mode, word, src, dst, slot, c0, c1)
    # conflicting accesses are ordered
    acc = {}
    for (r, role, ch), n in index.items():
        for region, w in accesses(mode, role, r, p, root, ch, ch % K, in_place):
            acc.setdefault(region[:-1], []).append((region, w, n))
    for lst in acc.values():
        for (ra, wa, na), (rb, wb, nb) in itertools.combinations(lst, 2):
            if na == nb or not (wa or wb) or not overlap(ra, rb):
                continue
            assert before(na, nb) or before(nb, na), "%s p=%d K=%d groups=%s chunks=%d root=%d in_place=%s: %s of %s by %s and %s by %s are unordered" % (
                mode, p, K, groups, nchunks, root, in_place, "write" if wa else "read", ra, nodes[na], "write" if wb else "read", nodes[nb])


@pytest.mark.parametrize("mode", MODES)
def test_pipelined_hand_shakes_order_every_slot_reuse(mode):
    for p in (2, 3, 4):
        for K in (1, 2, 4):
            for groups in ((1, 1, 1), (2, 2, 2), (2, 4, 2), (3, 1, 2)):
                for nchunks in (1, K, 2 * K + 1, 3 * K + 2):
                    for root in ((0, p - 1) if mode in ("BC_MC", "BC_PUSH", "RD_PUSH") else (0,)):
                        for in_place in ((False, True) if mode not in ("BC_MC", "BC_PUSH") else (False,)):
                            check(mode, p, K, groups, nchunks, root, in_place)


def test_model_sees_a_missing_reuse_wait():
    """Take the slot-reuse wait out of the push stage (as if a slot were refilled without asking its readers): the model objects."""
    real = flags

    def broken(mode, role, me, p, root):
        waits, sigs = real(mode, role, me, p, root)
        return ([w for w in waits if not w[2]] if role == 0 else waits), sigs
    globals()["flags"] = broken
    try:
        with pytest.raises(AssertionError, match="unordered"):
            check("AR2_PUSH", 3, 2, (1, 1, 1), 5, 0, False)
    finally:
        globals()["flags"] = real
