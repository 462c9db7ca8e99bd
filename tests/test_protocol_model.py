"""Exhaustive check of the flag protocols of the multi-rank kernels on a small
model: every interleaving of the ranks' steps is explored, and the run fails on
a deadlock, on a staging buffer that is overwritten before its owner has read
it, and on a load that finds anything but the data of the round it expects.

One modelled rank stands for thread block b of that rank: block b of a rank
only ever talks to block b of the other ranks, so the protocol of one block
index is the whole protocol.  Flag words are monotonic epoch counters per
(owner, channel, source); a wait is enabled once every watched word has reached
its target; stores are visible at once (the kernels order them with a release
store of the flag and an acquire load on the other side).  A step of a rank is
a wait, a signal, or a group of data accesses between two of those; accesses
of different ranks that no flag orders are tried in both orders, so a missing
wait shows up as a wrong tag.

The programs restate, step for step, the waits, stores, loads and signals of

  ar_twoshot_kernel        lock-step two-shot all-reduce
  zero_reduce_kernel       reduce-scatter of the sharded optimizer step
  zero_update_kernel       verdict exchange, update, all-gather
  gather_flow_kernel       staged all-gather / broadcast: pushing and copying blocks
  ar_nvls_inplace_kernel   in place on symmetric memory, followed by the
                           caller's next write to the buffer
  ar_flow_kernel           staged ring: copy-in, reducing and copy-out blocks
  allgather_kernel         stores only: push into the peers' gather boxes
  allgather_pull_kernel    publish in the outbox, peers pull (large blocks)

(dragon_b200/csrc/dgn_kernels.cuh, dgn_zero.cuh), including the bookkeeping
that carries over from one collective to the next -- epoch, parity, last "done"
per parity -- which is what makes back-to-back collectives safe.
"""

import collections
import itertools

import pytest

A, B, C, D = range(4)


class Rank(object):
    """Builds the step list of one rank (or of one warp role of a rank: the
    roles of a block run side by side and are explored as processes of their
    own); keeps the block state the kernels keep."""

    def __init__(self, me, n, role=0):
        self.me, self.n, self.role = me, n, role
        self.peers = [p for p in range(n) if p != me]
        self.steps = []
        self.epoch, self.ops, self.last_done, self.zero_ops, self.ll_ops = 0, 0, [0, 0], 0, 0
        self.joins = 0

    def local_set(self, name, value):
        """A counter in the block's shared memory, written by one role."""
        self.steps.append(("local_set", name, value))

    def local_wait(self, name, value):
        self.steps.append(("local_wait", name, value))

    def poll(self, key, tag):
        """Flag-in-data lines: spin until this rank's buffer holds `tag`, then it is read."""
        self.steps.append(("poll", key, tag))

    def wait(self, chan, sources, value):
        self.steps.append(("wait", chan, tuple(sources), value))

    def signal(self, chan, targets, value):
        # Every epoch a collective signals lies above the epoch the block had
        # when it began; together with `end` (below) this is why a flag left by
        # an earlier collective can never satisfy a wait of a later one.
        if chan != D:
            assert value > self.epoch, "signalled epoch {} is not above the base {}".format(value, self.epoch)
            self.high = max(getattr(self, "high", 0), value)
        self.steps.append(("signal", chan, tuple(targets), value))

    def data(self, *accesses):
        """One group of accesses, each of
        ("write", owner, key, tag)  store into a staging buffer; the previous content must have been read
        ("store", owner, key, tag)  store that may overwrite (in-place results, refilled chunk buffers)
        ("read", key, tag)          load from this rank's own buffer; marks it as read
        ("peek", owner, key, tag)   load that leaves the buffer as it is (through the switch, or re-read later)"""
        if accesses:
            self.steps.append(("data", tuple(accesses)))

    # what every flag-based kernel does first and last (begin_collective / end_collective)
    def begin(self):
        base, parity = self.epoch, self.ops & 1
        self.wait(B, self.peers, self.last_done[parity])
        return base, parity

    def end(self, parity, done):
        self.signal(B, self.peers, done)
        assert self.high <= done, "an epoch above the collective's last one ({}) was signalled".format(done)
        self.epoch, self.ops = done, self.ops + 1
        self.last_done[parity] = done


def _enabled(step, r, flags, bufs):
    kind = step[0]
    if kind == "wait":
        return all(flags.get((r, step[1], s), 0) >= step[3] for s in step[2])
    if kind == "local_wait":
        return flags.get((r, "local", step[1]), 0) >= step[2]
    if kind == "poll":
        got = bufs.get((r, step[1]))
        return got is not None and got[0] == step[2] and not got[1]
    return True


def _apply(step, r, flags, bufs):
    """Returns (flags, bufs) after `step` of a process of rank r; checks the data accesses."""
    kind = step[0]
    if kind in ("wait", "local_wait"):
        return flags, bufs
    if kind == "signal":
        nflags = dict(flags)
        for t in step[2]:
            assert nflags.get((t, step[1], r), 0) <= step[3], "flag went backwards"
            nflags[(t, step[1], r)] = step[3]
        return nflags, bufs
    if kind == "local_set":
        nflags = dict(flags)
        nflags[(r, "local", step[1])] = step[2]
        return nflags, bufs
    nbufs = dict(bufs)
    if kind == "poll":
        nbufs[(r, step[1])] = (step[2], True)
        return flags, nbufs
    for acc in step[1]:
        if acc[0] in ("write", "store"):
            _, owner, key, tag = acc
            old = nbufs.get((owner, key))
            assert acc[0] == "store" or old is None or old[1], \
                "rank {} overwrites {} of rank {} before it was read: {} -> {}".format(r, key, owner, old, tag)
            # What a plain "store" leaves is guarded by the tag checks of its
            # readers, not by the overwrite check.
            nbufs[(owner, key)] = (tag, acc[0] == "store")
        else:
            owner, key, tag = (r, acc[1], acc[2]) if acc[0] == "read" else acc[1:]
            got = nbufs.get((owner, key))
            assert got is not None and got[0] == tag, \
                "rank {} loads {} of rank {} and finds {} instead of {}".format(r, key, owner, got, tag)
            if acc[0] == "read":
                nbufs[(owner, key)] = (tag, True)
    return flags, nbufs


def explore(procs, limit=2000000):
    """All interleavings of the processes' data accesses; returns the number of
    states seen.  Waits, signals and local counters are taken as soon as they
    are enabled: flags only grow, so an enabled wait stays enabled and a signal
    or counter update can only enable others -- delaying one of them is the
    same as delaying whoever waits for it, which the search does anyway.  Only
    data accesses and polls, whose order across processes matters, branch."""
    n = len(procs)
    progs = [p.steps for p in procs]
    rank_of = [p.me for p in procs]
    start = (tuple(0 for _ in range(n)), frozenset(), frozenset())
    seen = {start}
    stack = [start]
    while stack:
        pcs, flag_items, buf_items = stack.pop()
        flags, bufs = dict(flag_items), dict(buf_items)
        # run every enabled step that is not a data access, to a fixed point
        progress = True
        pcs = list(pcs)
        while progress:
            progress = False
            for q in range(n):
                while pcs[q] < len(progs[q]):
                    step = progs[q][pcs[q]]
                    if step[0] in ("data", "poll") or not _enabled(step, rank_of[q], flags, bufs):
                        break
                    flags, bufs = _apply(step, rank_of[q], flags, bufs)
                    pcs[q] += 1
                    progress = True
        pcs = tuple(pcs)
        branches = [q for q in range(n) if pcs[q] < len(progs[q]) and progs[q][pcs[q]][0] in ("data", "poll")
                    and _enabled(progs[q][pcs[q]], rank_of[q], flags, bufs)]
        if not branches:
            assert all(pcs[q] >= len(progs[q]) for q in range(n)), "deadlock at program counters {}".format(pcs)
            continue
        for q in branches:
            nflags, nbufs = _apply(progs[q][pcs[q]], rank_of[q], flags, bufs)
            npcs = pcs[:q] + (pcs[q] + 1,) + pcs[q + 1:]
            state = (npcs, frozenset(nflags.items()), frozenset(nbufs.items()))
            if state not in seen:
                seen.add(state)
                assert len(seen) <= limit, "state space larger than expected"
                stack.append(state)
    return len(seen)


# ---- the kernels -------------------------------------------------------------------------

def twoshot_allreduce(rk, c, rounds):
    """ar_twoshot_kernel<T, TABLE, false>: gather(i-2), push(i), reduce(i-1) per iteration."""
    n, me = rk.n, rk.me
    base, parity = rk.begin()
    for i in range(rounds + 2):
        do_pull, do_push, do_reduce = i >= 2, i < rounds, 1 <= i <= rounds
        if i >= 2:
            rk.wait(B, rk.peers, base + 2 * (i - 2) + 2)
        if do_reduce:
            rk.wait(A, rk.peers, base + 2 * (i - 1) + 1)
        acc = []
        if do_pull:
            acc += [("read", (parity, i & 1, n + p), (c, i - 2, p, "reduced")) for p in rk.peers]
        if do_push:
            acc += [("write", p, (parity, i & 1, me), (c, i, me, "pushed")) for p in rk.peers]
        if do_reduce:
            acc += [("read", (parity, (i - 1) & 1, s), (c, i - 1, s, "pushed")) for s in rk.peers]
            acc += [("write", p, (parity, (i - 1) & 1, n + me), (c, i - 1, me, "reduced")) for p in rk.peers]
        rk.data(*acc)
        if do_push:
            rk.signal(A, rk.peers, base + 2 * i + 1)
        if do_reduce:
            rk.signal(B, rk.peers, base + 2 * (i - 1) + 2)
    rk.end(parity, base + 2 * rounds + 1)


def zero_reduce(rk, c, rounds):
    """zero_reduce_kernel: push(i), reduce(i-1)."""
    me = rk.me
    base, parity = rk.begin()
    for i in range(rounds + 1):
        do_push, do_reduce = i < rounds, i >= 1
        if do_push and i >= 2:
            rk.wait(B, rk.peers, base + 2 * (i - 2) + 2)
        if do_reduce:
            rk.wait(A, rk.peers, base + 2 * (i - 1) + 1)
        acc = []
        if do_push:
            acc += [("write", p, (parity, i & 1, me), (c, i, me, "pushed")) for p in rk.peers]
        if do_reduce:
            acc += [("read", (parity, (i - 1) & 1, s), (c, i - 1, s, "pushed")) for s in rk.peers]
        rk.data(*acc)
        if do_push:
            rk.signal(A, rk.peers, base + 2 * i + 1)
        if do_reduce:
            rk.signal(B, rk.peers, base + 2 * (i - 1) + 2)
    rk.end(parity, base + 2 * rounds + 1)


def zero_update(rk, c, rounds, check=True, overflow=False):
    """zero_update_kernel: verdict word on channel D, then update(i), gather(i-1)."""
    n, me = rk.n, rk.me
    base, parity = rk.begin()
    if check:
        tag = rk.zero_ops + 1
        rk.signal(D, rk.peers, tag)
        rk.wait(D, rk.peers, tag)
        rk.zero_ops = tag
    if not overflow:
        for i in range(rounds + 1):
            do_update, do_gather = i < rounds, i >= 1
            if do_update and i >= 2:
                rk.wait(B, rk.peers, base + 2 * (i - 2) + 2)
            if do_gather:
                rk.wait(A, rk.peers, base + 2 * (i - 1) + 1)
            acc = []
            if do_update:
                acc += [("write", p, (parity, i & 1, n + me), (c, i, me, "updated")) for p in rk.peers]
            if do_gather:
                acc += [("read", (parity, (i - 1) & 1, n + p), (c, i - 1, p, "updated")) for p in rk.peers]
            rk.data(*acc)
            if do_update:
                rk.signal(A, rk.peers, base + 2 * i + 1)
            if do_gather:
                rk.signal(B, rk.peers, base + 2 * (i - 1) + 2)
    rk.end(parity, base + 2 * rounds + 1)


def gather_roles(me, n, launches, depth):
    """gather_flow_kernel (staged all-gather and broadcast): the pushing blocks and
    the copying blocks of one rank as two processes.  `launches` lists (chunks,
    root, mode) of consecutive launches; root < 0: all-gather, every rank is a
    source; mode "scatter": broadcast whose root forwards shard j of every chunk
    to rank j's inbox, every rank then pushing its shard; mode "pull": all-gather
    whose sources store into their own ring only, the copying blocks loading
    from the sources' rings.  One "pushed" and one "freed" word per rank, raised
    to base + chunk + 1; a source writes chunk k into slot k % D of the rings
    once every rank has freed chunk k - D -- or, for the first D chunks,
    everything the launches before have pushed; a forwarding rank waits for the
    root's "pushed" instead.  Every rank is modelled as reading every region
    (the kernel skips the copy of a block that is in place already, which only
    removes reads)."""
    push, out = Rank(me, n, 0), Rank(me, n, 1)
    roles = [push, out]
    everyone = list(range(n))
    base = 0
    for c, (K, root, mode) in enumerate(launches):
        D = min(depth, K)
        scatter, pull = mode == "scatter", mode == "pull"
        sources = everyone if root < 0 or scatter else [root]
        if me in sources:
            region = me if len(sources) == n else 0
            for k in range(K):
                s = k % D
                if scatter and me != root:
                    push.wait("pushed", [root], base + k + 1)
                    push.data(("read", ("inbox", s), (c, k, "shard", me)))
                else:
                    push.wait("freed", everyone, base + max(0, k - D + 1))
                    if scatter:
                        push.data(*[("write", t, ("inbox", s), (c, k, "shard", t)) for t in everyone if t != root])
                targets = [me] if pull else everyone
                push.data(*[("write", t, ("gring", s, region), (c, k, me)) for t in targets])
                push.signal("pushed", everyone, base + k + 1)
        for k in range(K):
            out.wait("pushed", sources, base + k + 1)
            if pull:
                # every rank loads the source's one copy; the model marks a buffer as read
                # by its owner only, so the owner reads and the others peek
                out.data(*[("read" if j == me else "peek",) + ((("gring", k % D, j), (c, k, j)) if j == me else
                                                              (j, ("gring", k % D, j), (c, k, j))) for j in sources])
            else:
                out.data(*[("read", ("gring", k % D, j if len(sources) == n else 0), (c, k, j)) for j in sources])
            out.signal("freed", everyone, base + k + 1)
        for rk in roles:  # kernel boundary
            rk.local_set(("gleft", c, rk.role), 1)
        for rk in roles:
            for other in roles:
                rk.local_wait(("gleft", c, other.role), 1)
        base += K
    return roles


def nvls_inplace(rk, c):
    """The caller fills its symmetric buffer, ar_nvls_inplace_kernel reduces it in
    place, the caller reads the result (and, in the next call, refills it)."""
    n, me = rk.n, rk.me
    rk.data(*[("store", me, ("user", s), (c, "input")) for s in range(n)])
    base, parity = rk.begin()
    rk.signal(A, rk.peers, base + 1)
    rk.wait(A, rk.peers, base + 1)
    rk.data(*([("peek", t, ("user", me), (c, "input")) for t in range(n)] +      # multimem.ld_reduce
              [("store", t, ("user", me), (c, "result")) for t in range(n)]))    # multimem.st
    rk.end(parity, base + 2)
    rk.wait(B, rk.peers, base + 2)
    rk.data(*[("peek", me, ("user", s), (c, "result")) for s in range(n)])


def flow_roles(me, n, collectives, depth, groups=1):
    """ar_flow_kernel: the copy-in blocks, the reducing blocks (as `groups`
    processes that take chunks in turn: reducing warps work on different chunks
    at the same time) and the copy-out blocks of one rank as processes of their own.  `collectives` lists
    the number of chunks of consecutive launches; a launch ends when all roles
    have finished (the kernel boundary), and the epoch base grows by its chunk
    count.  Counters in_done / sw_done / out_done are per ring slot and local;
    ready / done flags are per ring slot and travel to the peers."""
    cin = Rank(me, n, 0)
    sws = [Rank(me, n, 1 + g) for g in range(groups)]
    cout = Rank(me, n, 1 + groups)
    roles = [cin] + sws + [cout]
    everyone = list(range(n))
    base = 0
    for c, K in enumerate(collectives):
        D = max(groups, min(depth, K) // groups * groups)
        for k in range(K):
            s, use = k % D, k // D + 1
            if k >= D:
                cin.local_wait(("out", c, s), use - 1)
            cin.data(*[("store", me, ("ring", s, sh), (c, k, "in")) for sh in everyone])
            cin.local_set(("in", c, s), use)
            cin.signal(("ready", s), cin.peers, base + k + 1)
        for g, sw in enumerate(sws):
            for k in range(g, K, groups):
                s, use = k % D, k // D + 1
                sw.local_wait(("in", c, s), use)
                sw.wait(("ready", s), sw.peers, base + k + 1)
                sw.data(*([("peek", t, ("ring", s, me), (c, k, "in")) for t in everyone] +     # ld_reduce / n loads
                          [("store", t, ("ring", s, me), (c, k, "out")) for t in everyone]))   # multimem.st / n stores
                sw.local_set(("sw", c, s), use)
                sw.signal(("done", s), sw.peers, base + k + 1)
        for k in range(K):
            s, use = k % D, k // D + 1
            cout.local_wait(("sw", c, s), use)
            cout.wait(("done", s), cout.peers, base + k + 1)
            cout.data(*[("peek", me, ("ring", s, sh), (c, k, "out")) for sh in everyone])
            cout.local_set(("out", c, s), use)
        # kernel boundary: the next launch starts when every block has left
        for rk in roles:
            rk.local_set(("left", c, rk.role), 1)
        for rk in roles:
            for other in roles:
                rk.local_wait(("left", c, other.role), 1)
        base += K
    return roles


def ll_oneshot(rk, c):
    """ar_oneshot_ll_kernel / allgather_ll_kernel: lines {data, flag} stored into
    every peer's inbox; the receiver polls the lines.  No flag words at all."""
    flag, parity = rk.ll_ops + 1, rk.ll_ops & 1
    rk.ll_ops += 1
    rk.data(*[("write", p, ("ll", parity, rk.me), flag) for p in rk.peers])
    for s in rk.peers:
        rk.poll(("ll", parity, s), flag)


def ll_twoshot(rk, c):
    """ar_twoshot_ll_kernel: slices to the owner, results back, all as lines."""
    flag, parity = rk.ll_ops + 1, rk.ll_ops & 1
    rk.ll_ops += 1
    rk.data(*[("write", p, ("ll2", parity, 0, rk.me), flag) for p in rk.peers])
    for s in rk.peers:
        rk.poll(("ll2", parity, 0, s), flag)
    rk.data(*[("write", p, ("ll2", parity, 1, rk.me), flag) for p in rk.peers])
    for s in rk.peers:
        rk.poll(("ll2", parity, 1, s), flag)


def allgather(rk, c, rounds):
    """allgather_kernel: every rank stores its slice into gather box [me] of every
    peer; the push of round i + 1 is issued before the boxes of round i are emptied."""
    n, me = rk.n, rk.me
    base, parity = rk.begin()

    def push(rnd):
        if rnd >= 2:
            rk.wait(B, rk.peers, base + 2 * (rnd - 2) + 2)
        rk.data(*[("write", p, (parity, rnd & 1, n + me), (c, rnd, me, "slice")) for p in rk.peers])
        rk.signal(A, rk.peers, base + 2 * rnd + 1)

    push(0)
    for rnd in range(rounds):
        if rnd + 1 < rounds:
            push(rnd + 1)
        rk.wait(A, rk.peers, base + 2 * rnd + 1)
        rk.data(*[("read", (parity, rnd & 1, n + p), (c, rnd, p, "slice")) for p in rk.peers])
        rk.signal(B, rk.peers, base + 2 * rnd + 2)
    rk.end(parity, base + 2 * rounds + 1)


def allgather_pull(rk, c, rounds):
    """allgather_pull_kernel: publish in the outbox, peers pull."""
    n = rk.n
    base, parity = rk.begin()
    for rnd in range(rounds):
        e_pub, e_got = base + 2 * rnd + 1, base + 2 * rnd + 2
        if rnd >= 2:
            rk.wait(B, rk.peers, base + 2 * (rnd - 2) + 2)
        rk.data(("store", rk.me, (parity, rnd & 1, n), (c, rnd, rk.me, "outbox")))
        rk.signal(A, rk.peers, e_pub)
        rk.wait(A, rk.peers, e_pub)
        rk.data(*[("peek", p, (parity, rnd & 1, n), (c, rnd, p, "outbox")) for p in rk.peers])
        rk.signal(B, rk.peers, e_got)
    rk.end(parity, base + 2 * rounds + 1)


def broadcast_pull(rk, c, rounds, root):
    """broadcast_kernel: the root publishes, the peers pull and acknowledge."""
    n = rk.n
    base, parity = rk.begin()
    for rnd in range(rounds):
        e_pub, e_got = base + 2 * rnd + 1, base + 2 * rnd + 2
        if rk.me == root:
            if rnd >= 2:
                rk.wait(B, rk.peers, base + 2 * (rnd - 2) + 2)
            rk.data(("store", root, (parity, rnd & 1, n), (c, rnd, "outbox")))
            rk.signal(A, rk.peers, e_pub)
        else:
            rk.wait(A, [root], e_pub)
            rk.data(("peek", root, (parity, rnd & 1, n), (c, rnd, "outbox")))
            rk.signal(B, [root], e_got)
    rk.end(parity, base + 2 * rounds + 1)


def broadcast_scatter(rk, c, rounds, root):
    """broadcast_scatter_kernel: scatter from the root, all-gather among the peers."""
    n, me = rk.n, rk.me
    base, parity = rk.begin()
    for i in range(rounds):
        half = i & 1
        e_a, e_b, e_c = base + 3 * i + 1, base + 3 * i + 2, base + 3 * i + 3
        if i >= 2:
            rk.wait(C, rk.peers, base + 3 * (i - 2) + 3)
        if me == root:
            acc = []
            for p in rk.peers:
                acc.append(("write", p, (parity, half, root), (c, i, p, "slice")))
                acc.append(("write", p, (parity, half, n + root), (c, i, root, "own")))
            rk.data(*acc)
            rk.signal(A, rk.peers, e_a)
            rk.signal(C, rk.peers, e_c)
        else:
            others = [q for q in rk.peers if q != root]
            rk.wait(A, [root], e_a)
            rk.data(*([("read", (parity, half, root), (c, i, me, "slice"))] +
                      [("write", q, (parity, half, n + me), (c, i, me, "fwd")) for q in others]))
            rk.signal(B, rk.peers, e_b)
            rk.wait(B, others, e_b)
            rk.data(*[("read", (parity, half, n + src), (c, i, src, "own" if src == root else "fwd"))
                      for src in rk.peers])
            rk.signal(C, rk.peers, e_c)
    rk.end(parity, base + 3 * rounds + 1)


DEPTH = 2  # kDepth of the warp-specialised kernels


def twoshot_ws_roles(me, n, collectives):
    """ar_twoshot_ws_kernel: pusher, reducer and gatherer of one block as three
    processes.  They start a collective together (begin_collective runs before
    the roles split) and meet before end_collective."""
    roles = [Rank(me, n, role) for role in range(3)]
    push, red, gat = roles
    for c, rounds in enumerate(collectives):
        base, parity = push.epoch, push.ops & 1
        for rk in roles:
            rk.wait(B, rk.peers, push.last_done[parity])
        for i in range(rounds):
            if i >= DEPTH:
                push.wait(B, push.peers, base + (i - DEPTH) + 1)
            push.data(*[("write", p, (parity, i % DEPTH, me), (c, i, me, "pushed")) for p in push.peers])
            push.signal(A, push.peers, base + i + 1)
        for j in range(rounds):
            red.wait(A, red.peers, base + j + 1)
            if j >= DEPTH:
                red.wait(C, red.peers, base + (j - DEPTH) + 1)
            red.data(*([("read", (parity, j % DEPTH, s), (c, j, s, "pushed")) for s in red.peers] +
                       [("write", p, (parity, j % DEPTH, n + me), (c, j, me, "reduced")) for p in red.peers]))
            red.signal(B, red.peers, base + j + 1)
        for j in range(rounds):
            gat.wait(B, gat.peers, base + j + 1)
            gat.data(*[("read", (parity, j % DEPTH, n + p), (c, j, p, "reduced")) for p in gat.peers])
            gat.signal(C, gat.peers, base + j + 1)
        _join_and_end(roles, c, parity, base + rounds + 1)
    return roles


def _join_and_end(roles, c, parity, done):
    """__syncthreads_or at the end of the role loops, then end_collective."""
    first = roles[0]
    for rk in roles:
        rk.local_set("joined{}".format(rk.role), c + 1)
    for rk in roles:
        for other in roles:
            rk.local_wait("joined{}".format(other.role), c + 1)
    first.signal(B, first.peers, done)
    assert all(getattr(rk, "high", 0) <= done for rk in roles)
    first.local_set("ended", c + 1)
    for rk in roles:
        rk.local_wait("ended", c + 1)
        rk.epoch, rk.ops = done, rk.ops + 1
        rk.last_done[parity] = done


def run_roles(n, build):
    procs = []
    for me in range(n):
        procs += build(me, n)
    return explore(procs)


def run(n, build):
    ranks = [Rank(r, n) for r in range(n)]
    for rk in ranks:
        build(rk)
    return explore(ranks)


# ---- tests ---------------------------------------------------------------------------------

@pytest.mark.parametrize("n,rounds", [(2, 1), (2, 5), (3, 4), (4, 3)])
def test_twoshot_allreduce_back_to_back(n, rounds):
    def build(rk):
        for c in range(3):  # three collectives: both parities are reused
            twoshot_allreduce(rk, c, rounds)
    assert run(n, build) > 0


@pytest.mark.parametrize("n,rounds", [(2, 1), (2, 5), (3, 3), (4, 3)])
def test_sharded_optimizer_steps_back_to_back(n, rounds):
    def build(rk):
        for c in range(3):
            zero_reduce(rk, 2 * c, rounds)
            zero_update(rk, 2 * c + 1, rounds, check=True, overflow=(c == 1))  # the middle step is skipped
    assert run(n, build) > 0


def test_sharded_step_between_other_collectives():
    def build(rk):
        twoshot_allreduce(rk, 0, 2)
        zero_reduce(rk, 1, 3)
        zero_update(rk, 2, 3, check=False)
        broadcast_scatter(rk, 3, 3, root=1)
        twoshot_allreduce(rk, 4, 1)
    assert run(2, build) > 0


@pytest.mark.parametrize("n,launches,depth", [
    (2, ((5, -1, ""), (1, 0, ""), (3, 1, "")), 2), (2, ((4, 1, "scatter"), (4, -1, "")), 3),
    (3, ((4, -1, ""), (3, 2, "scatter")), 2), (3, ((3, 0, "scatter"), (2, -1, ""), (2, 1, "")), 2),
    (3, ((3, -1, "pull"), (3, 1, "scatter"), (2, -1, "pull")), 2), (4, ((3, 1, "scatter"), (2, -1, "")), 2),
    (4, ((3, -1, "pull"),), 2)])
def test_staged_gather_and_broadcast(n, launches, depth):
    """More chunks than ring slots; all-gathers and broadcasts from different roots back to back."""
    assert run_roles(n, lambda me, n_: gather_roles(me, n_, launches, depth)) > 0


@pytest.mark.parametrize("n", [2, 3, 4])
def test_in_place_multicast_allreduce_and_buffer_reuse(n):
    def build(rk):
        for c in range(3):  # the caller refills the same buffer for every call
            nvls_inplace(rk, c)
    assert run(n, build) > 0


@pytest.mark.parametrize("n,collectives,depth,groups", [(2, (5, 1, 3), 2, 1), (2, (6, 2), 4, 2), (3, (4, 3), 2, 2),
                                                        (3, (5,), 3, 1), (4, (3, 2), 2, 1)])
def test_staged_ring_allreduce(n, collectives, depth, groups):
    """More chunks than ring slots, launches back to back, one and two groups of reducing blocks."""
    assert run_roles(n, lambda me, n_: flow_roles(me, n_, collectives, depth, groups)) > 0


@pytest.mark.parametrize("n", [2, 3, 4])
def test_low_latency_kernels_share_their_counter(n):
    """Flag-in-data kernels, two parities, no flag words: a peer cannot send
    collective k+2 before this rank has sent its part of k+1."""
    def build(rk):
        for c in range(5):
            (ll_twoshot if c in (1, 2) else ll_oneshot)(rk, c)
    assert run(n, build) > 0


@pytest.mark.parametrize("n,rounds", [(2, 4), (3, 3), (4, 3)])
def test_allgather_and_the_three_broadcasts(n, rounds):
    def build(rk):
        allgather(rk, 0, rounds)
        broadcast_pull(rk, 1, rounds, root=n - 1)
        if n > 2:
            broadcast_scatter(rk, 2, rounds, root=1)
        allgather_pull(rk, 3, rounds)
        allgather(rk, 4, 1)
        broadcast_pull(rk, 5, 1, root=0)
    assert run(n, build) > 0


def test_broadcast_scatter_four_ranks():
    assert run(4, lambda rk: broadcast_scatter(rk, 0, 3, root=2)) > 0


@pytest.mark.parametrize("n,collectives", [(2, (5, 1, 3)), (3, (4, 3)), (4, (3,))])
def test_warp_specialised_twoshot(n, collectives):
    assert run_roles(n, lambda me, n_: twoshot_ws_roles(me, n_, collectives)) > 0


def test_eight_ranks():
    """The rank count of the target machine, with fewer rounds."""
    assert run(8, lambda rk: [nvls_inplace(rk, c) for c in range(2)]) > 0
    assert run_roles(4, lambda me, n: flow_roles(me, n, (3,), 2, 1)) > 0
    assert run(8, lambda rk: [twoshot_allreduce(rk, c, 2) for c in range(2)]) > 0
    assert run(8, lambda rk: [(zero_reduce(rk, 2 * c, 3), zero_update(rk, 2 * c + 1, 3)) for c in range(2)]) > 0
    assert run_roles(4, lambda me, n: gather_roles(me, n, ((2, 3, "scatter"),), 1)) > 0
    assert run_roles(4, lambda me, n: gather_roles(me, n, ((2, -1, ""),), 1)) > 0
    assert run(8, lambda rk: broadcast_scatter(rk, 0, 3, root=5)) > 0
    assert run(5, lambda rk: allgather(rk, 0, 2)) > 0   # the pushing kernel branches more: five ranks


def test_the_model_catches_a_missing_wait():
    """The checker itself: without the wait for "pushed" a reduce stage can run
    before the peer's slice has arrived, and with the pusher running two rounds
    ahead unchecked a slice is overwritten before it was read; without a signal
    the ranks deadlock.  All three must be found."""
    def reduce_without_waiting_for_the_push(rk):
        me = rk.me
        base, parity = rk.begin()
        for i in range(3):
            acc = []
            if i < 2:
                acc += [("write", p, (parity, i & 1, me), (0, i, me, "pushed")) for p in rk.peers]
            if i >= 1:
                acc += [("read", (parity, (i - 1) & 1, s), (0, i - 1, s, "pushed")) for s in rk.peers]
            rk.data(*acc)
            if i < 2:
                rk.signal(A, rk.peers, base + 2 * i + 1)
        rk.end(parity, base + 5)

    with pytest.raises(AssertionError, match="finds"):
        run(2, reduce_without_waiting_for_the_push)

    def pusher_runs_ahead(rk):
        me = rk.me
        base, parity = rk.begin()
        for i in range(4):  # all pushes first, nothing holds them back
            rk.data(*[("write", p, (parity, i & 1, me), (0, i, me, "pushed")) for p in rk.peers])
            rk.signal(A, rk.peers, base + 2 * i + 1)
        for i in range(4):
            rk.wait(A, rk.peers, base + 2 * i + 1)
            rk.data(*[("read", (parity, i & 1, s), (0, i, s, "pushed")) for s in rk.peers])
        rk.end(parity, base + 9)

    with pytest.raises(AssertionError, match="overwrites"):
        run(2, pusher_runs_ahead)

    def no_signal(rk):
        base, parity = rk.begin()
        if rk.me == 0:
            rk.signal(A, rk.peers, base + 1)
        rk.wait(A, rk.peers, base + 1)
        rk.end(parity, base + 2)

    with pytest.raises(AssertionError, match="deadlock"):
        run(2, no_signal)
