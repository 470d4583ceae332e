"""The copy-engine all-gather of the column-sharded INT8 pipeline, checked as a protocol on the CPU.

`bench_infer.ShardedInt8MLP.forward` is run against a recording device: every call it makes (GEMM,
quantise, all-reduce, push, mark, wait) is written down with the stream it goes to and the buffers it
reads and writes.  The recorded programs of all ranks are then played on a small model of CUDA's
ordering rules -- in-order streams, events, collectives that end only after every rank has started
them, copies that write into a peer's buffer -- with random durations and slow ranks, over several
forward passes that re-use the same buffers.  Checked: no rank's buffer is ever written while its
owner still reads it (or read while being written), and every GEMM reads the codes of its own pass.
A control run with the closing all-reduce of a push left out must trip the checker."""
import random
from types import SimpleNamespace as NS

import pytest

import bench_infer

BASE = 1 << 44  # exported gather buffers live above this address; everything else is private


def gather_base(rank, layer):
    return BASE * (rank + 1) + (layer << 36)


class RecDev:
    LANE_BULK, LANE_SMALL = 0, 1

    def __init__(self, rank, small_lane, closing_collective=True):
        self.rank, self.small_lane, self.closing = rank, small_lane, closing_collective
        self.prog, self.step = [], 0

    def _lane(self, lane):
        return "small" if (lane == self.LANE_SMALL and self.small_lane) else "bulk"

    # compute-stream work
    def quant_rows_i8(self, A, M, K, Q, scale, amax_in=None):
        Q = getattr(Q, "ptr", Q)
        self.prog.append(NS(op="kernel", name="quant", reads=[], writes=[(Q, Q + M * K)], step=self.step))

    def _gemm(self, aq, shards, Mc, K):
        part = Mc * (K // shards)
        self.prog.append(NS(op="kernel", name="gemm", reads=[(aq + s * part, aq + (s + 1) * part) for s in range(shards)],
                            writes=[], step=self.step))

    def linear_i8_fwd_amax(self, aq, shards, sa, Wq, sw, bias, y, Mc, n, K, relu, amax):
        self._gemm(aq, shards, Mc, K)

    def linear_i8_fwd_sharded_a(self, aq, shards, sa, Wq, sw, bias, y, Mc, n, K, relu=False):
        self._gemm(aq, shards, Mc, K)

    # communication
    def allreduce_max_f32_async(self, ptr, n):
        self.prog.append(NS(op="coll", lane=self._lane(self.LANE_SMALL)))

    def allgather_push_async(self, src, peer_dst, nbytes):
        R = len(peer_dst)
        copies = []
        for i in range(1, R + 1):
            r = (self.rank + i) % R
            if peer_dst[r]:
                copies.append((peer_dst[r], peer_dst[r] + nbytes))
        self.prog.append(NS(op="push", src=(src, src + nbytes), copies=copies, step=self.step, closing=self.closing))

    def comm_mark(self, lane, slot):
        self.prog.append(NS(op="mark", lane=self._lane(lane), slot=slot))

    def comm_wait_mark(self, slot):
        self.prog.append(NS(op="waitmark", slot=slot))

    def comm_wait(self):
        self.prog.append(NS(op="commwait"))


def make_model(rank, R, C, dims, tokens, dev):
    m = object.__new__(bench_infer.ShardedInt8MLP)
    m.dev, m.R, m.rank, m.M, m.dims, m.C, m.Mc, m.push = dev, R, rank, tokens, dims, C, tokens // C, True
    m.layers = []
    for li in range(len(dims) - 1):
        n = dims[li + 1] // R
        priv = (li + 1) << 30
        L = dict(K=dims[li], N=dims[li + 1], n=n, Wq=NS(ptr=priv), sw=NS(ptr=priv + 1), bias=NS(ptr=priv + 2),
                 Y=NS(ptr=priv + (1 << 20)), amax=NS(ptr=priv + (2 << 20)), sa=NS(ptr=priv + (3 << 20)))
        if li + 1 < len(dims) - 1:
            L["q_all_ptr"] = gather_base(rank, li)
            L["peers"] = [None if r == rank else gather_base(r, li) for r in range(R)]
        else:
            L["q_all_ptr"] = priv + (4 << 20)
        m.layers.append(L)
    m.q_in, m.sa_in = NS(ptr=1 << 20), NS(ptr=2 << 20)
    return m


def record(R, C, small_lane, steps, closing=True, dims=(512, 1024, 512, 1024, 512), tokens=256):
    progs = []
    for rank in range(R):
        dev = RecDev(rank, small_lane, closing)
        model = make_model(rank, R, C, list(dims), tokens, dev)
        for s in range(steps):
            dev.step = s
            model.forward(NS(ptr=3 << 20))
        progs.append(dev.prog)
    return progs


def play(progs, rng):
    """Times every recorded call under CUDA's ordering rules; returns the accesses to gather buffers as
    (owner-global interval, 'r' | 'w', start, end, step, rank)."""
    R = len(progs)
    slow = [rng.choice([1.0, 1.0, 2.5, 6.0]) for _ in range(R)]
    ops = []       # every timed op: NS(rank, stream, deps, dur, coll, start, end, access)
    colls = {}     # (lane, index) -> list of its R ops

    def dur(kind, rank):
        base = {"gemm": 8.0, "quant": 1.5, "copy": 5.0, "coll": 1.0, "zero": 0.0}[kind]
        return base * rng.uniform(0.3, 2.0) * (slow[rank] if kind != "coll" else 1.0)

    for rank, prog in enumerate(progs):
        tail = {"compute": None, "bulk": None, "small": None}
        marks, n_coll = {}, {"bulk": 0, "small": 0}

        def add(stream, kind, deps=(), coll=None, access=()):
            o = NS(rank=rank, stream=stream, deps=[d for d in (tail[stream],) + tuple(deps) if d is not None],
                   dur=dur(kind, rank), coll=coll, start=None, end=None, access=list(access))
            ops.append(o)
            tail[stream] = o
            if coll is not None:
                colls.setdefault(coll, []).append(o)
            return o

        for c in prog:
            if c.op == "kernel":
                acc = [(iv, "r", c.step) for iv in c.reads if iv[0] >= BASE] + \
                      [(iv, "w", c.step) for iv in c.writes if iv[0] >= BASE]
                add("compute", c.name, access=acc)
            elif c.op == "coll":  # ordered behind the compute work enqueued so far
                add(c.lane, "coll", deps=[tail["compute"]], coll=(c.lane, n_coll[c.lane]))
                n_coll[c.lane] += 1
            elif c.op == "push":
                first = True
                for iv in c.copies:
                    add("bulk", "copy", deps=[tail["compute"]] if first else [], access=[(iv, "w", c.step), (c.src, "r", c.step)])
                    first = False
                if c.closing:
                    add("bulk", "coll", deps=[tail["compute"]] if first else [], coll=("bulk", n_coll["bulk"]))
                    n_coll["bulk"] += 1
            elif c.op == "mark":
                marks[c.slot] = tail[c.lane]
            elif c.op == "waitmark":
                add("compute", "zero", deps=[marks[c.slot]])
            elif c.op == "commwait":
                add("compute", "zero", deps=[tail["bulk"], tail["small"]])
    for group in colls.values():
        assert len(group) == R, "the ranks issue different numbers of collectives"
    pending = list(ops)
    while pending:
        progress, rest = False, []
        for o in pending:
            if o.start is None and all(d.end is not None for d in o.deps):
                o.start = max([d.end for d in o.deps], default=0.0)
                progress = True
                if o.coll is None:
                    o.end = o.start + o.dur
            if o.coll is not None and o.start is not None and o.end is None:
                group = colls[o.coll]
                if all(g.start is not None for g in group):  # it ends only after every rank has entered it
                    e = max(g.start for g in group) + group[0].dur
                    for g in group:
                        g.end = e
                    progress = True
            if o.end is None:
                rest.append(o)
        assert progress, "the recorded programs deadlock"
        pending = rest
    return [(iv, kind, o.start, o.end, step, o.rank) for o in ops for (iv, kind, step) in o.access]


def violations(accesses):
    """Overlapping intervals of one buffer: a write may not overlap a read or another write in time, and
    the last write that ended before a read started must belong to the read's own pass."""
    bad = []
    writes = [a for a in accesses if a[1] == "w"]
    reads = [a for a in accesses if a[1] == "r"]
    overlap = lambda x, y: x[0] < y[1] and y[0] < x[1]
    for rd in reads:
        feeding = None
        for w in writes:
            if not overlap(rd[0], w[0]):
                continue
            if w[2] < rd[3] and rd[2] < w[3]:
                bad.append(("written while read", w, rd))
            if w[3] <= rd[2] and (feeding is None or w[3] > feeding[3]):
                feeding = w
        if feeding is None or feeding[4] != rd[4]:
            bad.append(("reads another pass's data", feeding, rd))
    return bad


@pytest.mark.parametrize("R,C,small_lane", [(2, 2, True), (3, 2, True), (4, 2, False), (4, 4, True), (3, 1, False)])
def test_no_buffer_is_overwritten_while_it_is_read(R, C, small_lane):
    progs = record(R, C, small_lane, steps=3, dims=(384 * 4, 768 * 4, 384 * 4, 768 * 4, 384 * 4), tokens=64 * C)
    for trial in range(40):
        rng = random.Random(1000 * R + 10 * C + trial)
        acc = play(progs, rng)
        # every hidden layer's block is read by the next layer's GEMM on every rank in every pass
        assert sum(1 for a in acc if a[1] == "r" and a[0][0] >= BASE) > 0
        bad = violations(acc)
        assert not bad, bad[:2]


def test_the_checker_sees_a_push_without_its_closing_collective():
    """Control: without the one-word all-reduce behind the copies a rank may read a block before a
    slow peer's part has landed (and, over passes, be overwritten while reading)."""
    progs = record(3, 2, True, steps=3, closing=False, dims=(384 * 4, 768 * 4, 384 * 4, 768 * 4, 384 * 4), tokens=128)
    found = 0
    for trial in range(40):
        found += bool(violations(play(progs, random.Random(trial))))
    assert found > 0
