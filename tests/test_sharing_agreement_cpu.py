"""Host logic of the copy-engine all-gather set-up (bench_infer.ShardedInt8MLP._open_shared): the
ranks either all end up with their peers' buffers opened or all undo the set-up, whichever rank a
failure hits and at whichever step, and they make the same number of host exchanges on the way (an
unequal number would hang a real job).  Two ranks as threads over a fake device; no GPU."""
import threading

import pytest

import bench_infer
from vtl_b200.capi import VtlbError


class FakeDev:
    def __init__(self, rank, fail_alloc_at=None, fail_open_at=None):
        self.rank, self.fail_alloc_at, self.fail_open_at = rank, fail_alloc_at, fail_open_at
        self.allocs, self.opens, self.live, self.mapped, self.lanes = 0, 0, set(), set(), 0

    def shared_alloc(self, nbytes):
        if self.fail_alloc_at == self.allocs:
            raise VtlbError(-3, "out of memory (fake)")
        self.allocs += 1
        ptr = 0x1000 * (self.rank + 1) + self.allocs
        self.live.add(ptr)
        return ptr, bytes([self.rank, self.allocs]) * 32

    def shared_open(self, handle):
        assert len(handle) == 64
        if self.fail_open_at == self.opens:
            raise VtlbError(-2, "cannot open (fake)")
        self.opens += 1
        ptr = 0x100000 + 0x100 * handle[0] + handle[1]
        self.mapped.add(ptr)
        return ptr

    def shared_close(self, ptr):
        self.mapped.remove(ptr)

    def shared_free(self, ptr):
        self.live.remove(ptr)

    def comm_small_lane(self):
        self.lanes += 1


class Exchange:
    """obj -> [obj of rank 0, obj of rank 1] between two threads; counts the calls of each rank."""

    def __init__(self, world):
        self.world, self.slots, self.calls = world, [None] * world, [0] * world
        self.bar = threading.Barrier(world, timeout=20)

    def for_rank(self, rank):
        def exchange(obj):
            self.calls[rank] += 1
            self.slots[rank] = obj
            self.bar.wait()
            out = list(self.slots)
            self.bar.wait()
            return out
        return exchange


def run_two(devs, monkeypatch=None):
    ex, results, errors = Exchange(2), [None, None], []

    def worker(rank):
        try:
            m = object.__new__(bench_infer.ShardedInt8MLP)
            m.dev, m.R, m.rank, m.C, m.Mc = devs[rank], 2, rank, 2, 128
            m._shared, m._opened = [], []
            hidden = [dict(n=256), dict(n=128), dict(n=256)]
            results[rank] = (m._open_shared(hidden, ex.for_rank(rank)), hidden, m)
        except Exception as e:  # a broken barrier in the other thread ends up here
            errors.append((rank, repr(e)))

    ts = [threading.Thread(target=worker, args=(r,)) for r in range(2)]
    [t.start() for t in ts]
    [t.join(30) for t in ts]
    assert not errors, errors
    assert ex.calls[0] == ex.calls[1], f"unequal exchanges {ex.calls}: a real job would hang"
    return results


def test_all_ranks_share():
    devs = [FakeDev(0), FakeDev(1)]
    res = run_two(devs)
    for rank, (ok, hidden, m) in enumerate(res):
        assert ok and devs[rank].lanes == 1
        assert len(m._shared) == 3 and len(m._opened) == 3
        for L in hidden:
            assert L["peers"][rank] is None and L["peers"][1 - rank] in devs[rank].mapped
            assert L["q_all_ptr"] in devs[rank].live


@pytest.mark.parametrize("kw", [dict(fail_alloc_at=0), dict(fail_alloc_at=2), dict(fail_open_at=0), dict(fail_open_at=2)])
@pytest.mark.parametrize("bad_rank", [0, 1])
def test_a_failure_on_one_rank_undoes_the_set_up_on_all(kw, bad_rank):
    devs = [FakeDev(r, **(kw if r == bad_rank else {})) for r in range(2)]
    res = run_two(devs)
    for rank, (ok, hidden, m) in enumerate(res):
        assert not ok
        assert not devs[rank].live and not devs[rank].mapped, "a buffer or a mapping was left behind"
        assert devs[rank].lanes == 0 and not m._shared and not m._opened
        assert all("q_all_ptr" not in L and "peers" not in L and "handle" not in L for L in hidden)


def test_injected_failure_switch(monkeypatch):
    monkeypatch.setenv("VTLB_C5_FAIL_SHARING", "1")
    devs = [FakeDev(0), FakeDev(1)]
    res = run_two(devs)
    assert [r[0] for r in res] == [False, False]
    assert not devs[0].live and not devs[1].live
