"""Device-side batch assembly and the copy pipeline: the host mirror's DataLoader against the CPU
restatement of datasets/dataloader.v (indices and batches bit-exact), the gather / one-hot kernels,
and double-buffered host<->device copies overlapping compute."""
import ctypes as C

import numpy as np
import pytest

from oracle import dataloader as odl

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sess():
    from vtl_b200 import capi, host
    if capi.device_count() == 0:
        pytest.skip("no CUDA device")
    s = host.Session(0)
    yield s
    s.dev.sync()
    assert s.dev.check_status() == 0
    s.close()


@pytest.mark.parametrize("rows,row_elems", [(1, 1), (7, 3), (100, 784), (33, 3 * 32 * 32), (5, 1000001)])
def test_gather_rows(dev, rows, row_elems):
    rng = np.random.default_rng(rows + row_elems)
    src = rng.standard_normal((rows, row_elems)).astype(np.float32)
    idx = rng.integers(0, rows, size=2 * rows + 1).astype(np.int32)
    d_src, d_idx = dev.to_device(src), dev.to_device(idx)
    d_dst = dev.zeros((idx.size, row_elems))
    dev.gather_rows_f32(d_src, rows, row_elems, d_idx, idx.size, d_dst)
    assert np.array_equal(d_dst.numpy(), src[idx])
    for b in (d_src, d_idx, d_dst):
        b.free()


def test_gather_and_one_hot_refuse_out_of_range(dev):
    from vtl_b200.capi import VtlbError
    src = np.arange(12, dtype=np.float32).reshape(4, 3)
    d_src, d_dst = dev.to_device(src), dev.zeros((3, 3))
    for bad in (4, -1):
        d_idx = dev.to_device(np.array([0, bad, 2], np.int32))
        with pytest.raises(VtlbError, match="outside"):
            dev.gather_rows_f32(d_src, 4, 3, d_idx, 3, d_dst)
        d_idx.free()
    d_lab, d_out = dev.to_device(np.array([0, 3, 1], np.int32)), dev.zeros((3, 3))
    with pytest.raises(VtlbError, match="label is outside"):
        dev.one_hot_f32(d_lab, 3, 3, d_out)
    assert dev.check_status() == 0
    for b in (d_src, d_dst, d_lab, d_out):
        b.free()


def test_one_hot(dev):
    rng = np.random.default_rng(0)
    lab = rng.integers(0, 10, size=1000).astype(np.int32)
    d_lab, d_out = dev.to_device(lab), dev.zeros((1000, 10))
    dev.one_hot_f32(d_lab, 1000, 10, d_out)
    assert np.array_equal(d_out.numpy(), np.eye(10, dtype=np.float32)[lab])
    d_lab.free(); d_out.free()


@pytest.mark.parametrize("shuffle,drop_last,n,bs", [(True, True, 103, 16), (True, False, 103, 16),
                                                    (False, False, 10, 4), (True, True, 64, 64), (True, True, 5, 8)])
def test_loader_matches_oracle(sess, shuffle, drop_last, n, bs):
    from vtl_b200 import host
    rng = np.random.default_rng(n)
    data = rng.standard_normal((n, 3, 4, 4)).astype(np.float32)
    labels = np.eye(10, dtype=np.float32)[rng.integers(0, 10, n)]
    d_data, d_lab = sess.dev.to_device(data), sess.dev.to_device(labels)
    ours = host.DataLoader(sess, d_data, d_lab, batch_size=bs, shuffle=shuffle, drop_last=drop_last, seed=7)
    ref = odl.DataLoader(data, labels, batch_size=bs, shuffle=shuffle, drop_last=drop_last, seed=7)
    for epoch in range(3):
        assert ours.indices == ref.indices and len(ours) == len(ref) and ours.total_samples() == n
        for i in range(len(ref) + 1):
            want = ref.batch_with_labels(i)
            got = ours.batch_with_labels(i)
            if want is None:
                assert got is None
                continue
            f, l = got
            assert np.array_equal(f.numpy(), want[0]) and np.array_equal(l.numpy(), want[1])
            only = ours.batch(i)
            assert np.array_equal(only.numpy(), want[0])
            for b in (f, l, only):
                b.free()
        ours.reset()
        ref.reset()
    t, v = ours.split(0.2)
    rt, rv = ref.split(0.2)
    assert t.indices == rt.indices and v.indices == rv.indices and len(t) == len(rt) and len(v) == len(rv)
    if len(rv):
        b = v.batch(len(rv) - 1)
        assert np.array_equal(b.numpy(), rv.batch(len(rv) - 1))
        b.free()
    for x in (t, v, ours):
        x.close()
    d_data.free(); d_lab.free()


def test_loader_without_labels_and_bad_arguments(sess):
    from vtl_b200 import host
    from vtl_b200.capi import VtlbError
    data = np.arange(24, dtype=np.float32).reshape(6, 4)
    d = sess.dev.to_device(data)
    dl = host.DataLoader(sess, d, batch_size=4, shuffle=False, drop_last=False)
    assert dl.batch_with_labels(0) is None and len(dl) == 2
    b = dl.batch(1)
    assert np.array_equal(b.numpy(), data[4:])
    b.free(); dl.close()
    with pytest.raises(VtlbError, match="batch_size"):
        host.DataLoader(sess, d, batch_size=0)
    lab = sess.dev.to_device(np.zeros((5, 2), np.float32))
    with pytest.raises(VtlbError, match="first dimension"):
        host.DataLoader(sess, d, lab, batch_size=2)
    d.free(); lab.free()


def test_double_buffered_copies_overlap_compute_and_keep_order(dev):
    """Eight batches go in, ReLU runs on each, eight results come out, with the next copy-in and the
    previous copy-out in flight while a batch computes; every result must be its own batch's."""
    n, steps = 1 << 20, 8
    rng = np.random.default_rng(5)
    batches = [rng.standard_normal(n).astype(np.float32) for _ in range(steps)]
    h_in = [C.c_void_p() for _ in range(steps)]
    h_out = [C.c_void_p() for _ in range(steps)]
    for i in range(steps):
        assert dev.lib.vtlb_host_alloc(n * 4, C.byref(h_in[i])) == 0
        assert dev.lib.vtlb_host_alloc(n * 4, C.byref(h_out[i])) == 0
        C.memmove(h_in[i].value, batches[i].ctypes.data, n * 4)
    d_in = [dev.zeros(n), dev.zeros(n)]
    d_out = [dev.zeros(n), dev.zeros(n)]
    dev.copy_h2d_async(d_in[0], h_in[0].value, n * 4)
    for i in range(steps):
        dev.copy_wait(dev.COPY_IN_BEFORE_COMPUTE)
        if i + 1 < steps:
            dev.copy_h2d_async(d_in[(i + 1) % 2], h_in[i + 1].value, n * 4)
        dev.relu_fwd_f32(d_in[i % 2], d_out[i % 2], n)
        dev.copy_wait(dev.COPY_OUT_BEFORE_COMPUTE)
        dev.copy_d2h_async(h_out[i].value, d_out[i % 2], n * 4)
    dev.copy_wait(dev.COPY_OUT_DONE)
    for i in range(steps):
        got = np.frombuffer((C.c_float * n).from_address(h_out[i].value), np.float32)
        assert np.array_equal(got, np.maximum(batches[i], 0.0)), f"batch {i}"
    from vtl_b200.capi import VtlbError
    with pytest.raises(VtlbError, match="unknown bits"):
        dev.copy_wait(64)
    for h in h_in + h_out:
        dev.lib.vtlb_host_free(h)
    for b in d_in + d_out:
        b.free()
