"""The DataLoader oracle against the reference's rules, worked out by hand where they can be."""
import numpy as np

from oracle import dataloader as odl


def test_lcg_first_outputs():
    """state' = state * 6364136223846793005 + 1442695040888963407 (mod 2^64); seed 0 counts as 1."""
    a, c, m = 6364136223846793005, 1442695040888963407, 1 << 64
    r = odl.LcgRng(0)
    s1 = (1 * a + c) % m
    s2 = (s1 * a + c) % m
    assert r.next() == s1 == 7806831264735756412
    assert r.next() == s2
    assert odl.LcgRng(1).next() == s1
    assert odl.LcgRng(5).next() == (5 * a + c) % m


def test_shuffle_is_a_permutation_and_depends_on_seed_and_epoch():
    data = np.arange(40, dtype=np.float32).reshape(20, 2)
    a = odl.DataLoader(data, batch_size=4, shuffle=True, seed=3)
    b = odl.DataLoader(data, batch_size=4, shuffle=True, seed=3)
    c = odl.DataLoader(data, batch_size=4, shuffle=True, seed=4)
    assert sorted(a.indices) == list(range(20)) and a.indices == b.indices != c.indices
    first = list(a.indices)
    a.reset()
    assert a.epoch == 1 and sorted(a.indices) == list(range(20)) and a.indices != first
    # the epoch-1 order is the epoch-0 order shuffled again with seed + 1
    c2 = odl.DataLoader(data, batch_size=4, shuffle=False)
    c2.indices = list(first)
    c2.seed, c2.epoch, c2.shuffle = 3, 0, True
    c2.reset()
    assert c2.indices == a.indices


def test_hand_worked_shuffle_of_three():
    """n = 3, seed 0 (state 1): i = 2 swaps with next() % 3, i = 1 swaps with next() % 2."""
    a, c, m = 6364136223846793005, 1442695040888963407, 1 << 64
    s1 = (a + c) % m
    s2 = (s1 * a + c) % m
    idx = [0, 1, 2]
    j = s1 % 3
    idx[2], idx[j] = idx[j], idx[2]
    j = s2 % 2
    idx[1], idx[j] = idx[j], idx[1]
    dl = odl.DataLoader(np.zeros((3, 1), np.float32), batch_size=1, shuffle=True, seed=0)
    assert dl.indices == idx


def test_batches_len_and_drop_last():
    data = np.arange(30, dtype=np.float32).reshape(10, 3)
    labels = np.eye(10, dtype=np.float32)
    dl = odl.DataLoader(data, labels, batch_size=4, shuffle=False, drop_last=True)
    assert len(dl) == 2 and dl.batch(2) is None and dl.batch(-1) is None
    assert np.array_equal(dl.batch(1), data[4:8])
    dl2 = odl.DataLoader(data, labels, batch_size=4, shuffle=False, drop_last=False)
    assert len(dl2) == 3 and dl2.batch(2).shape == (2, 3) and dl2.batch(3) is None
    f, l = dl2.batch_with_labels(2)
    assert np.array_equal(f, data[8:]) and np.array_equal(l, labels[8:])
    assert odl.DataLoader(data, batch_size=4, shuffle=False).batch_with_labels(0) is None


def test_split():
    data = np.arange(20, dtype=np.float32).reshape(10, 2)
    dl = odl.DataLoader(data, batch_size=3, shuffle=True, seed=9)
    train, val = dl.split(0.25)
    assert train.indices == dl.indices[:8] and val.indices == dl.indices[8:]
    assert not train.shuffle and not val.shuffle and train.drop_last and not val.drop_last
    assert len(train) == 2 and len(val) == 1
