"""CPU restatement of the reference's DataLoader (TEST INFRASTRUCTURE ONLY).

Follows datasets/dataloader.v: index order (:179-224: 0..n-1, shuffled at creation when
shuffle is set), Fisher-Yates from the back driven by the LCG
state = state * 6364136223846793005 + 1442695040888963407 (mod 2^64), seeded with
seed + epoch, seed 0 replaced by 1 (:168-177, :316-331); batch ranges and drop_last (:41-63);
len (:146-154); reset (:160-165); split (:270-306).  Batches are row gathers of the dataset and
label arrays (:66-83, :107-141).

Parity: the reference's own tests for this file are not part of the hot path's golden vectors; the
LCG constants and the shuffle are restated from the source, and the first outputs of the generator
are pinned in tests/ as plain 64-bit arithmetic."""
from __future__ import annotations

import numpy as np

MASK = (1 << 64) - 1


class LcgRng:
    def __init__(self, seed: int):
        self.state = 1 if seed == 0 else seed & MASK

    def next(self) -> int:
        self.state = (self.state * 6364136223846793005 + 1442695040888963407) & MASK
        return self.state


class DataLoader:
    def __init__(self, dataset, labels=None, batch_size=32, shuffle=True, drop_last=True, seed=0):
        self.dataset, self.labels = dataset, labels
        self.batch_size, self.shuffle, self.drop_last, self.seed = batch_size, shuffle, drop_last, seed
        self.indices = list(range(dataset.shape[0]))
        self.epoch = 0
        if shuffle:
            self._shuffle()

    def _shuffle(self):
        rng = LcgRng((self.seed + self.epoch) & MASK)
        i = len(self.indices) - 1
        while i > 0:
            j = rng.next() % (i + 1)
            self.indices[i], self.indices[j] = self.indices[j], self.indices[i]
            i -= 1

    def reset(self):
        self.epoch += 1
        if self.shuffle:
            self._shuffle()

    def __len__(self):
        if not self.indices:
            return 0
        if self.drop_last:
            return len(self.indices) // self.batch_size
        return (len(self.indices) + self.batch_size - 1) // self.batch_size

    def _range(self, i):
        if not self.indices or i < 0:
            return None
        start = i * self.batch_size
        if start >= len(self.indices):
            return None
        end = start + self.batch_size
        if end > len(self.indices):
            if self.drop_last:
                return None
            end = len(self.indices)
        return start, end

    def batch(self, i):
        r = self._range(i)
        if r is None:
            return None
        return self.dataset[np.asarray(self.indices[r[0]:r[1]])]

    def batch_with_labels(self, i):
        r = self._range(i)
        if r is None or self.labels is None:
            return None
        idx = np.asarray(self.indices[r[0]:r[1]])
        return self.dataset[idx], self.labels[idx]

    def split(self, val_fraction):
        n = len(self.indices)
        val_size = int(float(n) * val_fraction)
        train_size = n - val_size
        train = DataLoader(self.dataset, self.labels, self.batch_size, False, self.drop_last, self.seed)
        train.indices, train.epoch = list(self.indices[:train_size]), self.epoch
        val = DataLoader(self.dataset, self.labels, self.batch_size, False, False, self.seed)
        val.indices, val.epoch = list(self.indices[train_size:]), 0
        return train, val
