"""Split a dataset over the ranks.

Rank 0 draws the index order (shuffled: ``random``; ordered by label: ``sorted`` = the
non-IID setting) and broadcasts it; every rank takes its slice of equal size
(``dl_code/pcode/datasets/partition_data.py:23-72``).  The shuffle is seeded with the run
seed (the reference uses the unseeded global ``random``)."""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist


class Partition:
    """Dataset-like view of a subset of indices."""

    def __init__(self, data, indices):
        self.data = data
        self.indices = indices

    def __len__(self):
        return len(self.indices)

    def __getitem__(self, index):
        return self.data[self.indices[index]]


class DataPartitioner:
    def __init__(self, data, partition_sizes, partition_type="random", seed=6, rank=0, on_cuda=False, group=None):
        self.data = data
        self.partition_sizes = list(partition_sizes)
        self.partition_type = partition_type
        self.data_size = len(data)
        indices = self._get_consistent_indices(seed, rank, on_cuda, group)
        self.partitions = []
        from_index = 0
        for frac in self.partition_sizes:
            to_index = from_index + int(frac * self.data_size)
            self.partitions.append(indices[from_index:to_index])
            from_index = to_index

    def _local_indices(self, seed):
        indices = np.arange(self.data_size)
        if self.partition_type == "random":
            np.random.RandomState(seed).shuffle(indices)
        elif self.partition_type == "sorted":
            targets = getattr(self.data, "targets", None)
            if targets is None:
                targets = [self.data[i][1] for i in range(self.data_size)]
            indices = np.argsort(np.asarray(targets), kind="stable")
        elif self.partition_type in (None, "origin"):
            pass
        else:
            raise NotImplementedError(self.partition_type)
        return indices

    def _get_consistent_indices(self, seed, rank, on_cuda, group):
        indices = self._local_indices(seed)
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            t = torch.from_numpy(indices.astype(np.int64))
            if on_cuda and dist.get_backend(group) == "nccl":
                t = t.cuda()
            dist.broadcast(t, src=0, group=group)
            indices = t.cpu().numpy()
        return list(indices)

    def use(self, partition_ind):
        return Partition(self.data, self.partitions[partition_ind])
