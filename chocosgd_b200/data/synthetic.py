"""Synthetic data of the benchmark shapes (no dataset files exist offline).

Images are N(0, 1) with uniform random labels; token streams are uniform over the
vocabulary.  Generation is a pure function of ``(seed, index)`` so ranks and restarts see
the same samples."""
from __future__ import annotations

import torch
from torch.utils.data import Dataset

SHAPES = {
    "synthetic_cifar10": ((3, 32, 32), 10),
    "synthetic_cifar100": ((3, 32, 32), 100),
    "synthetic_imagenet": ((3, 224, 224), 1000),
    "synthetic_mnist": ((1, 28, 28), 10),
}


class SyntheticImages(Dataset):
    def __init__(self, shape=(3, 32, 32), num_classes=10, size=50000, seed=0, materialize=None):
        self.shape, self.num_classes, self.size, self.seed = tuple(shape), num_classes, int(size), seed
        g = torch.Generator().manual_seed(seed)
        self.targets = torch.randint(0, num_classes, (self.size,), generator=g)
        n_el = self.size
        for s in self.shape:
            n_el *= s
        if materialize is None:
            materialize = n_el <= 64 * 1024 * 1024
        self.images = torch.randn((self.size,) + self.shape, generator=g) if materialize else None

    def __len__(self):
        return self.size

    def __getitem__(self, idx):
        if self.images is not None:
            return self.images[idx], int(self.targets[idx])
        g = torch.Generator().manual_seed(self.seed * 1000003 + int(idx))
        return torch.randn(self.shape, generator=g), int(self.targets[idx])


class SyntheticTokens:
    """A token stream batchified for truncated BPTT: ``[n_steps, global_batch]`` ids."""

    def __init__(self, n_tokens=33278, length=2_088_628, seed=0):
        g = torch.Generator().manual_seed(seed)
        self.n_tokens = n_tokens
        self.stream = torch.randint(0, n_tokens, (int(length),), generator=g)

    def batchify(self, global_batch):
        n = self.stream.numel() // global_batch
        return self.stream[: n * global_batch].view(global_batch, n).t().contiguous()
