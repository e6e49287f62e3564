"""Segment table of a flat parameter arena.

Every compression operator acts **per parameter tensor** (reference: the loops over
``zip(flatten_params, flatten_hat_params)``, ``dl_code/pcode/optim/parallel_choco_v.py:232-242``),
so a flat buffer always travels with the table of its segments.  Segments start on
32-element (128-byte) boundaries: one warp ballot produces one sign word that never
straddles two tensors, every segment is a legal 16-byte-aligned TMA / vector-load
base, and padding elements are kept at zero by all kernels.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import numpy as np

ALIGN = 32  # elements


def round_up(v: int, m: int) -> int:
    return (v + m - 1) // m * m


@dataclass
class Segments:
    sizes: List[int]  # logical element count of each tensor
    offsets: List[int]  # start of each tensor in the flat buffer (multiple of ALIGN)
    total: int  # padded length of the flat buffer (multiple of ALIGN)
    names: List[str]

    @staticmethod
    def from_sizes(sizes: Sequence[int], names: Sequence[str] = None, align: int = ALIGN) -> "Segments":
        offsets, off = [], 0
        for n in sizes:
            offsets.append(off)
            off += round_up(int(n), align)
        names = list(names) if names is not None else [f"t{i}" for i in range(len(sizes))]
        return Segments([int(s) for s in sizes], offsets, max(off, align), names)

    @property
    def n_segments(self) -> int:
        return len(self.sizes)

    @property
    def n_elements(self) -> int:
        """Logical (unpadded) number of elements."""
        return int(sum(self.sizes))

    def slices(self):
        for off, n in zip(self.offsets, self.sizes):
            yield slice(off, off + n)

    def keep_counts(self, compress_ratio: float) -> List[int]:
        """Per-tensor k of the sparsifiers: ``compress_ratio`` is the fraction *dropped*,
        k = max(1, int(n (1 - ratio)))  (``dl_code/pcode/utils/sparsification.py:22,45``)."""
        return [max(1, int(n * (1.0 - compress_ratio))) for n in self.sizes]

    def segment_of_element(self) -> np.ndarray:
        """int32 map flat position -> segment id (padding maps to the preceding segment)."""
        out = np.zeros(self.total, dtype=np.int32)
        for t, off in enumerate(self.offsets):
            out[off:] = t
        return out

    def valid_mask(self) -> np.ndarray:
        m = np.zeros(self.total, dtype=bool)
        for s in self.slices():
            m[s] = True
        return m
