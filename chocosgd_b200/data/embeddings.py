"""Pretrained word embeddings for the language model (``--rnn_use_pretrained_emb True``).

The reference lets torchtext attach GloVe vectors to its vocabulary and sizes the embedding
layer from them (``dl_code/pcode/create_model.py:44-76``).  Here a plain-text vector file
(``word v1 ... vd`` per line, the GloVe / fastText ``.txt`` / ``.vec`` layout) found under the
dataset folder is aligned with the corpus dictionary; words without a vector keep a small
uniform initialisation, as a freshly initialised embedding row would."""
from __future__ import annotations

import glob
import os
from typing import Optional

import torch

PATTERNS = ("glove*.txt", "*.vec", "vectors*.txt")


def find_vector_file(folder: str) -> Optional[str]:
    for pat in PATTERNS:
        hits = sorted(glob.glob(os.path.join(folder, pat)))
        if hits:
            return hits[0]
    return None


def load_vectors(path: str, word2idx, init_range: float = 0.1, seed: int = 0):
    """-> (weight [len(word2idx), d], number of dictionary words found in the file)."""
    dim, found, weight = None, 0, None
    with open(path, "r", encoding="utf8", errors="ignore") as f:
        for line in f:
            parts = line.rstrip().split(" ")
            if len(parts) < 3:
                continue  # fastText header line "<count> <dim>"
            if dim is None:
                dim = len(parts) - 1
                g = torch.Generator().manual_seed(seed)
                weight = (torch.rand(len(word2idx), dim, generator=g) * 2 - 1) * init_range
            i = word2idx.get(parts[0])
            if i is not None and len(parts) - 1 == dim:
                weight[i] = torch.tensor([float(v) for v in parts[1:]])
                found += 1
    if weight is None:
        raise ValueError(f"no vectors in {path}")
    return weight, found
