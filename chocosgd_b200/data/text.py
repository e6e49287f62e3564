"""Word-level corpus reader for wikitext-2 / PTB style folders
(``train.txt`` / ``valid.txt`` / ``test.txt``, also ``wiki.train.tokens`` naming).

The reference goes through legacy ``torchtext`` fields with a spacy tokenizer
(``dl_code/pcode/datasets/prepare_data.py:131-158``); neither package is needed here:
lines are split on whitespace and terminated by ``<eos>``."""
from __future__ import annotations

import os

import torch


class Dictionary:
    def __init__(self):
        self.word2idx = {}
        self.idx2word = []

    def add_word(self, word):
        if word not in self.word2idx:
            self.idx2word.append(word)
            self.word2idx[word] = len(self.idx2word) - 1
        return self.word2idx[word]

    def __len__(self):
        return len(self.idx2word)


class Corpus:
    NAMES = {
        "train": ("train.txt", "wiki.train.tokens", "ptb.train.txt"),
        "valid": ("valid.txt", "wiki.valid.tokens", "ptb.valid.txt"),
        "test": ("test.txt", "wiki.test.tokens", "ptb.test.txt"),
    }

    def __init__(self, path):
        self.dictionary = Dictionary()
        self.train = self.tokenize(self._find(path, "train"))
        self.valid = self.tokenize(self._find(path, "valid"))
        self.test = self.tokenize(self._find(path, "test"))

    def _find(self, path, split):
        for n in self.NAMES[split]:
            p = os.path.join(path, n)
            if os.path.exists(p):
                return p
        raise FileNotFoundError(f"no {split} file of a word-level corpus under {path}")

    def tokenize(self, path):
        ids = []
        with open(path, "r", encoding="utf8") as f:
            for line in f:
                for word in line.split() + ["<eos>"]:
                    ids.append(self.dictionary.add_word(word))
        return torch.tensor(ids, dtype=torch.int64)
