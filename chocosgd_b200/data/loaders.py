"""``define_dataset``: train/validation loaders for CV and the BPTT iterator for NLP
(``dl_code/pcode/create_dataset.py:17-204``).

``--data synthetic_*`` works offline; the on-disk datasets (cifar10/100, mnist, stl10, svhn,
imagenet folders, wikitext2 / ptb text files) are read through torchvision / plain text
files when present under ``--data_dir`` and fail with a clear error otherwise."""
from __future__ import annotations

import os

import torch
from torch.utils.data import DataLoader

from .partition import DataPartitioner
from .synthetic import SHAPES, SyntheticImages, SyntheticTokens
from .text import Corpus


def load_data_batch(device, _input, _target, non_blocking=True):
    """Host -> device copy of one batch (pinned memory makes it asynchronous)."""
    if device is not None and str(device) != "cpu":
        _input = _input.to(device, non_blocking=non_blocking)
        _target = _target.to(device, non_blocking=non_blocking)
    return _input, _target


def _cv_datasets(conf):
    name = conf.data
    if name.startswith("synthetic"):
        shape, classes = SHAPES.get(name, ((3, 32, 32), 10))
        n_train = conf.synthetic_size or (50000 if shape[-1] <= 32 else 2048)
        n_val = max(conf.batch_size, n_train // 5)
        return (
            SyntheticImages(shape, classes, n_train, seed=conf.manual_seed),
            SyntheticImages(shape, classes, n_val, seed=conf.manual_seed + 1),
        )
    if name in ("epsilon", "rcv1"):
        # feature-vector sets packed by `python -m chocosgd_b200.data.serialize --libsvm ...`
        from .lmdb_dataset import define_epsilon_or_rcv1_folder

        root = os.path.join(conf.data_dir, name)
        return (define_epsilon_or_rcv1_folder(os.path.join(root, f"{name}_train.lmdb")),
                define_epsilon_or_rcv1_folder(os.path.join(root, f"{name}_test.lmdb")))
    from .vision import get_vision_dataset

    return (
        get_vision_dataset(name, conf.data_dir, split="train", use_lmdb=conf.use_lmdb_data),
        get_vision_dataset(name, conf.data_dir, split="test", use_lmdb=conf.use_lmdb_data),
    )


def define_cv_dataset(conf, graph, run, force_shuffle=False):
    train, val = _cv_datasets(conf)
    world = graph.n_nodes
    if conf.partition_data:
        sizes = [1.0 / world for _ in range(world)]
        part = DataPartitioner(train, sizes, conf.partition_data, conf.manual_seed, graph.rank, graph.on_cuda)
        train_use = part.use(graph.rank)
    else:
        train_use = train
    pin = bool(conf.pin_memory and graph.on_cuda)
    train_loader = DataLoader(
        train_use, batch_size=conf.batch_size, shuffle=True, num_workers=conf.num_workers, pin_memory=pin,
        drop_last=False,
    )
    val_loader = DataLoader(
        val, batch_size=conf.batch_size, shuffle=False, num_workers=conf.num_workers, pin_memory=pin, drop_last=False
    )
    # epoch length: a rank that sees all data still only does 1/n of an epoch's batches.
    run.num_batches_train_per_device_per_epoch = (
        len(train_loader) if conf.partition_data else max(1, len(train_loader) // world)
    )
    run.num_whole_train_batches_per_worker = run.num_batches_train_per_device_per_epoch * conf.num_epochs
    run.num_warmup_train_batches_per_worker = run.num_batches_train_per_device_per_epoch * conf.lr_warmup_epochs
    run.num_iterations_per_worker = conf.num_iterations // world
    run.num_batches_val_per_device_per_epoch = len(val_loader)
    return {"train_loader": train_loader, "val_loader": val_loader}


class BPTTIterator:
    """Windows of ``bptt_len`` steps over a batchified stream; yields (text, target) of shape
    ``[bptt, global_batch]`` (the loop slices this rank's columns)."""

    def __init__(self, data, bptt_len, device=None):
        self.data = data if device is None else data.to(device)
        self.bptt_len = bptt_len

    def __len__(self):
        return max(0, (self.data.size(0) - 1 + self.bptt_len - 1) // self.bptt_len)

    def __iter__(self):
        n = self.data.size(0)
        for i in range(0, n - 1, self.bptt_len):
            seq = min(self.bptt_len, n - 1 - i)
            yield self.data[i:i + seq], self.data[i + 1:i + 1 + seq]


def define_nlp_dataset(conf, graph, run, device=None):
    world = graph.n_nodes
    if conf.data.startswith("synthetic"):
        n_tokens = 33278
        train = SyntheticTokens(n_tokens, conf.synthetic_size or 2_088_628, conf.manual_seed)
        val = SyntheticTokens(n_tokens, max(10000, (conf.synthetic_size or 2_088_628) // 10), conf.manual_seed + 1)
        train_ids, val_ids = train.stream, val.stream
    else:
        corpus = Corpus(os.path.join(conf.data_dir, conf.data))
        n_tokens, train_ids, val_ids = len(corpus.dictionary), corpus.train, corpus.valid
        if conf.rnn_use_pretrained_emb:
            from .embeddings import find_vector_file, load_vectors

            vec_file = find_vector_file(os.path.join(conf.data_dir, conf.data))
            if vec_file is not None:
                vectors, found = load_vectors(vec_file, corpus.dictionary.word2idx, seed=conf.manual_seed)
                print(f"=> {found} / {n_tokens} words initialised from {vec_file}")
    gb = conf.batch_size * world
    vectors = locals().get("vectors")

    def batchify(ids):
        n = ids.numel() // gb
        return ids[: n * gb].view(gb, n).t().contiguous()

    train_loader = BPTTIterator(batchify(train_ids), conf.rnn_bptt_len, device)
    val_loader = BPTTIterator(batchify(val_ids), conf.rnn_bptt_len, device)
    run.num_batches_train_per_device_per_epoch = len(train_loader)
    run.num_whole_train_batches_per_worker = len(train_loader) * conf.num_epochs
    run.num_warmup_train_batches_per_worker = len(train_loader) * conf.lr_warmup_epochs
    run.num_iterations_per_worker = conf.num_iterations // world
    run.num_batches_val_per_device_per_epoch = len(val_loader)
    return {"n_tokens": n_tokens, "train_loader": train_loader, "val_loader": val_loader,
            "emb_size": None if vectors is None else vectors.size(1), "vectors": vectors}


def define_dataset(conf, graph, run, force_shuffle=False, device=None):
    if "rnn_lm" in conf.arch:
        return define_nlp_dataset(conf, graph, run, device)
    return define_cv_dataset(conf, graph, run, force_shuffle)
