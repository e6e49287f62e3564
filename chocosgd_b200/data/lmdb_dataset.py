"""LMDB-packed image / feature datasets (``dl_code/pcode/datasets/loader/utils.py:30-204``,
``imagenet_folder.py``, ``epsilon_or_rcv1_folder.py``): records are msgpack / pyarrow
serialised ``(encoded image | feature vector, label)`` pairs keyed by index, with the key
list under ``__keys__`` and the count under ``__len__``.  The ``lmdb`` package is optional
and imported on first use."""
from __future__ import annotations

import io
import pickle

import numpy as np
import torch
from torch.utils.data import Dataset


def loads(buf):
    try:
        import msgpack

        return msgpack.loads(buf, raw=False)
    except Exception:
        return pickle.loads(buf)


class LMDBImageDataset(Dataset):
    def __init__(self, path, name, train=True, transform=None, is_image=True):
        try:
            import lmdb
        except ImportError as e:
            raise RuntimeError("--use_lmdb_data needs the 'lmdb' package") from e
        self.env = lmdb.open(path, subdir=False, readonly=True, lock=False, readahead=False, meminit=False)
        with self.env.begin(write=False) as txn:
            self.length = loads(txn.get(b"__len__"))
            self.keys = loads(txn.get(b"__keys__"))
        self.transform, self.is_image, self.name = transform, is_image, name

    def __len__(self):
        return self.length

    def __getitem__(self, index):
        with self.env.begin(write=False) as txn:
            rec = loads(txn.get(self.keys[index]))
        data, target = rec[0], rec[1]
        if self.is_image:
            from PIL import Image

            img = Image.open(io.BytesIO(data)).convert("RGB")
            if self.transform is not None:
                img = self.transform(img)
            else:
                img = torch.from_numpy(np.asarray(img)).permute(2, 0, 1).float().div_(255)
            return img, int(target)
        return torch.as_tensor(np.asarray(data, dtype=np.float32)), int(target)
