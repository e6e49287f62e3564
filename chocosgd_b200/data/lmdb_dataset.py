"""Datasets over packed record files (``data/serialize.py``): encoded images, or feature vectors
(epsilon / rcv1), addressed by index (``dl_code/pcode/datasets/loader/utils.py:30-204``,
``imagenet_folder.py:8-19``, ``epsilon_or_rcv1_folder.py:6-8``)."""
from __future__ import annotations

import io

import numpy as np
import torch
from torch.utils.data import Dataset

from .serialize import RecordStore, loads  # noqa: F401  (loads re-exported)


class LMDBImageDataset(Dataset):
    def __init__(self, path, name, train=True, transform=None, is_image=True):
        self.store = RecordStore(path)
        self.transform, self.is_image, self.name, self.train = transform, is_image, name, train

    def __len__(self):
        return len(self.store)

    def __getitem__(self, index):
        data, target = self.store[index][:2]
        if self.is_image:
            from PIL import Image

            img = Image.open(io.BytesIO(data)).convert("RGB")
            if self.transform is not None:
                return self.transform(img), int(target)
            return torch.from_numpy(np.asarray(img).copy()).permute(2, 0, 1).float().div_(255), int(target)
        return torch.from_numpy(np.array(data, dtype=np.float32)), int(target)


def define_epsilon_or_rcv1_folder(root):
    """Feature-vector dataset (``epsilon_<split>.lmdb`` / ``rcv1_<split>.lmdb``)."""
    return LMDBImageDataset(root, "features", is_image=False)
