"""On-disk vision datasets through torchvision (cifar10/100, mnist, stl10, svhn, imagenet
folders, downsampled imagenet) with the reference's augmentations
(``dl_code/pcode/datasets/prepare_data.py:19-120``): CIFAR pad-4 random crop + horizontal
flip + per-channel normalisation; ImageNet random-resized-crop 224 + flip / resize 256 +
centre crop.  LMDB-packed datasets (``--use_lmdb_data``) are read by ``lmdb_dataset``."""
from __future__ import annotations

import os


def _tv():
    try:
        import torchvision
        import torchvision.transforms as T
    except Exception as e:  # pragma: no cover
        raise RuntimeError("torchvision is needed for on-disk vision datasets") from e
    return torchvision, T


def get_vision_dataset(name, root, split="train", use_lmdb=False, download=False):
    tv, T = _tv()
    train = split == "train"
    root = os.path.join(root, name)
    if use_lmdb:
        from .lmdb_dataset import LMDBImageDataset

        return LMDBImageDataset(os.path.join(root, "train.lmdb" if train else "val.lmdb"), name, train)
    if name in ("cifar10", "cifar100"):
        if name == "cifar10":
            norm = T.Normalize((0.4914, 0.4822, 0.4465), (0.2023, 0.1994, 0.2010))
            cls = tv.datasets.CIFAR10
        else:
            norm = T.Normalize((0.5071, 0.4867, 0.4408), (0.2675, 0.2565, 0.2761))
            cls = tv.datasets.CIFAR100
        tf = ([T.RandomHorizontalFlip(), T.RandomCrop((32, 32), 4)] if train else []) + [T.ToTensor(), norm]
        return cls(root=root, train=train, transform=T.Compose(tf), download=download)
    if name == "mnist":
        tf = T.Compose([T.ToTensor(), T.Normalize((0.1307,), (0.3081,))])
        return tv.datasets.MNIST(root=root, train=train, transform=tf, download=download)
    if name == "stl10":
        tf = ([T.RandomHorizontalFlip(), T.RandomCrop((96, 96), 4)] if train else []) + [
            T.ToTensor(), T.Normalize((0.5, 0.5, 0.5), (0.5, 0.5, 0.5))]
        return tv.datasets.STL10(root=root, split="train" if train else "test", transform=T.Compose(tf),
                                 download=download)
    if name == "svhn":
        tf = T.Compose([T.ToTensor(), T.Normalize((0.5, 0.5, 0.5), (0.5, 0.5, 0.5))])
        if train:
            from torch.utils.data import ConcatDataset

            return ConcatDataset([
                tv.datasets.SVHN(root=root, split="train", transform=tf, download=download),
                tv.datasets.SVHN(root=root, split="extra", transform=tf, download=download),
            ])
        return tv.datasets.SVHN(root=root, split="test", transform=tf, download=download)
    if "imagenet" in name:
        norm = T.Normalize(mean=[0.485, 0.456, 0.406], std=[0.229, 0.224, 0.225])
        if "downsampled" in name:
            tf = ([T.RandomHorizontalFlip(), T.RandomCrop((32, 32), 4)] if train else []) + [T.ToTensor(), norm]
        elif train:
            tf = [T.RandomResizedCrop(224), T.RandomHorizontalFlip(), T.ToTensor(), norm]
        else:
            tf = [T.Resize(256), T.CenterCrop(224), T.ToTensor(), norm]
        return tv.datasets.ImageFolder(os.path.join(root, "train" if train else "val"), T.Compose(tf))
    raise NotImplementedError(name)
