"""Image augmentation toolkit, batched and device-resident.

The reference augments one PIL image at a time inside DataLoader worker processes
(``dl_code/pcode/datasets/loader/preprocess_toolkit.py:21-215``: scale / centre crop, pad +
random crop + flip, inception random-resized crop, colour jitter in random order, AlexNet-style
PCA lighting, normalisation).  Here every transform takes a float batch ``[B, C, H, W]`` in
[0, 1] on any device and draws one set of random parameters per image from a seeded generator,
so a whole batch is augmented by a handful of kernels after the host-to-device copy and the
DataLoader workers only decode.  ``get_transform`` returns the same recipes by dataset name;
``per_sample`` adapts a batch transform to the ``transform=`` argument of a dataset.
"""
from __future__ import annotations

import math
from typing import Callable, Optional, Sequence

import torch
import torch.nn.functional as F

IMAGENET_STATS = {"mean": [0.485, 0.456, 0.406], "std": [0.229, 0.224, 0.225]}
CIFAR10_STATS = {"mean": [0.4914, 0.4822, 0.4465], "std": [0.2023, 0.1994, 0.2010]}
IMAGENET_PCA = {
    "eigval": torch.tensor([0.2175, 0.0188, 0.0045]),
    "eigvec": torch.tensor([[-0.5675, 0.7192, 0.4009], [-0.5808, -0.0045, -0.8140], [-0.5836, -0.6948, 0.4203]]),
}
GRAY_WEIGHTS = (0.299, 0.587, 0.114)


def _rand(shape, gen, device):
    """Uniform draws from ``gen`` (on the generator's own device), delivered on ``device``."""
    if gen is None:
        return torch.rand(shape, device=device)
    return torch.rand(shape, generator=gen, device=gen.device).to(device)


class Transform:
    """Base class: ``__call__(batch, generator=None) -> batch``."""

    def __call__(self, x: torch.Tensor, generator: Optional[torch.Generator] = None) -> torch.Tensor:
        raise NotImplementedError


class Compose(Transform):
    def __init__(self, transforms: Sequence[Transform]):
        self.transforms = list(transforms)

    def __call__(self, x, generator=None):
        for t in self.transforms:
            x = t(x, generator)
        return x


class Normalize(Transform):
    def __init__(self, mean, std):
        self.mean, self.std = torch.tensor(mean).view(1, -1, 1, 1), torch.tensor(std).view(1, -1, 1, 1)

    def __call__(self, x, generator=None):
        return (x - self.mean.to(x)) / self.std.to(x)


class Resize(Transform):
    """Shorter side to ``size`` (bilinear, antialiased), aspect ratio kept."""

    def __init__(self, size: int):
        self.size = int(size)

    def __call__(self, x, generator=None):
        h, w = x.shape[-2:]
        if min(h, w) == self.size:
            return x
        s = self.size / min(h, w)
        return F.interpolate(x, size=(max(self.size, round(h * s)), max(self.size, round(w * s))), mode="bilinear",
                             align_corners=False, antialias=True)


class CenterCrop(Transform):
    def __init__(self, size: int):
        self.size = int(size)

    def __call__(self, x, generator=None):
        h, w = x.shape[-2:]
        t, l = (h - self.size) // 2, (w - self.size) // 2
        return x[..., t:t + self.size, l:l + self.size]


def _gather_windows(x, top, left, size):
    """One ``size x size`` window per image at (top[b], left[b]) with a single gather."""
    b, c, h, w = x.shape
    ar = torch.arange(size, device=x.device)
    rows = (top.view(b, 1) + ar.view(1, size)).clamp_(0, h - 1)      # [B, S]
    cols = (left.view(b, 1) + ar.view(1, size)).clamp_(0, w - 1)
    idx = rows.view(b, size, 1) * w + cols.view(b, 1, size)          # [B, S, S]
    flat = x.reshape(b, c, h * w)
    return flat.gather(2, idx.view(b, 1, size * size).expand(b, c, size * size)).view(b, c, size, size)


class RandomCrop(Transform):
    """Zero-pad by ``padding`` and cut a random ``size x size`` window per image."""

    def __init__(self, size: int, padding: int = 0):
        self.size, self.padding = int(size), int(padding)

    def __call__(self, x, generator=None):
        if self.padding:
            x = F.pad(x, [self.padding] * 4)
        b, _, h, w = x.shape
        top = (_rand((b,), generator, x.device) * (h - self.size + 1)).long()
        left = (_rand((b,), generator, x.device) * (w - self.size + 1)).long()
        return _gather_windows(x, top, left, self.size)


class RandomHorizontalFlip(Transform):
    def __call__(self, x, generator=None):
        flip = _rand((x.shape[0],), generator, x.device) < 0.5
        return torch.where(flip.view(-1, 1, 1, 1), x.flip(-1), x)


class RandomResizedCrop(Transform):
    """Inception crop: a random area fraction in ``scale`` and aspect ratio in ``ratio`` per image,
    resampled to ``size x size`` with one ``grid_sample`` for the whole batch."""

    def __init__(self, size: int, scale=(0.08, 1.0), ratio=(3.0 / 4.0, 4.0 / 3.0)):
        self.size, self.scale, self.ratio = int(size), scale, ratio

    def __call__(self, x, generator=None):
        b, _, h, w = x.shape
        dev = x.device
        area = self.scale[0] + _rand((b,), generator, dev) * (self.scale[1] - self.scale[0])
        logr = math.log(self.ratio[0]) + _rand((b,), generator, dev) * (math.log(self.ratio[1]) - math.log(self.ratio[0]))
        ar = torch.exp(logr)
        cw = torch.sqrt(area * ar).clamp(max=1.0)      # width / height of the crop as fractions of the image
        ch = torch.sqrt(area / ar).clamp(max=1.0)
        cx = (_rand((b,), generator, dev) * (1 - cw) + cw / 2) * 2 - 1     # crop centre in [-1, 1]
        cy = (_rand((b,), generator, dev) * (1 - ch) + ch / 2) * 2 - 1
        theta = torch.zeros(b, 2, 3, device=dev, dtype=x.dtype)
        theta[:, 0, 0], theta[:, 0, 2], theta[:, 1, 1], theta[:, 1, 2] = cw, cx, ch, cy
        grid = F.affine_grid(theta, (b, x.shape[1], self.size, self.size), align_corners=False)
        return F.grid_sample(x, grid, mode="bilinear", padding_mode="border", align_corners=False)


def grayscale(x):
    w = torch.tensor(GRAY_WEIGHTS, device=x.device, dtype=x.dtype).view(1, 3, 1, 1)
    return (x * w).sum(1, keepdim=True).expand_as(x)


class Brightness(Transform):
    def __init__(self, var):
        self.var = var

    def __call__(self, x, generator=None):
        a = _rand((x.shape[0], 1, 1, 1), generator, x.device) * self.var
        return x * (1 - a)            # lerp towards black


class Contrast(Transform):
    def __init__(self, var):
        self.var = var

    def __call__(self, x, generator=None):
        a = _rand((x.shape[0], 1, 1, 1), generator, x.device) * self.var
        mean = grayscale(x)[:, :1].mean(dim=(2, 3), keepdim=True)
        return torch.lerp(x, mean.expand_as(x), a)


class Saturation(Transform):
    def __init__(self, var):
        self.var = var

    def __call__(self, x, generator=None):
        a = _rand((x.shape[0], 1, 1, 1), generator, x.device) * self.var
        return torch.lerp(x, grayscale(x), a)


class RandomOrder(Transform):
    """Applies its transforms in an order drawn once per call."""

    def __init__(self, transforms):
        self.transforms = list(transforms)

    def __call__(self, x, generator=None):
        if generator is None:
            order = torch.randperm(len(self.transforms))
        else:
            order = torch.randperm(len(self.transforms), generator=generator, device=generator.device)
        for i in order.tolist():
            x = self.transforms[i](x, generator)
        return x


class ColorJitter(RandomOrder):
    def __init__(self, brightness=0.4, contrast=0.4, saturation=0.4):
        ts = []
        if brightness:
            ts.append(Brightness(brightness))
        if contrast:
            ts.append(Contrast(contrast))
        if saturation:
            ts.append(Saturation(saturation))
        super().__init__(ts)


class Lighting(Transform):
    """PCA lighting noise: ``rgb += eigvec (alpha * eigval)`` with ``alpha ~ N(0, alphastd)`` per image."""

    def __init__(self, alphastd, eigval=None, eigvec=None):
        self.alphastd = alphastd
        self.eigval = IMAGENET_PCA["eigval"] if eigval is None else eigval
        self.eigvec = IMAGENET_PCA["eigvec"] if eigvec is None else eigvec

    def __call__(self, x, generator=None):
        if self.alphastd == 0:
            return x
        if generator is None:
            alpha = torch.randn(x.shape[0], 3, device=x.device, dtype=x.dtype)
        else:
            alpha = torch.randn(x.shape[0], 3, generator=generator, device=generator.device, dtype=x.dtype).to(x.device)
        alpha = alpha * self.alphastd
        rgb = (alpha * self.eigval.to(x)).matmul(self.eigvec.to(x).t())       # [B, 3]
        return x + rgb.view(-1, 3, 1, 1)


# ---- recipes -------------------------------------------------------------------------------------------------
def _norm(normalize):
    return [Normalize(**normalize)] if normalize is not None else []


def scale_crop(input_size, scale_size=None, normalize=IMAGENET_STATS):
    ts = [CenterCrop(input_size)] + _norm(normalize)
    return Compose(([Resize(scale_size)] if scale_size and scale_size != input_size else []) + ts)


def scale_random_crop(input_size, scale_size=None, normalize=IMAGENET_STATS):
    ts = [RandomCrop(input_size)] + _norm(normalize)
    return Compose(([Resize(scale_size)] if scale_size and scale_size != input_size else []) + ts)


def pad_random_crop(input_size, scale_size=None, normalize=IMAGENET_STATS):
    padding = int(((scale_size or input_size) - input_size) / 2)
    return Compose([RandomCrop(input_size, padding=padding), RandomHorizontalFlip()] + _norm(normalize))


def inception_preprocess(input_size, normalize=IMAGENET_STATS):
    return Compose([RandomResizedCrop(input_size), RandomHorizontalFlip()] + _norm(normalize))


def inception_color_preprocess(input_size, normalize=IMAGENET_STATS):
    return Compose([RandomResizedCrop(input_size), RandomHorizontalFlip(), ColorJitter(0.4, 0.4, 0.4), Lighting(0.1)]
                   + _norm(normalize))


def get_transform(name="imagenet", input_size=None, scale_size=None, normalize=None, augment=True, color_process=False):
    """The reference's recipe table (``preprocess_toolkit.py:75-123``) by dataset name."""
    if "imagenet" in name:
        normalize = normalize or IMAGENET_STATS
        small = "downsampled" in name
        scale_size = scale_size or (36 if small else 256)
        input_size = input_size or (32 if small else 224)
        if augment:
            fn = inception_color_preprocess if color_process else inception_preprocess
            return fn(input_size, normalize=normalize)
        return scale_crop(input_size, scale_size, normalize)
    if "cifar" in name or name in ("svhn", "stl10"):
        normalize = normalize or (CIFAR10_STATS if name == "cifar10" else IMAGENET_STATS)
        input_size = input_size or (96 if name == "stl10" else 32)
        if augment:
            return pad_random_crop(input_size, scale_size or input_size + 8, normalize)
        return scale_crop(input_size, scale_size or input_size, normalize)
    if name == "mnist":
        normalize = normalize or {"mean": [0.5], "std": [0.5]}
        input_size = input_size or 28
        if augment:
            return pad_random_crop(input_size, scale_size or 32, normalize)
        return scale_crop(input_size, scale_size or input_size, normalize)
    raise NotImplementedError(name)


def per_sample(transform: Transform, generator: Optional[torch.Generator] = None) -> Callable:
    """Adapter for ``Dataset(transform=...)``: accepts one ``[C, H, W]`` float tensor or a PIL image."""

    def apply(img):
        if not torch.is_tensor(img):
            import numpy as np

            arr = np.asarray(img)
            if arr.ndim == 2:
                arr = arr[:, :, None]
            img = torch.from_numpy(arr.copy()).permute(2, 0, 1).float().div_(255)
        return transform(img.unsqueeze(0), generator)[0]

    return apply


class DeviceAugment:
    """Augments each training batch on the device it was copied to: ``aug(batch_uint8_or_float)``.
    uint8 input is scaled to [0, 1] first.  One seeded generator per rank keeps runs reproducible."""

    def __init__(self, transform: Transform, device, seed: int = 0):
        self.transform, self.device = transform, torch.device(device)
        self.generator = torch.Generator(device=self.device)
        self.generator.manual_seed(int(seed))

    def __call__(self, batch: torch.Tensor) -> torch.Tensor:
        x = batch.to(self.device, non_blocking=True)
        if x.dtype == torch.uint8:
            x = x.float().div_(255)
        return self.transform(x, self.generator)
