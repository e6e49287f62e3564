"""Compression operators.  ``reference`` holds the PyTorch oracles and the wire formats,
``segments`` the flat-arena segment table; the CUDA kernels live in ``ops``.

``SparsificationCompressor`` / ``QuantizationCompressor`` / ``SignCompressor`` and
``get_n_bits`` keep the reference's per-tensor API (``dl_code/pcode/utils/sparsification.py``)."""
from __future__ import annotations

import torch

from .reference import (Codec, QSGDCodec, RandomKCodec, SignCodec, TopKCodec, make_codec, qsgd_dequantize,
                        qsgd_quantize, qsgd_scale, random_k_indices, top_k)
from .segments import Segments


def get_n_bits(tensor: torch.Tensor) -> int:
    return 8 * tensor.nelement() * tensor.element_size()


class SparsificationCompressor:
    """Per-tensor top-k / random-k; ``compress_ratio`` is the fraction dropped."""

    def __init__(self, seed: int = 1234):
        self.seed, self._calls = seed, 0

    def get_top_k(self, x, ratio):
        k = max(1, int(x.nelement() * (1 - ratio)))
        return top_k(x, k)

    def get_mask(self, flatten_arr, indices):
        mask = torch.zeros_like(flatten_arr)
        mask[indices] = 1
        return mask.bool(), 1.0 - mask

    def get_random_k(self, x, ratio, is_biased=True):
        flat = x.reshape(-1)
        n = flat.nelement()
        k = max(1, int(n * (1 - ratio)))
        self._calls += 1
        idx = random_k_indices(n, k, self.seed, self._calls, 0, device=flat.device)
        vals = flat[idx]
        return (vals if is_biased else vals * (n / k)), idx

    def compress(self, arr, op, compress_ratio, is_biased):
        if "top_k" in op:
            return self.get_top_k(arr, compress_ratio)
        if "random_k" in op:
            return self.get_random_k(arr, compress_ratio)
        raise NotImplementedError(op)

    def uncompress(self, values, indices, selected_shapes, original_shapes):
        """Re-base tensor-local indices to flat offsets of the concatenated tensors."""
        out_v, out_i, off_sel, off_full = [], [], 0, 0
        for k, shape in zip(selected_shapes, original_shapes):
            n = shape[1] if isinstance(shape, (tuple, list)) and len(shape) == 2 and isinstance(shape[1], int) else int(
                torch.Size(shape).numel() if not isinstance(shape, int) else shape)
            out_v.append(values[off_sel:off_sel + k])
            out_i.append(indices[off_sel:off_sel + k].long() + off_full)
            off_sel += k
            off_full += n
        return torch.cat(out_v), torch.cat(out_i)


class QuantizationCompressor:
    def get_qsgd(self, x, s, is_biased=False):
        u = torch.rand_like(x.reshape(-1), dtype=torch.float32)
        norm, lv, neg = qsgd_quantize(x, s, u)
        return qsgd_dequantize(norm, lv, neg, s, qsgd_scale(x.nelement(), s, is_biased)).view_as(x)

    def compress(self, arr, op, quantize_level, is_biased):
        if quantize_level != 32:
            return self.get_qsgd(arr, 2 ** quantize_level - 1, is_biased)
        return arr

    def uncompress(self, arr):
        return arr


def SignCompressor():
    from ..ops.compress import SignCompressor as _S

    return _S()
