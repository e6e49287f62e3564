"""Stand-alone packing ops: native replacement of the external ``bit2byte`` extension.

``sign_pack(x) -> int32[ceil(n/32)]`` sets bit ``b`` of word ``w`` iff ``x[32 w + b] < 0``;
``sign_unpack(words, n, scale)`` returns ``+scale / -scale`` (zero decodes to ``+scale``).
CUDA tensors run the ballot kernel, CPU tensors the C++ twin.  ``SignCompressor`` keeps the
reference's class interface (``dl_code/pcode/utils/sparsification.py:126-163``)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def sign_pack(x: torch.Tensor) -> torch.Tensor:
    x = x.contiguous().view(-1).to(torch.float32)
    n = x.numel()
    words = torch.empty((n + 31) // 32, dtype=torch.int32, device=x.device)
    lib = _lib.load()
    if x.is_cuda:
        _lib.check(lib.sign_pack(_lib.ptr(x), n, _lib.ptr(words), _lib.stream_ptr()), "sign_pack")
    else:
        lib.cpu_sign_pack(_lib.ptr(x), n, _lib.ptr(words))
    return words


def sign_unpack(words: torch.Tensor, n: int, scale: float = 1.0) -> torch.Tensor:
    words = words.contiguous()
    out = torch.empty(n, dtype=torch.float32, device=words.device)
    lib = _lib.load()
    if words.is_cuda:
        _lib.check(lib.sign_unpack(_lib.ptr(words), n, _lib.ptr(out), float(scale), _lib.stream_ptr()), "sign_unpack")
    else:
        lib.cpu_sign_unpack(_lib.ptr(words), n, _lib.ptr(out), float(scale))
    return out


def sign_l1_compress(x: torch.Tensor):
    """Sign words and L1 norm of one CUDA fp32 tensor in a single kernel: ``(int32 words, 0-d norm)``."""
    x = x.contiguous().view(-1)
    assert x.is_cuda and x.dtype == torch.float32
    n = x.numel()
    lib = _lib.load()
    words = torch.empty((n + 31) // 32, dtype=torch.int32, device=x.device)
    norm = torch.empty(1, dtype=torch.float32, device=x.device)
    scratch = torch.empty(lib.sign_l1_scratch_bytes(n) // 4, dtype=torch.int32, device=x.device)
    _lib.check(lib.sign_l1_compress(_lib.ptr(x), n, _lib.ptr(words), _lib.ptr(norm), _lib.ptr(scratch),
                                    _lib.stream_ptr()), "sign_l1_compress")
    return words, norm[0]


def cpu_top_k(x: torch.Tensor, k: int):
    x = x.contiguous().view(-1).to(torch.float32).cpu()
    idx = torch.empty(k, dtype=torch.int32)
    val = torch.empty(k, dtype=torch.float32)
    _lib.load().cpu_top_k(_lib.ptr(x), x.numel(), k, _lib.ptr(idx), _lib.ptr(val))
    return val, idx.to(torch.int64)


def cpu_random_k_indices(n: int, k: int, seed: int, step: int, seg: int) -> torch.Tensor:
    idx = torch.empty(k, dtype=torch.int32)
    _lib.load().cpu_random_k_indices(n, k, seed & 0xFFFFFFFF, step, seg, _lib.ptr(idx))
    return idx.to(torch.int64)


def cpu_counter_uniform(seed: int, step: int, n: int) -> torch.Tensor:
    out = torch.empty(n, dtype=torch.float32)
    _lib.load().cpu_counter_uniform(seed & 0xFFFFFFFF, step, n, _lib.ptr(out))
    return out


class SignCompressor:
    """Interface of the reference's ``SignCompressor``: ``compress`` returns the packed sign
    words and the original size, ``uncompress`` the +/-1 tensor."""

    def packing(self, src_tensor):
        flat = src_tensor.reshape(-1)
        return sign_pack(flat), flat.numel()

    def unpacking(self, src_tensor, src_tensor_size):
        return sign_unpack(src_tensor, src_tensor_size, 1.0)

    def compress(self, src_tensor):
        return self.packing(src_tensor)

    def uncompress(self, src_tensor, src_tensor_size):
        return self.unpacking(src_tensor, src_tensor_size)

    def majority_vote(self, src_tensor_list):
        voter = torch.stack(list(src_tensor_list)).sum(dim=0)
        return torch.where(voter >= 0, torch.ones_like(voter), -torch.ones_like(voter))
