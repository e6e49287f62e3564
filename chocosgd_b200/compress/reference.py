"""Plain-PyTorch restatement of the four compression operators and their wire formats.

These functions are (a) the oracle the CUDA kernels are tested against, (b) the
implementation used on CPU / Gloo ranks and by the ``--gossip_impl nccl`` baseline
path.  Behaviour follows ``dl_code/pcode/utils/sparsification.py:17-163`` with the
deliberate differences listed next to each function.

Wire formats (all payloads are 1-d ``int32`` tensors; floats are bit-cast):

=========  ==========================================================================
sign       ``T`` fp32 per-tensor L1 norms, then one word per 32 flat positions of the
           *padded* arena, bit ``b`` of word ``w`` set iff ``d[32 w + b] < 0``
top-k      ``sum(k)`` int32 tensor-local indices, then ``sum(k)`` fp32 values
random-k   ``sum(k)`` fp32 values only: both ends regenerate the indices from
           ``(seed, step, tensor)`` with the same keyed permutation
qsgd       ``T`` fp32 per-tensor L2 norms, then for every group of 32 flat positions
           ``nbits + 1`` bit-plane words (level bit 0 .. nbits-1, then the sign plane)
=========  ==========================================================================
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch

from .segments import Segments

_M32 = 0xFFFFFFFF


# --------------------------------------------------------------------------------------
# counter-based hashing shared (bit for bit) with the CUDA kernels
# --------------------------------------------------------------------------------------
def mix32(x: torch.Tensor) -> torch.Tensor:
    """32-bit avalanche hash on int64 tensors holding uint32 values."""
    x = x & _M32
    x = x ^ (x >> 16)
    x = (x * 0x7FEB352D) & _M32
    x = x ^ (x >> 15)
    x = (x * 0x846CA68B) & _M32
    x = x ^ (x >> 16)
    return x


def _mix32_int(x: int) -> int:
    x &= _M32
    x ^= x >> 16
    x = (x * 0x7FEB352D) & _M32
    x ^= x >> 15
    x = (x * 0x846CA68B) & _M32
    x ^= x >> 16
    return x


def counter_uniform(seed: int, step: int, positions: torch.Tensor) -> torch.Tensor:
    """U[0,1) with 24 random bits, a pure function of (seed, step, flat position)."""
    base = _mix32_int((step * 0x9E3779B9 + 0x7F4A7C15) & _M32) ^ (seed & _M32)
    h = mix32(positions.to(torch.int64) ^ base)
    return (h >> 8).to(torch.float32) * (1.0 / 16777216.0)


def feistel_keys(seed: int, step: int, seg: int) -> List[int]:
    return [
        _mix32_int((seed & _M32) ^ _mix32_int((step * 0x9E3779B9 + seg * 0x85EBCA6B + r * 0xC2B2AE35 + 1) & _M32))
        for r in range(4)
    ]


def feistel_half_bits(n: int) -> int:
    bits = max(2, int(math.ceil(math.log2(n))) if n > 1 else 2)
    if bits % 2:
        bits += 1
    return bits // 2


def random_k_indices(n: int, k: int, seed: int, step: int, seg: int, device=None) -> torch.Tensor:
    """First ``k`` images of a keyed pseudo-random permutation of ``[0, n)``.

    A 4-round balanced Feistel network over the next even power of two, cycle-walked
    back into range, is a bijection on ``[0, n)``: the ``k`` indices are distinct, like
    ``np.random.choice(n, k, replace=False)`` in the reference
    (``dl_code/pcode/utils/sparsification.py:40-49``), but they are a pure function of
    ``(seed, step, tensor)`` so the receiver can regenerate them and no index travels."""
    if n == 1:
        return torch.zeros(k, dtype=torch.int64, device=device)
    hb = feistel_half_bits(n)
    mask = (1 << hb) - 1
    keys = feistel_keys(seed, step, seg)
    v = torch.arange(k, dtype=torch.int64, device=device)
    out = torch.full_like(v, -1)
    todo = torch.ones_like(v, dtype=torch.bool)
    for _ in range(64):
        left, right = v >> hb, v & mask
        for r in range(4):
            left, right = right, left ^ (mix32(right ^ keys[r]) & mask)
        v = (left << hb) | right
        done = todo & (v < n)
        out = torch.where(done, v, out)
        todo = todo & ~done
        if not bool(todo.any()):
            break
    assert not bool(todo.any())
    return out


# --------------------------------------------------------------------------------------
# element-level operators (one tensor)
# --------------------------------------------------------------------------------------
def top_k(x: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Values and indices of the ``k`` largest ``|x|``; ties resolved towards the lowest
    index and results ordered by index (``torch.topk(sorted=False)`` in the reference
    leaves both unspecified, ``dl_code/pcode/utils/sparsification.py:18-31``)."""
    flat = x.reshape(-1)
    order = torch.sort(flat.abs(), descending=True, stable=True).indices[:k]
    idx = torch.sort(order).values
    return flat[idx], idx


def qsgd_levels_from(quantize_level: Optional[int], qsgd_levels: Optional[int]) -> int:
    """``s``.  ``quantize_level`` counts bits (s = 2^b - 1, ``sparsification.py:114-117``);
    ``qsgd_levels`` is ``s`` itself (``convex_code/logistic.py:13-23``)."""
    if qsgd_levels is not None:
        return int(qsgd_levels)
    return 2 ** int(quantize_level) - 1


def qsgd_nbits(s: int) -> int:
    return max(1, int(math.ceil(math.log2(s + 1))))


def qsgd_scale(n: int, s: int, is_biased: bool) -> float:
    if not is_biased:
        return 1.0
    return 1.0 / (min(n / (s * s), math.sqrt(n) / s) + 1.0)


def qsgd_quantize(x: torch.Tensor, s: int, u: torch.Tensor):
    """-> (norm, integer levels, negative mask).  A zero tensor quantizes to zeros
    (the reference divides 0/0 there, ``dl_code/pcode/utils/sparsification.py:88-89``)."""
    flat = x.reshape(-1).to(torch.float32)
    norm = torch.sqrt(torch.sum(flat * flat))
    safe = torch.where(norm > 0, norm, torch.ones_like(norm))
    lvl = flat.abs() * (float(s) / safe)  # one fp32 division per tensor, one multiply per element
    fl = torch.floor(lvl)
    lv = fl + (u < (lvl - fl)).to(torch.float32)
    lv = torch.where(norm > 0, lv, torch.zeros_like(lv))
    return norm, lv.to(torch.int32), flat < 0


def qsgd_dequantize(norm, levels, neg, s: int, scale: float) -> torch.Tensor:
    mag = (scale * norm / s) * levels.to(torch.float32)
    return torch.where(neg, -mag, mag)


def pack_bits(neg: torch.Tensor) -> torch.Tensor:
    """bool[32 m] -> int32[m]; bit b of word w = neg[32 w + b].

    The reference packs row-strided through the external ``bit2byte`` extension
    (``dl_code/pcode/utils/sparsification.py:129-145``); the layout is private to the
    two ends of a link, so a contiguous layout (one warp ballot per word) is used."""
    m = neg.numel() // 32
    w = neg.reshape(m, 32).to(torch.int64)
    shifts = torch.arange(32, device=neg.device, dtype=torch.int64)
    words = (w << shifts).sum(dim=1)
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words)
    return words.to(torch.int32)


def unpack_bits(words: torch.Tensor) -> torch.Tensor:
    """int32[m] -> bool[32 m]."""
    w = words.to(torch.int64) & _M32
    shifts = torch.arange(32, device=words.device, dtype=torch.int64)
    return ((w.unsqueeze(1) >> shifts) & 1).to(torch.bool).reshape(-1)


def f2i(x: torch.Tensor) -> torch.Tensor:
    return x.contiguous().view(torch.int32)


def i2f(x: torch.Tensor) -> torch.Tensor:
    return x.contiguous().view(torch.float32)


# --------------------------------------------------------------------------------------
# segmented codecs on flat arenas
# --------------------------------------------------------------------------------------
class Codec:
    """Per-tensor compressor over a flat, segment-padded fp32 buffer."""

    name = "identity"
    is_sparse = False

    def __init__(self, segments: Segments):
        self.seg = segments

    def payload_words(self) -> int:
        return self.seg.total

    def n_bits(self) -> int:
        """Bits *accounted* per message, same formulas as the reference's loggers."""
        return 32 * self.seg.n_elements

    def compress(self, d: torch.Tensor, step: int = 0, src: int = 0) -> torch.Tensor:
        return f2i(d)

    def decompress(self, payload: torch.Tensor, step: int = 0, src: int = 0) -> torch.Tensor:
        return i2f(payload).clone()

    def sparse(self, payload: torch.Tensor, step: int = 0, src: int = 0):
        raise NotImplementedError

    def roundtrip(self, d: torch.Tensor, step: int = 0, src: int = 0) -> torch.Tensor:
        return self.decompress(self.compress(d, step, src), step, src)


class SignCodec(Codec):
    """q_t = ||d_t||_1 / n_t * sign(d_t), sign(0) = +1 (``parallel_choco_v.py:476-558``)."""

    name = "sign"

    def payload_words(self) -> int:
        return self.seg.n_segments + self.seg.total // 32

    def n_bits(self) -> int:
        return 32 * self.seg.n_segments + 32 * int(math.ceil(self.seg.n_elements / 32))

    def compress(self, d, step=0, src=0):
        norms = torch.stack([d[s].abs().sum() for s in self.seg.slices()]).to(torch.float32)
        return torch.cat([f2i(norms), pack_bits(d < 0)])

    def decompress(self, payload, step=0, src=0):
        t = self.seg.n_segments
        norms = i2f(payload[:t])
        neg = unpack_bits(payload[t:])
        out = torch.zeros(self.seg.total, dtype=torch.float32, device=payload.device)
        for i, s in enumerate(self.seg.slices()):
            mag = norms[i] / self.seg.sizes[i]
            out[s] = torch.where(neg[s], -mag, mag)
        return out


class TopKCodec(Codec):
    name = "compress_top_k"
    is_sparse = True

    def __init__(self, segments: Segments, compress_ratio: float):
        super().__init__(segments)
        self.ks = segments.keep_counts(compress_ratio)
        self.sum_k = int(sum(self.ks))

    def payload_words(self):
        return 2 * self.sum_k

    def n_bits(self):
        return 64 * self.sum_k

    def compress(self, d, step=0, src=0):
        vals, idxs = [], []
        for s, k in zip(self.seg.slices(), self.ks):
            v, i = top_k(d[s], k)
            vals.append(v)
            idxs.append(i.to(torch.int32))
        return torch.cat([torch.cat(idxs), f2i(torch.cat(vals))])

    def sparse(self, payload, step=0, src=0):
        """-> (flat positions int64, values fp32)."""
        idx = payload[: self.sum_k].to(torch.int64)
        val = i2f(payload[self.sum_k:])
        base = torch.cat(
            [torch.full((k,), off, dtype=torch.int64, device=payload.device) for off, k in zip(self.seg.offsets, self.ks)]
        )
        return idx + base, val

    def decompress(self, payload, step=0, src=0):
        pos, val = self.sparse(payload, step, src)
        out = torch.zeros(self.seg.total, dtype=torch.float32, device=payload.device)
        out[pos] = val
        return out


class RandomKCodec(TopKCodec):
    """Always the biased variant (no n/k rescale): the reference never forwards
    ``is_biased`` to ``get_random_k`` (``dl_code/pcode/utils/sparsification.py:59-60``)."""

    name = "compress_random_k"

    def __init__(self, segments, compress_ratio, seed: int = 1234):
        super().__init__(segments, compress_ratio)
        self.seed = seed

    def payload_words(self):
        return self.sum_k

    def _positions(self, step, device, src=0):
        return torch.cat(
            [
                random_k_indices(n, k, self.seed + 7919 * src, step, t, device) + off
                for t, (n, k, off) in enumerate(zip(self.seg.sizes, self.ks, self.seg.offsets))
            ]
        )

    def compress(self, d, step=0, src=0):
        return f2i(d[self._positions(step, d.device, src)])

    def sparse(self, payload, step=0, src=0):
        return self._positions(step, payload.device, src), i2f(payload)


class QSGDCodec(Codec):
    name = "quantize_qsgd"

    def __init__(self, segments, s: int, is_biased: bool = False, seed: int = 1234):
        super().__init__(segments)
        self.s = int(s)
        self.nbits = qsgd_nbits(self.s)
        self.is_biased = is_biased
        self.seed = seed
        self.accounted_level = None  # bits per element used by n_bits(); set by the factory

    def payload_words(self):
        return self.seg.n_segments + (self.seg.total // 32) * (self.nbits + 1)

    def n_bits(self):
        lvl = self.accounted_level if self.accounted_level is not None else self.nbits
        return int(self.seg.n_elements * lvl)

    def uniforms(self, step, device, src=0):
        return counter_uniform(self.seed + 7919 * src, step, torch.arange(self.seg.total, device=device))

    def compress(self, d, step=0, src=0, u: Optional[torch.Tensor] = None):
        u = self.uniforms(step, d.device, src) if u is None else u
        norms = torch.zeros(self.seg.n_segments, dtype=torch.float32, device=d.device)
        levels = torch.zeros(self.seg.total, dtype=torch.int32, device=d.device)
        for i, s in enumerate(self.seg.slices()):
            nrm, lv, _ = qsgd_quantize(d[s], self.s, u[s])
            norms[i] = nrm
            levels[s] = lv
        planes = [pack_bits(((levels >> b) & 1).to(torch.bool)) for b in range(self.nbits)]
        planes.append(pack_bits(d < 0))
        body = torch.stack(planes, dim=1).reshape(-1)  # group-major: nbits+1 words per 32 elements
        return torch.cat([f2i(norms), body])

    def decompress(self, payload, step=0, src=0):
        t = self.seg.n_segments
        norms = i2f(payload[:t])
        body = payload[t:].reshape(-1, self.nbits + 1)
        levels = torch.zeros(self.seg.total, dtype=torch.int32, device=payload.device)
        for b in range(self.nbits):
            levels |= unpack_bits(body[:, b].contiguous()).to(torch.int32) << b
        neg = unpack_bits(body[:, self.nbits].contiguous())
        out = torch.zeros(self.seg.total, dtype=torch.float32, device=payload.device)
        for i, s in enumerate(self.seg.slices()):
            scale = qsgd_scale(self.seg.sizes[i], self.s, self.is_biased)
            out[s] = qsgd_dequantize(norms[i], levels[s], neg[s], self.s, scale)
        return out


def make_codec(
    segments: Segments,
    comm_op: Optional[str],
    compress_ratio: Optional[float] = None,
    quantize_level: Optional[int] = None,
    qsgd_levels: Optional[int] = None,
    is_biased: bool = False,
    seed: int = 1234,
) -> Codec:
    if comm_op is None:
        return Codec(segments)
    if comm_op == "sign":
        return SignCodec(segments)
    if comm_op == "compress_top_k":
        return TopKCodec(segments, compress_ratio)
    if comm_op == "compress_random_k":
        return RandomKCodec(segments, compress_ratio, seed)
    if comm_op == "quantize_qsgd":
        if qsgd_levels is None and quantize_level is not None and int(quantize_level) >= 32:
            return Codec(segments)  # quantize_level == 32 is the identity (sparsification.py:118-119)
        c = QSGDCodec(segments, qsgd_levels_from(quantize_level, qsgd_levels), is_biased, seed)
        c.accounted_level = quantize_level if quantize_level is not None else None
        return c
    raise NotImplementedError(comm_op)
