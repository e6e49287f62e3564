import math

import numpy as np
import pytest
import torch

from chocosgd_b200.compress.reference import (
    QSGDCodec, RandomKCodec, SignCodec, TopKCodec, counter_uniform, make_codec, pack_bits, qsgd_scale,
    random_k_indices, top_k, unpack_bits,
)
from chocosgd_b200.compress.segments import Segments


def _flat(seg, seed=0):
    g = torch.Generator().manual_seed(seed)
    d = torch.zeros(seg.total)
    for s in seg.slices():
        d[s] = torch.randn(s.stop - s.start, generator=g)
    return d


SIZES = [10, 64, 33, 1, 1000, 31]


def test_segments_layout():
    seg = Segments.from_sizes(SIZES)
    assert all(o % 32 == 0 for o in seg.offsets)
    assert seg.total % 32 == 0 and seg.n_elements == sum(SIZES)
    assert seg.keep_counts(0.99) == [max(1, int(n * 0.01)) for n in SIZES]
    assert seg.keep_counts(0.5)[0] == 5


def test_pack_unpack_roundtrip():
    g = torch.Generator().manual_seed(1)
    neg = torch.rand(32 * 17, generator=g) < 0.5
    w = pack_bits(neg)
    assert w.dtype == torch.int32 and w.numel() == 17
    assert torch.equal(unpack_bits(w), neg)
    # explicit bit positions
    one = torch.zeros(64, dtype=torch.bool)
    one[3] = True
    one[32 + 31] = True
    w = pack_bits(one)
    assert int(w[0]) == 8 and int(w[1]) == -(2 ** 31)


def test_sign_codec_matches_definition():
    seg = Segments.from_sizes(SIZES)
    d = _flat(seg)
    d[seg.offsets[1] + 5] = 0.0  # sign(0) decodes to +1
    c = SignCodec(seg)
    q = c.roundtrip(d)
    for sl, n in zip(seg.slices(), seg.sizes):
        expect = d[sl].abs().sum() / n * torch.where(d[sl] < 0, -1.0, 1.0)
        torch.testing.assert_close(q[sl], expect)
    assert q[~torch.from_numpy(seg.valid_mask())].abs().sum() == 0
    assert c.n_bits() == 32 * len(SIZES) + 32 * math.ceil(sum(SIZES) / 32)
    assert c.compress(d).numel() == c.payload_words()


def test_topk_codec():
    seg = Segments.from_sizes(SIZES)
    d = _flat(seg, 3)
    c = TopKCodec(seg, 0.9)
    q = c.roundtrip(d)
    for sl, n, k in zip(seg.slices(), seg.sizes, c.ks):
        assert k == max(1, int(n * (1 - 0.9)))
        ref = np.zeros(n, dtype=np.float32)
        idx = np.argsort(-np.abs(d[sl].numpy()), kind="stable")[:k]
        ref[idx] = d[sl].numpy()[idx]
        np.testing.assert_array_equal(q[sl].numpy(), ref)
    assert c.n_bits() == 64 * sum(c.ks)
    # ties -> lowest index
    v, i = top_k(torch.tensor([1.0, -1.0, 1.0, 0.5]), 2)
    assert i.tolist() == [0, 1]


def test_random_k_is_a_permutation_prefix():
    for n in (1, 2, 3, 10, 1000, 4097):
        idx = random_k_indices(n, n, seed=5, step=2, seg=1)
        assert sorted(idx.tolist()) == list(range(n))
    a = random_k_indices(1000, 10, 5, 2, 1)
    assert torch.equal(a, random_k_indices(1000, 1000, 5, 2, 1)[:10])
    assert not torch.equal(a, random_k_indices(1000, 10, 5, 3, 1))


def test_random_k_uniformity():
    counts = np.zeros(50)
    for step in range(2000):
        for i in random_k_indices(50, 5, 11, step, 0).tolist():
            counts[i] += 1
    expect = 2000 * 5 / 50
    chi2 = ((counts - expect) ** 2 / expect).sum()
    assert chi2 < 100  # 49 dof: mean 49, this is > 4 sigma


def test_random_k_codec_no_indices_on_wire():
    seg = Segments.from_sizes(SIZES)
    d = _flat(seg, 4)
    c = RandomKCodec(seg, 0.5, seed=9)
    p = c.compress(d, step=3, src=2)
    assert p.numel() == sum(c.ks)
    q = c.decompress(p, step=3, src=2)
    nz = q != 0
    torch.testing.assert_close(q[nz], d[nz])
    assert int(nz.sum()) == sum(c.ks)


def test_qsgd_unbiased_and_levels():
    seg = Segments.from_sizes([512])
    d = _flat(seg, 5)
    c = QSGDCodec(seg, s=15)
    assert c.nbits == 4 and c.payload_words() == 1 + 16 * 5
    acc = torch.zeros_like(d)
    n_rep = 400
    for t in range(n_rep):
        q = c.roundtrip(d, step=t)
        lv = (q.abs() * 15 / d.norm()).round()
        assert lv.max() <= 15
        acc += q
    err = (acc / n_rep - d).abs().max()
    assert err < 0.05 * d.abs().max() + 4 * float(d.norm()) / 15 / math.sqrt(n_rep)
    # explicit s = 16 (convex-code spelling) needs 5 level bits
    assert QSGDCodec(seg, s=16).nbits == 5
    assert abs(qsgd_scale(2000, 16, True) - 1 / (min(2000 / 256, math.sqrt(2000) / 16) + 1)) < 1e-12


def test_qsgd_injected_uniforms_match_formula():
    seg = Segments.from_sizes([100])
    d = _flat(seg, 6)
    u = torch.rand(seg.total, generator=torch.Generator().manual_seed(0))
    c = QSGDCodec(seg, s=7, is_biased=True)
    q = c.decompress(c.compress(d, u=u))
    x = d[:100]
    norm = x.norm()
    lvl = 7 * x.abs() / norm
    lv = lvl.floor() + (u[:100] < (lvl - lvl.floor())).float()
    expect = qsgd_scale(100, 7, True) * torch.sign(x) * norm * lv / 7
    torch.testing.assert_close(q[:100], expect, rtol=1e-6, atol=1e-7)


def test_qsgd_zero_tensor_is_finite():
    seg = Segments.from_sizes([40])
    q = QSGDCodec(seg, 15).roundtrip(torch.zeros(seg.total))
    assert torch.isfinite(q).all() and q.abs().sum() == 0


def test_counter_uniform_range():
    u = counter_uniform(1, 2, torch.arange(100000))
    assert 0 <= float(u.min()) and float(u.max()) < 1
    assert abs(float(u.mean()) - 0.5) < 0.01


def test_factory():
    seg = Segments.from_sizes(SIZES)
    assert make_codec(seg, None).name == "identity"
    assert make_codec(seg, "sign").name == "sign"
    assert make_codec(seg, "compress_top_k", 0.9).name == "compress_top_k"
    assert make_codec(seg, "compress_random_k", 0.9).name == "compress_random_k"
    q = make_codec(seg, "quantize_qsgd", quantize_level=4)
    assert q.s == 15 and q.n_bits() == sum(SIZES) * 4
    assert make_codec(seg, "quantize_qsgd", quantize_level=32).name == "identity"
    assert make_codec(seg, "quantize_qsgd", qsgd_levels=16).s == 16
