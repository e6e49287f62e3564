"""Index arithmetic of the ImageNet stem kernels (``csrc/conv_stem_bf16.cu``) restated on the CPU: the K layout of
the im2col tile (7 filter rows x 8 window pixels x 3 channels, window starting one pixel left of the filter),
the placement of the filter in the B operand, and the 128-byte-swizzled shared-memory addresses."""
import torch
import torch.nn.functional as F

K_PAD = 176          # 7 * 24 = 168, plus one zero chunk of 8


def im2col_rows(x):
    """x [N, H, W, 3] -> A [N * H/2 * W/2, K_PAD] exactly as a producer thread gathers it."""
    n, h, w, _ = x.shape
    ho, wo = h // 2, w // 2
    a = torch.zeros(n * ho * wo, K_PAD, dtype=x.dtype)
    for p in range(n * ho * wo):
        ow, oh, img = p % wo, (p // wo) % ho, p // (wo * ho)
        w_start, h0 = 2 * ow - 4, 2 * oh - 3
        lo = -3 * w_start if w_start < 0 else 0
        hi = 3 * min(8, w - w_start)
        for r in range(7):
            hh = h0 + r
            if not 0 <= hh < h:
                continue
            row = x[img, hh].reshape(-1)                      # W * 3 floats
            for f in range(0, 24, 2):                        # twelve float2 loads
                if lo <= f < hi:
                    base = w_start * 3 + f
                    a[p, 24 * r + f] = row[base]
                    a[p, 24 * r + f + 1] = row[base + 1]
    return a


def filter_rows(wt):
    """wt [64, 7, 7, 3] -> B [64, K_PAD]: k = 24 r + 3 (s + 1) + c, window pixel 0 and the padding stay zero."""
    b = torch.zeros(wt.shape[0], K_PAD, dtype=wt.dtype)
    for i in range(wt.shape[0] * 147):
        co, e = divmod(i, 147)
        r, sc = divmod(e, 21)
        b[co, 24 * r + 3 + sc] = wt.reshape(-1)[i]
    return b


def test_im2col_layout_reproduces_the_convolution():
    torch.manual_seed(0)
    for n, h, w in ((1, 16, 16), (2, 12, 20)):
        x = torch.randn(n, h, w, 3, dtype=torch.float64)
        wt = torch.randn(64, 7, 7, 3, dtype=torch.float64)
        y = im2col_rows(x) @ filter_rows(wt).t()                                   # [pixels, 64]
        ref = F.conv2d(x.permute(0, 3, 1, 2), wt.permute(0, 3, 1, 2), None, 2, 3)   # [n, 64, h/2, w/2]
        torch.testing.assert_close(y.view(n, h // 2, w // 2, 64), ref.permute(0, 2, 3, 1), rtol=1e-10, atol=1e-10)
        # weight gradient: the same two matrices, contracted over the pixel
        dy = torch.randn(n * (h // 2) * (w // 2), 64, dtype=torch.float64)
        d = dy.t() @ im2col_rows(x)                                                # [64, K_PAD]
        xr = x.permute(0, 3, 1, 2).clone().requires_grad_()
        wr = wt.permute(0, 3, 1, 2).clone().requires_grad_()
        F.conv2d(xr, wr, None, 2, 3).backward(dy.view(n, h // 2, w // 2, 64).permute(0, 3, 1, 2))
        dw = torch.stack([d[:, 24 * r + 3 + sc] for r in range(7) for sc in range(21)], dim=1).view(64, 7, 7, 3)
        torch.testing.assert_close(dw, wr.grad.permute(0, 2, 3, 1), rtol=1e-9, atol=1e-9)


def swizzled_offset(row, k, rows_per_slab):
    """Byte offset of bf16 element (row, k) of a K-major tile cut into slabs of 64 k (128 bytes per row)."""
    q = k >> 3                                   # 16-byte chunk along K
    return (q >> 3) * rows_per_slab * 128 + row * 128 + (((q & 7) ^ (row & 7)) << 4) + (k & 7) * 2


def test_swizzled_addresses_are_a_bijection_and_keep_mma_steps_inside_a_slab():
    for rows in (128, 64, 176):                   # forward A, forward B, weight-gradient B
        ks = 192 if rows != 176 else 128          # 3 slabs forward, 2 slabs (128 pixels) in the weight gradient
        seen = set()
        for row in range(rows):
            for k in range(ks):
                off = swizzled_offset(row, k, rows)
                assert off % 2 == 0 and 0 <= off < (ks // 64) * rows * 128
                seen.add(off)
        assert len(seen) == rows * ks
    # one MMA reads K = 16 = two neighbouring chunks: both lie in the same slab and the same 128-byte row
    for ks_step in range(K_PAD // 16):
        q0, q1 = 2 * ks_step, 2 * ks_step + 1
        assert q0 >> 3 == q1 >> 3
    # the descriptor start of K step j inside a slab is 32 j bytes: chunk 2 j of row 0
    assert [swizzled_offset(0, 16 * j, 128) for j in range(4)] == [0, 32, 64, 96]
