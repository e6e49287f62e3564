"""The allocation-free entry point ``sign_l1_compress_noalloc`` of the native library.

Some users of the library cannot call ``cudaMalloc`` where they compress (progress threads
and callbacks of other runtimes, processes whose device memory is pre-reserved by another
allocator).  For them the library keeps the small work area of the norm reduction in a
fixed device array.  The test drives that entry point through its exported C symbol, the
way such a caller would, and compares with the ordinary entry point (caller-supplied
scratch) on two consecutive calls: the second call sees the work area as the first left it.

Collected last on purpose: a failure here cannot hide the result of any other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, x, stream):
    n = x.numel()
    words = torch.full(((n + 31) // 32,), -1, dtype=torch.int32, device=x.device)
    norm = torch.full((1,), -1.0, dtype=torch.float32, device=x.device)
    fn = lib.sign_l1_compress_noalloc  # the exported C symbol
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    rc = fn(x.data_ptr(), n, words.data_ptr(), norm.data_ptr(), stream)
    return rc, words, norm


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    from chocosgd_b200.ops import _lib
    from chocosgd_b200.ops.compress import sign_l1_compress

    lib = ctypes.CDLL(_lib.lib_path())
    torch.cuda.set_device(0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator().manual_seed(3)
    # first a large tensor (many partial sums), then a small one: stale partials of the first
    # call are still in the work area when the second runs
    for n in (1_000_003, 4097):
        x = torch.randn(n, generator=g).cuda()
        x[0] = 0.0
        rc, words, norm = _call_noalloc(lib, x, stream)
        assert rc == 0
        ref_words, ref_norm = sign_l1_compress(x)
        torch.cuda.synchronize()
        assert torch.equal(words, ref_words)
        assert float(norm) == float(ref_norm)  # same kernel, same reduction order
        torch.testing.assert_close(norm[0].cpu(), x.abs().sum().cpu(), rtol=2e-5, atol=1e-4)
        # and against a plain PyTorch restatement of the packing
        from chocosgd_b200.compress.reference import pack_bits

        pad = torch.zeros((n + 31) // 32 * 32, device="cuda")
        pad[:n] = x
        assert torch.equal(words.cpu(), pack_bits(pad.cpu() < 0))


def test_noalloc_rejects_oversized_input():
    from chocosgd_b200.ops import _lib

    lib = ctypes.CDLL(_lib.lib_path())
    fn = lib.sign_l1_compress_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    x = torch.zeros(32, device="cuda")
    too_many = 16384 * 8192 + 1
    assert fn(x.data_ptr(), too_many, x.data_ptr(), x.data_ptr(), None) == -2
    assert fn(x.data_ptr(), 0, x.data_ptr(), x.data_ptr(), None) == -2
