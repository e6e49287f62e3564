"""ctypes loader of the in-tree native library.

The library is built in-tree by ``chocosgd_b200.build_ext`` (``lib/libchoco_b200.so``) and
bound through its C ABI.  On a machine with a CUDA device the library is mandatory: ops
raise instead of silently falling back when it cannot be loaded."""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_float, c_int, c_int32, c_longlong, c_uint32, c_void_p

_LIB = None
_ERR = None


def lib_path() -> str:
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib", "libchoco_b200.so")


def load(build_if_missing: bool = True):
    """Return the loaded library (building it first when sources changed and nvcc exists)."""
    global _LIB, _ERR
    if _LIB is not None:
        return _LIB
    path = lib_path()
    try:
        if build_if_missing:
            from ..build_ext import build, is_current, nvcc_path

            if not is_current() and nvcc_path() is not None:
                build()
        _LIB = ctypes.CDLL(path)
        _declare(_LIB)
        _check_abi(_LIB)
    except Exception as e:  # pragma: no cover - exercised only on broken installs
        _ERR = e
        _LIB = None
        raise RuntimeError(f"native library {path} could not be loaded: {e}") from e
    return _LIB


def configure_pdl(mode: str = "auto", bf16: bool = False) -> bool:
    """Programmatic dependent launch for the library's kernels (``csrc/launch.cuh`` reads ``CHOCO_PDL`` at the
    first launch, so call this before any).  ``auto``: on for bf16-autocast training (measured on the ResNet-50
    step: 12.45 - 12.65 ms against 12.76 - 12.78 ms), off otherwise (the fp32 ResNet-20 step, about 140 kernels
    of 3 - 10 us, was slower with it).  A ``CHOCO_PDL`` already in the environment wins."""
    if "CHOCO_PDL" not in os.environ:
        on = mode == "on" or (mode == "auto" and bf16)
        os.environ["CHOCO_PDL"] = "1" if on else "0"
    return os.environ["CHOCO_PDL"] not in ("", "0")


def available() -> bool:
    try:
        load()
        return True
    except Exception:
        return False


def check(code: int, what: str = ""):
    if code != 0:
        msg = load().choco_cuda_error_string(code).decode()
        raise RuntimeError(f"CUDA error {code} ({msg}) in {what}")


MAX_PEERS = 16

#: kernels of this library launched so far by this process (the Python wrappers add their
#: launches; a training step captured in a CUDA graph replays the count taken while capturing)
LAUNCHES = [0]


def count(n: int = 1):
    LAUNCHES[0] += n


class SegTableC(Structure):
    _fields_ = [
        ("chunk_seg", c_void_p),
        ("chunk_start", c_void_p),
        ("chunk_valid", c_void_p),
        ("seg_start", c_void_p),
        ("seg_size", c_void_p),
        ("seg_first_chunk", c_void_p),
        ("seg_n_chunks", c_void_p),
        ("seg_wd", c_void_p),
        ("seg_k", c_void_p),
        ("seg_koff", c_void_p),
        ("n_chunks", c_int),
        ("n_segments", c_int),
        ("chunk_elems", c_int),
        ("total", c_int),
    ]


class ChocoParamsC(Structure):
    _fields_ = [
        ("x", c_void_p),
        ("g", c_void_p),
        ("m", c_void_p),
        ("x_hat", c_void_p),
        ("s", c_void_p),
        ("scratch_d", c_void_p),
        ("outbox", c_void_p),
        ("peer_inbox", c_void_p * MAX_PEERS),
        ("peer_flag", c_void_p * MAX_PEERS),
        ("my_inbox", c_void_p * MAX_PEERS),
        ("my_flag", c_void_p * MAX_PEERS),
        ("hyper", c_void_p),
        ("step", c_void_p),
        ("seg_count", c_void_p),
        ("done_count", c_void_p),
        ("partial", c_void_p),
        ("hist", c_void_p),
        ("chunk_cnt", c_void_p),
        ("sel", c_void_p),
        ("status", c_void_p),
        ("seg_g", c_void_p),
        ("wait_budget_ns", c_longlong),
        ("tab", SegTableC),
        ("w_self", c_float),
        ("w_peer", c_float * MAX_PEERS),
        ("n_peers", c_int),
        ("payload_words", c_int),
        ("body_off", c_int),
        ("rank", c_int),
        ("peer_rank", c_int * MAX_PEERS),
        ("seed", c_uint32),
        ("qsgd_s", c_int),
        ("qsgd_nbits", c_int),
        ("qsgd_biased", c_int),
        ("pad_", c_int),
    ]


def _declare(lib):
    vp, i, ll, f = c_void_p, c_int, c_longlong, c_float
    lib.choco_cuda_error_string.restype = ctypes.c_char_p
    lib.choco_cuda_error_string.argtypes = [i]
    sigs = {
        "choco_sign_step": [vp, i, i, i, i, vp],
        "choco_sign_step_range": [vp, i, i, i, i, i, vp],
        "fused_sgd_step": [vp, i, i, i, vp],
        "grad_clip_coef": [vp, i, i, f, vp, vp],
        "sign_pack": [vp, ll, vp, vp],
        "sign_unpack": [vp, ll, vp, f, vp],
        "sign_l1_compress": [vp, ll, vp, vp, vp, vp],
        "sign_l1_compress_noalloc": [vp, ll, vp, vp, vp],
        "symm_alloc": [POINTER(vp), ll],
        "symm_free": [vp],
        "symm_handle_size": [],
        "symm_get_handle": [vp, vp],
        "symm_open_handle": [vp, POINTER(vp)],
        "symm_close_handle": [vp],
        "symm_can_access_peer": [i, i],
        "choco_params_size": [],
        "choco_params_offset": [i],
        "choco_max_peers": [],
        "choco_hist_words": [],
    }
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = i
    lib.sign_l1_scratch_bytes.argtypes = [ll]
    lib.sign_l1_scratch_bytes.restype = ll
    for name, args in {
        "cpu_sign_pack": [vp, ll, vp],
        "cpu_sign_unpack": [vp, ll, vp, f],
        "cpu_top_k": [vp, i, i, vp, vp],
        "cpu_random_k_indices": [i, i, c_uint32, c_uint32, c_uint32, vp],
        "cpu_counter_uniform": [c_uint32, c_uint32, ll, vp],
    }.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = None
    # optional symbols (present once the corresponding source is compiled in)
    for name, args in {
        "choco_dense_prep": [vp, i, i, i, i, vp],
        "choco_qsgd_pack": [vp, i, i, vp],
        "choco_qsgd_pack_nbits": [vp, i, i, i, vp],
        "choco_qsgd_decode": [vp, i, i, vp],
        "choco_topk_hist": [vp, i, i, i, vp],
        "choco_topk_count": [vp, i, i, vp],
        "choco_topk_emit": [vp, i, i, vp],
        "choco_randk_emit": [vp, i, i, vp],
        "choco_sparse_decode": [vp, i, i, i, i, vp],
        "choco_sparse_decode_ex": [vp, i, i, i, i, i, vp],
        "choco_wait_flags": [vp, i, vp],
        "choco_publish": [vp, i, vp],
    }.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = i


def _check_abi(lib):
    if lib.choco_max_peers() != MAX_PEERS:
        raise RuntimeError("CHOCO_MAX_PEERS mismatch between the library and the bindings")
    if lib.choco_params_size() != ctypes.sizeof(ChocoParamsC):
        raise RuntimeError(
            f"ChocoParams layout mismatch: C {lib.choco_params_size()} vs ctypes {ctypes.sizeof(ChocoParamsC)}"
        )
    names = ["outbox", "hyper", "wait_budget_ns", "tab", "w_self", "n_peers", "seed"]
    for which, name in enumerate(names):
        if lib.choco_params_offset(which) != getattr(ChocoParamsC, name).offset:
            raise RuntimeError(f"ChocoParams.{name} offset mismatch")


def stream_ptr(stream=None):
    import torch

    s = stream if stream is not None else torch.cuda.current_stream()
    return c_void_p(s.cuda_stream)


def ptr(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)
