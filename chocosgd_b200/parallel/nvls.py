"""All-reduce through the NVSwitch (``csrc/nvls.cu``): ``multimem.ld_reduce`` / ``multimem.st`` on a
symmetric buffer that is also bound to an NVLink multicast object.

The buffer, the exchange of its peer addresses and the multicast binding come from
``torch.distributed._symmetric_memory`` (plumbing); the collective itself is ONE kernel of this
library per rank.  Used for the averaged-model evaluation (``train/loops.py``) and by
``CentralizedAggregation`` for flat fp32 tensors when ``enable()`` succeeded; everything falls back
to the process group's ``all_reduce`` when the device, the driver or the group has no multicast
support (``NvlsUnavailable``).  Counterpart of the reference's ``dist.all_reduce`` calls
(``dl_code/pcode/utils/communication.py:114-122, 173-181``).

A rank must not exit while its memory is bound to the multicast object of a group that keeps
running: ``close()`` (called from ``bootstrap.shutdown``) drops the buffers after a barrier, and the
elastic mode (``--elastic``), where ranks may leave, never creates one."""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..utils.error_handler import GossipTimeout


class NvlsUnavailable(RuntimeError):
    pass


class NvlsArgsC(ctypes.Structure):
    _fields_ = [
        ("mc", ctypes.c_void_p),
        ("local", ctypes.c_void_p),
        ("flags_local", ctypes.c_void_p),
        ("flags_peer", ctypes.c_void_p * (_lib.MAX_PEERS + 1)),
        ("epoch", ctypes.c_void_p),
        ("status", ctypes.c_void_p),
        ("n", ctypes.c_longlong),
        ("budget_ns", ctypes.c_longlong),
        ("scale", ctypes.c_float),
        ("rank", ctypes.c_int),
        ("world", ctypes.c_int),
    ]


def _declare():
    lib = _lib.load()
    if not getattr(lib, "_nvls_declared", False):
        lib.nvls_allreduce.argtypes = [ctypes.POINTER(NvlsArgsC), ctypes.c_int, ctypes.c_void_p]
        for n in ("nvls_allreduce", "nvls_args_size", "nvls_max_grid"):
            getattr(lib, n).restype = ctypes.c_int
        assert lib.nvls_args_size() == ctypes.sizeof(NvlsArgsC), "NvlsArgs layout mismatch"
        lib._nvls_declared = True
    return lib


FLAG_WORDS = 64  # flag array behind the data (one word per rank, padded to 256 bytes)


class NvlsAllReduce:
    """In-place sum / average of the first ``n`` floats of ``self.data`` over the ranks of ``group``."""

    def __init__(self, capacity: int, group=None, device=None, wait_budget_ms: float = 5000.0, sync: bool = True):
        if not (dist.is_available() and dist.is_initialized()):
            raise NvlsUnavailable("no process group")
        group = group if group is not None else dist.group.WORLD
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world < 2 or self.world > _lib.MAX_PEERS + 1:
            raise NvlsUnavailable(f"world size {self.world} outside 2 .. {_lib.MAX_PEERS + 1}")
        if os.environ.get("NCCL_NVLS_ENABLE", "1") == "0":
            raise NvlsUnavailable("multicast switched off (NCCL_NVLS_ENABLE=0)")
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        try:
            import torch.distributed._symmetric_memory as symm
        except Exception as e:  # pragma: no cover
            raise NvlsUnavailable(f"symmetric memory not importable: {e}")
        self.capacity = (int(capacity) + 4 * self.world - 1) // (4 * self.world) * (4 * self.world)
        total = self.capacity + FLAG_WORDS
        try:
            self.buf = symm.empty(total, dtype=torch.float32, device=self.device)
            self.handle = symm.rendezvous(self.buf, group)
            mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        except NvlsUnavailable:
            raise
        except Exception as e:
            raise NvlsUnavailable(f"symmetric-memory rendezvous failed: {type(e).__name__}: {e}")
        if mc == 0:
            raise NvlsUnavailable("the symmetric buffer has no multicast mapping on this system")
        self.buf.zero_()
        self.data = self.buf[: self.capacity]
        self.lib = _declare()
        with torch.cuda.device(self.device):
            self.max_grid = max(1, self.lib.nvls_max_grid())
        self.sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.epoch = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        a = NvlsArgsC()
        a.mc, a.local = mc, self.buf.data_ptr()
        a.flags_local = self.buf.data_ptr() + 4 * self.capacity
        ptrs = list(self.handle.buffer_ptrs)
        for r in range(self.world):
            a.flags_peer[r] = int(ptrs[r]) + 4 * self.capacity
        a.epoch, a.status = self.epoch.data_ptr(), self.status.data_ptr()
        a.budget_ns = int(wait_budget_ms * 1e6)
        a.rank, a.world = self.rank, self.world
        self.args = a
        # every rank's flags must be zero before anybody's first kernel can write one: a collective
        # (the barrier here, or the caller's own when sync=False) separates set-up from first use
        torch.cuda.synchronize(self.device)
        if sync:
            dist.barrier(group=group)

    def reduce_(self, n: int, average: bool = True, stream=None):
        """All-reduce ``self.data[:n]`` in place (asynchronous on the current stream).  Every rank calls it
        with the same ``n``."""
        n4 = (int(n) + 3) // 4 * 4
        if n4 > self.capacity:
            raise ValueError(f"{n} floats exceed the buffer's capacity {self.capacity}")
        if n4 != n:
            self.data[n:n4].zero_()
        a = self.args
        a.n, a.scale = n4, (1.0 / self.world) if average else 1.0
        grid = max(1, min(self.max_grid, 4 * self.sms, (n4 // 4 // self.world + 1023) // 1024))
        _lib.check(self.lib.nvls_allreduce(ctypes.byref(a), grid, _lib.stream_ptr(stream)), "nvls_allreduce")
        _lib.count(1)
        return self.data[:n]

    def all_reduce(self, x: torch.Tensor, average: bool = True) -> torch.Tensor:
        """``x`` (flat fp32 on this device) summed / averaged over the group; returns a view of the
        symmetric buffer (valid until the next call)."""
        n = x.numel()
        self.data[:n].copy_(x.reshape(-1))
        return self.reduce_(n, average).view_as(x)

    def check(self):
        st = self.status.tolist()
        if st[0] != 0:
            self.status.zero_()
            raise GossipTimeout(st[0], st[1], st[2])

    def close(self):
        self.args = None
        self.handle = None
        self.buf = self.data = None


_ACTIVE: Optional[NvlsAllReduce] = None
_TRIED = False


def enable(capacity: int, group=None, device=None) -> Optional[NvlsAllReduce]:
    """Create the process-wide all-reduce buffer (collective call: every rank of ``group``).  Returns None,
    with the reason recorded in ``why_not()``, when the system cannot do it; all ranks agree on the
    outcome (one ``all_reduce`` of a success flag) so that nobody waits for a kernel that others skip."""
    global _ACTIVE, _TRIED, _WHY
    if _ACTIVE is not None and _ACTIVE.capacity >= capacity:
        return _ACTIVE
    if _TRIED and _ACTIVE is None:
        return None          # the system said no once: do not rendezvous again at every evaluation
    _TRIED = True
    obj, _WHY = None, ""
    try:
        obj = NvlsAllReduce(capacity, group, device, sync=False)   # the all_reduce below is the barrier
    except NvlsUnavailable as e:
        _WHY = str(e)
    if dist.is_available() and dist.is_initialized():
        dev = torch.device(device if device is not None else (f"cuda:{torch.cuda.current_device()}" if torch.cuda.is_available() else "cpu"))
        on_gpu = dist.get_backend(group) == "nccl"
        ok = torch.tensor([1 if obj is not None else 0], dtype=torch.int32, device=dev if on_gpu else "cpu")
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok) == 0 and obj is not None:
            obj.close()
            obj, _WHY = None, "another rank could not create its buffer"
    _ACTIVE = obj
    return obj


_WHY = ""


def active() -> Optional[NvlsAllReduce]:
    return _ACTIVE


def why_not() -> str:
    return _WHY


def close():
    global _ACTIVE
    if _ACTIVE is not None:
        _ACTIVE.close()
        _ACTIVE = None
