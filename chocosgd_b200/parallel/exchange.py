"""Neighbour exchange over peer-mapped mailboxes (``csrc/exchange.cu``): the drop-in
replacement of ``DecentralizedAggregation`` (``torch.distributed`` send/recv) on NVLink.

``MailboxExchange.start(payload).wait()`` publishes a 1-d fp32/int32 payload to every graph
neighbour with in-kernel NVLink stores and returns ``{rank: tensor}`` (own payload included),
the contract of the reference's ``_agg(..., op="get_raw_sync_data")``
(``dl_code/pcode/utils/communication.py:246-287``).  On the complete graph the same call is an
all-gather by push (DGC, EF-signSGD).  ``mix_`` is the fused D-PSGD averaging."""
from __future__ import annotations

import ctypes

import torch

from ..ops import _lib
from ..utils.error_handler import GossipTimeout
from .symm import DistributedMailbox

MAXP = _lib.MAX_PEERS


class ExchangeArgsC(ctypes.Structure):
    _fields_ = [
        ("src", ctypes.c_void_p),
        ("peer_inbox", ctypes.c_void_p * MAXP),
        ("peer_flag", ctypes.c_void_p * MAXP),
        ("my_inbox", ctypes.c_void_p * MAXP),
        ("my_flag", ctypes.c_void_p * MAXP),
        ("w_peer", ctypes.c_float * MAXP),
        ("w_self", ctypes.c_float),
        ("counter", ctypes.c_void_p),
        ("status", ctypes.c_void_p),
        ("wait_budget_ns", ctypes.c_longlong),
        ("n_words", ctypes.c_longlong),
        ("slot_words", ctypes.c_longlong),
        ("n_peers", ctypes.c_int),
        ("seq", ctypes.c_uint32),
        ("peer_rank", ctypes.c_int * MAXP),
    ]


def _lib_ex():
    lib = _lib.load()
    if not getattr(lib, "_ex_declared", False):
        P = ctypes.POINTER(ExchangeArgsC)
        lib.mailbox_push.argtypes = [P, ctypes.c_void_p]
        lib.mailbox_wait.argtypes = [P, ctypes.c_void_p]
        lib.dpsgd_mix.argtypes = [P, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p]
        lib.sq_distance.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p,
                                    ctypes.c_void_p, ctypes.c_void_p]
        lib.sq_distance_blocks.argtypes = [ctypes.c_longlong]
        for n in ("mailbox_push", "mailbox_wait", "dpsgd_mix", "sq_distance", "sq_distance_blocks", "exchange_args_size"):
            getattr(lib, n).restype = ctypes.c_int
        assert lib.exchange_args_size() == ctypes.sizeof(ExchangeArgsC), "ExchangeArgs layout mismatch"
        lib._ex_declared = True
    return lib


class _Pending:
    def __init__(self, ex, data, n, dtype):
        self.ex, self.data, self.n, self.dtype = ex, data, n, dtype

    def wait(self):
        ex = self.ex
        if ex.args.n_peers:
            _lib.check(ex.lib.mailbox_wait(ctypes.byref(ex.args), _lib.stream_ptr()), "mailbox_wait")
        return self.data


class MailboxExchange:
    def __init__(self, graph, max_words: int, device, group=None, wait_budget_ms: float = 5000.0):
        self.lib = _lib_ex()
        self.rank, self.device = graph.rank, torch.device(device)
        self.neighbors_info = graph.get_neighborhood()
        self.slot_words = (int(max_words) + 3) // 4 * 4
        self.mailbox = DistributedMailbox(graph, self.slot_words, self.device, group)
        v = self.mailbox.view()
        self.peers = v.peers
        self.world_size = len(self.neighbors_info)
        a = ExchangeArgsC()
        for k, j in enumerate(v.peers):
            a.peer_inbox[k], a.peer_flag[k], a.my_inbox[k], a.my_flag[k] = (
                v.peer_inbox[k], v.peer_flag[k], v.my_inbox[k], v.my_flag[k])
            a.w_peer[k], a.peer_rank[k] = float(self.neighbors_info[j]), int(j)
        a.w_self = float(self.neighbors_info[self.rank])
        self.counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        a.counter, a.status = self.counter.data_ptr(), self.status.data_ptr()
        a.wait_budget_ns = int(wait_budget_ms * 1e6)
        a.slot_words, a.n_peers, a.seq = self.slot_words, len(v.peers), 0
        self.args = a
        self.stage = torch.zeros(self.slot_words, dtype=torch.int32, device=self.device)
        self.seq = 0

    def _slot_view(self, k, parity, n, dtype):
        base = self.mailbox.local
        off = (self.args.my_inbox[k] - self.mailbox.local.data_ptr()) // 4 + parity * self.slot_words
        return base[off:off + n].view(dtype)

    def start(self, data: torch.Tensor) -> _Pending:
        assert data.dim() == 1 and data.element_size() == 4 and data.is_cuda
        n = data.numel()
        if n > self.slot_words:
            raise ValueError("payload larger than the mailbox slot")
        src = data.contiguous()
        if n % 4 != 0 or src.data_ptr() % 16 != 0:
            self.stage[:n].copy_(src.view(torch.int32))
            src = self.stage
        a = self.args
        a.src, a.n_words, a.seq = src.data_ptr(), (n + 3) // 4 * 4, self.seq
        if a.n_peers:
            _lib.check(self.lib.mailbox_push(ctypes.byref(a), _lib.stream_ptr()), "mailbox_push")
        out = {self.rank: data}
        for k, j in enumerate(self.peers):
            out[j] = self._slot_view(k, self.seq & 1, n, data.dtype)
        self.seq += 1
        return _Pending(self, out, n, data.dtype)

    def _agg(self, data, op, force_wait=True, **kw):
        pending = self.start(data)
        if not force_wait:
            return [pending], pending.data
        local = pending.wait()
        if op == "avg":
            return sum(local.values()) / self.world_size
        if op == "weighted":
            return sum(t * self.neighbors_info[r] for r, t in local.items())
        if op == "get_raw_sync_data":
            return local
        raise NotImplementedError(op)

    def complete_wait(self, reqs):
        for r in reqs:
            r.wait()

    def mix_(self, x: torch.Tensor):
        """x <- sum_j w_ij x_j in place: push x, then one fused wait + weighted-sum kernel."""
        assert x.numel() % 4 == 0
        a = self.args
        a.src, a.n_words, a.seq = x.data_ptr(), x.numel(), self.seq
        if a.n_peers:
            _lib.check(self.lib.mailbox_push(ctypes.byref(a), _lib.stream_ptr()), "mailbox_push")
        _lib.check(self.lib.dpsgd_mix(ctypes.byref(a), x.data_ptr(), x.numel(), _lib.stream_ptr()), "dpsgd_mix")
        self.seq += 1
        return x

    def all_gather(self, data):
        """Payloads of all ranks in rank order (complete graph only)."""
        local = self.start(data).wait()
        return [local[r] for r in sorted(local)]

    def check(self):
        code, peer, seq, _ = self.status.tolist()
        if code != 0:
            raise GossipTimeout(code, peer, seq)

    def close(self):
        self.mailbox.close()


def sq_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Deterministic sum((a - b)^2) in float64 (0-d device tensor)."""
    lib = _lib_ex()
    a, b = a.contiguous().view(-1), b.contiguous().view(-1)
    assert a.is_cuda and a.dtype == torch.float32 and b.dtype == torch.float32 and a.numel() == b.numel()
    blocks = lib.sq_distance_blocks(a.numel())
    scratch = torch.empty(blocks + 2, dtype=torch.float64, device=a.device)
    out = torch.empty(1, dtype=torch.float64, device=a.device)
    _lib.check(lib.sq_distance(_lib.ptr(a), _lib.ptr(b), a.numel(), _lib.ptr(scratch), _lib.ptr(out),
                               _lib.stream_ptr()), "sq_distance")
    return out[0]
