"""Peer-mapped mailboxes: the memory the gossip kernels push into over NVLink.

Every rank owns one mailbox region::

    slot 0: [2][payload_words] uint32      payload buffers (step parity 0 / 1)
    slot 1: ...
    flags : one 128-byte line per slot     word 0 = number of payloads published so far

Slot ``k`` of rank ``i`` is written only by the ``k``-th neighbour of ``i`` (neighbours in
ascending rank order).  ``DistributedMailbox`` cudaMallocs the region, exports a CUDA IPC
handle and opens its neighbours' handles (exchanged once with ``all_gather_object``), which
gives this process ordinary device pointers into the neighbours' memory.  No
``torch.distributed`` call is made after construction.  ``LoopbackMailbox`` places all
logical ranks' regions on one device for single-GPU tests of the same kernels.

The reference moves the same payloads with ``dist.isend`` / ``dist.irecv`` of freshly
allocated tensors every step (``dl_code/pcode/utils/communication.py:246-287``).
"""
from __future__ import annotations

import ctypes
from typing import Dict, List

import torch
import torch.distributed as dist

FLAG_STRIDE_WORDS = 32  # one 128-byte line per flag


def region_words(n_slots: int, payload_words: int) -> int:
    return n_slots * 2 * payload_words + max(n_slots, 1) * FLAG_STRIDE_WORDS


def slot_offset_words(slot: int, payload_words: int) -> int:
    return slot * 2 * payload_words


def flag_offset_words(n_slots: int, slot: int, payload_words: int) -> int:
    return n_slots * 2 * payload_words + slot * FLAG_STRIDE_WORDS


class _RawCudaBuffer:
    """Exposes a raw device pointer to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes // 4,),
            "typestr": "<i4",
            "data": (ptr, False),
            "version": 3,
            "strides": None,
        }


def wrap_device_memory(ptr: int, nbytes: int, device) -> torch.Tensor:
    return torch.as_tensor(_RawCudaBuffer(ptr, nbytes), device=device)


class MailboxView:
    """Pointers one logical rank needs: where its neighbours write (local) and where it
    writes in each neighbour's region (remote)."""

    def __init__(self, rank, peers, my_inbox, my_flag, peer_inbox, peer_flag):
        self.rank = rank
        self.peers: List[int] = peers
        self.my_inbox: List[int] = my_inbox
        self.my_flag: List[int] = my_flag
        self.peer_inbox: List[int] = peer_inbox
        self.peer_flag: List[int] = peer_flag


def _view_from_bases(rank, neighbors: Dict[int, List[int]], bases: Dict[int, int], payload_words: int) -> MailboxView:
    peers = sorted(neighbors[rank])
    n_slots = len(peers)
    my_inbox = [bases[rank] + 4 * slot_offset_words(k, payload_words) for k in range(n_slots)]
    my_flag = [bases[rank] + 4 * flag_offset_words(n_slots, k, payload_words) for k in range(n_slots)]
    peer_inbox, peer_flag = [], []
    for j in peers:
        theirs = sorted(neighbors[j])
        slot = theirs.index(rank)
        peer_inbox.append(bases[j] + 4 * slot_offset_words(slot, payload_words))
        peer_flag.append(bases[j] + 4 * flag_offset_words(len(theirs), slot, payload_words))
    return MailboxView(rank, peers, my_inbox, my_flag, peer_inbox, peer_flag)


class LoopbackMailbox:
    """All logical ranks on one device (tests, single-GPU emulation)."""

    def __init__(self, neighbors: Dict[int, List[int]], payload_words: int, device):
        self.regions = {
            r: torch.zeros(region_words(len(nb), payload_words), dtype=torch.int32, device=device)
            for r, nb in neighbors.items()
        }
        bases = {r: t.data_ptr() for r, t in self.regions.items()}
        self.views = {r: _view_from_bases(r, neighbors, bases, payload_words) for r in neighbors}

    def view(self, rank) -> MailboxView:
        return self.views[rank]

    def close(self):
        self.regions = {}


class DistributedMailbox:
    """One process per GPU; neighbours' regions mapped through CUDA IPC."""

    def __init__(self, graph, payload_words: int, device, group=None):
        from ..ops import _lib

        self.lib = _lib.load()
        self.device = torch.device(device)
        self.rank = graph.rank
        neighbors = {r: graph.neighbors(r) for r in graph.ranks}
        my_peers = sorted(neighbors[self.rank])
        nbytes = 4 * region_words(len(my_peers), payload_words)
        nbytes = (nbytes + 2 * 1024 * 1024 - 1) // (2 * 1024 * 1024) * (2 * 1024 * 1024)
        self._ptr = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(self.lib.symm_alloc(ctypes.byref(self._ptr), nbytes), "symm_alloc")
            hsize = self.lib.symm_handle_size()
            hbuf = ctypes.create_string_buffer(hsize)
            _lib.check(self.lib.symm_get_handle(self._ptr, hbuf), "symm_get_handle")
            torch.cuda.synchronize()
        self.nbytes = nbytes
        self.local = wrap_device_memory(self._ptr.value, nbytes, self.device)
        info = {"rank": self.rank, "handle": bytes(hbuf.raw), "device": self.device.index}
        gathered = [None] * dist.get_world_size(group)
        dist.all_gather_object(gathered, info, group=group)
        self._opened = {}
        bases = {self.rank: self._ptr.value}
        with torch.cuda.device(self.device):
            for entry in gathered:
                r = entry["rank"]
                if r in my_peers:
                    p = ctypes.c_void_p()
                    _lib.check(self.lib.symm_open_handle(entry["handle"], ctypes.byref(p)), f"symm_open_handle({r})")
                    self._opened[r] = p
                    bases[r] = p.value
        # a rank only needs the bases of itself and of its neighbours
        self._view = _view_from_bases(self.rank, {r: neighbors[r] for r in [self.rank] + my_peers}, bases,
                                      payload_words)
        dist.barrier(group=group)

    def view(self, rank=None) -> MailboxView:
        return self._view

    def close(self):
        if self._ptr is None:
            return
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for p in self._opened.values():
                self.lib.symm_close_handle(p)
            self._opened = {}
            self.local = None
            self.lib.symm_free(self._ptr)
        self._ptr = None
