"""Column-wise (N) split of dense projections over the GPUs of one node, one
process per GPU, with the all-gather fused into the GEMV kernel.

Dense projections and the lm_head shard by output rows (the 8-row-interleaved
layout makes a shard a contiguous slice of the tensor's bytes). Every rank's
GEMV epilogue stores its output slice straight into the gathered vector of every
rank over NVLink (peer memory mapped with CUDA IPC) as (value, launch number)
pairs; the next GEMV polls the numbers of the elements it reads. No fence, no
collective call. ``torch.distributed`` is used
only to exchange the IPC handles and for barriers; no collective runs on the
data path.

Host-side helpers (``shard_rows``, ``sequence_number``) are plain functions so
that they can be tested on CPU.
"""
from __future__ import annotations

import ctypes as C

from . import capi
from .capi import QTYPE, check, lib

MAX_RANKS = 8


def shard_rows(N: int, world: int, rank: int, qtype: str = "q4_K") -> tuple[int, int]:
    """Rows [lo, hi) of an N-row projection owned by ``rank``: equal shards whose boundaries fall on multiples of 8
    rows for the 8-row-interleaved formats (a shard must be whole row groups)."""
    align = 8 if qtype in ("q4_K", "q4_0") else 1
    if N % (world * align):
        raise ValueError(f"N={N} does not split into {world} shards of whole {align}-row groups")
    per = N // world
    return rank * per, (rank + 1) * per


def shard_bytes(qtype: str, N: int, K: int, world: int, rank: int) -> tuple[int, int]:
    """Byte range of the tensor that holds the rank's rows."""
    bs, bb = {"q4_0": (32, 18), "q4_K": (256, 144), "q6_K": (256, 210)}[qtype]
    lo, hi = shard_rows(N, world, rank, qtype)
    row = K // bs * bb
    return lo * row, hi * row


def sequence_number(epoch: int, layers_per_epoch: int, layer: int) -> int:
    """Sequence number a launch publishes in its flag slots; it waits for every slot to show this number minus one
    (mirrors the device-side formula; the first launch ever, number 1, waits for nothing)."""
    return (epoch - 1) * layers_per_epoch + layer + 1


def expert_range(n_experts: int, world: int, rank: int) -> tuple[int, int]:
    """Experts [lo, hi) owned by ``rank`` under expert parallelism: equal contiguous blocks."""
    if n_experts % world:
        raise ValueError(f"{n_experts} experts do not split evenly over {world} ranks")
    per = n_experts // world
    return rank * per, (rank + 1) * per


class PeerBuffers:
    """Device buffers of this rank (zeroed) and the same buffers of every peer mapped through CUDA IPC.
    ``sizes``: bytes of each buffer. ``ptr(r, i)`` is buffer i of rank r as a device pointer valid in this process."""

    def __init__(self, sizes, group=None):
        import torch
        import torch.distributed as dist
        self.dist, self.torch, self.group = dist, torch, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > MAX_RANKS:
            raise ValueError("peer buffers span the GPUs of one node (at most 8 ranks)")
        L = lib()
        self._own, mine = [], []
        for n in sizes:
            p = C.c_void_p()
            check(L.nntr_cuda_malloc(C.byref(p), n))
            self._own.append(p.value)
            h = (C.c_ubyte * 64)()
            check(L.nntr_cuda_ipc_export(p.value, h))
            mine.append(bytes(h))
        if self.world > 1:
            allh = [None] * self.world
            dist.all_gather_object(allh, mine, group=group)
        else:
            allh = [mine]
        self._opened, self._ptrs = [], []
        for r in range(self.world):
            if r == self.rank:
                self._ptrs.append(list(self._own))
                continue
            row = []
            for hb in allh[r]:
                p = C.c_void_p()
                check(L.nntr_cuda_ipc_open((C.c_ubyte * 64).from_buffer_copy(hb), C.byref(p)))
                self._opened.append(p.value)
                row.append(p.value)
            self._ptrs.append(row)
        if self.world > 1:
            dist.barrier(group=group)

    def ptr(self, rank: int, i: int) -> int:
        return self._ptrs[rank][i]

    def close(self) -> None:
        L = lib()
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier(group=self.group)
        for p in self._opened:
            L.nntr_cuda_ipc_close(p)
        self._opened = []
        if self.world > 1:
            self.dist.barrier(group=self.group)
        for p in self._own:
            L.nntr_cuda_free(p)
        self._own = []


def check_ring_rows(ring: int, first_n: int | None, n: int) -> int:
    """With a ring of more than two gathered buffers every CTA keeps its own "done reading" slot and a launch checks the
    slots of as many CTAs as it runs itself, so every launch of the sequence must run the same number of CTAs: the group
    then takes launches of ONE size only (rows per rank). Two buffers count the CTAs of each launch separately and take
    any sizes. Returns the size to remember."""
    if ring > 2 and first_n is not None and n != first_n:
        raise ValueError(f"a ring of {ring} gathered buffers takes launches of one size only ({first_n} rows per rank, "
                         f"now {n}): use ring=2 for sequences of differently sized projections")
    return n if first_n is None else first_n


class NSplitGroup:
    """Per-process state of an N-split group: ``ring`` gathered vectors in rotation, a flag array and an epoch
    word in this rank's memory, and the peers' copies mapped through CUDA IPC."""

    def __init__(self, n_local: int, layers_per_epoch: int, group=None, ring: int = 2):
        import torch
        import torch.distributed as dist

        self.dist, self.torch = dist, torch
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > MAX_RANKS:
            raise ValueError("N-split groups span the GPUs of one node (at most 8 ranks)")
        if ring < 2 or ring > 16 or layers_per_epoch % ring:
            # the gathered buffers rotate per launch; if the launches of a pass were not a multiple of the ring, the first
            # launch of the next pass would not continue the rotation, and a buffer could be overwritten while a slower
            # rank (or the caller) still reads it: the "done reading" flags assume the rotation
            raise ValueError(f"layers_per_epoch must be a multiple of the ring of {ring} gathered buffers "
                             "(pad the sequence with more launches)")
        self.n_local, self.layers, self.ring = n_local, layers_per_epoch, ring
        L = lib()
        self._own = []
        nbytes = self.world * n_local * 8  # (fp32 value, launch number) per element

        def alloc(n):
            p = C.c_void_p()
            check(L.nntr_cuda_malloc(C.byref(p), n))
            self._own.append(p.value)
            return p.value

        self.buf = [alloc(nbytes) for _ in range(ring)]  # gathered vectors in rotation
        self.counter = alloc(8 * 512 * 8)  # flag array: [source rank][source CTA] sequence numbers
        self.epoch = alloc(8)
        # exchange IPC handles of buf[0], buf[1], counter
        mine = []
        for p in (*self.buf, self.counter):
            h = (C.c_ubyte * 64)()
            check(L.nntr_cuda_ipc_export(p, h))
            mine.append(bytes(h))
        if self.world > 1:
            allh = [None] * self.world
            dist.all_gather_object(allh, mine, group=group)
        else:
            allh = [mine]
        self._opened = []
        self.peer = []  # per rank: (buf0, buf1, counter) device pointers valid in THIS process
        for r in range(self.world):
            if r == self.rank:
                self.peer.append((*self.buf, self.counter))
                continue
            ptrs = []
            for hb in allh[r]:
                p = C.c_void_p()
                check(L.nntr_cuda_ipc_open((C.c_ubyte * 64).from_buffer_copy(hb), C.byref(p)))
                self._opened.append(p.value)
                ptrs.append(p.value)
            self.peer.append(tuple(ptrs))
        if self.world > 1:
            dist.barrier(group=group)

    def exchange(self, layer: int, x_tagged: bool = True) -> capi.Exchange:
        """Description of launch ``layer`` of the sequence: it writes gathered buffer layer % ring."""
        ex = capi.Exchange()
        ex.n_ranks, ex.rank = self.world, self.rank
        ex.ring = self.ring
        for r in range(self.world):
            ex.y[r] = self.peer[r][layer % self.ring]
            ex.flags[r] = self.peer[r][self.ring]
        ex.epoch = self.epoch
        ex.layers_per_epoch, ex.layer = self.layers, layer
        ex.x_tagged = 1 if x_tagged else 0
        return ex

    def input_ptr(self, layer: int, src_rank: int | None = None) -> int:
        """Where launch ``layer`` (>= 1) finds its activation: the slice rank ``src_rank`` (default: this rank)
        contributed to the previous gathered vector."""
        r = self.rank if src_rank is None else src_rank
        return self.buf[(layer - 1) % self.ring] + r * self.n_local * 8

    def gathered_ptr(self, layer: int) -> int:
        return self.buf[layer % self.ring]

    def bump_epoch(self, stream: int) -> None:
        check(lib().nntr_cuda_epoch_bump_dev(self.epoch, stream))

    def gemv(self, qtype: str, K: int, x_ptr: int, w_ptr: int, layer: int, stream: int, pdl: bool = False,
             x_tagged: bool = True, n_local: int | None = None) -> None:
        """Launch ``layer`` of the sequence. ``x_ptr`` is (a slice of) the previous gathered vector (``gathered_ptr`` /
        ``input_ptr``, tagged pairs) or, with ``x_tagged=False``, a plain fp32 vector. ``n_local``: this launch's rows
        per rank when the launches of the sequence differ in size (at most the group's ``n_local``)."""
        n = self.n_local if n_local is None else n_local
        if n > self.n_local:
            raise ValueError("a launch's rows per rank exceed the gathered buffers of the group")
        self._first_n = check_ring_rows(self.ring, getattr(self, "_first_n", None), n)
        ex = self.exchange(layer, x_tagged)
        check(lib().nntr_cuda_gemv_nsplit_dev(QTYPE[qtype], n, K, x_ptr, w_ptr, C.byref(ex),
                                              capi.GEMV_PDL if pdl else 0, stream))

    def gathered_numpy(self, layer: int, n_local: int | None = None):
        """Host copy of the gathered vector launch ``layer`` produced (synchronising; for checks)."""
        import numpy as np
        raw = np.empty(2 * self.world * (self.n_local if n_local is None else n_local), dtype=np.float32)
        check(lib().nntr_cuda_memcpy(raw.ctypes.data, self.gathered_ptr(layer), raw.nbytes, 2))
        return np.ascontiguousarray(raw[0::2])  # drop the launch numbers

    def close(self) -> None:
        L = lib()
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        for p in self._opened:
            L.nntr_cuda_ipc_close(p)
        self._opened = []
        if self.world > 1:
            self.dist.barrier()
        for p in self._own:
            L.nntr_cuda_free(p)
        self._own = []
