"""Head exchange over peer memory: landing buffers shared between the processes of one node (CUDA IPC) and the
one-kernel exchange of the library (`kvax_b200_head_exchange`).

Every rank owns one landing buffer per process group, used in two halves that alternate from exchange to
exchange.  An exchange is, on the stream of the caller: one kernel per tensor that stores this rank's part
straight into the peers' buffers in the layout the attention kernels read, a collective (everybody has
written), and a copy out of the landing buffer into ordinary tensors.  The half written now was read two
exchanges ago, and every rank has passed the collective of the exchange in between since then, after its
copy: nobody still reads it.  The kernels themselves wait for nobody.

If the buffers cannot be shared (no peer access between the GPUs, IPC not permitted in the container) every
rank learns so in the same collective and `exchange` returns None: the caller then takes the NCCL path.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from kvax_b200 import _lib

_arenas: dict = {}          # (group id, device index) -> PeerArena or False (sharing failed: do not try again)


class _RawCuda:
    """Device memory as an object torch.as_tensor can alias."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def _align(n: int) -> int:
    return (n + 255) // 256 * 256


class PeerArena:
    def __init__(self, group, device: torch.device, nbytes: int):
        lib = _lib.load()
        self.group, self.device, self.nbytes = group, device, nbytes
        self.cp = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.ptr = None
        self.peers: list[int] = []
        self.flag = torch.zeros(1, dtype=torch.int32, device=device)
        self.turn = 0                      # which half the next exchange lands in
        ok = 1
        handle = C.create_string_buffer(_lib.PEER_HANDLE_BYTES)
        with torch.cuda.device(device):
            p = C.c_void_p()
            if lib.kvax_b200_peer_buffer_alloc(nbytes, C.byref(p)) != 0 or not p.value:
                ok = 0
            else:
                self.ptr = p.value
                if lib.kvax_b200_peer_buffer_export(self.ptr, handle) != 0:
                    ok = 0
            handles = [None] * self.cp
            dist.all_gather_object(handles, handle.raw if ok else None, group=group)
            self.bases = (C.c_void_p * self.cp)()
            if ok and all(h is not None for h in handles):
                for r in range(self.cp):
                    if r == self.rank:
                        self.bases[r] = self.ptr
                        continue
                    q = C.c_void_p()
                    if lib.kvax_b200_peer_buffer_open(handles[r], C.byref(q)) != 0 or not q.value:
                        ok = 0
                        break
                    self.peers.append(q.value)
                    self.bases[r] = q.value
            else:
                ok = 0
            agreed = torch.tensor([ok], dtype=torch.int32, device=device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)
            self.ok = bool(int(agreed.item()))
            if self.ok:
                self.mem = torch.as_tensor(_RawCuda(self.ptr, nbytes), device=device)
            else:
                self.release()

    def release(self) -> None:
        """Collective: every rank first closes its views of the peers' buffers, then (after a barrier) frees its own --
        a buffer must not be freed while another process still has it open."""
        lib = _lib.load()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for q in self.peers:
                lib.kvax_b200_peer_buffer_close(q)
            self.peers = []
            dist.barrier(group=self.group)
            if self.ptr:
                lib.kvax_b200_peer_buffer_free(self.ptr)
                self.ptr = None

    def view(self, offset: int, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.mem[offset:offset + nbytes].view(dtype).view(shape)

    def barrier(self) -> None:
        """Orders the stream of every rank: what ran before it on any rank has completed when it completes."""
        dist.all_reduce(self.flag, group=self.group)


def _arena(group, device: torch.device, nbytes: int):
    key = (id(group), device.index)
    a = _arenas.get(key)
    if a is False:
        return None
    if a is not None and a.nbytes >= 2 * nbytes:
        return a
    if a is not None:                      # grow: every rank takes this branch together (same sizes everywhere)
        a.release()
    a = PeerArena(group, device, 2 * _align(nbytes + nbytes // 8))
    _arenas[key] = a if a.ok else False
    return a if a.ok else None


def exchange(tensors, to_heads: bool, cp: int, rank: int, group, permuted: bool, phase=None):
    """Head exchange of several batch-1 tensors at once.  to_heads: (1, S_loc, cp * Hl, D) -> (1, cp * S_loc, Hl, D)
    in natural token order; else the inverse.  Returns new tensors, or None when peer memory cannot be used."""
    import contextlib

    phase = phase or (lambda name: contextlib.nullcontext())
    lib = _lib.load()
    device = tensors[0].device
    offs, total = [], 0
    for x in tensors:
        offs.append(total)
        total += _align(x.numel() * x.element_size())
    arena = _arena(group, device, total)
    if arena is None:
        return None
    stream = torch.cuda.current_stream(device).cuda_stream
    outs_meta = []
    base = arena.turn * (arena.nbytes // 2)
    arena.turn ^= 1
    with phase("peer_push"), torch.cuda.device(device):
        for x, off in zip(tensors, offs):
            off += base
            x = x.contiguous()
            if to_heads:
                _, s_loc, heads, d = x.shape
                hl = heads // cp
                out_shape = (1, cp * s_loc, hl, d)
            else:
                _, s_all, hl, d = x.shape
                s_loc = s_all // cp
                out_shape = (1, s_loc, cp * hl, d)
            rc = lib.kvax_b200_head_exchange(x.data_ptr(), arena.bases, off, s_loc, cp, rank, hl, d * x.element_size(),
                                             int(permuted), int(to_heads), stream)
            _lib.check(rc, "kvax_b200_head_exchange")
            outs_meta.append((off, out_shape, x.dtype))
    with phase("peer_barrier"):
        arena.barrier()
    with phase("peer_copy_out"):
        return [arena.view(off, shape, dtype).clone() for off, shape, dtype in outs_meta]
