"""Slab delivery down a chain of GPUs by the copy engines (one process per GPU, no kernel, no SM).

The N-sharded GEMM needs the root's activation on every rank.  A ring broadcast by NCCL moves 18-26 GB/s per channel,
and every channel is a CTA that takes an SM from the persistent GEMM; the 138 MB activation of the 16384 x 57344 x 8192
problem then needs 1.1-1.9 ms around 8 ranks, longer than the 1.0 ms GEMM it should hide behind.  Here every rank
instead PUSHES each slab it holds into the next rank's activation buffer with a device-to-device copy (copy engines
over NVLink, about 25 us per 17 MB slab and hop), followed by a 4-byte copy into that rank's ready word.  A rank
forwards slab s as soon as its own ready word for s has arrived (a stream wait on the word), so the slabs stream down
the chain root -> root+1 -> ... one hop behind each other, and the consumer on every rank is the GEMM launch that waits
for the ready words (``B200_GEMM_BATCH_READY``).

Flow control: a rank may push the slabs of step i into buffer i % nbuf of its neighbour only when the neighbour has
finished with step i - nbuf in that buffer -- its GEMM has read it and its own forwarding has copied it on.  The
neighbour says so by copying the step number into the pusher's CREDIT word; the pusher's stream waits on that word.

Every rank owns one region of device memory that the neighbours map (``b200_ipc_alloc`` / ``b200_ipc_open``):

    [ nbuf x slabs x bytes_per_slab activation bytes | nbuf x slabs ready words | credit word | scratch words ]

All operations are expressed through three primitives on integer addresses -- ``copy(dst, src, nbytes)``,
``write(addr, value)``, ``wait(addr, value)`` -- queued on whatever stream is current; the CPU tests of this logic
replace them by eager stand-ins over host arrays.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Callable, Optional


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


@dataclass(frozen=True)
class RegionLayout:
    """Offsets inside a rank's shared region (identical on every rank)."""

    slabs: int
    bytes_per_slab: int
    nbuf: int

    @property
    def act_bytes(self) -> int:
        return self.nbuf * self.slabs * self.bytes_per_slab

    @property
    def ready_off(self) -> int:
        return _align(self.act_bytes)

    @property
    def credit_off(self) -> int:
        return _align(self.ready_off + 4 * self.nbuf * self.slabs)

    @property
    def scratch_off(self) -> int:
        return self.credit_off + 256

    @property
    def total_bytes(self) -> int:
        return self.scratch_off + 256

    def slab(self, buf: int, s: int) -> int:
        return (buf * self.slabs + s) * self.bytes_per_slab

    def ready(self, buf: int, s: int) -> int:
        return self.ready_off + 4 * (buf * self.slabs + s)


class CudaPeerOps:
    """The three primitives on the current CUDA stream, through the C ABI."""

    def __init__(self):
        import torch

        from . import _lib as L

        self._torch, self._L, self._lib = torch, L, L.lib()

    def _stream(self):
        return C.c_void_p(self._torch.cuda.current_stream().cuda_stream)

    def copy(self, dst: int, src: int, nbytes: int) -> None:
        self._L.check(self._lib.b200_stream_copy(C.c_void_p(dst), C.c_void_p(src), nbytes, self._stream()), "b200_stream_copy")

    def write(self, addr: int, value: int) -> None:
        self._L.check(self._lib.b200_flag_write(C.c_void_p(addr), value, self._stream()), "b200_flag_write")

    def wait(self, addr: int, value: int) -> None:
        self._L.check(self._lib.b200_flag_wait(C.c_void_p(addr), value, self._stream()), "b200_flag_wait")


class SlabChain:
    """One rank's part of the chain.  ``base`` is this rank's region, ``down`` / ``up`` the mapped regions of the next
    and the previous rank of the chain (None at the ends)."""

    def __init__(self, layout: RegionLayout, ops, base: int, down: Optional[int], up: Optional[int], is_root: bool):
        self.lay, self.ops = layout, ops
        self.base, self.down, self.up, self.is_root = base, down, up, is_root

    def forward(self, step: int, before_slab: Optional[Callable[[int], None]] = None) -> None:
        """Queue on the current (delivery) stream: this rank's share of moving the slabs of ``step`` down the chain.
        ``before_slab(s)`` is called on the root before slab s is touched (it makes the stream wait for whatever
        fills the slab)."""
        lay, ops = self.lay, self.ops
        buf, epoch = step % lay.nbuf, step + 1
        tmp = self.base + lay.scratch_off                       # a word of this rank that holds the epoch for the 4-byte copies
        if self.is_root:
            # the root's own GEMM: its slabs are local, their ready words are written first
            for s in range(lay.slabs):
                if before_slab is not None:
                    before_slab(s)
                ops.write(self.base + lay.ready(buf, s), epoch)
        if self.down is None:
            return
        if step >= lay.nbuf:
            # the neighbour must be done with what this buffer held before: step - nbuf
            ops.wait(self.base + lay.credit_off, step - lay.nbuf + 1)
        ops.write(tmp, epoch)
        for s in range(lay.slabs):
            if not self.is_root:
                ops.wait(self.base + lay.ready(buf, s), epoch)   # my copy of slab s has arrived
            ops.copy(self.down + lay.slab(buf, s), self.base + lay.slab(buf, s), lay.bytes_per_slab)
            ops.copy(self.down + lay.ready(buf, s), tmp, 4)      # ... and only then its ready word

    def credit(self, step: int) -> None:
        """Queue on the current (credit) stream, behind this rank's GEMM of ``step`` and its forwarding of ``step``:
        tell the previous rank that buffer ``step % nbuf`` may be overwritten."""
        if self.up is None:
            return
        tmp = self.base + self.lay.scratch_off + 64
        self.ops.write(tmp, step + 1)
        self.ops.copy(self.up + self.lay.credit_off, tmp, 4)


def chain_neighbours(rank: int, world: int, root: int):
    """(next rank, previous rank) of ``rank`` in the chain root, root+1, ... (mod world); None at the ends."""
    pos = (rank - root) % world
    down = (rank + 1) % world if pos + 1 < world else None
    up = (rank - 1) % world if pos > 0 else None
    return down, up
