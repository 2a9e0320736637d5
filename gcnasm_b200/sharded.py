"""Column-parallel (N-sharded) block-scale GEMM over the GPUs of one node.

The reference has no multi-GPU code.  Output columns are independent (no reduction crosses N), so rank r
keeps ``B[r*N/R:(r+1)*N/R, :]`` with its 128x128 scale blocks and produces ``C[:, r*N/R:(r+1)*N/R]``.  The only
exchange is the activation: A and its 1x128 scales are broadcast from the root over NCCL once per call.
The result stays N-sharded; an all-gather into ``[R, M, N/R]`` is optional.  One process per GPU,
``torch.distributed`` supplies the process group (NCCL on GPUs; gloo in the CPU tests of the host logic).

Two ways to run a call:

* ``op(a, sfa)`` / ``op.forward_bf16(x, ...)``: one broadcast of the whole activation, then the GEMM.
* ``op.step(i, ...)`` (``post`` + ``run``): the activation is cut into M slabs (``b200_slab_bytes``: each slab is one
  contiguous ``[rows x K bytes | K/128 x rows scales]`` piece).  The slabs are delivered one after the other on a
  side stream -- root: quantise or upload the slab; all: broadcast it; then a stream-ordered write of the slab's
  ready word -- while ONE persistent GEMM launch on the main stream consumes slab s as batch s as soon as its
  ready word shows the step's epoch (``B200_GEMM_BATCH_READY``).  Only the first slab's delivery is exposed, and
  with ``nbuf`` >= 2 activation buffers the delivery of step i+1 runs entirely behind the GEMM of step i.
"""
from __future__ import annotations

import contextlib
import os
from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n: int, world: int, rank: int, align: int = 128) -> Tuple[int, int]:
    """Columns [n0, n1) owned by ``rank``.  N/world must be a multiple of ``align`` (the scale block)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad world/rank")
    if n % world != 0 or (n // world) % align != 0:
        raise ValueError(f"N={n} does not split into {world} shards of whole {align}-column scale blocks")
    per = n // world
    return rank * per, (rank + 1) * per


def pick_slab_rows(m: int, want: int = 2048) -> int:
    """Rows per activation slab: the largest multiple of 256 (the GEMM's row tile) that divides M and is at most
    ``want``; M itself when there is none (one slab)."""
    best = 0
    for rows in range(256, min(m, want) + 1, 256):
        if m % rows == 0:
            best = rows
    return best or m


def slab_bytes(rows: int, k: int) -> int:
    """Bytes of one slab: rows x K e4m3 bytes followed by K/128 x rows fp32 scales (``b200_slab_bytes``)."""
    if k % 128 != 0 or rows % 4 != 0:
        raise ValueError("slabs need K % 128 == 0 and rows % 4 == 0")
    return rows * k + 4 * (k // 128) * rows


def default_comm_sms(world: int) -> int:
    """SMs to leave to NCCL beside the GEMM.  Measured on 8 x B200 (NVSwitch) with the 138 MB activation of the
    16384 x 57344 x 8192 problem: a ring broadcast moves 18-26 GB/s per channel (one CTA each), so 4 channels deliver the
    activation in 1.3 ms between 2 ranks but need 1.9 ms around 8, against GEMMs of 4.7 ms (2 ranks), 2.0 ms (4) and
    1.0-1.15 ms (8); 6 channels need 1.4 ms at 8 ranks, 8 channels 1.1 ms but cost the GEMM another round of tiles."""
    return 4 if world <= 2 else 6


def configure_overlap(world: int, sm_count: int = 148, comm_sms: Optional[int] = None) -> None:
    """Call before the process group is created.  The GEMM kernels are persistent -- one CTA per SM until the last
    tile -- so a collective that is to run BESIDE a GEMM needs SMs the GEMM does not occupy: the GEMM grid is capped at
    ``sm_count - comm_sms`` SMs and NCCL is held to ``comm_sms`` channels (one CTA each, no CTA clusters, so that any
    free SM will do).  Existing settings of the variables win."""
    if world <= 1:
        return
    if comm_sms is None:
        comm_sms = default_comm_sms(world)
    os.environ.setdefault("NCCL_MAX_NCHANNELS", str(comm_sms))
    os.environ.setdefault("NCCL_MIN_NCHANNELS", str(comm_sms))
    os.environ.setdefault("NCCL_CGA_CLUSTER_SIZE", "0")
    os.environ.setdefault("B200GEMM_MAX_SMS", str(sm_count - comm_sms))


class PeerDeliveryUnavailable(RuntimeError):
    """The GPUs of this job cannot map each other's memory (every rank raises it together)."""


@dataclass
class SlabPlan:
    m: int
    k: int
    rows: int            # rows per slab
    slabs: int
    bytes_per_slab: int
    nbuf: int


class ColumnShardedGemm:
    """Holds one rank's weight shard; ``__call__`` broadcasts the activation and runs the local GEMM."""

    def __init__(self, b_shard: torch.Tensor, sfb_shard: torch.Tensor, n_total: int, group=None,
                 gemm_fn: Optional[Callable] = None, out_dtype=torch.bfloat16, quant_fn: Optional[Callable] = None,
                 slab_gemm_fn: Optional[Callable] = None, flag_fn: Optional[Callable] = None,
                 upload_fn: Optional[Callable] = None, delivery: str = "nccl"):
        if delivery not in ("nccl", "peer"):
            raise ValueError("delivery is 'nccl' (slab broadcasts) or 'peer' (copy-engine pushes down a chain of GPUs)")
        self.delivery = delivery
        self.delivery_note = ""
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n0, self.n1 = shard_bounds(n_total, self.world, self.rank)
        if b_shard.shape[0] != self.n1 - self.n0:
            raise ValueError("weight shard has the wrong number of rows")
        if sfb_shard.shape[0] != (self.n1 - self.n0) // 128:
            raise ValueError("scale shard has the wrong number of block rows")
        self.b, self.sfb, self.n_total = b_shard, sfb_shard, n_total
        self.out_dtype = out_dtype
        if gemm_fn is None:
            from . import api

            gemm_fn = lambda a, b, sfa, sfb, out: api.gemm_a8w8_blockscale(a, b, sfa, sfb, out=out, out_dtype=self.out_dtype)
        self.gemm_fn = gemm_fn
        if quant_fn is None:
            def quant_fn(x, q, sfa):
                from . import api

                api.quantize_act_bf16_1x128(x, q=q, sfa=sfa)
        self.quant_fn = quant_fn
        # the three device-specific pieces of the slab path (replaced by host stand-ins in the CPU tests of the logic)
        if slab_gemm_fn is None:
            def slab_gemm_fn(a3, b, sfa3, sfb, out3, ready, epoch):
                from . import api

                api.gemm_a8w8_blockscale(a3, b, sfa3, sfb, out=out3, batch_ready=ready, batch_epoch=epoch)
        self.slab_gemm_fn = slab_gemm_fn
        if flag_fn is None:
            def flag_fn(ready, index, value):
                from . import api

                api.flag_write(ready, index, value)
        self.flag_fn = flag_fn
        if upload_fn is None:
            def upload_fn(a_host, sfa_host, buf, m, k, rows, slab):
                from . import _lib as L

                L.check(L.lib().b200_slab_upload(a_host.data_ptr(), sfa_host.data_ptr(), buf.data_ptr(), m, k, rows, slab,
                                                 torch.cuda.current_stream().cuda_stream), "b200_slab_upload")
        self.upload_fn = upload_fn
        self._act_buf = None
        self._plan: Optional[SlabPlan] = None
        self._bufs: List[torch.Tensor] = []
        self._ready: List[torch.Tensor] = []
        self._gemm_done: List[Optional[object]] = []
        self._posted: List[Optional[object]] = []
        self._comm = None
        self.overlap = True
        self._chain = None               # peer delivery: this rank's part of the chain (gcnasm_b200.peer.SlabChain)
        self._region = None              # ... and its shared region: (pointer, mapped neighbours)
        self._credit_stream = None
        self._fwd_done: List[Optional[object]] = []
        self._next_step = 0

    def check_agreement(self, m: int, k: int) -> None:
        """Host-side guard before a collective: every rank must be about to run the same (M, K).  A rank that
        disagrees would otherwise leave the others inside a broadcast of the wrong size; here all ranks raise."""
        if self.world == 1:
            return
        seen = [None] * self.world
        dist.all_gather_object(seen, (int(m), int(k)), group=self.group)
        if any(x != seen[0] for x in seen):
            raise ValueError(f"ranks disagree on the activation shape: {seen}")

    def broadcast_activation(self, a: torch.Tensor, sfa: torch.Tensor, root: int = 0):
        """A [M,K] e4m3 bytes and SFA [K/128, M]: valid on ``root``, allocated (same shape) elsewhere."""
        if self.world > 1:
            dist.broadcast(a, src=root, group=self.group)
            dist.broadcast(sfa, src=root, group=self.group)
        return a, sfa

    def __call__(self, a: torch.Tensor, sfa: torch.Tensor, root: int = 0, out: Optional[torch.Tensor] = None,
                 gather: bool = False, broadcast: bool = True):
        if broadcast:
            self.broadcast_activation(a, sfa, root)
        m = a.shape[0]
        if out is None:
            out = torch.empty((m, self.n1 - self.n0), dtype=self.out_dtype, device=a.device)
        self.gemm_fn(a, self.b, sfa, self.sfb, out)
        if not gather:
            return out
        return self.gather(out)

    def gather(self, out: torch.Tensor) -> torch.Tensor:
        """All-gather of the shards into ``[R, M, N/R]`` (rank r's columns are ``full[r]``)."""
        full = torch.empty((self.world,) + tuple(out.shape), dtype=out.dtype, device=out.device)
        if self.world > 1:
            dist.all_gather(list(full.unbind(0)), out.contiguous(), group=self.group)
        else:
            full[0] = out
        return full

    def activation_buffer(self, m: int, k: int, device) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """One flat buffer ``[M*K e4m3 bytes | (K/128)*M fp32 scales]`` and its two views.  Kept between calls."""
        need = m * k + 4 * (k // 128) * m
        if self._act_buf is None or self._act_buf.numel() != need or self._act_buf.device != torch.device(device):
            self._act_buf = torch.empty(need, dtype=torch.uint8, device=device)
        buf = self._act_buf
        return buf, buf[:m * k].view(m, k), buf[m * k:].view(torch.float32).view(k // 128, m)

    def forward_bf16(self, x: Optional[torch.Tensor], m: int, k: int, device, root: int = 0,
                     out: Optional[torch.Tensor] = None, gather: bool = False, check: bool = False):
        """bf16 activations ``x`` [M,K] (needed on ``root`` only) -> this rank's ``C[:, shard]``.

        The root quantises straight into the broadcast buffer (fused quantiser: one read of x, one write of the
        e4m3 bytes and of the scales in the GEMM's layout), the buffer travels as ONE broadcast, and every rank runs
        its GEMM on views of it: no fp32 copy of the activations, no separate scale tensor on the wire."""
        if m * k % 4 != 0:
            raise ValueError("M*K must be a multiple of 4 (the scales follow the bytes in one buffer)")
        if check:
            self.check_agreement(m, k)
        buf, a, sfa = self.activation_buffer(m, k, device)
        if self.rank == root:
            if x is None or tuple(x.shape) != (m, k):
                raise ValueError("the root needs the [M,K] activations")
            self.quant_fn(x, a, sfa)
        if self.world > 1:
            dist.broadcast(buf, src=root, group=self.group)
        return self(a, sfa, root=root, out=out, gather=gather, broadcast=False)

    # ------------------------------------------------------------------------------------------------------
    # slab pipeline
    # ------------------------------------------------------------------------------------------------------
    def plan_slabs(self, m: int, k: int, device, slab_rows: Optional[int] = None, nbuf: int = 2, root: int = 0) -> SlabPlan:
        """Allocates ``nbuf`` activation buffers in the slab layout and their ready words (one int32 per slab and
        buffer, never cleared: a step's epoch is its number + 1, and words only grow).  With peer delivery this is a
        collective call: the buffers live in a region the neighbours of the chain (which starts at ``root``) map."""
        rows = slab_rows or pick_slab_rows(m)
        if m % rows != 0:
            raise ValueError(f"M={m} is not a whole number of {rows}-row slabs")
        plan = SlabPlan(m, k, rows, m // rows, slab_bytes(rows, k), nbuf)
        device = torch.device(device)
        if self._plan != plan or not self._bufs or self._bufs[0].device != device:
            self.close()
            self._plan = plan
            self._next_step = 0
            peer = self.delivery == "peer" and device.type == "cuda" and self.world > 1
            if peer:
                try:
                    self._plan_peer_region(plan, device, root)
                except PeerDeliveryUnavailable as e:
                    # said out loud, not hidden: the slabs then travel by NCCL broadcasts (delivery_note tells the caller)
                    self.delivery, self.delivery_note, peer = "nccl", f"peer delivery unavailable ({e}); NCCL broadcasts instead", False
            if not peer:
                self._bufs = [torch.empty(plan.slabs * plan.bytes_per_slab, dtype=torch.uint8, device=device) for _ in range(nbuf)]
                self._ready = [torch.zeros(plan.slabs, dtype=torch.int32, device=device) for _ in range(nbuf)]
            self._gemm_done = [None] * nbuf
            self._posted = [None] * nbuf
            self._fwd_done = [None] * nbuf
            # high priority: when an SM frees up, a pending block of the delivery goes before a pending block of a GEMM
            self._comm = torch.cuda.Stream(device=device, priority=-1) if device.type == "cuda" else None
            self._credit_stream = torch.cuda.Stream(device=device, priority=-1) if peer else None
            # may a collective run BESIDE a GEMM that is waiting for it?  Only when the GEMM grid leaves SMs free
            # (configure_overlap); a single rank has no collective to starve, and peer delivery runs on the copy engines
            self.overlap = True
            if device.type == "cuda" and self.world > 1 and not peer:
                from . import _lib as L

                with torch.cuda.device(device):
                    self.overlap = L.lib().b200_sm_count() < torch.cuda.get_device_properties(device).multi_processor_count
        return plan

    def _plan_peer_region(self, plan: SlabPlan, device, root: int) -> None:
        import ctypes as C

        from . import _lib as L
        from .peer import CudaPeerOps, RegionLayout, SlabChain, chain_neighbours

        lay = RegionLayout(plan.slabs, plan.bytes_per_slab, plan.nbuf)
        down_rank, up_rank = chain_neighbours(self.rank, self.world, root)
        mapped = {}
        ptr, handle, why = C.c_void_p(), (C.c_ubyte * 64)(), ""
        with torch.cuda.device(device):
            # every rank goes through the same collectives whatever fails locally, then all agree on the outcome
            try:
                L.check(L.lib().b200_ipc_alloc(lay.total_bytes, C.byref(ptr), handle), "b200_ipc_alloc")
            except Exception as e:                                  # noqa: BLE001 (reported, and every rank falls back)
                why, ptr = str(e), C.c_void_p()
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle) if ptr.value else None, group=self.group)
            if not why and any(h is None for h in handles):
                why = "another rank could not allocate its region"
            if not why:
                try:
                    for r in {down_rank, up_rank} - {None}:
                        p = C.c_void_p()
                        L.check(L.lib().b200_ipc_open((C.c_ubyte * 64).from_buffer_copy(handles[r]), C.byref(p)), "b200_ipc_open")
                        mapped[r] = p.value
                except Exception as e:                              # noqa: BLE001
                    why = str(e)
            reasons = [None] * self.world
            dist.all_gather_object(reasons, why, group=self.group)
            if any(reasons):
                for p in mapped.values():
                    L.lib().b200_ipc_close(p)
                dist.barrier(group=self.group)
                if ptr.value:
                    L.lib().b200_ipc_free(ptr)
                raise PeerDeliveryUnavailable("; ".join(f"rank {i}: {w}" for i, w in enumerate(reasons) if w))

        class _Raw:                                                 # a torch tensor over the region, without a copy
            __cuda_array_interface__ = {"shape": (lay.total_bytes,), "typestr": "|u1", "data": (ptr.value, False), "version": 2}

        whole = torch.as_tensor(_Raw(), device=device)
        whole.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)                              # nobody pushes into a region that is still being cleared
        per = plan.slabs * plan.bytes_per_slab
        self._bufs = [whole[i * per:(i + 1) * per] for i in range(plan.nbuf)]
        words = whole[lay.ready_off:lay.ready_off + 4 * plan.nbuf * plan.slabs].view(torch.int32)
        self._ready = [words[i * plan.slabs:(i + 1) * plan.slabs] for i in range(plan.nbuf)]
        self._region = (ptr.value, mapped, whole)
        self._chain = SlabChain(lay, CudaPeerOps(), ptr.value, mapped.get(down_rank), mapped.get(up_rank), self.rank == root)
        self._chain_root = root

    def close(self) -> None:
        """Releases the peer-mapped region (a collective call when peer delivery is in use; a no-op otherwise)."""
        if self._region is None:
            return
        from . import _lib as L

        ptr, mapped, whole = self._region
        torch.cuda.synchronize(whole.device)
        dist.barrier(group=self.group)                              # every rank has stopped pushing
        self._bufs, self._ready, self._chain, self._region = [], [], None, None
        del whole
        with torch.cuda.device(self._comm.device):
            for p in mapped.values():
                L.lib().b200_ipc_close(p)
            dist.barrier(group=self.group)                          # ... and unmapped, before the owner frees
            L.lib().b200_ipc_free(ptr)
        self._plan = None

    def slab_views(self, buf_index: int):
        """(bytes [slabs, bytes_per_slab], A [slabs, rows, K], SFA [slabs, K/128, rows]) over activation buffer ``buf_index``."""
        p = self._plan
        buf = self._bufs[buf_index]
        kg = p.k // 128
        a3 = torch.as_strided(buf, (p.slabs, p.rows, p.k), (p.bytes_per_slab, p.k, 1))
        fbuf = buf.view(torch.float32)                     # (a buffer may itself be a slice of a larger region)
        sfa3 = torch.as_strided(fbuf, (p.slabs, kg, p.rows), (p.bytes_per_slab // 4, p.rows, 1),
                                storage_offset=fbuf.storage_offset() + p.rows * p.k // 4)
        return buf.view(p.slabs, p.bytes_per_slab), a3, sfa3

    def _on_comm(self):
        return torch.cuda.stream(self._comm) if self._comm is not None else contextlib.nullcontext()

    def post(self, step: int, *, a: Optional[torch.Tensor] = None, sfa: Optional[torch.Tensor] = None,
             x_bf16: Optional[torch.Tensor] = None, prefilled: bool = False, root: int = 0) -> None:
        """Delivers the activation of ``step`` slab by slab on the side stream (returns at once on a GPU).

        The root's source -- exactly one of: ``x_bf16`` [M,K] (device; quantised slab by slab by the fused quantiser),
        ``a`` + ``sfa`` on the device (already quantised, reference layouts: copied into the slabs), ``a`` + ``sfa``
        in pinned HOST memory (uploaded slab by slab), or ``prefilled=True`` (the caller has written the slabs of
        buffer ``step % nbuf`` itself through ``slab_views``, on the current stream) -- is ignored on the other ranks.
        Every slab is then broadcast, and its ready word is written behind the broadcast."""
        p = self._plan
        if p is None:
            raise RuntimeError("plan_slabs() first")
        buf_index = step % p.nbuf
        epoch = step + 1
        raw, a3, sfa3 = self.slab_views(buf_index)
        ready = self._ready[buf_index]
        is_root = self.rank == root
        if is_root and not prefilled and x_bf16 is None and (a is None or sfa is None):
            raise ValueError("the root needs the activation: x_bf16, a and sfa, or prefilled slabs")
        on_gpu = self._comm is not None
        from_host = is_root and not prefilled and x_bf16 is None and a.device.type == "cpu" and on_gpu
        filled: List[Optional[object]] = [None] * p.slabs
        if on_gpu and self._gemm_done[buf_index] is not None:
            # the buffer was last read by the GEMM of step - nbuf
            torch.cuda.current_stream().wait_event(self._gemm_done[buf_index])
            self._comm.wait_event(self._gemm_done[buf_index])
        if is_root and prefilled and on_gpu:
            self._comm.wait_stream(torch.cuda.current_stream())
        if is_root and not from_host and not prefilled:
            # Slabs that a KERNEL produces (the fused quantiser, a device copy) are filled on the caller's stream, ahead
            # of the GEMM launch that will consume them: a persistent GEMM that is already spinning on a ready word
            # occupies its SMs until the word arrives, and a producer kernel queued behind it on another stream could
            # wait for an SM forever.  Copies by the copy engines and NCCL (which has SMs set aside, see
            # configure_overlap) have no such dependency and run on the side stream.
            for s in range(p.slabs):
                r0, r1 = s * p.rows, (s + 1) * p.rows
                if x_bf16 is not None:
                    self.quant_fn(x_bf16[r0:r1], a3[s], sfa3[s])
                else:
                    a3[s].copy_(a[r0:r1], non_blocking=True)
                    sfa3[s].copy_(sfa[:, r0:r1], non_blocking=True)
                if on_gpu:
                    filled[s] = torch.cuda.Event()
                    filled[s].record()
        if self._chain is not None:
            if root != self._chain_root:
                raise ValueError("peer delivery was planned for another root")

            def before_slab(s):
                if from_host:
                    self.upload_fn(a, sfa, self._bufs[buf_index], p.m, p.k, p.rows, s)
                elif filled[s] is not None:
                    self._comm.wait_event(filled[s])

            with self._on_comm():
                self._chain.forward(step, before_slab if is_root else None)
                self._fwd_done[buf_index] = torch.cuda.Event()
                self._fwd_done[buf_index].record()
            return
        with self._on_comm():
            for s in range(p.slabs):
                if from_host:
                    self.upload_fn(a, sfa, self._bufs[buf_index], p.m, p.k, p.rows, s)
                if filled[s] is not None:
                    self._comm.wait_event(filled[s])
                if self.world > 1:
                    dist.broadcast(raw[s], src=root, group=self.group)
                self.flag_fn(ready, s, epoch)
            if on_gpu and not self.overlap:
                self._posted[buf_index] = torch.cuda.Event()
                self._posted[buf_index].record()

    def run(self, step: int, out: torch.Tensor) -> torch.Tensor:
        """One GEMM launch over all slabs of ``step`` (slab s = batch s, the shard's B shared by all batches); the
        kernel itself waits for each slab's ready word.  ``out``: ``[M, N/R]``, contiguous."""
        p = self._plan
        buf_index = step % p.nbuf
        _, a3, sfa3 = self.slab_views(buf_index)
        n = self.n1 - self.n0
        if tuple(out.shape) != (p.m, n) or not out.is_contiguous():
            raise ValueError("out must be a contiguous [M, N/R] tensor")
        if self._comm is not None and not self.overlap and self._posted[buf_index] is not None:
            # no SMs are set aside for the collective: a GEMM spinning on a ready word could starve the very
            # broadcast it waits for, so the launch is ordered behind the whole delivery instead
            torch.cuda.current_stream().wait_event(self._posted[buf_index])
        self.slab_gemm_fn(a3, self.b, sfa3, self.sfb, out.view(p.slabs, p.rows, n), self._ready[buf_index], step + 1)
        if self._comm is not None:
            ev = torch.cuda.Event()
            ev.record()
            self._gemm_done[buf_index] = ev
        if self._chain is not None:
            # this rank is done with the buffer once its GEMM has read it and its forwarding has copied it on
            with torch.cuda.stream(self._credit_stream):
                self._credit_stream.wait_event(self._gemm_done[buf_index])
                if self._fwd_done[buf_index] is not None:
                    self._credit_stream.wait_event(self._fwd_done[buf_index])
                self._chain.credit(step)
        return out

    def step(self, step: int, out: torch.Tensor, **source) -> torch.Tensor:
        """``post(step, **source)`` then ``run(step, out)``."""
        self.post(step, **source)
        return self.run(step, out)

    def forward_slabs(self, out: torch.Tensor, **source) -> torch.Tensor:
        """The slab pipeline with the step numbering kept here: call k of this method is step k (``plan_slabs`` first).
        ``source`` as for ``post`` (needed on the root only)."""
        step = self._next_step
        self._next_step += 1
        return self.step(step, out, **source)

    def check_rows(self, step: int, out: torch.Tensor, row0: int, rows: int = 128):
        """Recomputes ``rows`` output rows starting at ``row0`` (inside one slab) of this rank's shard with the
        one-thread-per-output checker kernel (the device mirror of the reference's host loop) from the activation
        buffer of ``step``, and returns (max|err|, max|ref|) against ``out``."""
        from . import api

        p = self._plan
        _, a3, sfa3 = self.slab_views(step % p.nbuf)
        s, r = divmod(row0, p.rows)
        if r + rows > p.rows:
            raise ValueError("the checked rows must lie inside one slab")
        ref = api.gemm_a8w8_blockscale(a3[s, r:r + rows], self.b, sfa3[s][:, r:r + rows], self.sfb, out_dtype=torch.float32,
                                       simple=True)
        got = out[row0:row0 + rows].float()
        return float((got - ref).abs().max().item()), float(ref.abs().max().item())
