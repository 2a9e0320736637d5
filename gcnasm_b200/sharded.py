"""Column-parallel (N-sharded) block-scale GEMM over the GPUs of one node.

The reference has no multi-GPU code.  Output columns are independent (no reduction crosses N), so rank r
keeps ``B[r*N/R:(r+1)*N/R, :]`` with its 128x128 scale blocks and produces ``C[:, r*N/R:(r+1)*N/R]``.  The only
exchange is the activation: A and its 1x128 scales are broadcast from the root over NCCL once per call.
The result stays N-sharded; an all-gather into ``[R, M, N/R]`` is optional.  One process per GPU,
``torch.distributed`` supplies the process group (NCCL on GPUs; gloo in the CPU tests of the host logic).
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

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


class ColumnShardedGemm:
    """Holds one rank's weight shard; ``__call__`` broadcasts the activation and runs the local GEMM."""

    def __init__(self, b_shard: torch.Tensor, sfb_shard: torch.Tensor, n_total: int, group=None,
                 gemm_fn: Optional[Callable] = None, out_dtype=torch.bfloat16, quant_fn: Optional[Callable] = None):
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
        self._act_buf = None

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
        full = torch.empty((self.world, m, self.n1 - self.n0), dtype=out.dtype, device=out.device)
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
