"""GPU, two or more devices: the N-sharded GEMM with both slab deliveries (NCCL broadcasts, copy-engine chain) as
one process per GPU over NCCL, checked on every rank against the oracle.  Skipped on a single-GPU machine."""
import os
import socket

import numpy as np
import pytest
import torch

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, tmp, delivery):
    import sys

    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"              # plain peer transfers only
    import torch.distributed as dist

    from gcnasm_b200.sharded import ColumnShardedGemm, configure_overlap, shard_bounds

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    if delivery == "nccl":
        configure_overlap(world, torch.cuda.get_device_properties(dev).multi_processor_count)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from gcnasm_b200 import api
    from oracle import oracle as O

    m, n, k, rows = 1024, 512 * world, 1024, 256
    qb, sfb = O.quant_128x128(O.fill_normal((n, k), 7, 1))
    n0, n1 = shard_bounds(n, world, rank)
    T = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(dev)
    op = ColumnShardedGemm(T(qb[n0:n1]), T(sfb[n0 // 128:n1 // 128]), n, out_dtype=torch.float32, delivery=delivery)
    op.plan_slabs(m, k, dev, slab_rows=rows, nbuf=2)
    ok = op.delivery == delivery                      # no silent change of delivery on a machine that can do both
    out = torch.zeros(m, n1 - n0, dtype=torch.float32, device=dev)
    for step in range(5):                             # more steps than buffers: credits / buffer reuse are exercised
        qa, sfa = O.quant_1x128(O.fill_normal((m, k), 100 + step, 0))
        if step % 2 == 0:
            src = dict(a=T(qa), sfa=T(sfa)) if rank == 0 else {}
        else:                                         # pinned host source on the root
            src = dict(a=torch.from_numpy(qa.copy()).pin_memory(), sfa=torch.from_numpy(sfa.copy()).pin_memory()) if rank == 0 else {}
        op.step(step, out, **src)
        torch.cuda.synchronize()
        ref = O.gemm_ref_blockscale(qa, qb[n0:n1], sfa, sfb[n0 // 128:n1 // 128])
        err, mref = O.max_err(ref, out.cpu().numpy())
        ok = ok and err <= 1e-2 * mref
        # what travelled is byte-identical to what the root sent
        _, a3, sfa3 = op.slab_views(step % 2)
        ok = ok and np.array_equal(a3.reshape(m, k).cpu().numpy(), qa)
        ok = ok and np.array_equal(torch.cat(list(sfa3), dim=1).cpu().numpy(), sfa)
    ok = ok and api.last_status() == 0
    full = op.gather(out)
    ok = ok and tuple(full.shape) == (world, m, n1 - n0)
    open(os.path.join(tmp, f"ok{rank}"), "w").write("1" if ok else "0")
    dist.barrier()
    op.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("delivery", ["peer", "nccl"])
def test_sharded_gemm_on_all_gpus(tmp_path, O, native, delivery):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path), delivery), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"ok{r}").read() == "1", f"rank {r} ({delivery})"
