"""CPU, world_size 2 over gloo: the host logic of the N-sharded GEMM (partitioning, activation broadcast,
optional all-gather).  The local GEMM is replaced by the oracle here -- this test covers the plumbing, the GPU
tests cover the kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def test_shard_bounds():
    from gcnasm_b200.sharded import shard_bounds

    assert shard_bounds(57344, 8, 3) == (21504, 28672)
    assert shard_bounds(7168, 1, 0) == (0, 7168)
    assert [shard_bounds(1024, 4, r) for r in range(4)] == [(0, 256), (256, 512), (512, 768), (768, 1024)]
    with pytest.raises(ValueError):
        shard_bounds(1000, 2, 0)          # 500 is not a whole number of 128-column scale blocks
    with pytest.raises(ValueError):
        shard_bounds(1024, 3, 0)
    with pytest.raises(ValueError):
        shard_bounds(1024, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, tmp):
    import sys

    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from gcnasm_b200.sharded import ColumnShardedGemm, shard_bounds
    from oracle import oracle as O

    m, n, k = 48, 512, 256
    a = O.cast_e4m3(O.fill_uniform((m, k), 3, 0, 0.0, 1.0))
    b = O.cast_e4m3(O.fill_uniform((n, k), 3, 1, -0.5, 0.5))
    sfa = O.fill_uniform((k // 128, m), 3, 2, 0.8, 1.2)
    sfb = O.fill_uniform((n // 128, k // 128), 3, 3, 0.8, 1.2)
    n0, n1 = shard_bounds(n, world, rank)

    def cpu_gemm(ta, tb, tsfa, tsfb, out):
        out.copy_(torch.from_numpy(O.gemm_ref_blockscale(ta.numpy(), tb.numpy(), tsfa.numpy(), tsfb.numpy())))

    op = ColumnShardedGemm(torch.from_numpy(b[n0:n1].copy()), torch.from_numpy(sfb[n0 // 128:n1 // 128].copy()), n,
                           gemm_fn=cpu_gemm, out_dtype=torch.float32)
    # only the root holds the activation; the others pass zero-filled buffers
    ta = torch.from_numpy(a.copy()) if rank == 0 else torch.zeros(m, k, dtype=torch.uint8)
    tsfa = torch.from_numpy(sfa.copy()) if rank == 0 else torch.zeros(k // 128, m)
    full = op(ta, tsfa, root=0, gather=True)
    assert np.array_equal(ta.numpy(), a) and np.array_equal(tsfa.numpy(), sfa)      # broadcast arrived
    ref = O.gemm_ref_blockscale(a, b, sfa, sfb)
    got = torch.cat([full[r] for r in range(world)], dim=1).numpy()
    ok = np.array_equal(got, ref)
    shard = op(ta, tsfa, broadcast=False)
    ok = ok and np.array_equal(shard.numpy(), ref[:, n0:n1])
    # bf16 activations: the root quantises into the single broadcast buffer, the others receive bytes + scales
    xf = O.fill_normal((m, k), 3, 4)
    xbits = O.f32_to_bf16_bits(xf)

    def cpu_quant(x, q, tsfa):
        qq, ss = O.quant_1x128(O.bf16_bits_to_f32(x.view(torch.int16).numpy().view(np.uint16)))
        q.copy_(torch.from_numpy(qq))
        tsfa.copy_(torch.from_numpy(ss))

    op2 = ColumnShardedGemm(torch.from_numpy(b[n0:n1].copy()), torch.from_numpy(sfb[n0 // 128:n1 // 128].copy()), n,
                            gemm_fn=cpu_gemm, out_dtype=torch.float32, quant_fn=cpu_quant)
    xb = torch.from_numpy(xbits.view(np.int16).copy()).view(torch.bfloat16) if rank == 0 else None
    shard2 = op2.forward_bf16(xb, m, k, "cpu", root=0)
    qa, sa = O.quant_1x128(O.bf16_bits_to_f32(xbits))
    ok = ok and np.array_equal(shard2.numpy(), O.gemm_ref_blockscale(qa, b, sa, sfb)[:, n0:n1])
    _, va, vs = op2.activation_buffer(m, k, "cpu")
    ok = ok and np.array_equal(va.numpy(), qa) and np.array_equal(vs.numpy(), sa)
    open(os.path.join(tmp, f"ok{rank}"), "w").write("1" if ok else "0")
    dist.barrier()
    dist.destroy_process_group()


def _worker_slabs(rank, world, port, tmp):
    """The slab pipeline's host logic on gloo: slab layout, ring of buffers, epochs, root-only sources."""
    import sys

    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from gcnasm_b200.sharded import ColumnShardedGemm, shard_bounds
    from oracle import oracle as O

    m, n, k, rows = 1024, 512, 256, 256           # 4 slabs
    b = O.cast_e4m3(O.fill_uniform((n, k), 5, 1, -0.5, 0.5))
    sfb = O.fill_uniform((n // 128, k // 128), 5, 3, 0.8, 1.2)
    n0, n1 = shard_bounds(n, world, rank)
    seen = []

    def cpu_slab_gemm(a3, tb, sfa3, tsfb, out3, ready, epoch):
        # what the kernel does: every slab's ready word must have reached the step's epoch before its bytes are read
        seen.append((ready.tolist(), epoch))
        assert all(int(v) >= epoch for v in ready.tolist())
        for s in range(a3.shape[0]):
            out3[s].copy_(torch.from_numpy(O.gemm_ref_blockscale(a3[s].contiguous().numpy(), tb.numpy(),
                                                                 sfa3[s].contiguous().numpy(), tsfb.numpy())))

    def cpu_quant(x, q, tsfa):
        qq, ss = O.quant_1x128(O.bf16_bits_to_f32(x.contiguous().view(torch.int16).numpy().view(np.uint16)))
        q.copy_(torch.from_numpy(qq))
        tsfa.copy_(torch.from_numpy(ss))

    def cpu_flag(ready, index, value):
        ready[index] = value

    op = ColumnShardedGemm(torch.from_numpy(b[n0:n1].copy()), torch.from_numpy(sfb[n0 // 128:n1 // 128].copy()), n,
                           out_dtype=torch.float32, slab_gemm_fn=cpu_slab_gemm, flag_fn=cpu_flag, quant_fn=cpu_quant)
    plan = op.plan_slabs(m, k, "cpu", slab_rows=rows, nbuf=2)
    ok = (plan.slabs, plan.bytes_per_slab) == (4, rows * k + 4 * (k // 128) * rows)
    out = torch.zeros(m, n1 - n0)
    for step in range(3):                          # three steps over two buffers: the ring wraps
        a = O.cast_e4m3(O.fill_uniform((m, k), 100 + step, 0, 0.0, 1.0))
        sfa = O.fill_uniform((k // 128, m), 100 + step, 2, 0.8, 1.2)
        src = dict(a=torch.from_numpy(a.copy()), sfa=torch.from_numpy(sfa.copy())) if rank == 0 else {}
        op.step(step, out, **src)
        ok = ok and np.array_equal(out.numpy(), O.gemm_ref_blockscale(a, b, sfa, sfb)[:, n0:n1])
        ok = ok and seen[-1] == ([step + 1] * 4, step + 1)
        # the slab layout itself: slab s = [rows of A | the slab's columns of SFA]
        raw, a3, sfa3 = op.slab_views(step % 2)
        ok = ok and np.array_equal(a3.reshape(m, k).numpy(), a)
        ok = ok and np.array_equal(torch.cat(list(sfa3), dim=1).numpy(), sfa)
        s1 = raw[1].numpy()
        ok = ok and np.array_equal(s1[:rows * k], a[rows:2 * rows].reshape(-1))
        ok = ok and np.array_equal(s1[rows * k:].view(np.float32).reshape(k // 128, rows), sfa[:, rows:2 * rows])
    # bf16 source: the root quantises slab by slab into the buffer
    xbits = O.f32_to_bf16_bits(O.fill_normal((m, k), 7, 4))
    xb = torch.from_numpy(xbits.view(np.int16).copy()).view(torch.bfloat16) if rank == 0 else None
    op.step(3, out, **(dict(x_bf16=xb) if rank == 0 else {}))
    qa, sa = O.quant_1x128(O.bf16_bits_to_f32(xbits))
    ok = ok and np.array_equal(out.numpy(), O.gemm_ref_blockscale(qa, b, sa, sfb)[:, n0:n1])
    full = op.gather(out)
    ok = ok and np.array_equal(torch.cat(list(full), dim=1).numpy(), O.gemm_ref_blockscale(qa, b, sa, sfb))
    if rank == 0:
        try:
            op.post(4)                             # the root without a source
            ok = False
        except ValueError:
            pass
    open(os.path.join(tmp, f"ok{rank}"), "w").write("1" if ok else "0")
    dist.barrier()
    dist.destroy_process_group()


def test_slab_pipeline_world2(tmp_path, O):
    world = 2
    mp.spawn(_worker_slabs, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"ok{r}").read() == "1"


def test_slab_geometry():
    from gcnasm_b200.sharded import pick_slab_rows, slab_bytes

    assert pick_slab_rows(16384) == 2048 and pick_slab_rows(4096) == 2048 and pick_slab_rows(4096, 1024) == 1024
    assert pick_slab_rows(768) == 768 and pick_slab_rows(1280) == 1280 and pick_slab_rows(2560) == 1280
    assert pick_slab_rows(300) == 300                        # no 256-multiple divides it: one slab
    assert slab_bytes(2048, 8192) == 2048 * 8192 + 64 * 2048 * 4
    with pytest.raises(ValueError):
        slab_bytes(2048, 8200)


def test_slab_bytes_matches_the_library(native):
    from gcnasm_b200.sharded import slab_bytes

    for rows, k in ((2048, 8192), (256, 128), (1024, 2048)):
        assert native.b200_slab_bytes(rows, k) == slab_bytes(rows, k)
    assert native.b200_slab_bytes(2048, 8200) == 0 and native.b200_slab_bytes(0, 128) == 0
    assert native.b200_slab_upload(None, None, None, 1, 128, 4, 0, None) == -1


def test_column_sharded_gemm_world2(tmp_path, O):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"ok{r}").read() == "1"


# ---- failures are made on the host: a rank that disagrees, a rank that leaves; nothing touches a GPU -----------
def _worker_disagree(rank, world, port, tmp):
    import sys

    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from gcnasm_b200.sharded import ColumnShardedGemm

    op = ColumnShardedGemm(torch.zeros(128, 256, dtype=torch.uint8), torch.zeros(1, 2), 256, gemm_fn=lambda *a: None,
                           quant_fn=lambda *a: None, out_dtype=torch.float32)
    k = 256 if rank == 0 else 384                     # rank 1 is about to run another problem
    try:
        op.forward_bf16(torch.zeros(16, k, dtype=torch.bfloat16), 16, k, "cpu", check=True)
        verdict = "no error"
    except ValueError as e:
        verdict = "ValueError" if "disagree" in str(e) else f"other: {e}"
    open(os.path.join(tmp, f"v{rank}"), "w").write(verdict)
    dist.barrier()
    dist.destroy_process_group()


def test_ranks_that_disagree_raise_on_every_rank(tmp_path):
    world = 2
    mp.spawn(_worker_disagree, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"v{r}").read() == "ValueError"


def _worker_leaves(rank, world, port, tmp):
    import datetime
    import sys
    import time

    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    from gcnasm_b200.sharded import ColumnShardedGemm

    dist.barrier()
    if rank == 1:
        os._exit(0)                                   # leaves between steps, with no collective of its own in flight
    op = ColumnShardedGemm(torch.zeros(128, 256, dtype=torch.uint8), torch.zeros(1, 2), 256, gemm_fn=lambda *a: None,
                           out_dtype=torch.float32)
    t0 = time.time()
    try:
        op(torch.zeros(16, 256, dtype=torch.uint8), torch.zeros(2, 16))
        verdict = "no error"
    except Exception as e:                            # gloo: connection closed by peer / timed out
        verdict = f"error after {time.time() - t0:.1f}s"
    open(os.path.join(tmp, "v0"), "w").write(verdict)
    os._exit(0)                                       # the group is broken: no orderly shutdown


def test_rank_that_leaves_ends_the_next_collective_with_an_error(tmp_path):
    """The survivor's next broadcast fails within the process-group timeout instead of waiting forever."""
    world = 2
    mp.spawn(_worker_leaves, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    verdict = open(tmp_path / "v0").read()
    assert verdict.startswith("error after"), verdict
    assert float(verdict.split()[2][:-1]) < 30.0
