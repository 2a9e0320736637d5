"""GPU parity: batched GEMM with one B for every batch, per-batch ready words (B200_GEMM_BATCH_READY), the
stream-ordered flag write, and the stream rules of the skinny-M path (per-stream split-K workspaces, weights
written by the previous kernel of the stream)."""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import assert_close
from test_gpu_gemm import DEV, T, e4m3, status_ok

pytestmark = pytest.mark.gpu


def _slab_problem(O, batch, m, n, k, seed):
    """`batch` activation slabs laid out the way the sharded path moves them: slab s = [A rows | SFA [K/128][m]]."""
    kg = k // 128
    a = e4m3(O, (batch * m, k), seed, 0, 0.0, 1.0)
    b = e4m3(O, (n, k), seed, 1, -0.5, 0.5)
    sfa = O.fill_uniform((kg, batch * m), seed, 2, 0.8, 1.2)
    sfb = O.fill_uniform((n // 128, kg), seed, 3, 0.8, 1.2)
    slab_bytes = m * k + 4 * kg * m
    buf = np.zeros(batch * slab_bytes, np.uint8)
    for s in range(batch):
        base = s * slab_bytes
        buf[base:base + m * k] = a[s * m:(s + 1) * m].reshape(-1)
        buf[base + m * k:base + slab_bytes] = np.ascontiguousarray(sfa[:, s * m:(s + 1) * m]).view(np.uint8).reshape(-1)
    return a, b, sfa, sfb, buf, slab_bytes


def _views(buf_t, batch, m, k, slab_bytes):
    kg = k // 128
    a_v = torch.as_strided(buf_t, (batch, m, k), (slab_bytes, k, 1))
    sfa_v = torch.as_strided(buf_t.view(torch.float32), (batch, kg, m), (slab_bytes // 4, m, 1), storage_offset=m * k // 4)
    return a_v, sfa_v


@pytest.mark.parametrize("batch,m,n,k", [(3, 256, 512, 1024), (2, 384, 768, 512), (4, 512, 256, 256)])
def test_shared_b_batched_blockscale(api, O, batch, m, n, k):
    a, b, sfa, sfb, buf, slab_bytes = _slab_problem(O, batch, m, n, k, 41)
    a_v, sfa_v = _views(T(buf), batch, m, k, slab_bytes)
    out = torch.zeros(batch * m, n, dtype=torch.float32, device=DEV)
    api.gemm_a8w8_blockscale(a_v, T(b), sfa_v, T(sfb), out=out.view(batch, m, n))
    status_ok(api)
    assert_close(O, out.cpu().numpy(), O.gemm_ref_blockscale(a, b, sfa, sfb), "slabs as batches, shared B")


def test_shared_b_batched_unscaled_and_simple(api, O):
    batch, m, n, k = 3, 256, 384, 512
    a = e4m3(O, (batch, m, k), 42, 0, 0.0, 1.0)
    b = e4m3(O, (n, k), 42, 1, -0.5, 0.5)
    c = api.gemm_a8w8(T(a), T(b), out_dtype=torch.float32)
    cs = api.gemm_a8w8(T(a), T(b), out_dtype=torch.float32, simple=True)
    status_ok(api)
    ref = O.gemm_ref_nt(a.reshape(batch * m, k), b).reshape(batch, m, n)
    assert_close(O, c.cpu().numpy(), ref, "shared B, unscaled")
    assert np.array_equal(cs.cpu().numpy(), ref)            # the checker kernel repeats the host loop bit for bit


def test_batch_ready_words_set_beforehand_and_by_flag_write(api, O):
    batch, m, n, k = 4, 256, 512, 1024
    a, b, sfa, sfb, buf, slab_bytes = _slab_problem(O, batch, m, n, k, 43)
    a_v, sfa_v = _views(T(buf), batch, m, k, slab_bytes)
    ref = O.gemm_ref_blockscale(a, b, sfa, sfb)
    ready = torch.zeros(batch, dtype=torch.int32, device=DEV)
    # epoch 1: the words are written on the launching stream, before the launch
    for s in range(batch):
        api.flag_write(ready, s, 1)
    out = torch.zeros(batch, m, n, dtype=torch.float32, device=DEV)
    api.gemm_a8w8_blockscale(a_v, T(b), sfa_v, T(sfb), out=out, batch_ready=ready, batch_epoch=1)
    status_ok(api)
    assert ready.cpu().tolist() == [1] * batch
    assert_close(O, out.cpu().numpy().reshape(batch * m, n), ref, "ready words, epoch 1")
    # words only grow: a later epoch is satisfied by any larger value, no clearing in between
    ready.fill_(7)
    out.zero_()
    api.gemm_a8w8_blockscale(a_v, T(b), sfa_v, T(sfb), out=out, batch_ready=ready, batch_epoch=5)
    status_ok(api)
    assert_close(O, out.cpu().numpy().reshape(batch * m, n), ref, "ready words, epoch 5 <= 7")


def test_batch_that_never_arrives_ends_as_a_status_code(api, O):
    """A ready word that nothing sets: the launch gives up after its bounded wait (about 2 s), the status word says
    which wait it was, and the context stays usable."""
    batch, m, n, k = 2, 256, 256, 256
    a, b, sfa, sfb, buf, slab_bytes = _slab_problem(O, batch, m, n, k, 44)
    a_v, sfa_v = _views(T(buf), batch, m, k, slab_bytes)
    ready = torch.zeros(batch, dtype=torch.int32, device=DEV)
    api.flag_write(ready, 0, 1)                                     # slab 0 arrives, slab 1 never does
    out = torch.zeros(batch, m, n, dtype=torch.float32, device=DEV)
    api.gemm_a8w8_blockscale(a_v, T(b), sfa_v, T(sfb), out=out, batch_ready=ready, batch_epoch=1)
    torch.cuda.synchronize()
    assert api.peek_status() == 8
    assert api.last_status() == 8                                   # reported once, then cleared
    assert api.last_status() == 0
    api.flag_write(ready, 1, 1)
    api.gemm_a8w8_blockscale(a_v, T(b), sfa_v, T(sfb), out=out, batch_ready=ready, batch_epoch=1)
    status_ok(api)
    assert_close(O, out.cpu().numpy().reshape(batch * m, n), O.gemm_ref_blockscale(a, b, sfa, sfb), "after the timeout")


def test_split_k_decode_on_two_streams(api, O):
    """Two skinny-M GEMMs that both split K run on two streams at once: each stream has its own workspace."""
    probs = []
    for seed, (m, n, k) in ((51, (16, 1024, 8192)), (52, (8, 512, 8192))):
        a = e4m3(O, (m, k), seed, 0, 0.0, 1.0)
        b = e4m3(O, (n, k), seed, 1, -0.5, 0.5)
        sfa = O.fill_uniform((k // 128, m), seed, 2, 0.8, 1.2)
        sfb = O.fill_uniform((n // 128, k // 128), seed, 3, 0.8, 1.2)
        probs.append((a, b, sfa, sfb, [T(x) for x in (a, b, sfa, sfb)], torch.zeros(m, n, dtype=torch.float32, device=DEV)))
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    torch.cuda.synchronize()
    for rep in range(6):
        for st, (a, b, sfa, sfb, dev, out) in zip(streams, probs):
            with torch.cuda.stream(st):
                api.gemm_a8w8_blockscale(dev[0], dev[1], dev[2], dev[3], out=out)
    status_ok(api)
    for a, b, sfa, sfb, dev, out in probs:
        assert_close(O, out.cpu().numpy(), O.gemm_ref_blockscale(a, b, sfa, sfb), "split-K on its own stream")


def test_weights_written_by_the_previous_kernel_of_the_stream(api, O):
    """shuffle_b -> skinny-M GEMM back to back on one stream, weights changing every round: without
    B200_GEMM_INPUTS_READY the GEMM reads its weights only after the shuffle has completed."""
    m, n, k = 16, 2048, 2048
    a = e4m3(O, (m, k), 61, 0, 0.0, 1.0)
    ws = [e4m3(O, (k, n), 61, 1 + r, -0.5, 0.5) for r in range(3)]
    a_d = T(a)
    w_d = [T(w) for w in ws]
    flat = torch.empty(n * k, dtype=torch.uint8, device=DEV)
    outs = []
    from gcnasm_b200 import _lib as L

    for r in range(3):
        L.check(L.lib().b200_shuffle_b(w_d[r].data_ptr(), flat.data_ptr(), n, k, 1, C.c_void_p(torch.cuda.current_stream().cuda_stream)), "shuffle")
        outs.append(api.flatmm_a8w8(a_d, flat, n, out_dtype=torch.float32))
    status_ok(api)
    for r in range(3):
        assert_close(O, outs[r].cpu().numpy(), O.gemm_ref_kn(a, ws[r]), f"round {r}")


def test_host_entry_argument_errors_leave_the_device_alone(api, native, O):
    from gcnasm_b200 import _lib as L
    from gcnasm_b200._lib import GemmArgs

    m, n, k = 256, 256, 256
    a = e4m3(O, (m, k), 71, 0, 0.0, 1.0)
    b = e4m3(O, (n, k), 71, 1, -0.5, 0.5)
    c = np.zeros((m, n), np.float32)
    g = GemmArgs()
    g.ptr_a, g.ptr_b, g.ptr_c = a.ctypes.data, b.ctypes.data, c.ctypes.data
    g.m, g.n, g.k, g.batch = m, n, k, 1
    g.stride_a, g.stride_b, g.stride_c = k, k, n
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert native.b200_gemm_a8w8_host(C.byref(g), st) == 0
    assert_close(O, c, O.gemm_ref_nt(a, b), "host entry")
    for field, value, want in (("m", -5, L.ERR_BAD_ARG), ("stride_a", 100, L.ERR_BAD_ARG), ("k", 250, L.ERR_BAD_ARG),
                               ("ptr_b", 0, L.ERR_BAD_ARG), ("stride_c", 1 << 62, L.ERR_BAD_ARG)):
        bad = GemmArgs.from_buffer_copy(g)
        setattr(bad, field, value)
        rc = native.b200_gemm_a8w8_host(C.byref(bad), st)
        assert rc in (want, L.ERR_UNSUPPORTED), (field, rc)
    c[:] = 0
    assert native.b200_gemm_a8w8_host(C.byref(g), st) == 0          # the cached buffers are still there and valid
    assert_close(O, c, O.gemm_ref_nt(a, b), "host entry after rejected calls")


def test_slab_pipeline_single_gpu_all_sources(api, O):
    """ColumnShardedGemm's slab path on one GPU (a world of 1: no collective, the same kernels and ready words):
    device operands, bf16 activations through the fused quantiser, and pinned host operands through b200_slab_upload."""
    from gcnasm_b200.sharded import ColumnShardedGemm

    m, n, k, rows = 1024, 512, 1024, 256
    xb_w = O.fill_normal((n, k), 81, 1)
    qb, sfb = O.quant_128x128(xb_w)
    op = ColumnShardedGemm(T(qb), T(sfb), n, out_dtype=torch.float32)
    plan = op.plan_slabs(m, k, DEV, slab_rows=rows, nbuf=2)
    assert plan.slabs == 4 and plan.bytes_per_slab == api.lib().b200_slab_bytes(rows, k)
    out = torch.zeros(m, n, dtype=torch.float32, device=DEV)
    step = 0
    # (1) quantised operands on the device, three steps so that the ring of two buffers wraps
    for r in range(3):
        qa, sfa = O.quant_1x128(O.fill_normal((m, k), 82 + r, 0))
        op.step(step, out, a=T(qa), sfa=T(sfa))
        status_ok(api)
        assert_close(O, out.cpu().numpy(), O.gemm_ref_blockscale(qa, qb, sfa, sfb), f"device source, step {step}")
        step += 1
    # (2) bf16 activations: quantised slab by slab into the buffer (bit-exact against the oracle quantiser)
    bits = O.f32_to_bf16_bits(O.fill_normal((m, k), 90, 0) * 3.0)
    x = torch.from_numpy(bits.view(np.int16).copy()).to(DEV).view(torch.bfloat16)
    op.step(step, out, x_bf16=x)
    status_ok(api)
    qa, sfa = O.quant_1x128(O.bf16_bits_to_f32(bits))
    _, a3, sfa3 = op.slab_views(step % 2)
    assert np.array_equal(a3.reshape(m, k).cpu().numpy(), qa)
    assert np.array_equal(torch.cat(list(sfa3), dim=1).cpu().numpy(), sfa)
    assert_close(O, out.cpu().numpy(), O.gemm_ref_blockscale(qa, qb, sfa, sfb), "bf16 source")
    err, ref = op.check_rows(step, out, 256 + 64, 128)
    assert err <= 1e-2 * ref
    step += 1
    # (3) pinned host operands in the reference layouts: uploaded slab by slab on the side stream
    qa, sfa = O.quant_1x128(O.fill_normal((m, k), 91, 0))
    ha = torch.from_numpy(qa.copy()).pin_memory()
    hs = torch.from_numpy(sfa.copy()).pin_memory()
    op.step(step, out, a=ha, sfa=hs)
    status_ok(api)
    raw, a3, sfa3 = op.slab_views(step % 2)
    assert np.array_equal(a3.reshape(m, k).cpu().numpy(), qa)
    assert np.array_equal(torch.cat(list(sfa3), dim=1).cpu().numpy(), sfa)
    assert_close(O, out.cpu().numpy(), O.gemm_ref_blockscale(qa, qb, sfa, sfb), "host source")
