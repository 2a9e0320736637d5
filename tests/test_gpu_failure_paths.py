"""GPU: failure paths that must end as a status, never as a hang or a stray write.

* a bounded device wait runs out (a barrier nothing signals, budget of a few milliseconds) -> status word, kernel
  returns, the context stays usable;
* canaries around and inside the output buffer stay untouched for ragged shapes on every kernel family.
No GPU is faulted, trapped or hung by these tests."""
import time

import numpy as np
import pytest
import torch

from test_gpu_gemm import DEV, T, assert_close, e4m3

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("polling", [0, 1])
def test_bounded_wait_runs_out_and_reports(api, native, O, polling):
    assert api.last_status() == 0
    t0 = time.time()
    rc = native.b200_selftest_bounded_wait(3000, polling, None)        # 3 ms budget
    assert rc == 0, "both waiting threads must give up and return"
    assert time.time() - t0 < 2.0
    assert api.last_status() == 7                                       # the self-test's code, reported once
    assert api.last_status() == 0
    # the context is still usable and the next GEMM is correct
    a, b = e4m3(O, (64, 256), 5, 0, 0.0, 1.0), e4m3(O, (128, 256), 5, 1, -0.5, 0.5)
    c = api.gemm_a8w8(T(a), T(b), out_dtype=torch.float32)
    assert_close(O, c.cpu().numpy(), O.gemm_ref_nt(a, b), "after the self-test")
    assert api.last_status() == 0
    assert native.b200_selftest_bounded_wait(10, 0, None) == -1         # budget out of range


CANARY = 0x7FC1                                                          # a bf16 NaN pattern no GEMM here produces


def _guarded(m, n, pad_cols, guard_rows):
    """bf16 output [m, n] inside a larger poisoned buffer: guard rows above and below, pad_cols after every row."""
    buf = torch.full((m + 2 * guard_rows, n + pad_cols), CANARY, dtype=torch.int16, device=DEV).view(torch.bfloat16)
    return buf, buf[guard_rows:guard_rows + m, :n]


def _check_canaries(buf, m, n, guard_rows):
    raw = buf.view(torch.int16).cpu().numpy().view(np.uint16)
    assert (raw[:guard_rows] == CANARY).all() and (raw[guard_rows + m:] == CANARY).all(), "rows outside C were written"
    assert (raw[guard_rows:guard_rows + m, n:] == CANARY).all(), "row padding was written"
    assert not (raw[guard_rows:guard_rows + m, :n] == CANARY).any(), "part of C was not written"


@pytest.mark.parametrize("m,n,k,tile", [
    (300, 384, 256, 4), (513, 640, 384, 4), (257, 896, 256, 7), (200, 384, 256, 8), (129, 256, 128, 6),   # pair tiles
    (100, 384, 256, 1), (130, 512, 256, 2),                                                               # single CTA
    (16, 384, 512, 3), (33, 1152, 1024, 3), (64, 256, 256, 3),                                            # decode
])
def test_block_scale_writes_only_c(api, O, m, n, k, tile):
    a, b = e4m3(O, (m, k), 6, 0, 0.0, 1.0), e4m3(O, (n, k), 6, 1, -0.5, 0.5)
    sfa = O.fill_uniform((k // 128, m), 6, 2, 0.8, 1.2)
    sfb = O.fill_uniform((n // 128, k // 128), 6, 3, 0.8, 1.2)
    buf, out = _guarded(m, n, pad_cols=24, guard_rows=3)                  # row pitch (n+24)*2 bytes: 16-byte multiple
    api.gemm_a8w8_blockscale(T(a), T(b), T(sfa), T(sfb), out=out, tile=tile)
    torch.cuda.synchronize()
    _check_canaries(buf, m, n, 3)
    assert_close(O, out.float().cpu().numpy(), O.gemm_ref_blockscale(a, b, sfa, sfb), f"guarded {m}x{n}x{k} tile {tile}")


@pytest.mark.parametrize("m,n,k,tile", [(300, 200, 272, 4), (140, 72, 144, 1), (1, 48, 64, 0), (40, 144, 528, 3)])
def test_unscaled_ragged_n_writes_only_c(api, O, m, n, k, tile):
    a, b = e4m3(O, (m, k), 7, 0, 0.0, 1.0), e4m3(O, (n, k), 7, 1, -0.5, 0.5)
    buf, out = _guarded(m, n, pad_cols=8, guard_rows=2)
    api.gemm_a8w8(T(a), T(b), out=out, tile=tile)
    torch.cuda.synchronize()
    _check_canaries(buf, m, n, 2)
    assert_close(O, out.float().cpu().numpy(), O.gemm_ref_nt(a, b), f"guarded unscaled {m}x{n}x{k}")
