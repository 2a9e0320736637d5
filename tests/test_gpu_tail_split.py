"""GPU parity of the split tail of the block-scale GEMM: the tiles of a partly filled last round of the persistent
schedule are computed as column parts (narrower MMAs over the full K) on otherwise idle CTA pairs.  Every element is
summed in the order of a whole tile, so the results must not depend on the split at all: checked against the oracle
on every element and bit for bit against the same problem on 256 x 128 tiles, which are never split."""
import numpy as np
import pytest
import torch

from conftest import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def T(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def inputs(O, m, n, k, seed):
    a = O.cast_e4m3(O.fill_uniform((m, k), seed, 0, 0.0, 1.0))
    b = O.cast_e4m3(O.fill_uniform((n, k), seed, 1, -0.5, 0.5))
    sfa = O.fill_uniform((k // 128, m), seed, 2, 0.8, 1.2)
    sfb = O.fill_uniform((n // 128, k // 128), seed, 3, 0.8, 1.2)
    return a, b, sfa, sfb


def done(api):
    torch.cuda.synchronize()
    assert api.last_status() == 0, "a bounded device wait expired"


def pairs(api):
    return api.lib().b200_sm_count() // 2


def expected_plan(api, m, n):
    tiles = ((m + 255) // 256) * ((n + 255) // 256)
    cap = pairs(api)
    full, rem = (tiles // cap) * cap, tiles % cap
    if not full or not rem:
        return None
    parts = 4 if rem * 4 <= cap else (2 if rem * 2 <= cap else 0)
    return (full, parts) if parts else None


# on 74 CTA pairs: 80 tiles -> 6 tail tiles in 4 parts; 98 tiles -> 24 tail tiles in 2 parts; ragged M edge; less than
# one round and 256 x 128 tiles are never split
@pytest.mark.parametrize("m,n,k,tile", [(2560, 2048, 512, 4), (1792, 3584, 512, 4), (2500, 2048, 640, 4), (512, 1024, 1024, 4),
                                        (2560, 2048, 512, 6)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_split_equals_whole(api, O, m, n, k, tile, out_dtype):
    a, b, sfa, sfb = inputs(O, m, n, k, 21)
    c = api.gemm_a8w8_blockscale(T(a), T(b), T(sfa), T(sfb), out_dtype=out_dtype, tile=tile)
    plan = api.last_tail_split()
    done(api)
    assert plan == (expected_plan(api, m, n) if tile == 4 else None)
    ref = O.gemm_ref_blockscale(a, b, sfa, sfb, out_bf16=out_dtype == torch.bfloat16)
    if out_dtype == torch.bfloat16:
        ref = O.bf16_bits_to_f32(ref)
    assert_close(O, c.float().cpu().numpy(), ref, f"tail {m}x{n}x{k}")
    # 256 x 128 tiles are never split: the same sums in the same order
    c6 = api.gemm_a8w8_blockscale(T(a), T(b), T(sfa), T(sfb), out_dtype=out_dtype, tile=6)
    assert api.last_tail_split() is None
    done(api)
    assert torch.equal(c, c6), "a split tile differs from a whole one"


def test_whole_rounds_then_tail(api, O):
    """80 tiles of 256 x 256: one whole round on the GPU's CTA pairs, then the remaining tiles as column parts; bf16
    through the bulk-store epilogue for the whole tiles and the staged stores for the parts."""
    m, n, k = 2560, 2048, 2048
    xa = O.fill_normal((m, k), 77, 0)
    xb = O.fill_normal((n, k), 77, 1)
    qa, sfa = O.quant_1x128(xa)
    qb, sfb = O.quant_128x128(xb)
    ref = O.bf16_bits_to_f32(O.gemm_ref_blockscale(qa, qb, sfa, sfb, out_bf16=True))
    outs = []
    for _ in range(3):
        c = api.gemm_a8w8_blockscale(T(qa), T(qb), T(sfa), T(sfb), out_dtype=torch.bfloat16, tile=4)
        plan = api.last_tail_split()
        done(api)
        outs.append(c)
    assert plan == expected_plan(api, m, n)
    assert_close(O, outs[0].float().cpu().numpy(), ref, "whole rounds + tail")
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    c6 = api.gemm_a8w8_blockscale(T(qa), T(qb), T(sfa), T(sfb), out_dtype=torch.bfloat16, tile=6)
    done(api)
    assert torch.equal(outs[0], c6)


def test_batched_shared_b_with_tail(api, O):
    """Slabs of A against one B (the sharded GEMM's launch): 5 x 4 x 4 = 80 tiles, the last 6 in parts."""
    B, m, n, k = 5, 1024, 1024, 512
    a = O.cast_e4m3(O.fill_uniform((B, m, k), 5, 0, 0.0, 1.0))
    b = O.cast_e4m3(O.fill_uniform((n, k), 5, 1, -0.5, 0.5))
    sfa = O.fill_uniform((B, k // 128, m), 5, 2, 0.8, 1.2)
    sfb = O.fill_uniform((n // 128, k // 128), 5, 3, 0.8, 1.2)
    c = api.gemm_a8w8_blockscale(T(a), T(b), T(sfa), T(sfb), out_dtype=torch.float32, tile=4).cpu().numpy()
    assert api.last_tail_split() == expected_plan(api, B * m, n)
    done(api)
    for i in range(B):
        assert_close(O, c[i], O.gemm_ref_blockscale(a[i], b, sfa[i], sfb), f"slab {i}")


def test_ragged_columns_and_strided_output(api, O):
    """N = 2176 leaves the last tile column with 128 valid columns (parts 2 and 3 of its tiles lie outside the matrix);
    the output is a view with a row pitch that is not a multiple of 16 bytes, so the parts take the scalar store path."""
    m, n, k = 2560, 2176, 512
    a, b, sfa, sfb = inputs(O, m, n, k, 41)
    ref = O.gemm_ref_blockscale(a, b, sfa, sfb)
    c = api.gemm_a8w8_blockscale(T(a), T(b), T(sfa), T(sfb), out_dtype=torch.float32, tile=4)
    assert api.last_tail_split() == expected_plan(api, m, n)
    done(api)
    assert_close(O, c.cpu().numpy(), ref, "ragged columns")
    wide = torch.full((m, n + 3), -7.0, dtype=torch.float32, device=DEV)
    api.gemm_a8w8_blockscale(T(a), T(b), T(sfa), T(sfb), out=wide[:, :n], tile=4)
    done(api)
    assert torch.equal(wide[:, :n], c) and torch.all(wide[:, n:] == -7.0)


def test_overlapped_launches_with_tail(api, O):
    """B200_GEMM_INPUTS_READY chains: launches that start while their predecessor drains, each with a split tail, writing
    the same C -- the last one wins, and nothing changes against launches in plain order."""
    m, n, k = 2560, 2048, 512
    sets = [[T(x) for x in inputs(O, m, n, k, 50 + j)] for j in range(3)]
    want = [api.gemm_a8w8_blockscale(*s, out_dtype=torch.bfloat16, tile=4) for s in sets]
    done(api)
    shared = torch.empty_like(want[0])
    for _ in range(3):
        for s in sets:
            api.gemm_a8w8_blockscale(*s, out=shared, tile=4, inputs_ready=True)
    done(api)
    assert torch.equal(shared, want[2])
