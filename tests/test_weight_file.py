"""CPU: the weight-file format (host code of libb200gemm.so): round trips, header contents, and every way a file
can be wrong -- truncated, flipped byte, foreign magic, buffers too small."""
import ctypes as C
import os

import numpy as np
import pytest

from gcnasm_b200 import _lib as L
from gcnasm_b200 import B200Error, weights


def _case(O, n, k, seed):
    w = O.fill_normal((n, k), seed, 0)
    q, sfb = O.quant_128x128(w)
    return q, sfb


def test_round_trip_block_scaled_flat(tmp_path, O):
    n, k = 256, 384
    q, sfb = _case(O, n, k, 31)
    flat = O.shuffle_b_nk(q)
    path = str(tmp_path / "w.b2w")
    weights.save(path, flat, sfb, n, k, b_layout=L.B_FLAT_16x16, scale_mode=L.SCALE_BLOCK)
    info = weights.stat(path)
    assert (info.n, info.k, info.b_layout, info.scale_mode) == (n, k, L.B_FLAT_16x16, L.SCALE_BLOCK)
    assert info.data_bytes == n * k and info.scale_bytes == 4 * (n // 128) * (k // 128)
    assert os.path.getsize(path) == 128 + n * k + info.scale_bytes           # n*k is a multiple of 64 here
    info2, data, scales = weights.load(path)
    assert info2 == info
    assert np.array_equal(data, flat) and np.array_equal(scales, sfb)
    # the flat image in the file is the reference's shuffle of the [N,K] operand
    assert np.array_equal(O.unshuffle_b(data, n, k).T, q)


def test_round_trip_other_scale_modes(tmp_path, O):
    n, k = 144, 128                          # n*k = 18432: padded to a multiple of 64 anyway; n not a multiple of 128
    q = O.cast_e4m3(O.fill_uniform((n, k), 32, 0, -2.0, 2.0))
    p = str(tmp_path / "plain.b2w")
    weights.save(p, q, None, n, k)
    info, data, scales = weights.load(p)
    assert scales is None and np.array_equal(data.reshape(n, k), q) and info.scale_mode == L.SCALE_NONE
    p = str(tmp_path / "tensor.b2w")
    weights.save(p, q, np.array([0.125], np.float32), n, k, scale_mode=L.SCALE_TENSOR)
    _, _, s = weights.load(p)
    assert s.tolist() == [0.125]
    p = str(tmp_path / "mx.b2w")
    atoms = np.arange(2 * 512, dtype=np.uint32).astype(np.uint8)             # ceil(144/128) * (128/128) atoms of 512 B
    weights.save(p, q, atoms, n, k, scale_mode=L.SCALE_MX)
    info, _, s = weights.load(p)
    assert info.scale_bytes == 1024 and np.array_equal(s, atoms)
    with pytest.raises(B200Error):                                           # block scales need N % 128 == 0
        weights.save(str(tmp_path / "bad.b2w"), q, np.zeros(4, np.float32), n, k, scale_mode=L.SCALE_BLOCK)


def test_padding_between_operand_and_scales(tmp_path, O):
    n, k = 16, 16 * 3                        # 768 bytes: already a multiple of 64 -> choose 16 x 16*5 = 1280 too
    for kk in (48, 80, 16):
        q = O.cast_e4m3(O.fill_uniform((n, kk), 33, 0, -1.0, 1.0))
        p = str(tmp_path / f"p{kk}.b2w")
        weights.save(p, q, np.array([2.0], np.float32), n, kk, scale_mode=L.SCALE_TENSOR)
        assert os.path.getsize(p) == 128 + (n * kk + 63) // 64 * 64 + 4
        _, data, s = weights.load(p)
        assert np.array_equal(data.reshape(n, kk), q) and s[0] == 2.0


def test_corruption_truncation_and_foreign_files(tmp_path, O):
    n, k = 128, 256
    q, sfb = _case(O, n, k, 34)
    path = str(tmp_path / "w.b2w")
    weights.save(path, q, sfb, n, k, scale_mode=L.SCALE_BLOCK)
    blob = bytearray(open(path, "rb").read())
    # one flipped operand byte -> checksum mismatch
    bad = bytearray(blob)
    bad[128 + 1000] ^= 0x10
    open(tmp_path / "flip.b2w", "wb").write(bad)
    with pytest.raises(B200Error) as e:
        weights.load(str(tmp_path / "flip.b2w"))
    assert e.value.code == L.ERR_CORRUPT
    # one flipped scale byte
    bad = bytearray(blob)
    bad[-1] ^= 0x01
    open(tmp_path / "flip2.b2w", "wb").write(bad)
    with pytest.raises(B200Error) as e:
        weights.load(str(tmp_path / "flip2.b2w"))
    assert e.value.code == L.ERR_CORRUPT
    # truncated
    open(tmp_path / "short.b2w", "wb").write(blob[:-5])
    with pytest.raises(B200Error) as e:
        weights.stat(str(tmp_path / "short.b2w"))
    assert e.value.code == L.ERR_IO
    # foreign magic, and a header whose sizes disagree
    bad = bytearray(blob)
    bad[0:4] = b"NOPE"
    open(tmp_path / "magic.b2w", "wb").write(bad)
    with pytest.raises(B200Error) as e:
        weights.stat(str(tmp_path / "magic.b2w"))
    assert e.value.code == L.ERR_BAD_ARG
    with pytest.raises(B200Error) as e:
        weights.stat(str(tmp_path / "missing.b2w"))
    assert e.value.code == L.ERR_IO
    # caller's buffers too small
    data = np.empty(n * k - 1, np.uint8)
    rc = L.lib().b200_weight_file_read(path.encode(), data.ctypes.data, data.nbytes, None, 0)
    assert rc == L.ERR_TOO_LARGE


def test_header_layout_is_fixed(tmp_path, O):
    """Byte offsets of the header fields (a file written today must stay readable)."""
    n, k = 128, 128
    q, sfb = _case(O, n, k, 35)
    path = str(tmp_path / "w.b2w")
    weights.save(path, q, sfb, n, k, scale_mode=L.SCALE_BLOCK)
    raw = open(path, "rb").read()
    assert raw[:8] == b"B200WGT1"
    assert np.frombuffer(raw, np.int32, 3, 8).tolist() == [1, L.B_NK_ROWMAJOR, L.SCALE_BLOCK]
    assert np.frombuffer(raw, np.int64, 4, 24).tolist() == [n, k, n * k, 4]
    h = 1469598103934665603
    for b in q.tobytes() + sfb.tobytes():
        h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    assert int(np.frombuffer(raw, np.uint64, 1, 56)[0]) == h
    assert C.sizeof(weights.WeightDesc) == 128


def test_overflowing_header_is_rejected(tmp_path, O):
    """A header whose N and K would overflow the size arithmetic (corrupt or hostile file) is a bad argument."""
    n, k = 128, 128
    q, sfb = _case(O, n, k, 36)
    path = str(tmp_path / "w.b2w")
    weights.save(path, q, sfb, n, k, scale_mode=L.SCALE_BLOCK)
    blob = bytearray(open(path, "rb").read())
    for nn, kk in ((1 << 62, 1 << 62), ((1 << 31) + 128, 128), (3 << 40, 3 << 22)):
        bad = bytearray(blob)
        bad[24:40] = np.array([nn, kk], np.int64).tobytes()
        bad[40:48] = np.array([(nn * kk) & 0x7FFFFFFFFFFFFFFF], np.int64).tobytes()      # whatever the product wraps to
        open(tmp_path / "huge.b2w", "wb").write(bad)
        with pytest.raises(B200Error) as e:
            weights.stat(str(tmp_path / "huge.b2w"))
        assert e.value.code == L.ERR_BAD_ARG
    rc = L.lib().b200_weight_file_write(str(tmp_path / "x.b2w").encode(), L.B_NK_ROWMAJOR, L.SCALE_NONE, 1 << 40, 1 << 40,
                                        q.ctypes.data, None)
    assert rc == L.ERR_BAD_ARG
