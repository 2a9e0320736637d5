"""GPU: the HBM bandwidth probe reads every byte (word checksum, bit-exact) and copies bit-identically."""
import os
import re
import subprocess

import numpy as np
import pytest
import torch

from conftest import ROOT
from test_gpu_gemm import DEV

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nbytes", [16, 4096 + 16, 1 << 20, (1 << 20) * 37 + 48, 300 << 20])
def test_membw_read_checksum_and_copy(api, nbytes):
    g = torch.Generator(device="cpu").manual_seed(nbytes)
    src = torch.randint(-2**31, 2**31 - 1, (nbytes // 4,), dtype=torch.int32, generator=g).to(DEV)
    want = int(src.cpu().numpy().view(np.uint32).sum(dtype=np.uint64) & 0xFFFFFFFF)
    got = api.membw_read(src)
    assert int(got.cpu().numpy().view(np.uint32)[0]) == want
    again = api.membw_read(src, got)                     # accumulates
    assert int(again.cpu().numpy().view(np.uint32)[0]) == (2 * want) & 0xFFFFFFFF
    dst = torch.zeros_like(src)
    api.membw_copy(src, dst)
    assert torch.equal(src, dst)


def test_membw_rejects_ragged(api):
    from gcnasm_b200 import B200Error

    with pytest.raises(B200Error):
        api.membw_read(torch.zeros(5, dtype=torch.int32, device=DEV))          # 20 bytes


def test_bandwidth_driver_single_size():
    exe = os.path.join(ROOT, "gcnasm_b200", "bin", "bandwidth_memread")
    out = subprocess.run([exe, "67092480"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    lines = [l for l in out.stdout.splitlines() if "GB/s" in l]
    assert len(lines) == 2 and "[ro]" in lines[0] and "[rw]" in lines[1]
    for l in lines:
        gbs = float(re.search(r"([0-9.]+)\(GB/s\)", l).group(1))
        assert gbs > 500.0, l                      # a 256 MB stream on any working B200 is far above this
