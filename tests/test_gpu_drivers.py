"""GPU: the three C++ host drivers keep the reference's command line and self-check."""
import os
import re
import subprocess

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu
BIN = os.path.join(ROOT, "gcnasm_b200", "bin")


@pytest.fixture(scope="module")
def drivers(native):
    from gcnasm_b200 import build

    build.build_drivers()
    return BIN


def run(drivers, name, *args):
    out = subprocess.run([os.path.join(drivers, name), *args, "--warmup", "5", "--iters", "10"], capture_output=True,
                         text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    return out.stdout


def test_gemm_a8w8_8wave_default_and_flags(drivers):
    out = run(drivers, "gemm_a8w8_8wave")                               # reference defaults: 256x512x256, batch 8
    assert "Launching GEMM kernel: M=256, N=512, K=256" in out
    assert out.count("VALID") >= 9 and "ALL BATCHES VALID" in out and "FAIL" not in out
    assert re.search(r"Kernel Performance: avg_time=\d+\.\d+ ms, \d+\.\d+ TFlops", out)
    out = run(drivers, "gemm_a8w8_8wave", "-m", "256", "-n", "512", "-k", "1024", "-b", "1", "--scale", "tensor", "--out", "bf16")
    assert "ALL BATCHES VALID" in out


def test_gemm_a8w8_8wave_rejects_bad_size(drivers):
    out = subprocess.run([os.path.join(drivers, "gemm_a8w8_8wave"), "-m", "0"], capture_output=True, text=True)
    assert out.returncode == 1 and "Invalid problem size" in out.stderr


def test_blockscale_driver(drivers):
    out = run(drivers, "gemm_a8w8_blockscale", "-m=512", "-n=768", "-k=1024", "-b=2", "-v=1")
    assert "Validating GPU results against CPU reference" in out and "ALL BATCHES VALID" in out
    out = run(drivers, "gemm_a8w8_blockscale", "-m", "512", "-n", "768", "-k", "1024", "-b", "1", "-v", "1", "--dist", "n01", "--out", "bf16")
    assert "ALL BATCHES VALID" in out
    out = run(drivers, "gemm_a8w8_blockscale", "-m", "256", "-n", "384", "-k", "512", "-b", "1", "-v", "1", "--scale", "mx")
    assert "ALL BATCHES VALID" in out
    out = run(drivers, "gemm_a8w8_blockscale", "-m", "256", "-n", "384", "-k", "512", "-b", "1")       # -v defaults to 0
    assert "VALID" not in out and "Kernel Performance" in out
    bad = subprocess.run([os.path.join(drivers, "gemm_a8w8_blockscale"), "-n", "500"], capture_output=True, text=True)
    assert bad.returncode == 1 and "multiples of GROUP_M/GROUP_N/GROUP_K" in bad.stderr


def test_flatmm_driver(drivers):
    out = run(drivers, "flatmm_a8w8")
    assert "Shuffling B matrix for FlatMM layout (batch=8)" in out and "BIT-EXACT" in out
    assert "Launching FlatMM kernel: M=256, N=512, K=256" in out and "ALL BATCHES VALID" in out
    out = run(drivers, "flatmm_a8w8", "-m", "16", "-n", "2304", "-k", "1024", "-b", "1", "--scale", "block", "--out", "bf16")
    assert "ALL BATCHES VALID" in out and "tile_config=3" in out


def test_flatmm_weight_file_round_trip(drivers, tmp_path):
    """--save-weights after the shuffle, then --load-weights instead of it: same self-check, no shuffle pass; the
    file is the reference's flat image plus the block scales."""
    from gcnasm_b200 import _lib as L
    from gcnasm_b200 import weights

    wfile = str(tmp_path / "decode.b2w")
    shape = ["-m", "16", "-n", "1024", "-k", "1024", "-b", "1", "--scale", "block", "--out", "bf16"]
    out = run(drivers, "flatmm_a8w8", *shape, "--save-weights", wfile)
    assert "BIT-EXACT" in out and "ALL BATCHES VALID" in out and f"Wrote {wfile}" in out
    info = weights.stat(wfile)
    assert (info.n, info.k, info.b_layout, info.scale_mode) == (1024, 1024, L.B_FLAT_16x16, L.SCALE_BLOCK)
    out = run(drivers, "flatmm_a8w8", *shape, "--load-weights", wfile)
    assert "no shuffle pass" in out and "Shuffling B" not in out and "ALL BATCHES VALID" in out and "FAIL" not in out
    # a file for another shape is refused
    bad = subprocess.run([os.path.join(drivers, "flatmm_a8w8"), "-m", "16", "-n", "2048", "-k", "1024", "-b", "1", "--scale", "block",
                          "--load-weights", wfile], capture_output=True, text=True)
    assert bad.returncode == 1 and "not what this run asks for" in bad.stderr


def test_gemm_a16w16_driver(drivers):
    out = run(drivers, "gemm_a16w16")                                   # reference defaults: 256x512x128, batch 8, bf16 out
    assert "Launching GEMM kernel: M=256, N=512, K=128" in out
    assert out.count("VALID") >= 9 and "ALL BATCHES VALID" in out and "FAIL" not in out
    assert re.search(r"Kernel Performance: avg_time=\d+\.\d+ ms, \d+\.\d+ TFlops", out)
    out = run(drivers, "gemm_a16w16", "--flat", "-m", "300", "-n", "1024", "-k", "512", "-b", "2")
    assert "BIT-EXACT" in out and "ALL BATCHES VALID" in out and "Launching FlatMM kernel" in out


def test_blockscale_driver_bf16_activations(drivers):
    """--act-bf16: activations handed over in bf16 and quantised by the fused kernel; the driver's host check (which
    reads the device-made operand and scales back) must still pass, for fp32 block scales and for MX."""
    out = run(drivers, "gemm_a8w8_blockscale", "-m", "512", "-n", "768", "-k", "1024", "-b", "2", "-v", "1", "--dist", "n01",
              "--act-bf16", "--out", "bf16")
    assert "fused quantiser" in out and "FAIL" not in out and out.count("VALID") >= 2
    out = run(drivers, "gemm_a8w8_blockscale", "-m", "300", "-n", "512", "-k", "512", "-b", "1", "-v", "1", "--scale", "mx",
              "--act-bf16")
    assert "fused quantiser" in out and "FAIL" not in out and "VALID" in out


def test_blockscale_driver_overlap_flag(drivers):
    """--overlap flags the benchmark loop's launches as independent; the self-check and the result lines stay the same."""
    out = run(drivers, "gemm_a8w8_blockscale", "-m", "1024", "-n", "1792", "-k", "1024", "-b", "1", "-v", "1", "--overlap")
    assert "FAIL" not in out and "VALID" in out
    assert re.search(r"Kernel Performance: avg_time=\d+\.\d+ ms, \d+\.\d+ TFlops", out)


def test_blockscale_driver_sharded_over_gpus(drivers):
    """--gpus R: one host process, B sharded along N, the activation pushed from GPU to GPU by the copy engines and
    consumed slab by slab through ready words; every shard is checked on its own GPU."""
    import torch

    gpus = min(torch.cuda.device_count(), 4)
    if gpus < 2:
        pytest.skip("needs at least two GPUs")
    out = run(drivers, "gemm_a8w8_blockscale", "--gpus", str(gpus), "-m", "1024", "-n", str(512 * gpus), "-k", "1024", "-b", "1",
              "-v", "1", "--out", "bf16", "--json")
    assert f"gpus={gpus}" in out and "ALL SHARDS VALID" in out and "FAIL" not in out
    assert out.count("VALID") == gpus + 1
    assert '"status": 0' in out
    bad = subprocess.run([os.path.join(drivers, "gemm_a8w8_blockscale"), "--gpus", "64", "-b", "1"], capture_output=True, text=True)
    assert bad.returncode == 1 and "CUDA device" in bad.stderr
