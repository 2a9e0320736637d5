"""Builds ``oracle/_ref``: the reference's OWN host checkers, compiled here with g++.  TEST INFRASTRUCTURE ONLY.

The reference's translation units are HIP programs (device kernels on an external template library), so they
cannot be compiled as files.  Their host-side checkers, however, are plain C++/OpenMP.  This script cuts exactly
those functions -- unmodified, located by their signature and closed by brace matching -- out of a reference
checkout into a scratch directory, compiles ``ref_shim.cc`` (which includes them) twice, and deletes the scratch
directory again, so that only binaries remain:

    oracle/_ref/libref_strict.so   -O3 -fno-fast-math -ffp-contract=off   (IEEE evaluation order)
    oracle/_ref/libref_fast.so     -O3 -ffast-math                        (the flags of the reference's Makefiles)
    oracle/_ref/MANIFEST.json      which lines of which file went in, their SHA-256, the flags

``oracle/_ref`` is never committed.  The tests use it to check the C restatement (``oracle.c``) against the
reference's code on the same seeded inputs, and ``tests/golden/make_ref_golden.py`` uses it to produce the
committed fixtures that pin the restatement where no reference checkout is at hand.

Usage: ``python oracle/ref_build.py [reference_root]`` (default: the REFERENCE_ROOT environment variable).
"""
from __future__ import annotations

import hashlib
import json
import os
import re
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
DEFAULT_ROOTS = (os.environ.get("REFERENCE_ROOT"), "/root/reference")

# (output name, file within the reference, regex of the line that opens the function, take the `template<...>` line above it)
PIECES = [
    ("a8w8_valid_vector", "opus_gemm/gemm_a8w8_8wave.cc", r"^bool valid_vector\(const T\* ref", True),
    ("a8w8_gemm_ref", "opus_gemm/gemm_a8w8_8wave.cc", r"^void gemm_ref\(const host_fp8_t\* a", False),
    ("bs_valid_vector", "opus_gemm/block_scale_gemm/gemm_a8w8_blockscale_host.cc", r"^bool valid_vector\(const T\* ref", True),
    ("bs_gemm_ref", "opus_gemm/block_scale_gemm/gemm_a8w8_blockscale_host.cc", r"^void gemm_ref\(const host_fp8_t\* a", False),
    ("fmm_gemm_ref", "opus_fmm/flatmm_a8w8_gfx950.cc", r"^void gemm_ref\(const host_fp8_t\* a", False),
    ("fmm_shuffle_b", "opus_fmm/flatmm_a8w8_gfx950.cc", r"^void shuffle_b\(const DataType\* b_input", True),
    ("a16_gemm_ref", "opus_gemm/gemm_a16w16_8wave.cc", r"^void gemm_ref\(const bf16_t\* a", False),
    ("fmm16_gemm_ref", "opus_fmm/flatmm_a16w16_gfx950.cc", r"^void gemm_ref\(const bf16_t\* a", False),
    ("fmm16_shuffle_b", "opus_fmm/flatmm_a16w16_gfx950.cc", r"^void shuffle_b\(const DataType\* b_input", True),
]
# the two constants shuffle_b reads from its Traits argument, per flatmm program
TRAITS = [
    ("fmm_a8w8_traits", "opus_fmm/flatmm_a8w8_gfx950.cc"),
    ("fmm_a16w16_traits", "opus_fmm/flatmm_a16w16_gfx950.cc"),
]
STRICT = ["-O3", "-fno-fast-math", "-ffp-contract=off"]
FAST = ["-O3", "-ffast-math"]   # opus_gemm/block_scale_gemm/Makefile:5, opus_fmm/Makefile


def find_root(arg=None):
    for cand in (arg, *DEFAULT_ROOTS):
        if cand and os.path.isdir(os.path.join(cand, "opus_gemm")):
            return cand
    return None


def cut_function(lines, start_re, with_template):
    """Returns (first, last) 1-based inclusive line numbers of the function whose opening line matches."""
    hits = [i for i, l in enumerate(lines) if re.search(start_re, l)]
    if len(hits) != 1:
        raise RuntimeError(f"expected exactly one match of {start_re!r}, found {len(hits)}")
    first = hits[0]
    if with_template:
        if not lines[first - 1].lstrip().startswith("template"):
            raise RuntimeError(f"no template header above {start_re!r}")
        first -= 1
    depth, seen = 0, False
    for j in range(hits[0], len(lines)):
        for ch in lines[j]:
            if ch == "{":
                depth += 1
                seen = True
            elif ch == "}":
                depth -= 1
        if seen and depth == 0:
            return first + 1, j + 1
    raise RuntimeError(f"unbalanced braces after {start_re!r}")


def traits_constants(text):
    out = {}
    for name in ("W_N", "W_K"):
        m = re.search(r"static constexpr int %s\s*=\s*(\d+)\s*;" % name, text)
        if not m:
            raise RuntimeError(f"{name} not found")
        out[name] = int(m.group(1))
    return out


def build(reference_root=None, force=False, quiet=True):
    """Builds oracle/_ref from a reference checkout.  Returns the output directory, or None when no checkout exists."""
    root = find_root(reference_root)
    if root is None:
        return None
    manifest_path = os.path.join(OUT, "MANIFEST.json")
    shim = os.path.join(HERE, "ref_shim.cc")
    libs = [os.path.join(OUT, "libref_strict.so"), os.path.join(OUT, "libref_fast.so")]
    if not force and all(os.path.exists(p) for p in libs + [manifest_path]):
        newest_src = max(os.path.getmtime(shim), os.path.getmtime(os.path.abspath(__file__)))
        if min(os.path.getmtime(p) for p in libs) >= newest_src:
            return OUT
    scratch = os.path.join(OUT, "cut")
    os.makedirs(scratch, exist_ok=True)
    manifest = {"reference_root": root, "pieces": [], "traits": {}, "flags": {"strict": STRICT, "fast": FAST}}
    try:
        for name, rel, start_re, with_template in PIECES:
            with open(os.path.join(root, rel)) as f:
                lines = f.read().split("\n")
            first, last = cut_function(lines, start_re, with_template)
            body = "\n".join(lines[first - 1:last]) + "\n"
            with open(os.path.join(scratch, name + ".inc"), "w") as f:
                f.write(body)
            manifest["pieces"].append({"name": name, "file": rel, "lines": [first, last],
                                       "sha256": hashlib.sha256(body.encode()).hexdigest()})
        with open(os.path.join(scratch, "ref_traits.inc"), "w") as f:
            for struct, rel in TRAITS:
                with open(os.path.join(root, rel)) as src:
                    consts = traits_constants(src.read())
                manifest["traits"][struct] = dict(consts, file=rel)
                f.write("struct %s { static constexpr int W_N = %d; static constexpr int W_K = %d; };\n"
                        % (struct, consts["W_N"], consts["W_K"]))
        cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
        for lib, flags in zip(libs, (STRICT, FAST)):
            cmd = ["g++", "-std=c++17", "-fopenmp", "-fPIC", "-shared", "-Wall", "-Wno-unused-function", *flags,
                   "-I", scratch, "-I", cuda_inc, "-o", lib, shim]
            subprocess.check_call(cmd, stdout=subprocess.DEVNULL if quiet else None)
        with open(manifest_path, "w") as f:
            json.dump(manifest, f, indent=1)
    finally:
        shutil.rmtree(scratch, ignore_errors=True)     # the cut lines are reference source: binaries only stay
    return OUT


def available() -> bool:
    return all(os.path.exists(os.path.join(OUT, n)) for n in ("libref_strict.so", "libref_fast.so"))


if __name__ == "__main__":
    out = build(sys.argv[1] if len(sys.argv) > 1 else None, force=True, quiet=False)
    if out is None:
        print("no reference checkout found; oracle/_ref not built")
        sys.exit(1)
    with open(os.path.join(out, "MANIFEST.json")) as f:
        for p in json.load(f)["pieces"]:
            print("%-18s %s:%d-%d" % (p["name"], p["file"], p["lines"][0], p["lines"][1]))
