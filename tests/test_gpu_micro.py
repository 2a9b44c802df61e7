"""Micro-benchmark of the grouped GEMM's MMA <-> promotion pipeline (tests/micro/gemm_pipeline_probe.cu),
compiled with nvcc and run on one SM: it gives the cycles per K block of each part of the loop in isolation
and guards the handshake of ptx.cuh (bounded waits, TMEM allocation and release) in isolation."""
import re
import shutil
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_gemm_pipeline_probe(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        pytest.skip("nvcc not available on this machine")
    exe = tmp_path / "probe"
    src = ROOT / "tests" / "micro" / "gemm_pipeline_probe.cu"
    subprocess.run([nvcc, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-I",
                    str(ROOT / "fp8-moe-dev_b200" / "csrc"), "-o", str(exe), str(src)], check=True, capture_output=True)
    r = subprocess.run([str(exe), "1", "4000"], capture_output=True, text=True, timeout=120)
    print(r.stdout)
    assert r.returncode == 0, r.stdout + r.stderr
    cyc = {m.group(1): float(m.group(2)) for m in re.finditer(r"^(\w+)\s+([\d.]+) cycles", r.stdout, re.M)}
    # a K block is 4 MMAs of 128 cycles: the tensor pipe's floor
    assert 500 <= cyc["mma_only"] <= 560, cyc
    assert cyc["drain"] < 700 and cyc["promote_packed"] <= cyc["promote_scalar"] + 1, cyc
    # 128-column instructions re-read A per half: no faster per column
    assert cyc["mma_only_n128"] >= cyc["mma_only"], cyc
    # the operand ring's barrier work on the issuing thread is not hidden by the tensor pipe ...
    assert cyc["ring"] > cyc["promote_packed"] + 100, cyc
    # ... and a second issuing thread takes most of it back (in this probe; the kernel itself did not gain from one)
    assert cyc["ring_scales_two"] < cyc["ring_scales"] - 100, cyc
    assert cyc["ring_scales_relayed"] < cyc["ring_scales"], cyc
    # a real TMA producer behind the ring (48 KB per K block) changes little: the data movement is not the cost
    assert abs(cyc["ring_scales_tma"] - cyc["ring_scales"]) < 60, cyc
    assert abs(cyc["ring_scales_two_tma"] - cyc["ring_scales_two"]) < 60, cyc
    # a row-scale load that misses L1, pending while the warp polls the accumulator barrier, holds the warp up
    # (issuing it two blocks ahead does not help); issued after the wait it is free again
    assert cyc["ring_far_tma"] > cyc["ring_scales_tma"] + 80, cyc
    assert cyc["ring_far2_two_tma"] > cyc["ring_scales_two_tma"] + 150, cyc
    assert cyc["ring_farlate_two_tma"] < cyc["ring_far_two_tma"] - 150, cyc
