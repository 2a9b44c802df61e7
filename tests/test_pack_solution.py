"""The flashinfer-bench packaging: a flat solution/cuda folder that compiles on its own for
sm_100a and exports the reference's entry point (no GPU needed: compile and link only)."""
import importlib.util
import re
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _load_packer():
    spec = importlib.util.spec_from_file_location("pack_solution", ROOT / "fp8-moe-dev_b200" / "pack_solution.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_packed_solution_is_self_contained_and_builds(tmp_path):
    out = _load_packer().pack(tmp_path)
    cfg = (tmp_path / "config.toml").read_text()
    assert 'entry_point = "moe_fp8.cu::run"' in cfg and "destination_passing_style = true" in cfg
    names = {p.name for p in out.iterdir()}
    assert "moe_fp8.cu" in names
    for p in out.iterdir():   # every quoted include resolves inside the folder
        for inc in re.findall(r'#include\s+"([^"]+)"', p.read_text()):
            assert inc in names, f"{p.name} includes {inc}, which is not in the package"
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    tvm_ffi = pytest.importorskip("tvm_ffi")
    troot = Path(tvm_ffi.__file__).resolve().parent
    incs = ["-I", str(troot / "include"), "-I", str(troot / "3rdparty" / "dlpack" / "include")]
    cus = sorted(out.glob("*.cu"))

    def compile_one(src):
        obj = src.with_suffix(".o")
        r = subprocess.run([nvcc, "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler",
                            "-fPIC", *incs, "-c", str(src), "-o", str(obj)], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr[-2000:]
        return obj

    with ThreadPoolExecutor(4) as ex:
        objs = list(ex.map(compile_one, cus))
    so = tmp_path / "solution.so"
    r = subprocess.run([nvcc, "-shared", "-o", str(so), *map(str, objs), "-cudart", "static", "-L", str(troot / "lib"),
                        "-ltvm_ffi", "-lpthread", "-ldl", "-lrt"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    syms = subprocess.run(["nm", "-D", "--defined-only", str(so)], capture_output=True, text=True).stdout
    assert "__tvm_ffi_run" in syms and "moe_fp8_b200_run" in syms
