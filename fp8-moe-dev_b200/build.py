"""In-tree build of the CUDA library (sm_100a only).

`build()` compiles csrc/*.cu with nvcc into `libmoe_fp8_b200.so` next to this file and,
when the TVM-FFI headers are importable, the thin `__tvm_ffi_run` shim into
`libmoe_fp8_b200_tvm.so`.  Objects are rebuilt only when a source or header is newer.
The CUDA runtime is linked statically and the driver API is reached through
cudaGetDriverEntryPoint, so the library loads (and its symbols can be listed) on a
machine without a GPU driver.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
LIB = HERE / "libmoe_fp8_b200.so"
TVM_LIB = HERE / "libmoe_fp8_b200_tvm.so"
INCLUDE = HERE.parent / "include"

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]
CU_SOURCES = ["routing.cu", "gemm.cu", "moe_api.cu", "noalloc.cu", "quantize.cu", "decode.cu"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC")
    return cand


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def _run(cmd) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]} ({r.returncode})")


def build(verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h")) + [Path(__file__)]
    sources = [s for s in CU_SOURCES if (CSRC / s).exists()]
    objs = []
    for src in sources:
        o = OBJ / (src + ".o")
        if _stale(o, [CSRC / src] + headers):
            cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(INCLUDE), "-c", str(CSRC / src), "-o", str(o)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            _run(cmd)
        objs.append(o)
    if _stale(LIB, objs):
        _run([_nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static",
              "-Xlinker", "--no-undefined", "-lpthread", "-ldl", "-lrt"])
    build_tvm_shim()
    return LIB


def build_tvm_shim():
    """`__tvm_ffi_run` with the reference's 11-argument signature on top of the C ABI."""
    src = CSRC / "tvm_ffi_shim.cc"
    if not src.exists():
        return None
    try:
        import tvm_ffi  # noqa: F401
    except Exception:
        return None
    root = Path(tvm_ffi.__file__).resolve().parent
    inc, lib = root / "include", root / "lib"
    if not (inc / "tvm" / "ffi" / "function.h").exists():
        return None
    if _stale(TVM_LIB, [src, LIB, *INCLUDE.glob("*.h")]):
        dl = root / "3rdparty" / "dlpack" / "include"
        _run(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-o", str(TVM_LIB), str(src),
              "-I", str(INCLUDE), "-I", str(inc), "-I", str(dl), "-I", "/usr/local/cuda/include",
              "-L", str(HERE), "-l:libmoe_fp8_b200.so", "-L", str(lib), "-ltvm_ffi",
              f"-Wl,-rpath,{lib}", "-Wl,-rpath,$ORIGIN"])
    return TVM_LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
