"""Package the library as a flashinfer-bench CUDA solution: the layout the reference is
benchmarked in (README.md:133-155 of the reference: a runner workspace whose config.toml
names `entry_point = "moe_fp8.cu::run"`, `destination_passing_style = true`, and a flat
`solution/cuda/` folder that the runner compiles with tvm_ffi for sm_100a).

    python fp8-moe-dev_b200/pack_solution.py /path/to/runner

writes /path/to/runner/config.toml and /path/to/runner/solution/cuda/ holding this package's
CUDA sources, its headers (include paths flattened) and the TVM-FFI entry point under the file
name the runner expects.  Unlike the reference's solution it needs no CUTLASS include path, no
TRTLLM cubin path and no -lcuda: plain `nvcc -std=c++17 -gencode arch=compute_100a,code=sm_100a`
on every file, linked with -ltvm_ffi -ldl.
"""
from __future__ import annotations

import re
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
INCLUDE = HERE.parent / "include"
ENTRY_FILE = "moe_fp8.cu"   # the reference's entry point is moe_fp8.cu::run

CONFIG_TOML = """\
[build]
language = "cuda"
entry_point = "moe_fp8.cu::run"
destination_passing_style = true
"""


def _flatten_includes(text: str) -> str:
    """`#include "../../include/x.h"` -> `#include "x.h"`: everything sits in one folder."""
    return re.sub(r'#include\s+"(?:[^"]*/)?([^"/]+)"', r'#include "\1"', text)


def pack(dest) -> Path:
    dest = Path(dest)
    out = dest / "solution" / "cuda"
    out.mkdir(parents=True, exist_ok=True)
    files = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))
    for f in files:
        (out / f.name).write_text(_flatten_includes(f.read_text()))
    shim = (CSRC / "tvm_ffi_shim.cc").read_text()
    (out / ENTRY_FILE).write_text(_flatten_includes(shim))
    (dest / "config.toml").write_text(CONFIG_TOML)
    return out


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    print(pack(sys.argv[1]))
