"""B200 (sm_100a) FP8 block-scaled MoE layer: host-side mirror of the reference operator
on top of the C ABI in include/moe_fp8_b200.h.  Import name: fp8_moe_dev_b200 (the folder
name holds a hyphen, so the repo root's __graft_entry__.load_package() registers it)."""
from . import _lib  # noqa: F401
from .op import MoeError, MoeLayer, expert_loads, run  # noqa: F401
