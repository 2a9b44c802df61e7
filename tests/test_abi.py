"""C-ABI checks that need no GPU: the library loads, exports every symbol the header
declares, and its host-only entry points behave."""
import ctypes as C
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    names = []
    for h in sorted((ROOT / "include").glob("*.h")):
        txt = h.read_text()
        names += re.findall(r"MOE_FP8_B200_API\s+[\w\s\*]+?\b(moe_fp8_b200_\w+)\s*\(", txt)
    return names


def test_header_declares_the_path():
    names = declared_symbols()
    for must in ("moe_fp8_b200_create", "moe_fp8_b200_run", "moe_fp8_b200_run_host", "moe_fp8_b200_destroy"):
        assert must in names


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg._lib.load()
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"
    for name in pkg._lib.EXPORTS:
        assert name in declared_symbols()


def test_version_and_sizing(pkg):
    lib = pkg._lib.load()
    assert lib.moe_fp8_b200_version() >= 1
    for T, E in ((1, 32), (16, 32), (1024, 32), (12288, 256), (16384, 32)):
        cap = lib.moe_fp8_b200_row_capacity(T, E)
        assert cap % 128 == 0
        # every (token, expert) pair plus up to 127 pad rows per non-empty expert must fit
        assert cap >= 8 * T + 127 * min(E, 8 * T)
        ws = lib.moe_fp8_b200_workspace_bytes(T, E)
        # A1 + A2 + Y rows dominate: 7168 + 2048 + 2*7168 bytes each
        assert ws >= cap * (7168 + 2048 + 14336)
        assert ws < cap * (7168 + 2048 + 14336) * 1.2 + (1 << 22)
    assert lib.moe_fp8_b200_workspace_bytes(0, 32) == 0
    assert lib.moe_fp8_b200_row_capacity(16, 1000) == 0


def test_reference_policy_matches_oracle_restatement(pkg, oracle):
    """Two independent restatements of kernel/moe_fp8.cu:508-591, 2732-2790 (product host code
    and oracle) agree for every T the reference special-cases and a sweep around them."""
    special = [1, 2, 7, 14, 15, 16, 31, 32, 33, 52, 53, 54, 55, 56, 57, 58, 59, 62, 80, 81, 900, 901, 902, 1024,
               2048, 2049, 9999, 10000, 11948, 12288, 12999, 13000, 14107, 14108, 16384, 20000]
    for T in special + list(range(1, 200)):
        got = pkg._lib.reference_policy(T)
        want = oracle.policy(T, True).as_dict()
        for k, v in want.items():
            assert got[k] == pytest.approx(v, abs=0), (T, k, got[k], v)


def test_policy_known_answers(pkg):
    p = pkg._lib.reference_policy
    assert p(1)["prune"] == 0 and p(1)["skip_zero_weight"] == 0
    assert p(16)["prune"] == 0 and p(16)["skip_zero_weight"] == 1
    assert p(15)["prune"] == 1
    assert p(1024)["prune"] == 1 and p(1024)["drop_third"] == 0 and p(1024)["renorm"] == 1
    assert p(12288)["drop_third"] == 1 and abs(p(12288)["drop_third_frac"] - 0.34) < 1e-7
    assert p(16384)["drop_third"] == 1 and abs(p(16384)["drop_third_frac"] - 0.30) < 1e-7
    q = p(14107)
    assert q["renorm"] == 0 and abs(q["drop_second_frac_2"] - 0.302) < 1e-7 and abs(q["drop_second_frac_ge3"] - 0.303) < 1e-7
    assert abs(p(901)["drop_third_frac"] - 0.24) < 1e-7 and abs(p(901)["drop_second_frac_2"] - 0.245) < 1e-7
    assert p(32)["drop_second_frac_2"] == 0.0 and abs(p(32)["drop_third_frac"] - 0.25) < 1e-7


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_create_fails_loudly_without_a_gpu(pkg):
    lib = pkg._lib.load()
    h = C.c_void_p()
    rc = lib.moe_fp8_b200_create(C.byref(h), 0, 16, 32)
    assert rc != 0 and not h.value
    assert lib.moe_fp8_b200_last_error(None)
    with pytest.raises(pkg.MoeError):
        pkg.MoeLayer(16, 32, 0)


def test_create_rejects_bad_arguments(pkg):
    lib = pkg._lib.load()
    h = C.c_void_p()
    assert lib.moe_fp8_b200_create(C.byref(h), 0, 0, 32) == -1
    assert lib.moe_fp8_b200_create(C.byref(h), 0, 16, 48) == -1
    assert lib.moe_fp8_b200_create(None, 0, 16, 32) == -1
    assert b"num_local_experts" in lib.moe_fp8_b200_last_error(None) or lib.moe_fp8_b200_last_error(None)


def test_shaped_create_checks_the_shape_before_touching_a_device(pkg):
    lib = pkg._lib.load()
    Shape = pkg._lib.Shape
    h = C.c_void_p()
    bad = [(7168 + 128, 2048, 8, 8, 4), (0, 2048, 8, 8, 4), (8192 + 256, 2048, 8, 8, 4), (7168, 2048 + 64, 8, 8, 4),
           (7168, 0, 8, 8, 4), (7168, 2048, 0, 8, 4), (7168, 2048, 9, 8, 4), (7168, 2048, 8, 3, 1),
           (7168, 2048, 8, 8, 0), (7168, 2048, 8, 8, 9), (7168, 2048, 8, 4, 5)]
    for sh in bad:
        rc = lib.moe_fp8_b200_create_shaped(C.byref(h), 0, 16, 32, C.byref(Shape(*sh)))
        assert rc == pkg._lib.ERR_INVALID_ARGUMENT and not h.value, sh
        assert b"shape" in lib.moe_fp8_b200_last_error(None)
        assert lib.moe_fp8_b200_workspace_bytes_shaped(16, 32, C.byref(Shape(*sh))) == 0
    # one kept group of 32 experts still supplies 8 picks
    assert lib.moe_fp8_b200_workspace_bytes_shaped(16, 32, C.byref(Shape(7168, 2048, 8, 8, 1))) > 0
    # NULL and the reference's values size exactly like the plain entry point
    ref = lib.moe_fp8_b200_workspace_bytes(1024, 32)
    assert lib.moe_fp8_b200_workspace_bytes_shaped(1024, 32, None) == ref
    assert lib.moe_fp8_b200_workspace_bytes_shaped(1024, 32, C.byref(Shape(7168, 2048, 8, 8, 4))) == ref
    small = lib.moe_fp8_b200_workspace_bytes_shaped(1024, 32, C.byref(Shape(1024, 512, 4, 4, 2)))
    cap = lib.moe_fp8_b200_row_capacity(1024, 32)
    assert cap * (1024 + 512 + 2048) <= small < ref


def test_tvm_ffi_shim_exports_run(pkg):
    shim = ROOT / "fp8-moe-dev_b200" / "libmoe_fp8_b200_tvm.so"
    if not shim.exists():
        pytest.skip("tvm_ffi headers not available at build time")
    import tvm_ffi
    mod = tvm_ffi.load_module(str(shim))
    assert mod.implements_function("run")


def test_product_never_touches_the_oracle():
    """No file of the package may import, load or mention the oracle (or any CPU fallback)."""
    for f in (ROOT / "fp8-moe-dev_b200").rglob("*"):
        if f.suffix in (".py", ".cu", ".cuh", ".cc", ".h") and f.is_file():
            txt = f.read_text()
            assert "oracle" not in txt.lower(), f


def test_exchange_buffer_sizing(pkg):
    """moe_fp8_b200_exchange_bytes: flags + two parities of [world][ceil(T/world)] bf16 rows and
    presence bytes; zero for an invalid world size; monotonic in T."""
    lib = pkg._lib.load()
    for world in (1, 2, 4, 8):
        prev = 0
        for T in (0, 1, 7, 8, 9, 1000, 12288, 16384):
            per = (T + world - 1) // world
            n = lib.moe_fp8_b200_exchange_bytes(T, world)
            rows = 2 * world * per * 7168 * 2
            assert n >= 256 + rows + 2 * world * per
            assert n <= 256 + rows + 2 * (world * (per + 15) + 256)
            assert n >= prev
            prev = n
    for world in (0, 3, 5, 16, -1):
        assert lib.moe_fp8_b200_exchange_bytes(128, world) == 0
    assert lib.moe_fp8_b200_exchange_bytes(-1, 2) == 0


def test_exchange_regions_do_not_depend_on_the_call(pkg):
    """The receive buffer's regions are fixed by (capacity, world): the two parities' rows and presence
    bytes are disjoint, inside the buffer, and a call with fewer tokens than the capacity writes inside
    the region of its own parity (it uses the first ceil(T / world) rows of every source's slot)."""
    lib = pkg._lib.load()
    for world in (2, 4, 8):
        for cap in (96, 1000, 12288):
            off = (C.c_size_t * 4)()
            size = (C.c_size_t * 2)()
            assert lib.moe_fp8_b200_exchange_regions(cap, world, off, size) == 0
            total = lib.moe_fp8_b200_exchange_bytes(cap, world)
            assert off[0] >= 4 * world and off[1] == off[0] + size[0] and off[2] == off[1] + size[0]
            assert off[3] == off[2] + size[1] and off[3] + size[1] <= total
            slot_rows = (cap + world - 1) // world
            assert size[0] == world * slot_rows * 7168 * 2
            for T in (1, 33, cap // 2, cap):
                per = (T + world - 1) // world
                # last byte a source can write for this T: slot of the last source, row per - 1
                last = ((world - 1) * slot_rows + per) * 7168 * 2
                assert last <= size[0], (world, cap, T)
    assert lib.moe_fp8_b200_exchange_regions(128, 3, (C.c_size_t * 4)(), (C.c_size_t * 2)()) == -1


def test_python_binding_constants_match_the_header(pkg):
    txt = (ROOT / "include" / "moe_fp8_b200.h").read_text()
    consts = dict(re.findall(r"(MOE_FP8_B200_(?:OPT|BUF|ERR)\w+)\s*=\s*(-?\d+)", txt))
    L = pkg._lib
    assert int(consts["MOE_FP8_B200_OPT_REFERENCE_PRUNING"]) == L.OPT_REFERENCE_PRUNING
    assert int(consts["MOE_FP8_B200_OPT_EXACT_SILU"]) == L.OPT_EXACT_SILU
    assert int(consts["MOE_FP8_B200_OPT_STAGE_TIMING"]) == L.OPT_STAGE_TIMING
    assert int(consts["MOE_FP8_B200_OPT_STOP_AFTER_STAGE"]) == L.OPT_STOP_AFTER_STAGE
    assert int(consts["MOE_FP8_B200_OPT_DECODE_KERNEL"]) == L.OPT_DECODE_KERNEL
    assert int(consts["MOE_FP8_B200_OPT_EXPERT_STRIDE"]) == L.OPT_EXPERT_STRIDE
    assert int(consts["MOE_FP8_B200_OPT_WAIT_LIMIT_US"]) == L.OPT_WAIT_LIMIT_US
    assert int(consts["MOE_FP8_B200_OPT_WEIGHT_PRELAYOUT"]) == L.OPT_WEIGHT_PRELAYOUT
    assert int(consts["MOE_FP8_B200_OPT_SMALL_BATCH_RING"]) == L.OPT_SMALL_BATCH_RING
    for name, val in L.BUF.items():
        assert int(consts["MOE_FP8_B200_BUF_" + name.upper()]) == val, name
    assert int(re.search(r"MOE_FP8_B200_DECODE_MAX_TOKENS\s+(\d+)", txt).group(1)) == L.DECODE_MAX_TOKENS
    assert int(re.search(r"MOE_FP8_B200_NOALLOC_MAX_TOKENS\s+(\d+)", txt).group(1)) == L.NOALLOC_MAX_TOKENS
    # struct layouts the ctypes mirror must reproduce (LP64)
    assert C.sizeof(L.Args) == 8 * 8 + 8 + 8 + 8 + 8
    assert C.sizeof(L.Exchange) == 8 * 8 + 8 + 4 + 4 + 8
    assert C.sizeof(L.Unfinalized) == 5 * 8 + 8
