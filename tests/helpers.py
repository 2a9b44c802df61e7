"""Shared helpers of the test-suite: seeded cases, the reference loader, error metrics."""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np
import torch

import __graft_entry__ as entry

ROOT = Path(__file__).resolve().parent.parent
REF_LIB = ROOT / "oracle" / "_ref" / "libref_moe.so"
DIAG_DIR = Path(os.environ["MOE_TEST_DIAG_DIR"]) if os.environ.get("MOE_TEST_DIAG_DIR") else None
H, I, N1, NE, TOPK = 7168, 2048, 4096, 256, 8
RSF = 2.5


def np_u16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint16).cpu().numpy()


def np_u8(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint8).cpu().numpy()


def save_diag(name: str, **arrays):
    """Keep arrays of a failing comparison for offline reading (only when MOE_TEST_DIAG_DIR names a folder)."""
    if DIAG_DIR is None:
        return
    try:
        DIAG_DIR.mkdir(parents=True, exist_ok=True)
        np.savez_compressed(DIAG_DIR / f"{name}.npz", **arrays)
    except Exception:
        pass


_shards = {}


def gpu_shard(offset: int, E: int, base_seed: int = 1000):
    """Weights of experts [offset, offset+E) on the GPU (CUDA generator), cached per session."""
    key = (offset, E, base_seed)
    if key not in _shards:
        entry.load_package()
        from fp8_moe_dev_b200 import gen
        # shards are kept for the whole session (a 32-expert shard is 1.4 GB, all 256 experts 11.3 GB): a
        # freed shard's addresses could be handed to the next one, which handles that remember weights by
        # address would take for the old tensors
        if len(_shards) >= 12:
            _shards.pop(next(iter(_shards)))
            torch.cuda.empty_cache()
        _shards[key] = gen.make_shard(offset, E, base_seed, device="cuda", out_device="cuda")
    return _shards[key]


def cpu_inputs(T: int, seed: int = 0, skew: bool = False):
    entry.load_package()
    from fp8_moe_dev_b200 import gen
    logits, bias = gen.make_routing(T, seed, skew)
    hidden, hscale = gen.make_hidden(T, seed + 1)
    return logits, bias, hidden, hscale


def run_layer(layer, inputs, weights, offset, rsf=RSF, out=None):
    logits, bias, hidden, hscale = [x.cuda() for x in inputs]
    w1, s1, w2, s2 = weights
    T = logits.shape[0]
    if out is None:
        out = torch.full((T, H), float("nan"), dtype=torch.bfloat16, device="cuda")
    # The handle remembers what it derived from the weight tensors BY ADDRESS.  Test fixtures free shards
    # and generate others, which the allocator may place at the same addresses: tell the handle.
    layer.invalidate_weights()
    layer.run(logits, bias, hidden, hscale, w1, s1, w2, s2, offset, rsf, out)
    layer.check()
    return out


# ------------------------------------------------------------------ reference library
_ref_mod = None


def reference_available() -> bool:
    return REF_LIB.exists()


def reference_module():
    global _ref_mod
    if _ref_mod is None:
        import tvm_ffi
        _ref_mod = tvm_ffi.load_module(str(REF_LIB))
    return _ref_mod


_ref_scales_alive = []


def reference_run(inputs, weights, offset, rsf=RSF):
    """The unmodified reference operator on fresh device buffers.  Its caches key on pointers: the routing
    result on the input pointers (kernel/moe_fp8.cu:2696-2702) and a transposed copy of the weight scales
    on the scale pointers (:3007-3014, 3501-3508), with no way to invalidate either.  The inputs are
    therefore cloned per call, and the scales are cloned into tensors that stay allocated for the whole
    session, so that no later call can present other scales at an address the reference has seen."""
    logits, bias, hidden, hscale = [x.cuda().clone() for x in inputs]
    w1, s1, w2, s2 = weights
    s1, s2 = s1.clone(), s2.clone()
    _ref_scales_alive.append((s1, s2))
    T = logits.shape[0]
    out = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")
    reference_module().run(logits, bias, hidden, hscale, w1, s1, w2, s2, int(offset), float(rsf), out)
    torch.cuda.synchronize()
    return out


_harness = None


def harness():
    global _harness
    if _harness is None:
        reference_module()  # makes sure dependencies are resolved the same way
        _harness = C.CDLL(str(REF_LIB))
        _harness.ref_harness_route.restype = C.c_int
        _harness.ref_harness_dispatch.restype = C.c_int
    return _harness


def reference_routing(logits: torch.Tensor, bias: torch.Tensor):
    """topk_idx int32 [T,8], topk_weight fp32 [T,8] from the reference's own routing kernel."""
    T = logits.shape[0]
    lg, bs = logits.cuda().contiguous(), bias.cuda().contiguous()
    idx = torch.zeros(T, TOPK, dtype=torch.int32, device="cuda")
    w = torch.zeros(T, TOPK, dtype=torch.float32, device="cuda")
    cnt = torch.zeros(T, dtype=torch.int32, device="cuda")
    vp = lambda t: C.c_void_p(t.data_ptr())
    rc = harness().ref_harness_route(vp(lg), vp(bs), C.c_int(T), vp(idx), vp(w), vp(cnt), C.c_void_p(0))
    torch.cuda.synchronize()
    assert rc == 0, rc
    return idx.cpu().numpy(), w.cpu().numpy()


def reference_dispatch_arrays(logits: torch.Tensor, bias: torch.Tensor, offset: int, rsf: float = RSF):
    """The reference's dispatch tables for this T as arrays: dict(variant, expert_count [32], pair_n [T],
    pair_le [T,8], pair_w fp32 [T,8] in stored order, offsets [33], padded [32], expert_token_list [32,T])."""
    T = logits.shape[0]
    lg, bs = logits.cuda().contiguous(), bias.cuda().contiguous()
    i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device="cuda")
    f32 = lambda *s: torch.zeros(*s, dtype=torch.float32, device="cuda")
    idx, w, tlc = i32(T, TOPK), f32(T, TOPK), i32(T)
    ecount, elist, eweight = i32(32), i32(32, T), f32(32, T)
    pcode, pweight = i32(T, TOPK), f32(T, TOPK)
    offs, padded, scratch = i32(33), i32(32), i32(80)
    vp = lambda t: C.c_void_p(t.data_ptr())
    rc = harness().ref_harness_dispatch(vp(lg), vp(bs), C.c_int(T), C.c_int(offset), C.c_float(rsf), vp(idx), vp(w),
                                        vp(tlc), vp(ecount), vp(elist), vp(eweight), vp(pcode), vp(pweight),
                                        vp(offs), vp(padded), vp(scratch), C.c_void_p(0))
    torch.cuda.synchronize()
    assert rc >= 0, rc
    pair_n = np.minimum(tlc.cpu().numpy(), TOPK).astype(np.int32)
    pair_le = (pcode.cpu().numpy().view(np.uint32) >> 24).astype(np.int32)
    return dict(variant=rc, expert_count=ecount.cpu().numpy(), pair_n=pair_n, pair_le=pair_le,
                pair_w=pweight.cpu().numpy(), offsets=offs.cpu().numpy(), padded=padded.cpu().numpy(),
                expert_token_list=elist.cpu().numpy())


def reference_dispatch(logits: torch.Tensor, bias: torch.Tensor, offset: int, rsf: float = RSF):
    """As reference_dispatch_arrays, with `pairs` = per-token list of (local expert, weight) in stored order."""
    d = reference_dispatch_arrays(logits, bias, offset, rsf)
    pairs = []
    for t in range(logits.shape[0]):
        pairs.append([(int(d["pair_le"][t, p]), np.float32(d["pair_w"][t, p])) for p in range(int(d["pair_n"][t]))])
    d["pairs"] = pairs
    return d


def pairs_digest(pair_n: np.ndarray, pair_le: np.ndarray, pair_w: np.ndarray) -> str:
    """Order-independent digest of a dispatch result: sha256 over the (token, local expert, weight bits)
    triples of all kept pairs, sorted by token, then expert, then bits."""
    import hashlib
    pair_n = np.asarray(pair_n).astype(np.int64)
    T = pair_n.shape[0]
    keep = np.arange(TOPK)[None, :] < pair_n[:, None]
    tok = np.broadcast_to(np.arange(T, dtype=np.int64)[:, None], (T, TOPK))[keep]
    le = np.asarray(pair_le).astype(np.int64)[keep]
    bits = np.ascontiguousarray(pair_w, dtype=np.float32).view(np.uint32).astype(np.int64)[keep]
    order = np.lexsort((bits, le, tok))
    packed = np.stack([tok[order], le[order], bits[order]], axis=1)
    return hashlib.sha256(np.ascontiguousarray(packed).tobytes()).hexdigest()[:32]


# ------------------------------------------------------------------ metrics
def error_stats(got: np.ndarray, want: np.ndarray) -> dict:
    got = got.astype(np.float64)
    want = want.astype(np.float64)
    diff = np.abs(got - want)
    den = np.linalg.norm(want)
    return dict(
        max_abs=float(diff.max()) if diff.size else 0.0,
        mean_abs=float(diff.mean()) if diff.size else 0.0,
        rel_l2=float(np.linalg.norm(got - want) / den) if den > 0 else float(np.linalg.norm(got - want)),
        contest_ratio=float((diff <= 1.0 + 0.3 * np.abs(want)).mean()) if diff.size else 1.0,
        cosine=float((got * want).sum() / (np.linalg.norm(got) * den)) if den > 0 and np.linalg.norm(got) > 0 else 1.0,
    )


def gpu_pair_arrays(layer, T: int):
    """(pair_n [T], pair_le [T,8], slot [T,8], pair_w fp32 [T,8]) of the last run."""
    pc = layer.read("pair_count", T).astype(np.int32)
    code = layer.read("pair_code", T * TOPK).reshape(T, TOPK)
    pw = layer.read("pair_weight", T * TOPK).reshape(T, TOPK)
    return pc, (code >> 24).astype(np.int32), (code & 0xFFFFFF).astype(np.int32), pw


def gpu_pairs(layer, T: int):
    """Per-token [(local expert, slot, weight)] of the last run, expert_count, expert_offset."""
    pc, le, slot, pw = gpu_pair_arrays(layer, T)
    pairs = [[(int(le[t, p]), int(slot[t, p]), np.float32(pw[t, p])) for p in range(int(pc[t]))]
             for t in range(T)]
    return pairs, layer.read("expert_count", layer.num_local_experts), layer.read("expert_offset",
                                                                                  layer.num_local_experts + 1)


