"""TEST INFRASTRUCTURE -- numpy/ctypes front end of the CPU oracle (oracle/moe_oracle.c).

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs
import this module.  Nothing under fp8-moe-dev_b200/ does.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "liboracle.so"
H, I, N1, NE, TOPK = 7168, 2048, 4096, 256, 8


class Policy(C.Structure):
    _fields_ = [("prune", C.c_int), ("skip_zero_weight", C.c_int), ("keep_limit", C.c_int), ("drop_third", C.c_int),
                ("drop_third_frac", C.c_float), ("drop_second_frac_2", C.c_float),
                ("drop_second_frac_ge3", C.c_float), ("renorm", C.c_int)]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


def build() -> Path:
    r = subprocess.run(["make", "-C", str(HERE)], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + r.stdout + r.stderr)
    return LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            build()
        _lib = C.CDLL(str(LIB_PATH))
        _lib.oracle_layer.restype = C.c_long
        _lib.oracle_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _c(a, dt):
    a = np.ascontiguousarray(a, dtype=dt)
    return a


class shape:
    """Context manager: the oracle computes another shape of the layer inside the block (the library's
    setting is process-wide), the reference's 7168 / 2048 / 8 / 8 / 4 outside."""

    def __init__(self, hidden=7168, inter=2048, top_k=8, n_group=8, topk_group=4):
        self.args = (hidden, inter, top_k, n_group, topk_group)

    def __enter__(self):
        global H, I, N1
        if lib().oracle_set_shape(*map(C.c_int, self.args)) != 0:
            raise ValueError(f"oracle: unusable shape {self.args}")
        H, I, N1 = self.args[0], self.args[1], 2 * self.args[1]
        return self

    def __exit__(self, *exc):
        global H, I, N1
        lib().oracle_set_shape(*map(C.c_int, (7168, 2048, 8, 8, 4)))
        H, I, N1 = 7168, 2048, 4096
        return False


def num_threads() -> int:
    return lib().oracle_num_threads()


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    codes = _c(codes, np.uint8)
    out = np.empty(codes.shape, np.float32)
    lib().oracle_e4m3_decode(_p(codes), _p(out), C.c_long(codes.size))
    return out


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint8)
    lib().oracle_e4m3_encode(_p(x), _p(out), C.c_long(x.size))
    return out


def quantize_rows(x_bf16: np.ndarray):
    """bf16 codes [T, K] (uint16) -> (e4m3 codes [T, K] uint8, scales fp32 [K/128, T])."""
    x = _c(x_bf16, np.uint16)
    T, K = x.shape
    q = np.empty((T, K), np.uint8)
    sc = np.empty((K // 128, T), np.float32)
    lib().oracle_quantize_rows(_p(x), C.c_long(T), C.c_long(K), _p(q), _p(sc))
    return q, sc


def bf16_encode(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().oracle_bf16_encode(_p(x), _p(out), C.c_long(x.size))
    return out


def bf16_decode(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def route(logits: np.ndarray, bias_bf16: np.ndarray):
    """-> (idx int32 [T,8] in selection order, weights fp32 [T,8])."""
    logits = _c(logits, np.float32)
    bias_bf16 = _c(bias_bf16, np.uint16)
    T = logits.shape[0]
    idx = np.empty((T, TOPK), np.int32)
    w = np.empty((T, TOPK), np.float32)
    lib().oracle_route(_p(logits), _p(bias_bf16), C.c_int(T), _p(idx), _p(w))
    return idx, w


def route_margin(logits: np.ndarray, bias_bf16: np.ndarray) -> np.ndarray:
    logits = _c(logits, np.float32)
    bias_bf16 = _c(bias_bf16, np.uint16)
    T = logits.shape[0]
    m = np.empty(T, np.float32)
    lib().oracle_route_margin(_p(logits), _p(bias_bf16), C.c_int(T), _p(m))
    return m


def policy(T: int, reference_pruning: bool = True) -> Policy:
    p = Policy()
    lib().oracle_policy(C.c_int(T), C.c_int(int(reference_pruning)), C.byref(p))
    return p


def dispatch(idx, w, local_expert_offset: int, num_local_experts: int, pol: Policy, rsf: float):
    """-> (pair_count [T], pair_le [T,8], pair_w [T,8], expert_count [E])."""
    idx = _c(idx, np.int32)
    w = _c(w, np.float32)
    T = idx.shape[0]
    pc = np.zeros(T, np.int32)
    ple = np.full((T, TOPK), -1, np.int32)
    pw = np.zeros((T, TOPK), np.float32)
    ec = np.zeros(num_local_experts, np.int32)
    lib().oracle_dispatch(_p(idx), _p(w), C.c_int(T), C.c_int(local_expert_offset), C.c_int(num_local_experts),
                          C.byref(pol), C.c_float(rsf), _p(pc), _p(ple), _p(pw), _p(ec))
    return pc, ple, pw, ec


def expert_rows(hidden, hidden_scale, tokens, w1, s1, w2, s2, faithful=True, exact_silu=False, want_all=False):
    """All rows of one expert.  Returns y [rows, 7168] fp32 (bf16-valued when faithful) and,
    with want_all, also (d [rows,4096], a2 codes [rows,2048], sfa2 [rows,16])."""
    hidden = _c(hidden, np.uint8)
    hidden_scale = _c(hidden_scale, np.float32)
    tokens = _c(tokens, np.int32)
    T = hidden.shape[0]
    rows = tokens.shape[0]
    y = np.empty((rows, H), np.float32)
    d = np.empty((rows, N1), np.float32) if want_all else None
    a2 = np.zeros((rows, I), np.uint8) if want_all else None
    sf = np.empty((rows, I // 128), np.float32) if want_all else None
    lib().oracle_expert_rows(_p(hidden), _p(hidden_scale), C.c_int(T), _p(tokens), C.c_int(rows),
                             _p(_c(w1, np.uint8)), _p(_c(s1, np.float32)), _p(_c(w2, np.uint8)),
                             _p(_c(s2, np.float32)), C.c_int(int(faithful)), C.c_int(int(exact_silu)), _p(y), _p(d),
                             _p(a2), _p(sf))
    return (y, d, a2, sf) if want_all else y


def combine(y, pair_count, row_of_pair, pair_w):
    """out[t] = bf16(sum_p y[row_of_pair[t, p]] * pair_w[t, p]), fp32 FMA in pair order -> bf16 codes [T, 7168]."""
    y = _c(y, np.float32)
    pair_count = _c(pair_count, np.int32)
    row_of_pair = _c(row_of_pair, np.int32)
    pair_w = _c(pair_w, np.float32)
    T = pair_count.shape[0]
    out = np.empty((T, H), np.uint16)
    lib().oracle_combine(_p(y), _p(pair_count), _p(row_of_pair), _p(pair_w), C.c_int(T), _p(out))
    return out


def layer(logits, bias_bf16, hidden, hidden_scale, w1, s1, w2, s2, local_expert_offset, rsf, mode="faithful",
          reference_pruning=True, exact_silu=False):
    """Whole layer on the host.  mode "faithful" = the reference pipeline's rounding points,
    "fp32" = the layer's definition.  Returns (out bf16 codes [T,7168] uint16, routed rows)."""
    logits = _c(logits, np.float32)
    T = logits.shape[0]
    E = w1.shape[0]
    out = np.empty((T, H), np.uint16)
    M = lib().oracle_layer(_p(logits), _p(_c(bias_bf16, np.uint16)), _p(_c(hidden, np.uint8)),
                           _p(_c(hidden_scale, np.float32)), _p(_c(w1, np.uint8)), _p(_c(s1, np.float32)),
                           _p(_c(w2, np.uint8)), _p(_c(s2, np.float32)), C.c_int(T), C.c_int(local_expert_offset),
                           C.c_int(E), C.c_float(rsf), C.c_int(0 if mode == "faithful" else 1),
                           C.c_int(int(reference_pruning)), C.c_int(int(exact_silu)), _p(out))
    return out, int(M)
