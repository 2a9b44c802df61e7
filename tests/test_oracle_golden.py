"""Pins the CPU oracle to the reference: the fixtures in tests/golden/ hold what the
reference's own GPU code produced on a B200 (routing kernel, dispatch kernels for all eight
shard offsets, bf16 output of `run` for one shard) for seeded inputs that are regenerated
here from the seeds.  tests/golden/make_golden.py is the script that wrote them."""
import hashlib
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import cpu_inputs, np_u16, np_u8

GOLDEN = Path(__file__).resolve().parent / "golden"
CASES = ["t1", "t7", "t16", "t40"]
BIG = ["t32", "t53", "t80", "t901", "t14107", "t12288", "t16384skew"]
_experts = {}


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()[:16]


def load(name):
    f = GOLDEN / f"ref_{name}.npz"
    assert f.exists(), f"{f} missing: regenerate with tests/golden/make_golden.py on a B200"
    return np.load(f)


def expert(e):
    from fp8_moe_dev_b200 import gen
    if e not in _experts:
        _experts[e] = gen.make_expert(e)
    return _experts[e]


@pytest.mark.parametrize("name", CASES)
def test_inputs_regenerate_identically(pkg, name):
    g = load(name)
    logits, bias, hidden, hscale = cpu_inputs(int(g["T"]), seed=int(g["seed"]))
    assert sha(logits.numpy()) == str(g["sha_logits"])
    assert sha(np_u8(hidden)) == str(g["sha_hidden"])
    assert sha(hscale.numpy()) == str(g["sha_hscale"])
    e = int(g["first_used_expert"])
    if e >= 0:
        assert sha(np_u8(expert(int(g["offset"]) + e)[0])) == str(g["sha_w1_first_used"])


@pytest.mark.parametrize("name", CASES)
def test_routing_against_reference_kernel(pkg, oracle, name):
    g = load(name)
    T = int(g["T"])
    logits, bias, _, _ = cpu_inputs(T, seed=int(g["seed"]))
    idx, w = oracle.route(logits.numpy(), np_u16(bias))
    ref_idx = g["topk_idx"]
    ref_w = g["topk_weight_bits"].view(np.float32)
    margin = oracle.route_margin(logits.numpy(), np_u16(bias))
    safe = margin > 1e-5
    assert safe.mean() >= 0.9
    assert np.array_equal(idx[safe], ref_idx[safe]), "selection (and its order) differs from the reference"
    # CPU expf vs the GPU's ex2.approx: a few ulp
    assert np.allclose(w[safe], ref_w[safe], rtol=4e-6, atol=0)


@pytest.mark.parametrize("name", CASES)
def test_dispatch_against_reference_kernels(pkg, oracle, name):
    """Given the reference's routing output, the oracle's policy + dispatch must reproduce the
    reference's per-expert counts and (expert, weight) pairs bit for bit, for every shard."""
    g = load(name)
    T = int(g["T"])
    ref_idx = g["topk_idx"]
    ref_w = g["topk_weight_bits"].view(np.float32)
    pol = oracle.policy(T, True)
    assert {0: (0, 0), 1: (1, 0), 2: (0, 1)}[int(g["variant"])] == (pol.prune, pol.skip_zero_weight)
    pair_w = g["pair_w_bits"].view(np.float32)
    for s in range(8):
        pc, ple, pw, ec = oracle.dispatch(ref_idx, ref_w, 32 * s, 32, pol, float(g["rsf"]))
        assert np.array_equal(ec, g["expert_count"][s])
        assert np.array_equal(pc, g["pair_n"][s])
        for t in range(T):
            n = int(pc[t])
            mine = [(int(ple[t, p]), np.float32(pw[t, p]).tobytes()) for p in range(n)]
            theirs = [(int(g["pair_le"][s, t, p]), np.float32(pair_w[s, t, p]).tobytes()) for p in range(n)]
            if int(g["variant"]) == 2:   # unfused dispatch stores pairs in atomic order
                mine, theirs = sorted(mine), sorted(theirs)
            assert mine == theirs, (s, t)


@pytest.mark.parametrize("name", CASES)
def test_layer_output_against_reference_run(pkg, oracle, name):
    g = load(name)
    T, offset = int(g["T"]), int(g["offset"])
    logits, bias, hidden, hscale = cpu_inputs(T, seed=int(g["seed"]))
    used = np.nonzero(g["expert_count"][offset // 32])[0]
    w1 = np.zeros((32, 4096, 7168), np.uint8)
    s1 = np.ones((32, 32, 56), np.float32)
    w2 = np.zeros((32, 7168, 2048), np.uint8)
    s2 = np.ones((32, 56, 16), np.float32)
    for e in used:
        q1, a1, q2, a2 = expert(offset + int(e))
        w1[e], s1[e], w2[e], s2[e] = np_u8(q1), a1.numpy(), np_u8(q2), a2.numpy()
    out, rows = oracle.layer(logits.numpy(), np_u16(bias), np_u8(hidden), hscale.numpy(), w1, s1, w2, s2, offset,
                             float(g["rsf"]))
    assert rows == int(g["expert_count"][offset // 32].sum())
    got = oracle.bf16_decode(out)
    want = oracle.bf16_decode(g["out_bf16"])
    diff = np.abs(got - want)
    ratio = float((diff <= 1.0 + 0.3 * np.abs(want)).mean())      # the reference's stated tolerance
    rel = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    print(f"{name}: max_abs={diff.max():.4g} mean_abs={diff.mean():.4g} rel_l2={rel:.3g}")
    assert ratio >= 0.99
    assert rel < 1e-2, rel          # rounding-point-faithful restatement: far inside that tolerance
    assert np.array_equal(want == 0, got == 0) or rel < 1e-3
    _ = torch


# ------------------------------------------------------------------ the T-keyed branches, at size
def load_big(name):
    f = GOLDEN / f"ref_big_{name}.npz"
    assert f.exists(), f"{f} missing: regenerate with tests/golden/make_golden.py OUT big on a B200"
    return np.load(f)


@pytest.mark.parametrize("name", BIG)
def test_big_policy_and_dispatch_on_sampled_tokens(pkg, oracle, name):
    """Fed with the reference's own routing result for 512 evenly spaced tokens, the oracle's policy for
    this T and its dispatch reproduce the reference's pairs bit for bit, in stored order, for every shard
    (the fused pruning variant stores pairs in descending-weight order: deterministic)."""
    g = load_big(name)
    T = int(g["T"])
    pol = oracle.policy(T, True)
    assert int(g["variant"]) == 1 and pol.prune == 1
    idx = g["sample_topk_idx"].astype(np.int32)
    w = g["sample_topk_weight_bits"].view(np.float32)
    for s in range(8):
        pc, ple, pw, _ = oracle.dispatch(idx, w, 32 * s, 32, pol, float(g["rsf"]))
        want_le = g["sample_pair_le"][s].astype(np.int32)
        want_n = (want_le >= 0).sum(1)
        assert np.array_equal(pc, want_n), (name, s)
        live = want_le >= 0
        assert np.array_equal(np.where(live, ple, -1), want_le), (name, s)
        assert np.array_equal(np.where(live, pw.view(np.uint32), 0), g["sample_pair_w_bits"][s]), (name, s)


@pytest.mark.parametrize("name", BIG)
def test_big_counts_from_the_oracles_own_routing(pkg, oracle, name):
    """Whole batch on the host: oracle routing (CPU expf, a few ulp from the GPU's weights) + policy +
    dispatch give the reference's per-expert rows and per-token pair counts, except for tokens that sit
    within rounding of a drop threshold or of a routing tie."""
    g = load_big(name)
    T = int(g["T"])
    from fp8_moe_dev_b200 import gen
    logits, bias = gen.make_routing(T, int(g["seed"]), bool(int(g["skew"])))
    assert sha(logits.numpy()) == str(g["sha_logits"])
    idx, w = oracle.route(logits.numpy(), np_u16(bias))
    samp = g["sample_tokens"]
    same = (idx[samp] == g["sample_topk_idx"].astype(np.int32)).all(1)
    assert same.mean() >= 0.995, same.mean()
    pol = oracle.policy(T, True)
    off_tokens = 0
    for s in range(8):
        pc, _, _, ec = oracle.dispatch(idx, w, 32 * s, 32, pol, float(g["rsf"]))
        bad = int((pc != g["pair_n"][s].astype(np.int32)).sum())
        off_tokens += bad
        assert np.abs(ec - g["expert_count"][s]).sum() <= 2 * bad, (name, s)
    assert off_tokens <= max(2, T // 2000), (name, off_tokens)


def test_big_output_sample_t12288(pkg, oracle):
    """bf16 output rows of the reference's `run` at T = 12288 (drop-third policy, 128-row padding, its
    CUTLASS / TRTLLM GEMMs) for tokens whose rows lie in two experts: the oracle's expert arithmetic and
    combine, fed with the reference's pairs for those tokens, reproduce them."""
    g = load_big("t12288")
    T, offset = int(g["T"]), int(g["out_offset"])
    from fp8_moe_dev_b200 import gen
    hidden, hscale = gen.make_hidden(T, int(g["seed"]) + 1)
    toks = g["out_tokens"]
    assert sha(np_u8(hidden)[toks]) == str(g["sha_hidden_rows"])
    n, le, wbits = g["out_pair_n"], g["out_pair_le"], g["out_pair_w_bits"]
    ea, eb = [int(x) for x in g["out_experts"]]
    hid_s = np_u8(hidden)[toks]
    hs_s = np.ascontiguousarray(hscale.numpy()[:, toks])
    y_rows, row_of_pair = [], np.zeros((len(toks), 8), np.int32)
    base = 0
    for e in (ea, eb):
        q1, a1, q2, a2 = expert(offset + e)
        if e == ea:
            assert sha(np_u8(q1)) == str(g["sha_w1_a"])
        sel = [(i, p) for i in range(len(toks)) for p in range(int(n[i])) if int(le[i, p]) == e]
        local = np.array([i for i, _ in sel], np.int32)
        y = oracle.expert_rows(hid_s, hs_s, local, np_u8(q1), a1.numpy(), np_u8(q2), a2.numpy(), faithful=True)
        for r, (i, p) in enumerate(sel):
            row_of_pair[i, p] = base + r
        y_rows.append(y)
        base += len(sel)
    out = oracle.combine(np.concatenate(y_rows), n.astype(np.int32), row_of_pair, wbits.view(np.float32))
    got = oracle.bf16_decode(out)
    want8 = oracle.bf16_decode(g["out_bf16_cols8"])
    assert np.all(got[n == 0] == 0) and np.all(want8[n == 0] == 0)
    diff = np.abs(got[:, ::8] - want8)
    rel = float(np.linalg.norm(got[:, ::8] - want8) / np.linalg.norm(want8))
    ratio = float((diff <= 1.0 + 0.3 * np.abs(want8)).mean())
    print(f"t12288 sample: max_abs={diff.max():.4g} mean_abs={diff.mean():.4g} rel_l2={rel:.3g}")
    assert ratio >= 0.99 and rel < 1e-2, (ratio, rel)
    assert np.allclose(got.astype(np.float64).sum(1), g["out_row_sum"], rtol=0, atol=2e-2 * np.maximum(g["out_row_abs_sum"], 1.0))
