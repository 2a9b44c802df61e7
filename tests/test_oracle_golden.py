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
