"""Parity tests proper (B200): every stage of the CUDA layer, called through the C ABI,
against the CPU oracle on the same seeded inputs, and against the reference's own GPU
kernels (oracle/_ref, built from the reference sources) where those can be reached."""
import numpy as np
import pytest
import torch

import helpers as hp
from helpers import H, I, RSF, TOPK

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def layer32(pkg):
    lay = pkg.MoeLayer(1024, 32, 0)
    lay.set_decode_kernel(False)   # these tests look at the staged chain's intermediates; the decode kernel has its own file
    yield lay
    lay.close()


def _oracle_dispatch_from_gpu_routing(oracle, layer, T, offset, E, reference_pruning=True):
    idx = layer.read("topk_idx", T * TOPK).reshape(T, TOPK)
    w = layer.read("topk_weight", T * TOPK).reshape(T, TOPK)
    pol = oracle.policy(T, reference_pruning)
    return idx, w, oracle.dispatch(idx, w, offset, E, pol, RSF)


# ------------------------------------------------------------------------- routing
@pytest.mark.parametrize("T", [1, 2, 16, 33, 129, 1024])
def test_routing_matches_oracle(pkg, oracle, layer32, T):
    inputs = hp.cpu_inputs(T, seed=T)
    hp.run_layer(layer32, inputs, hp.gpu_shard(0, 32), 0)
    idx = layer32.read("topk_idx", T * TOPK).reshape(T, TOPK)
    w = layer32.read("topk_weight", T * TOPK).reshape(T, TOPK)
    oidx, ow = oracle.route(inputs[0].numpy(), hp.np_u16(inputs[1]))
    margin = oracle.route_margin(inputs[0].numpy(), hp.np_u16(inputs[1]))
    safe = margin > 1e-5
    assert safe.mean() > 0.9
    assert np.array_equal(np.sort(idx[safe], 1), np.sort(oidx[safe], 1))
    same_order = np.all(idx == oidx, axis=1)
    assert same_order.mean() > 0.95
    assert np.allclose(w[same_order], ow[same_order], rtol=5e-6, atol=1e-9)
    assert np.allclose(w.sum(1), 1.0, atol=1e-5)


@pytest.mark.parametrize("T", [1, 7, 16, 40, 1024])
def test_routing_bit_exact_vs_reference_kernels(pkg, layer32, T):
    if not hp.reference_available():
        pytest.skip("oracle/_ref/libref_moe.so not built")
    inputs = hp.cpu_inputs(T, seed=100 + T)
    hp.run_layer(layer32, inputs, hp.gpu_shard(0, 32), 0)
    idx = layer32.read("topk_idx", T * TOPK).reshape(T, TOPK)
    w = layer32.read("topk_weight", T * TOPK).reshape(T, TOPK)
    ridx, rw = hp.reference_routing(inputs[0], inputs[1])
    assert np.array_equal(idx, ridx)
    assert np.array_equal(w.view(np.uint32), rw.view(np.uint32)), "routing weights differ in bits"


@pytest.mark.parametrize("T,offset", [(1, 0), (7, 32), (16, 0), (15, 64), (40, 0), (129, 224), (1024, 96)])
def test_dispatch_bit_exact_vs_reference_kernels(pkg, layer32, T, offset):
    if not hp.reference_available():
        pytest.skip("oracle/_ref/libref_moe.so not built")
    inputs = hp.cpu_inputs(T, seed=200 + T)
    hp.run_layer(layer32, inputs, hp.gpu_shard(0, 32), offset)
    pairs, ecount, _ = hp.gpu_pairs(layer32, T)
    ref = hp.reference_dispatch(inputs[0], inputs[1], offset)
    assert np.array_equal(ecount, ref["expert_count"])
    for t in range(T):
        mine = sorted((le, w.tobytes()) for le, _, w in pairs[t])
        theirs = sorted((le, w.tobytes()) for le, w in ref["pairs"][t])
        assert mine == theirs, (t, pairs[t], ref["pairs"][t])
        if ref["variant"] != 2:  # stored order is deterministic in the fused variants
            assert [le for le, _, _ in pairs[t]] == [le for le, _ in ref["pairs"][t]]


# ------------------------------------------------------------------------- dispatch / permute
@pytest.mark.parametrize("T,offset,pruning", [(1, 0, True), (16, 0, True), (33, 32, True), (129, 0, False),
                                               (1024, 64, True)])
def test_dispatch_and_permute(pkg, oracle, layer32, T, offset, pruning):
    inputs = hp.cpu_inputs(T, seed=300 + T)
    layer32.set_reference_pruning(pruning)
    try:
        hp.run_layer(layer32, inputs, hp.gpu_shard(0, 32), offset)
    finally:
        layer32.set_reference_pruning(True)
    idx, w, (pc, ple, pw, ec) = _oracle_dispatch_from_gpu_routing(oracle, layer32, T, offset, 32, pruning)
    pairs, ecount, eoff = hp.gpu_pairs(layer32, T)
    assert np.array_equal(ecount, ec)
    padded = (ec + 127) // 128 * 128
    assert np.array_equal(eoff, np.concatenate([[0], np.cumsum(padded)]))
    assert layer32.read("num_tiles", 1)[0] == padded.sum() // 128
    M = int(eoff[-1])
    row_token = layer32.read("row_token", M) if M else np.zeros(0, np.int32)
    a1 = layer32.read("a1", M * H).reshape(M, H) if M else None
    sfa1 = np.stack([layer32.read("sfa1", M, kb * layer32.row_capacity) for kb in range(56)]) if M else None
    hidden = hp.np_u8(inputs[2])
    hscale = inputs[3].numpy()
    pair_row = layer32.read("pair_row", T * TOPK).reshape(T, TOPK)
    slots = [set() for _ in range(32)]
    for t in range(T):
        assert list(pair_row[t]) == [int(eoff[le]) + slot for le, slot, _ in pairs[t]] + [-1] * (TOPK - len(pairs[t]))
        got = [(le, wt.tobytes()) for le, _, wt in pairs[t]]
        want = [(int(ple[t, p]), np.float32(pw[t, p]).tobytes()) for p in range(pc[t])]
        assert got == want, (t, pairs[t])
        for le, slot, _ in pairs[t]:
            assert 0 <= slot < ec[le] and slot not in slots[le]
            slots[le].add(slot)
            row = eoff[le] + slot
            assert row_token[row] == t
            assert np.array_equal(a1[row], hidden[t])
            assert np.array_equal(sfa1[:, row], hscale[:, t])
    for le in range(32):
        assert slots[le] == set(range(ec[le]))


# ------------------------------------------------------------------------- GEMM1 + SwiGLU + requant
def _rows_by_expert(layer, T):
    pairs, ecount, eoff = hp.gpu_pairs(layer, T)
    M = int(eoff[-1])
    row_token = layer.read("row_token", M)
    return ecount, eoff, row_token


@pytest.mark.parametrize("T,pruning", [(1, True), (16, True), (129, False)])
def test_gemm1_swiglu_requant_vs_oracle(pkg, oracle, layer32, T, pruning):
    offset = 0
    inputs = hp.cpu_inputs(T, seed=400 + T)
    weights = hp.gpu_shard(0, 32)
    layer32.set_reference_pruning(pruning)
    try:
        hp.run_layer(layer32, inputs, weights, offset)
    finally:
        layer32.set_reference_pruning(True)
    ecount, eoff, row_token = _rows_by_expert(layer32, T)
    M = int(eoff[-1])
    if M == 0:
        pytest.skip("no local rows for this seed")
    cap = layer32.row_capacity
    a2 = layer32.read("a2", M * I).reshape(M, I)
    sfa2 = np.stack([layer32.read("sfa2", M, kb * cap) for kb in range(16)])  # [16, M]
    y = oracle.bf16_decode(layer32.read("y", M * H)).reshape(M, H)
    hidden, hscale = hp.np_u8(inputs[2]), inputs[3].numpy()
    w1, s1, w2, s2 = weights
    checked = 0
    for e in np.nonzero(ecount)[0][:6]:
        r0, n = int(eoff[e]), int(ecount[e])
        tokens = row_token[r0:r0 + n].astype(np.int32)
        oy, od, oa2, osf = oracle.expert_rows(hidden, hscale, tokens, hp.np_u8(w1[e]), s1[e].cpu().numpy(),
                                              hp.np_u8(w2[e]), s2[e].cpu().numpy(), faithful=True, want_all=True)
        g_scale = sfa2[:, r0:r0 + n].T  # [n, 16]
        g_deq = oracle.e4m3_decode(a2[r0:r0 + n]).reshape(n, 16, 128) * g_scale[:, :, None]
        o_deq = oracle.e4m3_decode(oa2).reshape(n, 16, 128) * osf[:, :, None]
        st = hp.error_stats(g_deq, o_deq)
        code_match = float((a2[r0:r0 + n] == oa2).mean())
        scale_rel = np.abs(g_scale - osf) / osf
        if not (st["rel_l2"] < 2e-2 and code_match > 0.9 and np.median(scale_rel) < 1e-3):
            hp.save_diag(f"gemm1_T{T}_e{e}", a2=a2[r0:r0 + n], oa2=oa2, sfa2=g_scale, osf=osf, d=od, tokens=tokens)
        assert st["rel_l2"] < 2e-2, (e, st, code_match)
        assert code_match > 0.9, (e, code_match)
        assert np.median(scale_rel) < 1e-3 and scale_rel.max() < 5e-2, (e, scale_rel.max())
        # GEMM2 in isolation: from the GPU's own A2 / sA2, in float64 on the host
        w2f = oracle.e4m3_decode(hp.np_u8(w2[e])).reshape(H, 16, 128).astype(np.float64)
        a2f = oracle.e4m3_decode(a2[r0:r0 + n]).reshape(n, 16, 128).astype(np.float64)
        sw = s2[e].cpu().numpy().astype(np.float64)  # [56, 16]
        raw = np.einsum("rkb,hkb->rhk", a2f, w2f)
        ref_y = (raw * (g_scale[:, None, :].astype(np.float64) * np.repeat(sw, 128, axis=0)[None])).sum(-1)
        sy = hp.error_stats(y[r0:r0 + n], ref_y)
        if not sy["rel_l2"] < 6e-3:
            hp.save_diag(f"gemm2_T{T}_e{e}", y=y[r0:r0 + n], ref=ref_y)
        assert sy["rel_l2"] < 6e-3, (e, sy)
        assert np.abs(y[r0:r0 + n] - ref_y).max() <= 2 ** -7 * np.abs(ref_y).max() + 1e-3
        checked += 1
    assert checked > 0


# ------------------------------------------------------------------------- whole layer
@pytest.mark.parametrize("T,offset", [(1, 0), (16, 0), (33, 32), (129, 224)])
def test_layer_vs_oracle(pkg, oracle, layer32, T, offset):
    inputs = hp.cpu_inputs(T, seed=500 + T)
    weights = hp.gpu_shard(offset, 32)
    out = hp.run_layer(layer32, inputs, weights, offset)
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all()
    w1, s1, w2, s2 = weights
    ref, rows = oracle.layer(inputs[0].numpy(), hp.np_u16(inputs[1]), hp.np_u8(inputs[2]), inputs[3].numpy(),
                             hp.np_u8(w1), s1.cpu().numpy(), hp.np_u8(w2), s2.cpu().numpy(), offset, RSF)
    want = oracle.bf16_decode(ref)
    st = hp.error_stats(got, want)
    pc = layer32.read("pair_count", T)
    assert int(pc.sum()) == rows
    # tokens without a local expert are exact zeros
    assert np.all(got[pc == 0] == 0)
    if rows:
        assert st["rel_l2"] < 2e-2, st
        assert st["contest_ratio"] >= 0.999, st
        fp32, _ = oracle.layer(inputs[0].numpy(), hp.np_u16(inputs[1]), hp.np_u8(inputs[2]), inputs[3].numpy(),
                               hp.np_u8(w1), s1.cpu().numpy(), hp.np_u8(w2), s2.cpu().numpy(), offset, RSF,
                               mode="fp32")
        if T < 32:  # no pruning below 32 tokens: the definition is the same function
            sd = hp.error_stats(got, oracle.bf16_decode(fp32))
            assert sd["rel_l2"] < 8e-2 and sd["cosine"] > 0.995, sd


@pytest.mark.parametrize("T,offset", [(1, 0), (16, 0), (40, 32), (1024, 0)])
def test_layer_vs_reference_gpu_build(pkg, layer32, T, offset):
    """Output parity with the reference's own GPU run on identical inputs: within
    atol 1.0 / rtol 0.3 on >= 99 % of the elements (the reference's stated tolerance),
    plus the tighter relative-L2 bound that is meaningful for O(1) outputs."""
    if not hp.reference_available():
        pytest.skip("oracle/_ref/libref_moe.so not built")
    inputs = hp.cpu_inputs(T, seed=600 + T)
    weights = hp.gpu_shard(offset, 32)
    out = hp.run_layer(layer32, inputs, weights, offset).float().cpu().numpy()
    ref = hp.reference_run(inputs, weights, offset).float().cpu().numpy()
    st = hp.error_stats(out, ref)
    print(f"T={T} offset={offset} vs reference: {st}")
    assert st["contest_ratio"] >= 0.99, st
    if np.abs(ref).max() > 0:
        assert st["rel_l2"] < 3e-2, st


# ------------------------------------------------------------------------- the benchmark's sizes
GOLDEN = __import__("pathlib").Path(__file__).resolve().parent / "golden"
BIG = [("t32", 32, False), ("t53", 53, False), ("t80", 80, False), ("t901", 901, False), ("t14107", 14107, False),
       ("t12288", 12288, False), ("t16384skew", 16384, True)]


@pytest.fixture(scope="module")
def layer_big(pkg):
    lay = pkg.MoeLayer(16384, 32, 0)
    yield lay
    lay.close()


def _sha(a):
    import hashlib
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()[:16]


@pytest.mark.parametrize("name,T,skew", BIG)
def test_dispatch_bit_exact_at_benchmark_sizes(pkg, layer_big, name, T, skew):
    """Routing + the T-keyed pruning dispatch (drop-third at T >= 10000, the per-T constants) against what
    the reference's own kernels gave for the same seeded logits (fixtures written on a B200 by
    tests/golden/make_golden.py) and, when the reference library is present, against those kernels run
    live: top-8 indices and weight bits of every token, per-expert rows, every token's pair count and all
    (token, expert, weight bits) pairs, for shard offsets 0, 96 and 224."""
    from fp8_moe_dev_b200 import gen
    g = np.load(GOLDEN / f"ref_big_{name}.npz")
    logits, bias = gen.make_routing(T, int(g["seed"]), skew)
    assert _sha(logits.numpy()) == str(g["sha_logits"])
    dev = [logits.cuda(), bias.cuda(), torch.zeros(T, H, dtype=torch.float8_e4m3fn, device="cuda"),
           torch.ones(56, T, device="cuda")]
    w1, s1, w2, s2 = hp.gpu_shard(0, 32)
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    layer_big.set_stop_after_stage(1)
    try:
        for offset in (0, 96, 224):
            layer_big.run(*dev, w1, s1, w2, s2, offset, RSF, out)
            layer_big.check()
            idx = layer_big.read("topk_idx", T * TOPK).reshape(T, TOPK)
            w = layer_big.read("topk_weight", T * TOPK).reshape(T, TOPK)
            assert _sha(idx) == str(g["sha_topk_idx"]) and _sha(w.view(np.uint32)) == str(g["sha_topk_weight_bits"])
            pc, le, slot, pw = hp.gpu_pair_arrays(layer_big, T)
            ec = layer_big.read("expert_count", 32)
            s = offset // 32
            assert np.array_equal(ec, g["expert_count"][s]), (name, offset)
            assert np.array_equal(pc, g["pair_n"][s].astype(np.int32)), (name, offset)
            assert hp.pairs_digest(pc, le, pw) == str(g["pairs_digest"][s]), (name, offset)
            # slots of an expert are a permutation of 0 .. rows-1, offsets are the 128-padded prefix sums
            live = np.arange(TOPK)[None, :] < pc[:, None]
            key = np.sort(le[live].astype(np.int64) * (1 << 24) + slot[live])
            want = np.concatenate([e * (1 << 24) + np.arange(ec[e], dtype=np.int64) for e in range(32)])
            assert np.array_equal(key, want)
            eoff = layer_big.read("expert_offset", 33)
            assert np.array_equal(eoff, np.concatenate([[0], np.cumsum((ec + 127) // 128 * 128)]))
            if hp.reference_available():
                d = hp.reference_dispatch_arrays(logits, bias, offset)
                assert d["variant"] == 1
                assert hp.pairs_digest(d["pair_n"], d["pair_le"], d["pair_w"]) == hp.pairs_digest(pc, le, pw)
    finally:
        layer_big.set_stop_after_stage(0)


@pytest.mark.parametrize("T,offset", [(12288, 0), (12288, 160)])
def test_layer_vs_reference_gpu_build_at_t12288(pkg, layer_big, T, offset):
    """One 32-expert shard at the benchmark's batch size, both libraries in one process on the same device
    tensors: drop-third pruning, several 128-row tiles per expert, a persistent schedule of a few thousand
    tiles.  Gate: >= 99 % within atol 1 / rtol 0.3 and rel-L2 < 3e-2; for offset 0 the tokens of the
    committed fixture (whose rows lie in two experts, generated on the CPU here) are also compared with
    what the reference printed when the fixture was made."""
    if not hp.reference_available():
        pytest.skip("oracle/_ref/libref_moe.so not built")
    from fp8_moe_dev_b200 import gen
    inputs = hp.cpu_inputs(T, seed=0)
    weights = hp.gpu_shard(offset, 32)
    g = np.load(GOLDEN / "ref_big_t12288.npz")
    if offset == int(g["out_offset"]):
        weights = tuple(x.clone() for x in weights)
        for e in g["out_experts"]:
            for dst, src in zip(weights, gen.make_expert(offset + int(e))):
                dst[int(e)].copy_(src)
    out = hp.run_layer(layer_big, inputs, weights, offset)
    rows_ours = int(layer_big.read("pair_count", T).sum())
    ref = hp.reference_run(inputs, weights, offset)
    rows_ref = int(hp.reference_dispatch_arrays(inputs[0], inputs[1], offset)["pair_n"].sum())
    st = hp.error_stats(out.float().cpu().numpy(), ref.float().cpu().numpy())
    print(f"T={T} offset={offset} rows {rows_ours} vs reference {rows_ref}: {st}")
    assert rows_ours == rows_ref
    assert st["contest_ratio"] >= 0.99 and st["rel_l2"] < 3e-2, st
    if offset == int(g["out_offset"]):
        toks = torch.from_numpy(g["out_tokens"]).cuda()
        got8 = out[toks][:, ::8].float().cpu().numpy()
        want8 = (g["out_bf16_cols8"].astype(np.uint32) << 16).view(np.float32)
        sg = hp.error_stats(got8, want8)
        print(f"fixture tokens: {sg}")
        assert sg["contest_ratio"] >= 0.99 and sg["rel_l2"] < 3e-2, sg
        assert np.all(got8[g["out_pair_n"] == 0] == 0)


@pytest.mark.parametrize("T,skew", [(2048, False), (12288, False), (16384, True)])
def test_256_expert_chain_vs_sum_of_reference_shard_runs(pkg, T, skew):
    """All 256 experts in one handle (the benchmark's one-GPU configuration: a tile schedule over 256
    experts, 70+ tiles per persistent CTA at the large sizes) against the fp32 sum of the reference's
    eight 32-expert `run` calls on the same inputs."""
    if not hp.reference_available():
        pytest.skip("oracle/_ref/libref_moe.so not built")
    inputs = hp.cpu_inputs(T, seed=0, skew=skew)
    weights = hp.gpu_shard(0, 256)
    lay = pkg.MoeLayer(T, 256, 0)
    try:
        out = hp.run_layer(lay, inputs, weights, 0).float()
        rows = int(lay.read("pair_count", T).sum())
        ec = lay.read("expert_count", 256)
    finally:
        lay.close()
    total = torch.zeros(T, H, device="cuda")
    rows_ref = 0
    for s in range(8):
        sl = slice(32 * s, 32 * s + 32)
        total += hp.reference_run(inputs, tuple(x[sl] for x in weights), 32 * s).float()
        d = hp.reference_dispatch_arrays(inputs[0], inputs[1], 32 * s)
        rows_ref += int(d["pair_n"].sum())
        assert np.array_equal(ec[sl], d["expert_count"]), s
    st = hp.error_stats(out.cpu().numpy(), total.cpu().numpy())
    print(f"T={T} skew={skew} rows {rows} (reference {rows_ref}) max rows/expert {int(ec.max())}: {st}")
    assert rows == rows_ref
    assert st["contest_ratio"] >= 0.99 and st["rel_l2"] < 1.5e-2, st


def test_exact_silu_option_changes_only_the_activation(pkg, oracle, layer32):
    T, offset = 16, 0
    inputs = hp.cpu_inputs(T, seed=700)
    weights = hp.gpu_shard(0, 32)
    layer32.set_exact_silu(True)
    try:
        out = hp.run_layer(layer32, inputs, weights, offset).float().cpu().numpy()
    finally:
        layer32.set_exact_silu(False)
    w1, s1, w2, s2 = weights
    ref, _ = oracle.layer(inputs[0].numpy(), hp.np_u16(inputs[1]), hp.np_u8(inputs[2]), inputs[3].numpy(),
                          hp.np_u8(w1), s1.cpu().numpy(), hp.np_u8(w2), s2.cpu().numpy(), offset, RSF,
                          exact_silu=True)
    st = hp.error_stats(out, oracle.bf16_decode(ref))
    assert st["rel_l2"] < 2e-2, st


# ------------------------------------------------------------------------- properties
def test_scaling_factor_is_linear(pkg, layer32):
    T = 64
    inputs = hp.cpu_inputs(T, seed=800)
    weights = hp.gpu_shard(0, 32)
    a = hp.run_layer(layer32, inputs, weights, 0, rsf=1.0).float()
    b = hp.run_layer(layer32, inputs, weights, 0, rsf=2.0).float()
    assert torch.allclose(b, 2 * a, rtol=2 ** -7, atol=1e-6)


def test_token_permutation_permutes_outputs(pkg, layer32):
    T = 96
    inputs = hp.cpu_inputs(T, seed=801)
    weights = hp.gpu_shard(0, 32)
    out = hp.run_layer(layer32, inputs, weights, 0)
    perm = torch.randperm(T, generator=torch.Generator().manual_seed(5))
    pin = (inputs[0][perm].contiguous(), inputs[1], inputs[2][perm].contiguous(), inputs[3][:, perm].contiguous())
    out_p = hp.run_layer(layer32, pin, weights, 0)
    assert torch.equal(out_p.cpu(), out.cpu()[perm]), "rows depend on their position in the batch"


def test_runs_are_deterministic_and_see_new_contents(pkg, layer32):
    """Same pointers, new contents -> new result (the reference would replay cached routing)."""
    T = 48
    inputs = [x.cuda() for x in hp.cpu_inputs(T, seed=802)]
    other = [x.cuda() for x in hp.cpu_inputs(T, seed=803)]
    w1, s1, w2, s2 = hp.gpu_shard(0, 32)
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    layer32.run(*inputs, w1, s1, w2, s2, 0, RSF, out)
    first = out.clone()
    layer32.run(*inputs, w1, s1, w2, s2, 0, RSF, out)
    assert torch.equal(first, out)
    for dst, src in zip(inputs, other):
        dst.copy_(src)
    layer32.run(*inputs, w1, s1, w2, s2, 0, RSF, out)
    layer32.check()
    fresh = torch.empty_like(out)
    layer32.run(*other, w1, s1, w2, s2, 0, RSF, fresh)
    layer32.check()
    assert torch.equal(out, fresh) and not torch.equal(out, first)


def test_cuda_graph_capture_and_replay(pkg, layer32):
    T = 16
    inputs = [x.cuda() for x in hp.cpu_inputs(T, seed=804)]
    other = [x.cuda() for x in hp.cpu_inputs(T, seed=805)]
    w1, s1, w2, s2 = hp.gpu_shard(0, 32)
    out = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")
    layer32.run(*inputs, w1, s1, w2, s2, 0, RSF, out)  # warm-up outside capture (tensor maps encoded)
    eager = out.clone()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            layer32.run(*inputs, w1, s1, w2, s2, 0, RSF, out)
    torch.cuda.current_stream().wait_stream(s)
    out.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    for dst, src in zip(inputs, other):
        dst.copy_(src)
    g.replay()
    torch.cuda.synchronize()
    want = torch.empty_like(out)
    layer32.run(*other, w1, s1, w2, s2, 0, RSF, want)
    layer32.check()
    assert torch.equal(out, want)


def test_shard_sum_identity_64_experts(pkg):
    """One pass over 64 local experts == sum of the two 32-expert shard passes."""
    T = 64
    inputs = hp.cpu_inputs(T, seed=806)
    wa = hp.gpu_shard(0, 32)
    wb = hp.gpu_shard(32, 32)
    lay32 = pkg.MoeLayer(T, 32, 0)
    lay64 = pkg.MoeLayer(T, 64, 0)
    try:
        oa = hp.run_layer(lay32, inputs, wa, 0).float()
        ob = hp.run_layer(lay32, inputs, wb, 32).float()
        wcat = tuple(torch.cat([x, y]) for x, y in zip(wa, wb))
        oc = hp.run_layer(lay64, inputs, wcat, 0).float()
        del wcat
    finally:
        lay32.close()
        lay64.close()
    ref = oa + ob
    assert torch.allclose(oc, ref, rtol=2 ** -6, atol=2e-2)
    st = hp.error_stats(oc.cpu().numpy(), ref.cpu().numpy())
    assert st["rel_l2"] < 6e-3, st


# ------------------------------------------------------------------------- boundary behaviour
def test_host_pointer_entry_point(pkg, layer32):
    T = 16
    inputs = hp.cpu_inputs(T, seed=807)
    w1, s1, w2, s2 = hp.gpu_shard(0, 32)
    dev = hp.run_layer(layer32, inputs, (w1, s1, w2, s2), 0).cpu()
    host_out = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()
    pinned = [x.pin_memory() for x in (inputs[0], inputs[2], inputs[3])]
    layer32.run_host(pinned[0], inputs[1].cuda(), pinned[1], pinned[2], w1, s1, w2, s2, 0, RSF, host_out)
    assert torch.equal(host_out, dev)


def test_errors_are_reported_not_swallowed(pkg, layer32):
    T = 2048  # above the handle's capacity of 1024
    inputs = hp.cpu_inputs(T, seed=808)
    with pytest.raises(pkg.MoeError) as ei:
        hp.run_layer(layer32, inputs, hp.gpu_shard(0, 32), 0)
    assert ei.value.code == -3
    small = hp.cpu_inputs(4, seed=809)
    w1, s1, w2, s2 = hp.gpu_shard(0, 32)
    out = torch.empty(4, H, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(pkg.MoeError):
        layer32.run(*[x.cuda() for x in small], w1, s1, w2, s2, 999, RSF, out)
    # a shard is a whole block of 32 experts inside the 256: no offset between blocks, none hanging over
    for bad in (16, 48, 240, 256, -32):
        with pytest.raises(pkg.MoeError) as ei:
            layer32.run(*[x.cuda() for x in small], w1, s1, w2, s2, bad, RSF, out)
        assert ei.value.code == -1 and "multiple of 32" in str(ei.value)
    lay64 = pkg.MoeLayer(4, 64, 0)
    try:
        w64 = tuple(torch.cat([x, x]) for x in (w1, s1, w2, s2))
        with pytest.raises(pkg.MoeError):
            lay64.run(*[x.cuda() for x in small], *w64, 224, RSF, out)   # 224 + 64 > 256
        lay64.run(*[x.cuda() for x in small], *w64, 192, RSF, out)
        lay64.check()
        del w64
    finally:
        lay64.close()
    with pytest.raises((TypeError, ValueError)):
        layer32.run(small[0].cuda().half(), *[x.cuda() for x in small[1:]], w1, s1, w2, s2, 0, RSF, out)
    # empty batch is a no-op, as in the reference
    empty = [torch.empty(0, 256, device="cuda"), small[1].cuda(),
             torch.empty(0, H, device="cuda", dtype=torch.float8_e4m3fn), torch.empty(56, 0, device="cuda")]
    layer32.run(*empty, w1, s1, w2, s2, 0, RSF, torch.empty(0, H, dtype=torch.bfloat16, device="cuda"))


def test_token_with_no_local_expert_gets_zeros(pkg, layer32):
    T = 8
    logits = torch.full((T, 256), -10.0)
    logits[:, 200:208] = 5.0  # every token routes to group 6 only
    bias = torch.zeros(256, dtype=torch.bfloat16)
    _, _, hidden, hscale = hp.cpu_inputs(T, seed=810)
    out = hp.run_layer(layer32, (logits, bias, hidden, hscale), hp.gpu_shard(0, 32), 0)
    assert torch.count_nonzero(out) == 0
    assert layer32.read("num_tiles", 1)[0] == 0


def test_tvm_ffi_entry_point_matches_c_abi(pkg, layer32):
    from pathlib import Path
    shim = Path(pkg.__file__).parent / "libmoe_fp8_b200_tvm.so"
    if not shim.exists():
        pytest.skip("shim not built")
    import tvm_ffi
    mod = tvm_ffi.load_module(str(shim))
    T = 16
    inputs = hp.cpu_inputs(T, seed=811)
    w1, s1, w2, s2 = hp.gpu_shard(0, 32)
    want = hp.run_layer(layer32, inputs, (w1, s1, w2, s2), 0)
    dev = [x.cuda() for x in inputs]
    out = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")
    mod.run(dev[0], dev[1], dev[2], dev[3], w1, s1, w2, s2, 0, RSF, out)
    torch.cuda.synchronize()
    assert torch.equal(out, want)


def test_pipelined_host_entry_point(pkg, layer32):
    """run_host_async / host_wait: five calls kept two deep in flight over rotating pinned buffers
    give, call by call, what the synchronous device-pointer run gives for the same inputs."""
    T = 300
    weights = hp.gpu_shard(0, 32)
    raw = [hp.cpu_inputs(T, seed=1700 + i) for i in range(3)]
    bias = raw[0][1]
    sets = [(r[0], bias, r[2], r[3]) for r in raw]
    want = [hp.run_layer(layer32, s, weights, 0).cpu() for s in sets]
    assert not torch.equal(want[0], want[1])
    pinned = [[x.pin_memory() for x in (s[0], s[2], s[3])] for s in sets]
    outs = [torch.zeros(T, H, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    bias_dev = bias.cuda()
    tickets = []
    for i in range(5):
        if i >= 2:   # the buffer about to be reused holds call i-2's result
            layer32.host_wait(tickets[i - 2])
            assert torch.equal(outs[i % 2], want[(i - 2) % 3]), f"call {i - 2}"
            outs[i % 2].zero_()
        p = pinned[i % 3]
        tickets.append(layer32.run_host_async(p[0], bias_dev, p[1], p[2], *weights, 0, RSF, outs[i % 2]))
    for i in (3, 4):
        layer32.host_wait(tickets[i])
        assert torch.equal(outs[i % 2], want[i % 3]), f"call {i}"
    layer32.host_wait(tickets[0])   # long finished: returns at once
    layer32.check()
    with pytest.raises(Exception):
        layer32.host_wait(99)


@pytest.mark.parametrize("T,offset,decode", [(3, 160, True), (8, 224, True), (9, 0, False), (17, 96, False),
                                             (31, 32, False), (47, 128, False), (64, 192, False), (5, 64, False)])
def test_layer_vs_oracle_across_the_path_boundaries(pkg, oracle, T, offset, decode):
    """Batch sizes on both sides of the internal path choices (decode kernel up to 8 tokens, chain
    with and without the small-batch GEMM instantiation, exact / pruning dispatch from 32 tokens on),
    every shard offset once: same bounds against the oracle as the fixed cases above."""
    lay = pkg.MoeLayer(64, 32, 0)
    lay.set_decode_kernel(decode)
    try:
        inputs = hp.cpu_inputs(T, seed=3000 + T)
        weights = hp.gpu_shard(offset, 32)
        got = hp.run_layer(lay, inputs, weights, offset).float().cpu().numpy()
        pc = lay.read("pair_count", T)
    finally:
        lay.close()
    w1, s1, w2, s2 = weights
    ref, rows = oracle.layer(inputs[0].numpy(), hp.np_u16(inputs[1]), hp.np_u8(inputs[2]), inputs[3].numpy(),
                             hp.np_u8(w1), s1.cpu().numpy(), hp.np_u8(w2), s2.cpu().numpy(), offset, RSF)
    assert np.isfinite(got).all() and int(pc.sum()) == rows
    assert np.all(got[pc == 0] == 0)
    if rows:
        st = hp.error_stats(got, oracle.bf16_decode(ref))
        assert st["rel_l2"] < 2e-2 and st["contest_ratio"] >= 0.999, st


def test_strided_expert_placement_sums_to_the_full_layer(pkg):
    """Strided placement (multi-GPU wrapper): four handles holding every 4th expert produce, together,
    the pairs of the 256-expert layer -- same per-shard policy, other owner -- so their outputs sum
    to the one-handle result; rows are spread evenly over the handles."""
    T, S = 160, 4
    from fp8_moe_dev_b200 import gen
    inputs = hp.cpu_inputs(T, seed=4000)
    full = pkg.MoeLayer(T, 256, 0)
    w_full = hp.gpu_shard(0, 256)
    want = hp.run_layer(full, inputs, w_full, 0).float().cpu()
    pc_full = int(full.read("pair_count", T).sum())
    full.close()
    del w_full
    total = torch.zeros(T, H)
    rows = []
    for phase in range(S):
        lay = pkg.MoeLayer(T, 256 // S, 0)
        lay.set_expert_stride(S)
        w = gen.make_experts(range(phase, 256, S), device="cuda", out_device="cuda")
        total += hp.run_layer(lay, inputs, w, phase).float().cpu()
        rows.append(int(lay.read("pair_count", T).sum()))
        with pytest.raises(Exception):
            hp.run_layer(lay, inputs, w, S)   # phase out of range
        lay.close()
        del w
    assert sum(rows) == pc_full
    assert max(rows) <= 1.25 * pc_full / S
    st = hp.error_stats(total.numpy(), want.numpy())
    assert st["rel_l2"] < 1e-2, st     # four bf16 partial outputs added in fp32 vs one bf16 output
    bad = pkg.MoeLayer(T, 32, 0)
    with pytest.raises(Exception):
        bad.set_expert_stride(4)       # 32 * 4 != 256
    bad.close()


def test_load_aware_expert_placement_sums_to_the_full_layer(pkg):
    """Table placement from measured loads: four handles, experts dealt longest-first by the routed
    rows of the batch itself, sum to the 256-expert result and carry nearly equal numbers of rows."""
    T, S = 192, 4
    from fp8_moe_dev_b200 import gen
    from fp8_moe_dev_b200.dist import balanced_expert_ids
    inputs = hp.cpu_inputs(T, seed=4100)
    loads = pkg.expert_loads(inputs[0].cuda(), inputs[1].cuda(), RSF)
    full = pkg.MoeLayer(T, 256, 0)
    w_full = hp.gpu_shard(0, 256)
    want = hp.run_layer(full, inputs, w_full, 0).float().cpu()
    assert loads == [int(x) for x in full.read("expert_count", 256)]
    pc_full = int(full.read("pair_count", T).sum())
    full.close()
    del w_full
    ids = balanced_expert_ids(loads, S)
    total = torch.zeros(T, H)
    rows = []
    for r in range(S):
        lay = pkg.MoeLayer(T, 256 // S, 0)
        lay.set_expert_map(ids[r])
        w = gen.make_experts(ids[r], device="cuda", out_device="cuda")
        total += hp.run_layer(lay, inputs, w, 0).float().cpu()
        rows.append(int(lay.read("pair_count", T).sum()))
        assert rows[-1] == sum(loads[e] for e in ids[r])
        lay.close()
        del w
    assert sum(rows) == pc_full and max(rows) <= 1.05 * pc_full / S + 8
    st = hp.error_stats(total.numpy(), want.numpy())
    assert st["rel_l2"] < 1e-2, st
    bad = pkg.MoeLayer(T, 64, 0)
    with pytest.raises(Exception):
        bad.set_expert_map(list(range(10)))     # 64 slots need 64 experts
    bad.set_expert_map(None)
    bad.close()


# ------------------------------------------------------------------------- failure reporting
def test_device_status_is_sticky_until_checked(pkg):
    """A failure that a kernel recorded survives later runs until the host reads it.  The failure is
    injected from the host (a status word and a stale grid-barrier count copied into the control block, as
    a decode launch that gave up half-way would leave them); nothing on the GPU faults or hangs.  Two more
    runs are enqueued, check() must still report the failure, and after it the next run is correct again."""
    T = 4
    inputs = hp.cpu_inputs(T, seed=5000)
    weights = hp.gpu_shard(0, 32)
    lay = pkg.MoeLayer(64, 32, 0)
    try:
        good = hp.run_layer(lay, inputs, weights, 0).clone()
        for chain_T in (4, 40):    # the decode kernel (T <= 8) and the five-kernel chain
            inp = inputs if chain_T == 4 else hp.cpu_inputs(chain_T, seed=5001)
            want = hp.run_layer(lay, inp, weights, 0).clone()
            lay.inject_device_status(105, stale_barrier_arrivals=7)
            dev = [x.cuda() for x in inp]
            out = torch.zeros(chain_T, H, dtype=torch.bfloat16, device="cuda")
            for _ in range(2):
                lay.run(*dev, *weights, 0, RSF, out)
            with pytest.raises(pkg.MoeError) as ei:
                lay.check()
            assert ei.value.code == -4 and "105" in str(ei.value)
            lay.check()            # reported once, then clear
            again = hp.run_layer(lay, inp, weights, 0)
            assert torch.equal(again, want)
        assert torch.equal(hp.run_layer(lay, inputs, weights, 0), good)
    finally:
        lay.close()


def test_exchange_wait_runs_out_and_is_reported(pkg):
    """The fused combine + reduce-scatter's bounded wait, made to run out on ONE GPU without any fault:
    a two-rank exchange whose two receive buffers are plain local allocations, of which only rank 0's
    call is ever issued, with the wait limit set to 2 ms.  The owner step finds no flag from rank 1,
    gives up after the limit, the kernel completes, check() reports the exchange timeout, and the next
    ordinary run on the handle is correct."""
    T = 64
    lib = pkg._lib.load()
    inputs = hp.cpu_inputs(T, seed=5100)
    weights = hp.gpu_shard(0, 32)
    lay = pkg.MoeLayer(T, 32, 0)
    try:
        want = hp.run_layer(lay, inputs, weights, 0).clone()
        nbytes = int(lib.moe_fp8_b200_exchange_bytes(T, 2))
        bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
        owned = torch.full((T // 2, H), 7.0, dtype=torch.bfloat16, device="cuda")
        lay.set_wait_limit_us(2000)
        dev = [x.cuda() for x in inputs]
        torch.cuda.synchronize()
        import time
        t0 = time.perf_counter()
        lay.run_reduce_scatter(*dev, *weights, 0, RSF, owned, [b.data_ptr() for b in bufs], nbytes, 0, 2, 1)
        with pytest.raises(pkg.MoeError) as ei:
            lay.check()
        dt = time.perf_counter() - t0
        assert ei.value.code == -4 and "104" in str(ei.value), str(ei.value)
        assert dt < 0.5, f"the wait took {dt:.3f} s with a 2 ms limit"
        assert torch.count_nonzero(owned) == 0     # a step that gave up writes zeros, not stale rows
        lay.set_wait_limit_us(1000000)
        assert torch.equal(hp.run_layer(lay, inputs, weights, 0), want)
    finally:
        lay.close()


def test_weight_scale_prelayout_follows_pointers_and_invalidation(pkg, layer32):
    """The handle keeps a copy of the weight scales in the GEMMs' order, keyed by the scale tensors'
    addresses: other tensors are picked up by themselves, new contents under the same addresses after
    invalidate_weights()."""
    T = 40
    dev = [x.cuda() for x in hp.cpu_inputs(T, seed=6000)]
    w1, s1, w2, s2 = hp.gpu_shard(0, 32)
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")

    def run(sa, sb):
        layer32.run(*dev, w1, sa, w2, sb, 0, RSF, out)
        layer32.check()
        return out.clone()

    layer32.invalidate_weights()
    base = run(s1, s2)
    s1b, s2b = (s1 * 2.0).contiguous(), s2.clone()
    doubled = run(s1b, s2b)                       # other addresses: seen at once
    assert not torch.equal(doubled, base)
    s1b.copy_(s1)                                 # same addresses, old contents back
    assert torch.equal(run(s1b, s2b), doubled), "the pre-laid-out copy is keyed by address"
    layer32.invalidate_weights()
    assert torch.equal(run(s1b, s2b), base)
    layer32.invalidate_weights()


@pytest.mark.parametrize("T,offset", [(3, 96), (9, 0), (40, 32), (300, 96), (1024, 0)])
def test_tile_ordered_weight_copies_change_nothing(pkg, T, offset):
    """MOE_FP8_B200_OPT_WEIGHT_PRELAYOUT: the GEMMs read the weights from the handle's tile-ordered copies (one
    contiguous 32 KB piece per tile and K block) and every bit of the result stays the same, also after the option
    has been switched off again (the copies are freed) and on once more."""
    dev = [x.cuda() for x in hp.cpu_inputs(T, seed=6100 + T)]
    w = hp.gpu_shard(offset, 32)
    lay = pkg.MoeLayer(T, 32, 0)
    try:
        lay.set_decode_kernel(False)
        outs = []
        for on in (False, True, False, True):
            lay.set_weight_prelayout(on)
            out = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")
            lay.run(*dev, *w, offset, RSF, out)
            lay.check()
            outs.append(out)
        assert outs[0].float().abs().sum() > 0
        for o in outs[1:]:
            assert torch.equal(o.view(torch.int16), outs[0].view(torch.int16))
    finally:
        lay.close()


def test_tile_ordered_weight_copies_follow_pointers_and_invalidation(pkg):
    T = 64
    dev = [x.cuda() for x in hp.cpu_inputs(T, seed=6200)]
    w1, s1, w2, s2 = hp.gpu_shard(0, 32)
    lay = pkg.MoeLayer(T, 32, 0)
    try:
        lay.set_weight_prelayout(True)
        out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")

        def run(wa, wb):
            lay.run(*dev, wa, s1, wb, s2, 0, RSF, out)
            lay.check()
            return out.clone()

        base = run(w1, w2)
        w1b = w1.clone()
        w1b.view(torch.uint8)[:, :, :128] ^= 0x80          # flip the signs of the first K block of every row
        w2b = w2.clone()
        changed = run(w1b, w2b)                            # other addresses: seen at once
        assert not torch.equal(changed, base)
        w1b.copy_(w1)                                      # same addresses, old contents back
        assert torch.equal(run(w1b, w2b), changed), "the copies are keyed by address"
        lay.invalidate_weights()
        assert torch.equal(run(w1b, w2b), base)
    finally:
        lay.close()


@pytest.mark.parametrize("T,offset", [(5, 0), (9, 32), (16, 0), (40, 96), (64, 0), (65, 0)])
def test_small_batch_ring_changes_nothing(pkg, T, offset):
    """Batches of 5 to 64 tokens run the GEMMs with 64-row activation boxes and a fourth operand stage
    (MOE_FP8_B200_OPT_SMALL_BATCH_RING, on by default): same arithmetic in the same order, so the results are
    bit-identical to the three-stage kernel's.  The handle has seen a larger batch before, so that the rows the
    64-row boxes leave out hold stale data, not zeros."""
    w = hp.gpu_shard(offset, 32)
    lay = pkg.MoeLayer(512, 32, 0)
    try:
        lay.set_decode_kernel(False)
        big = [x.cuda() for x in hp.cpu_inputs(512, seed=6400)]
        out_big = torch.empty(512, H, dtype=torch.bfloat16, device="cuda")
        lay.run(*big, *w, offset, RSF, out_big)
        lay.check()
        dev = [x.cuda() for x in hp.cpu_inputs(T, seed=6400 + T)]
        outs = []
        for on in (True, False, True):
            lay.set_small_batch_ring(on)
            out = torch.full((T, H), float("nan"), dtype=torch.bfloat16, device="cuda")
            lay.run(*dev, *w, offset, RSF, out)
            lay.check()
            outs.append(out)
        assert torch.isfinite(outs[0].float()).all() and outs[0].float().abs().sum() > 0
        for o in outs[1:]:
            assert torch.equal(o.view(torch.int16), outs[0].view(torch.int16))
    finally:
        lay.close()
