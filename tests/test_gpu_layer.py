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
    slots = [set() for _ in range(32)]
    for t in range(T):
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
