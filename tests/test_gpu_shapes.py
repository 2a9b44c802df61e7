"""Other shapes of the layer (B200): hidden / intermediate sizes and routing constants that the reference
compiles in (kernel/moe_fp8.cu:292-304) are run-time values of a handle made with create_shaped.  The CUDA
chain is compared with the CPU oracle set to the same shape; the reference's own GPU build exists for
7168 / 2048 / 8 / 8 / 4 only, so the oracle (pinned against the reference at that shape) is the checker here."""
import numpy as np
import pytest
import torch

import helpers as hp
from helpers import RSF, TOPK

pytestmark = pytest.mark.gpu

# (hidden, intermediate) with K-block counts 8/4, 16/6, 2/32 (GEMM2 uses both halves of the scale registers'
# first word), 64/1 (the largest hidden, a one-block intermediate) and 40/3
GEOMETRIES = [(1024, 512), (2048, 768), (256, 4096), (8192, 128), (5120, 384)]


def _inputs(T, seed, hidden, skew=False):
    from fp8_moe_dev_b200 import gen
    logits, bias = gen.make_routing(T, seed, skew)
    q, sc = gen.make_hidden(T, seed + 1, hidden=hidden)
    return logits, bias, q, sc


def _shard(offset, E, hidden, inter, seed=4000):
    from fp8_moe_dev_b200 import gen
    return gen.make_shard(offset, E, seed, device="cuda", out_device="cuda", hidden=hidden, inter=inter)


def _run(layer, inputs, weights, offset, hidden):
    logits, bias, q, sc = [x.cuda() for x in inputs]
    T = logits.shape[0]
    out = torch.full((T, hidden), float("nan"), dtype=torch.bfloat16, device="cuda")
    layer.invalidate_weights()
    layer.run(logits, bias, q, sc, *weights, offset, RSF, out)
    layer.check()
    return out


def _oracle_layer(oracle, inputs, weights, offset, mode="faithful", pruning=True):
    w1, s1, w2, s2 = weights
    return oracle.layer(inputs[0].numpy(), hp.np_u16(inputs[1]), hp.np_u8(inputs[2]), inputs[3].numpy(), hp.np_u8(w1),
                        s1.cpu().numpy(), hp.np_u8(w2), s2.cpu().numpy(), offset, RSF, mode=mode,
                        reference_pruning=pruning)


@pytest.mark.parametrize("hidden,inter", GEOMETRIES)
@pytest.mark.parametrize("T,offset,pruning", [(3, 0, True), (40, 32, True), (300, 0, False)])
def test_layer_of_another_geometry_vs_oracle(pkg, oracle, hidden, inter, T, offset, pruning):
    layer = pkg.MoeLayer(512, 32, 0, hidden=hidden, intermediate=inter)
    try:
        layer.set_reference_pruning(pruning)
        inputs = _inputs(T, 900 + T, hidden)
        weights = _shard(offset, 32, hidden, inter)
        got = _run(layer, inputs, weights, offset, hidden).float().cpu().numpy()
        assert np.isfinite(got).all()
        with oracle.shape(hidden, inter):
            ref, rows = _oracle_layer(oracle, inputs, weights, offset, pruning=pruning)
            # routing and dispatch tables: bit-exact against the oracle given the GPU's own routing result
            idx = layer.read("topk_idx", T * TOPK).reshape(T, TOPK)
            w = layer.read("topk_weight", T * TOPK).reshape(T, TOPK)
            opc, ople, opw, oec = oracle.dispatch(idx, w, offset, 32, oracle.policy(T, pruning), RSF)
        pc, le, slot, pw = hp.gpu_pair_arrays(layer, T)
        assert np.array_equal(pc, opc)
        keep = np.arange(TOPK)[None, :] < pc[:, None]
        assert np.array_equal(le[keep], ople[keep])
        assert np.array_equal(pw.view(np.uint32)[keep], opw.view(np.uint32)[keep])
        assert np.array_equal(layer.read("expert_count", 32), oec)
        assert int(pc.sum()) == rows
        want = oracle.bf16_decode(ref)
        assert np.all(got[pc == 0] == 0)
        st = hp.error_stats(got, want)
        assert st["rel_l2"] < 2e-2, st
        assert st["contest_ratio"] >= 0.999, st
    finally:
        layer.close()


def test_intermediates_of_another_geometry_vs_oracle(pkg, oracle):
    """Packed rows, GEMM1 + SwiGLU + requantisation and GEMM2 rows of one shape, stage by stage."""
    hidden, inter, T, offset = 2048, 768, 130, 64
    layer = pkg.MoeLayer(256, 32, 0, hidden=hidden, intermediate=inter)
    try:
        inputs = _inputs(T, 77, hidden)
        weights = _shard(offset, 32, hidden, inter)
        _run(layer, inputs, weights, offset, hidden)
        M = layer.row_capacity
        eoff = layer.read("expert_offset", 33)
        ecnt = layer.read("expert_count", 32)
        row_token = layer.read("row_token", M)
        a1 = layer.read("a1", M * hidden).reshape(M, hidden)
        sfa1 = layer.read("sfa1", (hidden // 128) * M).reshape(hidden // 128, M)
        a2 = layer.read("a2", M * inter).reshape(M, inter)
        sfa2 = layer.read("sfa2", (inter // 128) * M).reshape(inter // 128, M)
        y = layer.read("y", M * hidden).reshape(M, hidden)
        hq, hs = hp.np_u8(inputs[2]), inputs[3].numpy()
        w1, s1, w2, s2 = weights
        checked = 0
        with oracle.shape(hidden, inter):
            for e in np.flatnonzero(ecnt)[:6]:
                r0, n = int(eoff[e]), int(ecnt[e])
                toks = row_token[r0:r0 + n]
                assert np.array_equal(a1[r0:r0 + n], hq[toks])
                assert np.array_equal(sfa1[:, r0:r0 + n], hs[:, toks])
                oy, od, oa2, osf = oracle.expert_rows(hq, hs, toks, hp.np_u8(w1[e]), s1[e].cpu().numpy(), hp.np_u8(w2[e]),
                                                      s2[e].cpu().numpy(), want_all=True)
                # e4m3 payloads within one code step where the scale agrees, scales to fp32 rounding of the maximum
                assert np.allclose(sfa2[:, r0:r0 + n].T, osf, rtol=2e-2)
                ga2 = oracle.e4m3_decode(a2[r0:r0 + n]) * np.repeat(sfa2[:, r0:r0 + n].T, 128, axis=1)
                wa2 = oracle.e4m3_decode(oa2) * np.repeat(osf, 128, axis=1)
                assert hp.error_stats(ga2, wa2)["rel_l2"] < 3e-2
                gy = oracle.bf16_decode(y[r0:r0 + n])
                assert hp.error_stats(gy, oy)["rel_l2"] < 2e-2
                checked += 1
        assert checked > 0
    finally:
        layer.close()


@pytest.mark.parametrize("top_k,n_group,topk_group", [(8, 8, 4), (4, 4, 2), (6, 1, 1), (2, 8, 1), (8, 2, 1), (1, 8, 8)])
def test_other_routing_constants_vs_oracle(pkg, oracle, top_k, n_group, topk_group):
    hidden, inter, T = 512, 256, 700
    layer = pkg.MoeLayer(1024, 256, 0, hidden=hidden, intermediate=inter, top_k=top_k, n_group=n_group,
                         topk_group=topk_group)
    try:
        layer.set_reference_pruning(False)
        inputs = _inputs(T, 31 + top_k, hidden, skew=(n_group == 2))
        weights = _shard(0, 256, hidden, inter, seed=5000)
        got = _run(layer, inputs, weights, 0, hidden).float().cpu().numpy()
        idx = layer.read("topk_idx", T * TOPK).reshape(T, TOPK)
        w = layer.read("topk_weight", T * TOPK).reshape(T, TOPK)
        with oracle.shape(hidden, inter, top_k, n_group, topk_group):
            oidx, ow = oracle.route(inputs[0].numpy(), hp.np_u16(inputs[1]))
            margin = oracle.route_margin(inputs[0].numpy(), hp.np_u16(inputs[1]))
            ref, rows = _oracle_layer(oracle, inputs, weights, 0, pruning=False)
        assert np.all(idx[:, top_k:] == -1) and np.all(w[:, top_k:] == 0)
        assert np.all((idx[:, :top_k] >= 0) & (idx[:, :top_k] < 256))
        # the picks come from at most topk_group groups of 256 / n_group experts
        groups = idx[:, :top_k] // (256 // n_group)
        assert max(len(set(g)) for g in groups) <= topk_group
        safe = margin > 1e-5
        assert safe.mean() > 0.9
        assert np.array_equal(np.sort(idx[safe], 1), np.sort(oidx[safe], 1))
        same = np.all(idx == oidx, axis=1)
        assert same.mean() > 0.95
        assert np.allclose(w[same], ow[same], rtol=5e-6, atol=1e-9)
        assert np.allclose(w.sum(1), 1.0, atol=1e-5)
        pc = layer.read("pair_count", T)
        assert np.all(pc[safe] == top_k)   # all 256 experts are local and nothing is pruned
        if same.all():
            assert int(pc.sum()) == rows
        st = hp.error_stats(got[same], oracle.bf16_decode(ref)[same])
        assert st["rel_l2"] < 2e-2 and st["contest_ratio"] >= 0.999, st
    finally:
        layer.close()


def test_reference_geometry_with_other_routing_constants(pkg, oracle):
    """7168 / 2048 keep their compile-time kernels; only the routing kernel takes the run-time constants."""
    T, offset = 64, 96
    layer = pkg.MoeLayer(64, 32, 0, top_k=4, n_group=4, topk_group=2)
    try:
        inputs = hp.cpu_inputs(T, seed=4242)
        weights = hp.gpu_shard(offset, 32)
        got = hp.run_layer(layer, inputs, weights, offset).float().cpu().numpy()
        with oracle.shape(7168, 2048, 4, 4, 2):
            ref, rows = _oracle_layer(oracle, inputs, weights, offset)
            oidx, _ = oracle.route(inputs[0].numpy(), hp.np_u16(inputs[1]))
            margin = oracle.route_margin(inputs[0].numpy(), hp.np_u16(inputs[1]))
        idx = layer.read("topk_idx", T * TOPK).reshape(T, TOPK)
        safe = margin > 1e-5
        assert safe.mean() > 0.9
        assert np.array_equal(idx[safe], oidx[safe])
        assert np.all(idx[:, 4:] == -1)
        if np.array_equal(idx, oidx):
            assert int(layer.read("pair_count", T).sum()) == rows
        st = hp.error_stats(got, oracle.bf16_decode(ref))
        assert st["rel_l2"] < 2e-2 and st["contest_ratio"] >= 0.999, st
    finally:
        layer.close()


def test_default_shape_handle_is_the_reference_handle(pkg):
    import ctypes as C
    a = pkg.MoeLayer(64, 32, 0)
    b = pkg.MoeLayer(64, 32, 0, hidden=7168, intermediate=2048, top_k=8, n_group=8, topk_group=4)
    c = pkg.MoeLayer(64, 32, 0, hidden=1024, intermediate=512, top_k=4, n_group=4, topk_group=2)
    try:
        lib = pkg._lib.load()
        for lay, want in ((a, (7168, 2048, 8, 8, 4)), (b, (7168, 2048, 8, 8, 4)), (c, (1024, 512, 4, 4, 2))):
            sh = pkg._lib.Shape()
            assert lib.moe_fp8_b200_get_shape(lay._h, C.byref(sh)) == 0
            assert (sh.hidden, sh.intermediate, sh.top_k, sh.n_group, sh.topk_group) == want
        c.close()
        inputs = hp.cpu_inputs(48, seed=9)
        weights = hp.gpu_shard(0, 32)
        x = hp.run_layer(a, inputs, weights, 0)
        y = hp.run_layer(b, inputs, weights, 0)
        assert torch.equal(x.view(torch.int16), y.view(torch.int16))
        assert np.array_equal(a.read("topk_idx", 48 * TOPK), b.read("topk_idx", 48 * TOPK))
        # the slot part of a pair code is handed out by atomics (order of arrival); the expert part is not
        assert np.array_equal(a.read("pair_code", 48 * TOPK) >> 24, b.read("pair_code", 48 * TOPK) >> 24)
        assert np.array_equal(a.read("pair_weight", 48 * TOPK), b.read("pair_weight", 48 * TOPK))
    finally:
        a.close()
        b.close()


def test_quantize_hidden_of_another_length_is_bit_exact(pkg, oracle):
    from fp8_moe_dev_b200 import gen
    for hidden, T in [(1024, 77), (384 * 2, 5), (8192, 33)]:
        layer = pkg.MoeLayer(128, 32, 0, hidden=hidden, intermediate=256)
        try:
            x = gen._gen("cpu", 5).randn(T, hidden).to(torch.bfloat16)
            x[0, :128] = 0          # an all-zero block
            x[1, 130] = 3.0e38      # a huge maximum
            q, sc = layer.quantize_hidden(x.cuda())
            torch.cuda.synchronize()
            oq, osc = oracle.quantize_rows(hp.np_u16(x))
            assert np.array_equal(hp.np_u8(q), oq)
            assert np.array_equal(sc.cpu().numpy().view(np.uint32), osc.view(np.uint32))
        finally:
            layer.close()


def test_host_entry_points_of_another_geometry(pkg, oracle):
    hidden, inter, T = 1024, 512, 50
    layer = pkg.MoeLayer(64, 32, 0, hidden=hidden, intermediate=inter)
    try:
        inputs = _inputs(T, 12, hidden)
        weights = _shard(0, 32, hidden, inter)
        dev = _run(layer, inputs, weights, 0, hidden)
        pinned = [x.pin_memory() for x in inputs]
        out = torch.empty(T, hidden, dtype=torch.bfloat16).pin_memory()
        layer.run_host(pinned[0], inputs[1].cuda(), pinned[2], pinned[3], *weights, 0, RSF, out)
        assert torch.equal(out.view(torch.int16), dev.cpu().view(torch.int16))
        out2 = torch.empty(T, hidden, dtype=torch.bfloat16).pin_memory()
        ticket = layer.run_host_async(pinned[0], inputs[1].cuda(), pinned[2], pinned[3], *weights, 0, RSF, out2)
        layer.host_wait(ticket)
        assert torch.equal(out2.view(torch.int16), dev.cpu().view(torch.int16))
    finally:
        layer.close()


def test_paths_that_exist_for_the_reference_geometry_only_are_refused(pkg):
    hidden, inter, T = 1024, 512, 16
    layer = pkg.MoeLayer(64, 32, 0, hidden=hidden, intermediate=inter)
    try:
        inputs = [x.cuda() for x in _inputs(T, 3, hidden)]
        weights = _shard(0, 32, hidden, inter)
        owned = torch.empty(T, hidden, dtype=torch.bfloat16, device="cuda")
        buf = torch.zeros(1 << 22, dtype=torch.uint8, device="cuda")
        with pytest.raises(pkg.MoeError) as ei:
            layer.run_reduce_scatter(*inputs, *weights, 0, RSF, owned, [buf.data_ptr()], buf.numel(), 0, 1, 1)
        assert ei.value.code == pkg._lib.ERR_UNSUPPORTED
        # the layer is still usable afterwards
        out = _run(layer, [x.cpu() for x in inputs], weights, 0, hidden)
        assert torch.isfinite(out.float()).all()
    finally:
        layer.close()


@pytest.mark.parametrize("hidden,inter", [(1024, 512), (2048, 768), (256, 4096)])
def test_tile_ordered_weight_copies_of_another_geometry(pkg, hidden, inter):
    """The weight pre-layout option with other hidden / intermediate sizes: bit-identical results."""
    T, offset = 150, 64
    layer = pkg.MoeLayer(256, 32, 0, hidden=hidden, intermediate=inter)
    try:
        inputs = _inputs(T, 1300, hidden)
        weights = _shard(offset, 32, hidden, inter)
        plain = _run(layer, inputs, weights, offset, hidden)
        layer.set_weight_prelayout(True)
        tiled = _run(layer, inputs, weights, offset, hidden)
        assert plain.float().abs().sum() > 0
        assert torch.equal(plain.view(torch.int16), tiled.view(torch.int16))
    finally:
        layer.close()
