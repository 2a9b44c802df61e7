"""The single-kernel decode path (batches of at most 8 tokens, B200): against the CPU oracle,
against the staged five-kernel chain on the same inputs, against the reference's GPU build, and
its behaviour under CUDA graphs and repeated calls."""
import numpy as np
import pytest
import torch

import helpers as hp
from helpers import H, RSF, TOPK

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def layers(pkg):
    dec = pkg.MoeLayer(64, 32, 0)          # decode kernel on (default)
    chain = pkg.MoeLayer(64, 32, 0)
    chain.set_decode_kernel(False)
    yield dec, chain
    dec.close()
    chain.close()


def _tables(layer, T):
    pc = layer.read("pair_count", T)
    code = layer.read("pair_code", T * TOPK).reshape(T, TOPK)
    pw = layer.read("pair_weight", T * TOPK).reshape(T, TOPK)
    return (layer.read("topk_idx", T * TOPK).copy(), layer.read("topk_weight", T * TOPK).view(np.uint32).copy(), pc.copy(),
            [[(int(code[t, p] >> 24), int(pw[t, p].view(np.uint32))) for p in range(int(pc[t]))] for t in range(T)],
            layer.read("expert_count", layer.num_local_experts).copy())


@pytest.mark.parametrize("T,offset", [(1, 0), (1, 96), (2, 32), (3, 224), (5, 0), (8, 64), (8, 0)])
def test_decode_kernel_vs_oracle_and_chain(pkg, oracle, layers, T, offset):
    dec, chain = layers
    inputs = hp.cpu_inputs(T, seed=1100 + 17 * T + offset)
    weights = hp.gpu_shard(offset, 32)
    got_t = hp.run_layer(dec, inputs, weights, offset)
    tab_dec = _tables(dec, T)
    want_chain = hp.run_layer(chain, inputs, weights, offset)
    tab_chain = _tables(chain, T)
    # routing and dispatch tables: identical (slots inside an expert are an order, compared as sets)
    assert np.array_equal(tab_dec[0], tab_chain[0]) and np.array_equal(tab_dec[1], tab_chain[1])
    assert np.array_equal(tab_dec[2], tab_chain[2]) and tab_dec[3] == tab_chain[3]
    assert np.array_equal(tab_dec[4], tab_chain[4])
    got = got_t.float().cpu().numpy()
    assert np.isfinite(got).all()
    w1, s1, w2, s2 = weights
    ref, rows = oracle.layer(inputs[0].numpy(), hp.np_u16(inputs[1]), hp.np_u8(inputs[2]), inputs[3].numpy(),
                             hp.np_u8(w1), s1.cpu().numpy(), hp.np_u8(w2), s2.cpu().numpy(), offset, RSF)
    assert int(tab_dec[2].sum()) == rows
    assert np.all(got[tab_dec[2] == 0] == 0)
    if rows:
        st = hp.error_stats(got, oracle.bf16_decode(ref))
        assert st["rel_l2"] < 2e-2 and st["contest_ratio"] >= 0.999, st
        # against the chain: the same arithmetic except the fp32 summation order inside GEMM1
        sc = hp.error_stats(got, want_chain.float().cpu().numpy())
        print(f"T={T} offset={offset} rows={rows} decode vs chain: {sc}")
        assert sc["rel_l2"] < 5e-3, sc


@pytest.mark.parametrize("T,offset", [(1, 96), (4, 0), (8, 32)])
def test_decode_kernel_vs_reference_gpu_build(pkg, layers, T, offset):
    if not hp.reference_available():
        pytest.skip("oracle/_ref/libref_moe.so not built")
    dec, _ = layers
    inputs = hp.cpu_inputs(T, seed=1200 + T)
    weights = hp.gpu_shard(offset, 32)
    out = hp.run_layer(dec, inputs, weights, offset).float().cpu().numpy()
    ref = hp.reference_run(inputs, weights, offset).float().cpu().numpy()
    st = hp.error_stats(out, ref)
    print(f"T={T} offset={offset} decode kernel vs reference: {st}")
    assert st["contest_ratio"] >= 0.99, st
    if np.abs(ref).max() > 0:
        assert st["rel_l2"] < 3e-2, st


def test_decode_kernel_all_256_experts(pkg, oracle):
    """Eight tokens over all 256 experts of one GPU: 64 active experts, every row distinct."""
    T = 8
    lay = pkg.MoeLayer(T, 256, 0)
    chain = pkg.MoeLayer(T, 256, 0)
    chain.set_decode_kernel(False)
    try:
        inputs = hp.cpu_inputs(T, seed=1300)
        weights = hp.gpu_shard(0, 256)
        got = hp.run_layer(lay, inputs, weights, 0)
        want = hp.run_layer(chain, inputs, weights, 0)
        assert int(lay.read("pair_count", T).sum()) == T * TOPK
        st = hp.error_stats(got.float().cpu().numpy(), want.float().cpu().numpy())
        assert st["rel_l2"] < 5e-3, st
    finally:
        lay.close()
        chain.close()


def test_decode_kernel_is_deterministic_and_graph_capturable(pkg, layers):
    dec, _ = layers
    T = 4
    inputs = [x.cuda() for x in hp.cpu_inputs(T, seed=1400)]
    other = [x.cuda() for x in hp.cpu_inputs(T, seed=1401)]
    w1, s1, w2, s2 = hp.gpu_shard(0, 32)
    out = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")
    dec.run(*inputs, w1, s1, w2, s2, 0, RSF, out)
    dec.check()
    eager = out.clone()
    for _ in range(5):
        out.zero_()
        dec.run(*inputs, w1, s1, w2, s2, 0, RSF, out)
        dec.check()
        assert torch.equal(out, eager)
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            dec.run(*inputs, w1, s1, w2, s2, 0, RSF, out)
    torch.cuda.current_stream().wait_stream(s)
    out.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    for dst, src in zip(inputs, other):
        dst.copy_(src)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    want = torch.empty_like(out)
    dec.run(*other, w1, s1, w2, s2, 0, RSF, want)
    dec.check()
    assert torch.equal(out, want)


def test_decode_kernel_exact_silu_and_chain_agree(pkg, layers):
    dec, chain = layers
    T = 6
    inputs = hp.cpu_inputs(T, seed=1500)
    weights = hp.gpu_shard(32, 32)
    dec.set_exact_silu(True)
    chain.set_exact_silu(True)
    try:
        a = hp.run_layer(dec, inputs, weights, 32).float().cpu().numpy()
        b = hp.run_layer(chain, inputs, weights, 32).float().cpu().numpy()
    finally:
        dec.set_exact_silu(False)
        chain.set_exact_silu(False)
    c = hp.run_layer(dec, inputs, weights, 32).float().cpu().numpy()
    assert hp.error_stats(a, b)["rel_l2"] < 5e-3
    assert not np.array_equal(a, c)   # the option does reach the kernel


def test_decode_routing_equals_chain_routing_on_many_batches_and_ties(pkg, layers):
    """The decode kernel selects experts by counting instead of argmax rounds: its picks, their
    order and weights must equal the staged routing kernel's bit for bit, also when scores tie
    (coarsely quantised logits, zero bias: dozens of equal scores per token)."""
    dec, chain = layers
    T = 8
    weights = hp.gpu_shard(0, 32)
    g = torch.Generator().manual_seed(77)
    zero_bias = torch.zeros(256, dtype=torch.bfloat16)
    for trial in range(24):
        logits, bias, hidden, hscale = hp.cpu_inputs(T, seed=2000 + trial)
        if trial % 2:
            logits = (torch.randn(T, 256, generator=g) * 1.5).round() / 2      # heavy ties
            bias = zero_bias
        if trial % 6 == 5:
            logits = torch.zeros(T, 256)                                        # everything ties
        inputs = (logits.contiguous(), bias, hidden, hscale)
        hp.run_layer(dec, inputs, weights, 0)
        td = _tables(dec, T)
        hp.run_layer(chain, inputs, weights, 0)
        tc = _tables(chain, T)
        assert np.array_equal(td[0], tc[0]), f"trial {trial}: expert picks differ"
        assert np.array_equal(td[1], tc[1]), f"trial {trial}: weights differ"
        assert np.array_equal(td[2], tc[2]) and td[3] == tc[3] and np.array_equal(td[4], tc[4])
