"""CPU checks of the oracle itself: number formats against torch, routing and dispatch
invariants, and the two oracle modes against each other on a tiny case."""
import numpy as np
import pytest
import torch

from helpers import RSF, cpu_inputs, np_u16, np_u8


def test_e4m3_codec_matches_torch(oracle):
    rng = np.random.default_rng(0)
    x = np.concatenate([
        rng.standard_normal(200000).astype(np.float32) * 100,
        rng.standard_normal(200000).astype(np.float32) * 0.01,
        np.array([0.0, -0.0, 448.0, -448.0, 447.9, 2 ** -9, 2 ** -10, 1.5 * 2 ** -9, 0.0146484375], np.float32),
    ])
    x = np.clip(x, -448, 448)
    got = oracle.e4m3_encode(x)
    want = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(got, want)
    dec = oracle.e4m3_decode(np.arange(256, dtype=np.uint8))
    tdec = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    ok = ~np.isnan(tdec)
    assert np.array_equal(dec[ok], tdec[ok])
    # saturation (torch gives NaN above the range, the GPU conversion and the oracle saturate)
    assert oracle.e4m3_encode(np.array([1e6, -1e6, 465.0], np.float32)).tolist() == [0x7E, 0xFE, 0x7E]


def test_bf16_codec_matches_torch(oracle):
    x = np.random.default_rng(1).standard_normal(100000).astype(np.float32) * 37
    got = oracle.bf16_encode(x)
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.uint16).numpy()
    assert np.array_equal(got, want)
    assert np.array_equal(oracle.bf16_decode(got), torch.from_numpy(x).to(torch.bfloat16).float().numpy())


def test_routing_invariants_and_torch_cross_check(oracle):
    T = 512
    logits, bias, _, _ = cpu_inputs(T, seed=3)
    idx, w = oracle.route(logits.numpy(), np_u16(bias))
    assert idx.shape == (T, 8) and w.shape == (T, 8)
    assert np.all((idx >= 0) & (idx < 256))
    for t in range(T):
        assert len(set(idx[t].tolist())) == 8
        assert len(set((idx[t] // 32).tolist())) <= 4
    assert np.allclose(w.sum(1), 1.0, atol=1e-6)
    # independent statement of the same definition in torch (grouped top-k on sigmoid + bias)
    s = torch.sigmoid(logits)
    sb = s + bias.float()
    gs = sb.view(T, 8, 32).topk(2, dim=-1).values.sum(-1)
    keep = torch.zeros(T, 8, dtype=torch.bool)
    keep.scatter_(1, gs.topk(4, dim=-1).indices, True)
    masked = sb.masked_fill(~keep.repeat_interleave(32, dim=1), -1e30)
    tidx = masked.topk(8, dim=-1).indices
    margin = oracle.route_margin(logits.numpy(), np_u16(bias))
    safe = margin > 1e-5
    assert safe.mean() > 0.95
    a = np.sort(idx[safe], axis=1)
    b = np.sort(tidx.numpy()[safe], axis=1)
    assert np.array_equal(a, b)
    tw = torch.gather(s, 1, torch.from_numpy(idx).long())
    tw = tw / tw.sum(1, keepdim=True)
    assert np.allclose(w, tw.numpy(), rtol=2e-6, atol=1e-8)
    # selection order = descending biased score
    sel = torch.gather(sb, 1, torch.from_numpy(idx).long()).numpy()
    assert np.all(np.diff(sel, axis=1) <= 1e-7)


def test_routing_tie_order_follows_the_reference_butterfly(oracle):
    """Equal scores at lanes 8 and 16 of one warp resolve to lane 16 (bit-reversed lane order,
    kernel/moe_fp8.cu:416-420); equal scores in two warps resolve to the lower warp (:427-431)."""
    logits = np.full((2, 256), -20.0, np.float32)
    bias = np.zeros(256, np.uint16)
    logits[0, 8] = logits[0, 16] = 3.0      # same warp 0
    logits[0, 40] = 2.0                     # so that the group has two positive scores
    logits[1, 5] = logits[1, 37] = 3.0      # warps 0 and 1, same lane
    idx, _ = oracle.route(logits, bias)
    assert idx[0, 0] == 16 and idx[0, 1] == 8
    assert idx[1, 0] == 5 and idx[1, 1] == 37


def test_dispatch_exact_and_pruned(oracle):
    T = 2048
    logits, bias, _, _ = cpu_inputs(T, seed=5)
    idx, w = oracle.route(logits.numpy(), np_u16(bias))
    exact = oracle.policy(T, reference_pruning=False)
    pruned = oracle.policy(T, reference_pruning=True)
    assert not exact.prune and pruned.prune
    for off in (0, 96, 224):
        pc, ple, pw, ec = oracle.dispatch(idx, w, off, 32, exact, RSF)
        local = (idx >= off) & (idx < off + 32)
        assert np.array_equal(pc, local.sum(1))
        assert ec.sum() == local.sum()
        pc2, ple2, pw2, ec2 = oracle.dispatch(idx, w, off, 32, pruned, RSF)
        assert np.all(pc2 <= 3) and np.all(pc2 <= pc) and np.all((pc2 > 0) == (pc > 0))
        for t in np.nonzero(pc > pc2)[0][:50]:
            # renormalised: kept weights sum to the local weight mass
            assert pw2[t, :pc2[t]].sum() == pytest.approx(pw[t, :pc[t]].sum(), rel=1e-5)
            assert np.all(np.diff(pw2[t, :pc2[t]]) <= 0)
        same = pc == pc2
        for t in np.nonzero(same)[0][:50]:
            assert sorted(ple[t, :pc[t]].tolist()) == sorted(ple2[t, :pc2[t]].tolist())
    # 256 local experts = 8 shards: the union of the 8 shard dispatches
    pc_all, ple_all, pw_all, ec_all = oracle.dispatch(idx, w, 0, 256, pruned, RSF)
    tot = np.zeros(256, np.int64)
    for s in range(8):
        _, _, _, ec = oracle.dispatch(idx, w, 32 * s, 32, pruned, RSF)
        tot[32 * s:32 * s + 32] = ec
    assert np.array_equal(tot, ec_all)


def test_faithful_and_fp32_modes_agree_on_a_tiny_case(oracle, pkg):
    from fp8_moe_dev_b200 import gen
    T = 2
    logits, bias, hidden, hscale = cpu_inputs(T, seed=0)
    idx, _ = oracle.route(logits.numpy(), np_u16(bias))
    e = int(idx[0, 0])
    w1, s1, w2, s2 = gen.make_shard(e // 32 * 32, 32) if False else (None,) * 4
    # one expert is enough: build a 32-expert shard whose other experts are never selected
    q1, a1, q2, a2 = gen.make_expert(e)
    tokens = np.array([0, 1], np.int32)
    y_f, d, a2c, sf = oracle.expert_rows(np_u8(hidden), hscale.numpy(), tokens, np_u8(q1), a1.numpy(), np_u8(q2),
                                         a2.numpy(), faithful=True, want_all=True)
    y_d = oracle.expert_rows(np_u8(hidden), hscale.numpy(), tokens, np_u8(q1), a1.numpy(), np_u8(q2), a2.numpy(),
                             faithful=False)
    rel = np.linalg.norm(y_f - y_d) / np.linalg.norm(y_d)
    assert rel < 0.08, rel
    assert np.isfinite(y_f).all() and sf.min() > 0
    # independent numpy statement of GEMM1 for a few columns
    hq = oracle.e4m3_decode(np_u8(hidden)).reshape(T, 56, 128)
    wq = oracle.e4m3_decode(np_u8(q1)[:256]).reshape(256, 56, 128)
    raw = np.einsum("tkb,nkb->tnk", hq.astype(np.float64), wq.astype(np.float64))
    sc = hscale.numpy().T[:, None, :] * a1.numpy()[:2].repeat(128, 0)[None, :, :]
    ref = (raw * sc).sum(-1)
    assert np.allclose(d[:, :256], ref, rtol=1e-2, atol=1e-2)
    del w1, s1, w2, s2


def test_quantize_rows_matches_the_torch_definition(oracle, pkg):
    """Quantise-on-entry: the C restatement against torch's fp32 statement of the same scheme
    (1x128 blocks, scale = amax / 448 or 1, payload e4m3(x / scale)), bit for bit."""
    from fp8_moe_dev_b200 import gen
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(19, 7168, generator=g) * (0.01 + 5 * torch.rand(19, 1, generator=g))).to(torch.bfloat16)
    x[4, 256:384] = 0
    x[6] = 0
    x[7, 0] = -2.5e38
    q, s = gen.quantize_rows_1x128(x)
    oq, os_ = oracle.quantize_rows(np_u16(x))
    assert np.array_equal(np_u8(q), oq)
    assert np.array_equal(s.numpy().view(np.uint32), os_.view(np.uint32))
    assert os_.shape == (56, 19) and float(os_[2, 4]) == 1.0 and int(oq[4, 256:384].max()) == 0
