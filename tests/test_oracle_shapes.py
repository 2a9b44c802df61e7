"""The CPU oracle set to other shapes of the layer (oracle.shape) against an independent numpy statement of the
layer's definition: routing with other top_k / n_group / topk_group constants, and the fp32 layer (dequantised
GEMMs, exact SiLU, no pruning) with other hidden / intermediate sizes.  The reference itself exists for one shape
only, so this is what stands behind the oracle where tests/test_gpu_shapes.py uses it as the checker."""
import numpy as np
import pytest
import torch

import __graft_entry__ as entry


def _bf16_to_f32(u16):
    return (u16.astype(np.uint32) << 16).view(np.float32)


def _numpy_route(logits, bias_f32, top_k, n_group, topk_group):
    T = logits.shape[0]
    s = (1.0 / (1.0 + np.exp(-logits.astype(np.float32)))).astype(np.float32)
    sb = s + bias_f32[None, :]
    gsize = 256 // n_group
    g = sb.reshape(T, n_group, gsize)
    top2 = np.sort(g, axis=2)[:, :, -2:].sum(axis=2)
    keep = np.argsort(-top2, axis=1, kind="stable")[:, :topk_group]
    mask = np.zeros((T, n_group), bool)
    np.put_along_axis(mask, keep, True, axis=1)
    masked = np.where(np.repeat(mask, gsize, axis=1), sb, -np.inf)
    idx = np.argsort(-masked, axis=1, kind="stable")[:, :top_k]
    w = np.take_along_axis(s, idx, axis=1)
    w = w / (w.sum(axis=1, keepdims=True) + 1e-20)
    return idx, w.astype(np.float32)


@pytest.mark.parametrize("top_k,n_group,topk_group", [(8, 8, 4), (4, 4, 2), (6, 1, 1), (2, 8, 1), (8, 2, 1), (1, 8, 8)])
def test_oracle_routing_with_other_constants(oracle, top_k, n_group, topk_group):
    entry.load_package()
    from fp8_moe_dev_b200 import gen
    T = 300
    logits, bias = gen.make_routing(T, 70 + top_k)
    lg, bs = logits.numpy(), bias.view(torch.uint16).numpy()
    with oracle.shape(7168, 2048, top_k, n_group, topk_group):
        idx, w = oracle.route(lg, bs)
        margin = oracle.route_margin(lg, bs)
    nidx, nw = _numpy_route(lg, _bf16_to_f32(bs), top_k, n_group, topk_group)
    assert np.all(idx[:, top_k:] == -1) and np.all(w[:, top_k:] == 0)
    safe = margin > 1e-6   # away from ties the two statements must pick the same experts
    assert safe.mean() > 0.95
    assert np.array_equal(np.sort(idx[safe, :top_k], 1), np.sort(nidx[safe], 1))
    order_same = np.all(idx[:, :top_k] == nidx, axis=1)
    assert order_same[safe].mean() > 0.98
    assert np.allclose(w[order_same, :top_k], nw[order_same], rtol=2e-6, atol=1e-9)
    # after the block the oracle is back on the reference's constants
    ridx, _ = oracle.route(lg, bs)
    assert np.all(ridx >= 0)


@pytest.mark.parametrize("hidden,inter,top_k,n_group,topk_group", [(256, 128, 8, 8, 4), (512, 384, 4, 4, 2)])
def test_oracle_fp32_layer_of_another_shape(oracle, hidden, inter, top_k, n_group, topk_group):
    entry.load_package()
    from fp8_moe_dev_b200 import gen
    T, E, offset, rsf = 24, 32, 64, 2.5
    logits, bias = gen.make_routing(T, 5)
    q, sc = gen.make_hidden(T, 6, hidden=hidden)
    w1, s1, w2, s2 = gen.make_shard(offset, E, 900, hidden=hidden, inter=inter)
    lg, bs = logits.numpy(), bias.view(torch.uint16).numpy()
    with oracle.shape(hidden, inter, top_k, n_group, topk_group):
        out, rows = oracle.layer(lg, bs, q.view(torch.uint8).numpy(), sc.numpy(), w1.view(torch.uint8).numpy(), s1.numpy(),
                                 w2.view(torch.uint8).numpy(), s2.numpy(), offset, rsf, mode="fp32")
        idx, w = oracle.route(lg, bs)
    got = oracle.bf16_decode(out)
    # the definition in numpy, from the oracle's own routing result (checked above)
    a = oracle.e4m3_decode(q.view(torch.uint8).numpy()) * np.repeat(sc.numpy().T, 128, axis=1)
    W1 = oracle.e4m3_decode(w1.view(torch.uint8).numpy()) * np.repeat(np.repeat(s1.numpy(), 128, axis=1), 128, axis=2)
    W2 = oracle.e4m3_decode(w2.view(torch.uint8).numpy()) * np.repeat(np.repeat(s2.numpy(), 128, axis=1), 128, axis=2)
    want = np.zeros((T, hidden), np.float64)
    n_rows = 0
    for t in range(T):
        for k in range(top_k):
            le = int(idx[t, k]) - offset
            if 0 <= le < E:
                d = W1[le].astype(np.float64) @ a[t].astype(np.float64)
                x1, x2 = d[:inter], d[inter:]
                v = x2 / (1.0 + np.exp(-x2)) * x1
                want[t] += float(w[t, k]) * rsf * (W2[le].astype(np.float64) @ v)
                n_rows += 1
    assert rows == n_rows
    err = np.abs(got - want)
    assert np.all(err <= 2e-2 * np.abs(want) + 1e-2 * np.abs(want).max()), float(err.max())
    den = np.linalg.norm(want)
    assert den > 0 and np.linalg.norm(got - want) / den < 5e-3
