"""The operators either side of the layer (B200): quantise-on-entry against the CPU oracle and
the torch definition, and the layer without its final combine against the complete layer."""
import numpy as np
import pytest
import torch

import helpers as hp
from helpers import H, RSF

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def layer32(pkg):
    lay = pkg.MoeLayer(1024, 32, 0)
    lay.set_decode_kernel(False)   # these tests look at the staged chain's intermediates; the decode kernel has its own file
    yield lay
    lay.close()


def _activations(T, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g) * (0.05 + 4.0 * torch.rand(T, 1, generator=g))
    x = x.to(torch.bfloat16)
    if T > 3:
        x[3, 128:256] = 0          # an all-zero block: scale 1, payload 0
        x[2, 5] = 3.0e38           # a huge value: its block saturates at +-448 and flushes the rest
        x[1] = 0
    return x


@pytest.mark.parametrize("T", [1, 7, 8, 9, 129, 1000])
def test_quantize_hidden_bit_exact_vs_oracle(pkg, oracle, layer32, T):
    x = _activations(T, 900 + T)
    q, s = layer32.quantize_hidden(x.cuda())
    torch.cuda.synchronize()
    want_q, want_s = oracle.quantize_rows(hp.np_u16(x))
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), want_q)
    assert np.array_equal(s.cpu().numpy().view(np.uint32), want_s.view(np.uint32))
    # and the torch statement of the same definition
    from fp8_moe_dev_b200 import gen
    tq, ts = gen.quantize_rows_1x128(x)
    assert torch.equal(q.cpu().view(torch.uint8), tq.view(torch.uint8))
    assert torch.equal(s.cpu(), ts)


def test_quantize_hidden_roundtrip_error_bound(pkg, layer32):
    """Size-independent property at a full-size batch: |x - q * scale| <= scale * 2^-4 * 448 / 16
    (half an e4m3 step at the top binade) for every element."""
    T = 12288
    g = torch.Generator(device="cuda").manual_seed(7)
    x = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16)
    q, s = layer32.quantize_hidden(x)
    deq = q.float().view(T, H // 128, 128) * s.t().contiguous().unsqueeze(-1)
    err = (deq - x.float().view(T, H // 128, 128)).abs()
    bound = s.t().contiguous().unsqueeze(-1) * (16.0 * (1 + 1e-4))   # half of the largest e4m3 step (32), plus fp32 slack
    assert bool((err <= bound).all())
    amax = x.float().view(T, H // 128, 128).abs().amax(-1)
    assert torch.equal(s.t().contiguous(), amax / 448.0) or torch.allclose(s.t(), amax / 448.0, rtol=2e-7, atol=0)


def test_quantize_feeds_the_layer(pkg, layer32):
    """quantize_hidden output is accepted as the layer's input pair and gives the same result as
    the host-quantised pair."""
    T = 40
    logits, bias, hidden, hscale = hp.cpu_inputs(T, seed=910)
    x = (hidden.float().view(T, H // 128, 128) * hscale.t().contiguous().unsqueeze(-1)).view(T, H).to(torch.bfloat16)
    from fp8_moe_dev_b200 import gen
    hq, hs = gen.quantize_rows_1x128(x)
    weights = hp.gpu_shard(0, 32)
    want = hp.run_layer(layer32, (logits, bias, hq, hs), weights, 0).cpu()
    q, s = layer32.quantize_hidden(x.cuda())
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    layer32.run(logits.cuda(), bias.cuda(), q, s, *weights, 0, RSF, out)
    layer32.check()
    assert torch.equal(out.cpu(), want)


@pytest.mark.parametrize("T,offset", [(1, 0), (16, 0), (129, 32), (1024, 0)])
def test_unfinalized_plus_finalize_equals_run(pkg, layer32, T, offset):
    inputs = hp.cpu_inputs(T, seed=920 + T)
    weights = hp.gpu_shard(offset, 32)
    want = hp.run_layer(layer32, inputs, weights, offset).cpu()
    dev = [t.cuda() for t in inputs]
    v = layer32.run_unfinalized(*dev, *weights, offset, RSF)
    layer32.check()
    # the combine restated in torch from the returned views (fp32, pair order)
    cnt = v["pair_count"].long()
    code = v["pair_code"].long() & 0xFFFFFFFF
    rows = v["expert_offset"].long()[code >> 24] + (code & 0xFFFFFF)
    acc = torch.zeros(T, H, dtype=torch.float32, device="cuda")
    mag = torch.zeros(T, H, dtype=torch.float32, device="cuda")
    for p in range(8):
        live = (cnt > p)
        r = torch.where(live, rows[:, p], torch.zeros_like(rows[:, p]))
        contrib = v["y"][r].float() * v["pair_weight"][:, p:p + 1]
        acc = torch.where(live.unsqueeze(-1), acc + contrib, acc)
        mag = torch.where(live.unsqueeze(-1), mag + contrib.abs(), mag)
    manual = acc.to(torch.bfloat16).cpu()
    # torch rounds the product before the add where the kernel uses a fused multiply-add: the two
    # can differ by fp32 rounding of the terms (which cancellation magnifies relative to the sum)
    # and then in the last bf16 bit
    diff = (manual.float() - want.float()).abs()
    assert bool((diff <= 2 ** -7 * want.float().abs() + 2 ** -20 * mag.cpu() + 1e-30).all())
    assert float((manual != want).float().mean()) < 0.02
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    layer32.finalize(T, out)
    layer32.check()
    assert torch.equal(out.cpu(), want)


def test_quantize_hidden_every_bf16_maximum(pkg, oracle, layer32):
    """Every positive finite bf16 value (subnormals included) as a block maximum: the scale
    amax / 448 and the payloads must match the oracle's divisions bit for bit."""
    codes = np.arange(1, 0x7F80, dtype=np.uint16)
    T = (codes.size + 55) // 56
    x16 = np.zeros((T, 56, 128), np.uint16)
    flat = x16.reshape(T * 56, 128)
    flat[:codes.size, 0] = codes
    # companions below the maximum: the same value with a smaller exponent / other significand, negated
    comp = torch.from_numpy(codes.view(np.int16).copy()).view(torch.bfloat16).float()
    for j, f in enumerate((0.5, -0.7109375, 0.33203125, -0.0625, 0.9921875, -0.001953125), start=1):
        flat[:codes.size, j * 7] = hp.np_u16((comp * f).to(torch.bfloat16))
    x = torch.from_numpy(x16.reshape(T, 7168).view(np.int16).copy()).view(torch.bfloat16)
    q, s = layer32.quantize_hidden(x.cuda())
    torch.cuda.synchronize()
    want_q, want_s = oracle.quantize_rows(hp.np_u16(x))
    assert np.array_equal(s.cpu().numpy().view(np.uint32), want_s.view(np.uint32))
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), want_q)
