"""The multi-GPU plan on CPU: expert / token ownership and the cross-rank sum over a
world of two gloo ranks (the same code path runs over NCCL on the GPUs)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_expert_and_token_ranges(pkg):
    from fp8_moe_dev_b200.dist import expert_range, token_range
    for world in (1, 2, 4, 8):
        seen = []
        for r in range(world):
            off, n = expert_range(r, world)
            assert n == 256 // world and off == r * n and off % 32 == 0
            seen += list(range(off, off + n))
        assert seen == list(range(256))
        for T in (1, 7, 16, 1000, 12288):
            cover = []
            for r in range(world):
                lo, hi = token_range(r, world, T)
                cover += list(range(lo, hi))
            assert cover == list(range(T))
    with pytest.raises(ValueError):
        expert_range(0, 3)
    with pytest.raises(ValueError):
        expert_range(2, 2)


def _worker(rank, world, port, T, q):
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    sys.path.insert(0, str(root))
    import __graft_entry__ as entry
    entry.load_package()
    from fp8_moe_dev_b200.dist import combine_partials, expert_range, token_range
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(1234)
        # the 8 shard outputs of a pretend layer; rank r owns shards of its expert range
        shards = torch.randn(8, T, 64, generator=g)
        off, n = expert_range(rank, world)
        mine = shards[off // 32:(off + n) // 32].sum(0)
        full = combine_partials(mine.clone(), "all_reduce")
        ok = torch.allclose(full, shards.sum(0), atol=1e-5)
        part = combine_partials(mine.clone(), "reduce_scatter")
        lo, hi = token_range(rank, world, T)
        ok = ok and torch.allclose(part[:hi - lo], shards.sum(0)[lo:hi], atol=1e-5)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T", [8, 13])
def test_two_rank_combine_over_gloo(T):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, T, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    res = dict(q.get(timeout=10) for _ in range(world))
    assert res == {0: True, 1: True}


def test_shard_sum_identity_on_the_oracle(oracle):
    """Dispatching 64 local experts equals the union of two 32-expert shard dispatches, which
    is what makes `sum over ranks of partial outputs` the full layer."""
    from helpers import RSF, cpu_inputs, np_u16
    T = 256
    logits, bias, _, _ = cpu_inputs(T, seed=9)
    idx, w = oracle.route(logits.numpy(), np_u16(bias))
    pol = oracle.policy(T)
    pc, ple, pw, ec = oracle.dispatch(idx, w, 64, 64, pol, RSF)
    pa = oracle.dispatch(idx, w, 64, 32, pol, RSF)
    pb = oracle.dispatch(idx, w, 96, 32, pol, RSF)
    assert np.array_equal(ec, np.concatenate([pa[3], pb[3]]))
    assert np.array_equal(pc, pa[0] + pb[0])
    for t in range(T):
        want = [(int(pa[1][t, p]), float(pa[2][t, p])) for p in range(pa[0][t])] + \
               [(int(pb[1][t, p]) + 32, float(pb[2][t, p])) for p in range(pb[0][t])]
        got = [(int(ple[t, p]), float(pw[t, p])) for p in range(pc[t])]
        assert got == want


def _gather_worker(rank, world, port, T, q):
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    sys.path.insert(0, str(root))
    import __graft_entry__ as entry
    entry.load_package()
    from fp8_moe_dev_b200.dist import gather_token_slices
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(99)
        logits = torch.randn(T, 256, generator=g)
        hidden = torch.randint(0, 256, (T, 64), generator=g, dtype=torch.uint8)   # narrow stand-in for [T, 7168]
        scale = torch.rand(56, T, generator=g)
        per = T // world
        lo = rank * per
        # what a rank has after copying only its token slice from host memory
        my_logits = torch.full((T, 256), float("nan"))
        my_hidden = torch.zeros(T, 64, dtype=torch.uint8)
        parts = torch.full((world, 56, per), float("nan"))
        my_logits[lo:lo + per] = logits[lo:lo + per]
        my_hidden[lo:lo + per] = hidden[lo:lo + per]
        parts[rank] = scale[:, lo:lo + per]
        out_scale = torch.empty(56, T)
        gather_token_slices(my_logits, my_hidden, parts, out_scale, rank, world)
        ok = torch.equal(my_logits, logits) and torch.equal(my_hidden, hidden) and torch.equal(out_scale, scale)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_token_slices_are_gathered_into_the_replicated_inputs():
    """The multi-GPU host path: each rank brings its token slice, everybody ends with all tokens
    and with the [56, T] scale matrix in the layer's layout (two gloo ranks)."""
    world, T = 2, 24
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gather_worker, args=(r, world, port, T, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    res = dict(q.get(timeout=10) for _ in range(world))
    assert res == {0: True, 1: True}


def test_balanced_expert_placement(pkg):
    """Longest-first placement by load: every rank gets 256/world experts, every expert exactly one
    rank, and the heaviest rank stays close to the mean even for heavy-tailed loads."""
    from fp8_moe_dev_b200.dist import balanced_expert_ids, expert_ids
    g = torch.Generator().manual_seed(5)
    loads = (torch.rand(256, generator=g) ** -0.5 * 100).clamp(max=2500).tolist()   # heavy tail: a few experts 10x the median
    for world in (1, 2, 4, 8):
        ids = balanced_expert_ids(loads, world)
        assert [len(x) for x in ids] == [256 // world] * world
        assert sorted(sum(ids, [])) == list(range(256))
        tot = [sum(loads[e] for e in x) for x in ids]
        assert max(tot) <= 1.08 * sum(tot) / world
        if world == 8:
            contiguous = [sum(loads[e] for e in expert_ids(r, world)) for r in range(world)]
            assert max(tot) < max(contiguous)
    assert balanced_expert_ids(loads, 4) == balanced_expert_ids(list(loads), 4)   # deterministic
    with pytest.raises(ValueError):
        balanced_expert_ids(loads[:100], 4)
