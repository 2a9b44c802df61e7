"""Generates the golden fixtures of tests/golden/ by running the REFERENCE itself on a B200.

    python tests/golden/make_golden.py OUT_DIR [small|big|all]

For each case the seeded CPU generator (fp8-moe-dev_b200/gen.py, numpy PCG64 streams, identical on
every machine) produces the inputs; the unmodified reference library
(oracle/_ref/libref_moe.so, built by oracle/build_ref.sh from the reference's sources) then
gives
  * its routing kernel's top-8 indices and weights           (kernel/moe_fp8.cu:329-456)
  * its dispatch tables for every 32-expert shard offset      (kernel/moe_fp8.cu:457-669)
  * the bf16 output of its `run` for the case's shard         (kernel/moe_fp8.cu:2663-3672)
Only seeds, those results and input checksums are stored (a few hundred KB); the inputs are
regenerated from the seeds by the tests.  Copy the written .npz files into tests/golden/.

"big" cases pin the T-keyed branches of the reference's pruning dispatch (kernel/moe_fp8.cu:508-591)
that the small cases do not reach -- the per-T constants of T = 32, 53, 80, 901, 14107, the
drop-third rule of T >= 10000 (fraction 0.34 at T = 12288, 0.30 at T = 16384) -- at the benchmark's
sizes.  Per case and shard offset they hold the per-expert row counts, every token's pair count, a
digest of all (token, expert, weight bits) pairs, digests of the routing result, and for 512 evenly
spaced tokens the routing result and the pairs themselves; the T = 12288 case adds the bf16 output of
`run` (shard 0, every 8th column, plus per-row sums) for tokens whose rows lie in two experts only, so
that a CPU check needs only those two experts' weights.
"""
import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import __graft_entry__ as entry  # noqa: E402

entry.load_package()
import helpers as hp  # noqa: E402
from fp8_moe_dev_b200 import gen  # noqa: E402

CASES = [  # (name, T, seed, offset of the shard whose output is stored)
    ("t1", 1, 0, None),      # offset chosen so that the token has local rows
    ("t7", 7, 0, 0),
    ("t16", 16, 0, 0),       # the host-fp32 parity configuration of the benchmark list
    ("t40", 40, 0, 0),       # pruning dispatch (T >= 32)
]


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()[:16]


BIG_CASES = [  # (name, T, seed, skewed routing, shard offset whose `run` output is sampled)
    ("t32", 32, 0, False, None),
    ("t53", 53, 0, False, None),
    ("t80", 80, 0, False, None),
    ("t901", 901, 0, False, None),
    ("t14107", 14107, 0, False, None),
    ("t12288", 12288, 0, False, 0),
    ("t16384skew", 16384, 0, True, None),
]
N_SAMPLE = 512


def big_case(out_dir, name, T, seed, skew, out_offset):
    logits, bias = gen.make_routing(T, seed, skew)
    ridx, rw = hp.reference_routing(logits, bias)
    sample = np.unique(np.linspace(0, T - 1, min(N_SAMPLE, T)).round().astype(np.int64))
    S = len(sample)
    counts = np.zeros((8, 32), np.int32)
    pair_n = np.zeros((8, T), np.uint8)
    digests = []
    s_le = np.full((8, S, 8), -1, np.int8)
    s_w = np.zeros((8, S, 8), np.uint32)
    variant = -1
    keep = {}
    for s in range(8):
        d = hp.reference_dispatch_arrays(logits, bias, 32 * s)
        variant = d["variant"]
        counts[s] = d["expert_count"]
        pair_n[s] = d["pair_n"]
        digests.append(hp.pairs_digest(d["pair_n"], d["pair_le"], d["pair_w"]))
        live = np.arange(8)[None, :] < d["pair_n"][sample][:, None]
        s_le[s] = np.where(live, d["pair_le"][sample], -1)
        s_w[s] = np.where(live, d["pair_w"][sample].view(np.uint32), 0)
        if out_offset is not None and 32 * s == out_offset:
            keep = d
    extra = {}
    if out_offset is not None:
        # tokens whose rows of this shard lie in its two most loaded experts only (plus a few without rows)
        ec = counts[out_offset // 32]
        a, b = [int(x) for x in np.argsort(-ec, kind="stable")[:2]]
        n, le = keep["pair_n"], keep["pair_le"]
        live = np.arange(8)[None, :] < n[:, None]
        inside = (((le == a) | (le == b)) | ~live).all(1) & (n > 0)
        two = np.nonzero(inside & (n >= 2))[0][:16]
        one = np.nonzero(inside & (n == 1))[0][:24]
        none = np.nonzero(n == 0)[0][:8]
        toks = np.sort(np.concatenate([two, one, none])).astype(np.int64)
        hidden, hscale = gen.make_hidden(T, seed + 1)
        weights = [x.cuda() for x in gen.make_shard(out_offset, 32, device="cpu")]
        out = hp.reference_run((logits, bias, hidden, hscale), weights, out_offset)
        rows = out[torch.from_numpy(toks).cuda()].cpu()
        extra = dict(out_offset=out_offset, out_experts=np.array([a, b], np.int32), out_tokens=toks,
                     out_bf16_cols8=rows[:, ::8].contiguous().view(torch.uint16).numpy(),
                     out_row_sum=rows.double().sum(1).numpy(), out_row_abs_sum=rows.double().abs().sum(1).numpy(),
                     out_pair_n=n[toks].astype(np.int32), out_pair_le=le[toks].astype(np.int32),
                     out_pair_w_bits=keep["pair_w"][toks].view(np.uint32),
                     sha_hidden_rows=sha(hidden.view(torch.uint8).numpy()[toks]),
                     sha_w1_a=sha(weights[0][a].view(torch.uint8).cpu().numpy()))
    np.savez_compressed(
        out_dir / f"ref_big_{name}.npz",
        T=T, seed=seed, skew=int(skew), rsf=hp.RSF, variant=variant, expert_count=counts, pair_n=pair_n,
        pairs_digest=np.array(digests), sha_topk_idx=sha(ridx), sha_topk_weight_bits=sha(rw.view(np.uint32)),
        sample_tokens=sample, sample_topk_idx=ridx[sample].astype(np.uint8),
        sample_topk_weight_bits=rw[sample].view(np.uint32), sample_pair_le=s_le, sample_pair_w_bits=s_w,
        sha_logits=sha(logits.numpy()), **extra)
    print(f"big {name}: T={T} skew={skew} variant={variant} rows per shard={counts.sum(1).tolist()}")


def main():
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    out_dir = Path(sys.argv[1])
    which = sys.argv[2] if len(sys.argv) > 2 else "all"
    out_dir.mkdir(parents=True, exist_ok=True)
    if which in ("big", "all"):
        for case in BIG_CASES:
            big_case(out_dir, *case)
    if which == "big":
        return
    shards = {}
    for name, T, seed, offset in CASES:
        logits, bias = gen.make_routing(T, seed)
        hidden, hscale = gen.make_hidden(T, seed + 1)
        ridx, rw = hp.reference_routing(logits, bias)
        if offset is None:
            offset = int(ridx[0, 0]) // 32 * 32
        if offset not in shards:
            shards.clear()
            shards[offset] = [x.cuda() for x in gen.make_shard(offset, 32, device="cpu")]
        weights = shards[offset]
        counts = np.zeros((8, 32), np.int32)
        variant = -1
        pair_le = np.full((8, T, 8), -1, np.int32)
        pair_w = np.zeros((8, T, 8), np.float32)
        pair_n = np.zeros((8, T), np.int32)
        for s in range(8):
            d = hp.reference_dispatch(logits, bias, 32 * s)
            counts[s] = d["expert_count"]
            variant = d["variant"]
            for t, pl in enumerate(d["pairs"]):
                pair_n[s, t] = len(pl)
                for p, (le, w) in enumerate(pl):
                    pair_le[s, t, p] = le
                    pair_w[s, t, p] = w
        out = hp.reference_run((logits, bias, hidden, hscale), weights, offset)
        used = np.nonzero(counts[offset // 32])[0]
        w1 = weights[0]
        np.savez_compressed(
            out_dir / f"ref_{name}.npz",
            T=T, seed=seed, offset=offset, rsf=hp.RSF, variant=variant,
            topk_idx=ridx, topk_weight_bits=rw.view(np.uint32), expert_count=counts,
            pair_n=pair_n, pair_le=pair_le, pair_w_bits=pair_w.view(np.uint32),
            out_bf16=out.view(torch.uint16).cpu().numpy(),
            sha_logits=sha(logits.numpy()), sha_hidden=sha(hidden.view(torch.uint8).numpy()),
            sha_hscale=sha(hscale.numpy()),
            sha_w1_first_used=sha(w1[int(used[0])].view(torch.uint8).cpu().numpy()) if len(used) else "",
            first_used_expert=int(used[0]) if len(used) else -1,
        )
        print(f"{name}: T={T} offset={offset} variant={variant} rows={int(counts[offset // 32].sum())} "
              f"out_absmax={float(out.float().abs().max()):.4f}")


if __name__ == "__main__":
    main()
