"""Generates the golden fixtures of tests/golden/ by running the REFERENCE itself on a B200.

    python tests/golden/make_golden.py [OUT_DIR]        (default gpurun_out/golden)

For each case the seeded CPU generator (fp8-moe-dev_b200/gen.py, numpy PCG64 streams, identical on
every machine) produces the inputs; the unmodified reference library
(oracle/_ref/libref_moe.so, built by oracle/build_ref.sh from the reference's sources) then
gives
  * its routing kernel's top-8 indices and weights           (kernel/moe_fp8.cu:329-456)
  * its dispatch tables for every 32-expert shard offset      (kernel/moe_fp8.cu:457-669)
  * the bf16 output of its `run` for the case's shard         (kernel/moe_fp8.cu:2663-3672)
Only seeds, those results and input checksums are stored (a few hundred KB); the inputs are
regenerated from the seeds by the tests.  Copy the written .npz files into tests/golden/.
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


def main():
    out_dir = Path(sys.argv[1]) if len(sys.argv) > 1 else ROOT / "gpurun_out" / "golden"
    out_dir.mkdir(parents=True, exist_ok=True)
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
