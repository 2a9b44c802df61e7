"""Expert-parallel form of the layer on one NVSwitch box: the 256 experts are split evenly
over the G ranks of a torch.distributed group (rank r holds experts [r*256/G, (r+1)*256/G),
i.e. local_expert_offset = 256/G * r), every rank routes all T tokens and computes its own
experts, and the bf16 partial outputs are summed over NVLink.  The reference has no
multi-GPU code; its `local_expert_offset` argument (kernel/moe_fp8.cu:2668, 462-463) is the
hook this builds on.

The reduction is the path's one exchange step.  `partial -> all_reduce` (every rank ends
with the full [T,7168] output), `partial -> reduce_scatter` (rank r ends with tokens
[r*T/G, (r+1)*T/G)), both through NCCL, or `fused`: the combine kernel itself stores each
token's row into the owning rank's receive buffer over NVLink (plain peer stores into
symmetric memory) and the owner adds what arrived, so no partial [T,7168] tensor and no
separate collective exist.  The host-side planning (who owns which experts / tokens) is plain
Python so that it can be tested with gloo ranks on CPU.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

NE = 256


def expert_range(rank: int, world: int) -> Tuple[int, int]:
    """(local_expert_offset, num_local_experts) of `rank` among `world` ranks."""
    if world not in (1, 2, 4, 8):
        raise ValueError("world size must be 1, 2, 4 or 8 (256 experts, 32 per routing group)")
    if not 0 <= rank < world:
        raise ValueError("rank outside the group")
    per = NE // world
    return rank * per, per


def expert_ids(rank: int, world: int, placement: str = "contiguous"):
    """Global ids of the experts `rank` holds, in local order.  "contiguous": the reference's blocks
    (local_expert_offset = 256/world * rank); "strided": every world-th expert starting at `rank`, so
    that each rank carries an equal share of every routing group."""
    off, n = expert_range(rank, world)
    if placement == "contiguous":
        return list(range(off, off + n))
    if placement == "strided":
        return list(range(rank, NE, world))
    raise ValueError(f"unknown placement {placement!r}")


def balanced_expert_ids(loads, world: int):
    """Places the 256 experts on `world` ranks, 256/world each, so that the ranks' total loads are
    as equal as a greedy longest-first assignment makes them: experts in decreasing load, each to the
    least loaded rank that still has a free slot.  `loads`: 256 per-expert row counts of a
    calibration batch.  Returns one sorted id list per rank (the same on every rank: ties by id)."""
    loads = [float(x) for x in loads]
    if len(loads) != NE:
        raise ValueError("loads must have 256 entries")
    expert_range(0, world)   # validates world
    cap = NE // world
    order = sorted(range(NE), key=lambda e: (-loads[e], e))
    total = [0.0] * world
    ids = [[] for _ in range(world)]
    for e in order:
        r = min((r for r in range(world) if len(ids[r]) < cap), key=lambda r: (total[r], r))
        ids[r].append(e)
        total[r] += loads[e]
    return [sorted(x) for x in ids]


def token_range(rank: int, world: int, T: int) -> Tuple[int, int]:
    """Token slice [lo, hi) that `rank` owns after a reduce-scatter (T padded up to a multiple of world)."""
    per = (T + world - 1) // world
    lo = min(rank * per, T)
    return lo, min(lo + per, T)


def combine_partials(partial: torch.Tensor, mode: str = "all_reduce", group=None,
                     scatter_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sum the ranks' partial outputs.  Works on any backend (NCCL on GPUs, gloo on CPU)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return partial
    if mode == "all_reduce":
        dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
        return partial
    if mode == "reduce_scatter":
        T = partial.shape[0]
        per = (T + world - 1) // world
        if per * world != T:
            padded = partial.new_zeros((per * world,) + tuple(partial.shape[1:]))
            padded[:T].copy_(partial)
            partial = padded
        if scatter_out is None:
            scatter_out = partial.new_empty((per,) + tuple(partial.shape[1:]))
        dist.reduce_scatter_tensor(scatter_out, partial, op=dist.ReduceOp.SUM, group=group)
        return scatter_out
    raise ValueError(f"unknown mode {mode!r}")


def gather_token_slices(logits: torch.Tensor, hidden_u8: torch.Tensor, scale_parts: torch.Tensor,
                        scale_out: torch.Tensor, rank: int, world: int, group=None) -> None:
    """Completes the replicated inputs from per-rank token slices, in place.  On entry rank r has
    filled rows [r*per, (r+1)*per) of `logits` [T,256] and `hidden_u8` [T,7168] and its own
    `scale_parts[r]` ([56, per]: its columns of the [56,T] scale matrix); on return every rank
    holds all rows, and `scale_out` [56,T] holds the scales in the layer's layout.  Any backend."""
    T = logits.shape[0]
    per = T // world
    lo = rank * per
    if world > 1:
        # flat views: every rank's piece is one contiguous run at offset rank * count (in-place gather)
        for t, mine in ((logits, logits[lo:lo + per]), (hidden_u8, hidden_u8[lo:lo + per]), (scale_parts, scale_parts[rank])):
            dist.all_gather_into_tensor(t.view(-1), mine.reshape(-1), group=group)
    scale_out.view(scale_out.shape[0], world, per).copy_(scale_parts.permute(1, 0, 2))


class ShardedMoe:
    """One rank's share of the 256-expert layer plus the cross-rank sum."""

    def __init__(self, max_tokens: int, rank: Optional[int] = None, world: Optional[int] = None,
                 device: Optional[int] = None, group=None, placement: str = "contiguous", loads=None):
        from .op import MoeLayer
        if rank is None:
            rank = dist.get_rank(group) if dist.is_initialized() else 0
        if world is None:
            world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank, self.world, self.group = rank, world, group
        self.local_expert_offset, self.num_local_experts = expert_range(rank, world)
        self.placement = placement
        # the weights passed to run() must be these experts, in this order
        self.expert_ids = (balanced_expert_ids(loads, world)[rank] if placement == "balanced"
                           else expert_ids(rank, world, placement))
        self.layer = MoeLayer(max_tokens, self.num_local_experts, device)
        if placement == "strided" and world > 1:
            self.layer.set_expert_stride(world)
            self.local_expert_offset = rank   # the phase
        elif placement == "balanced" and world > 1:
            self.layer.set_expert_map(self.expert_ids)   # placed by measured load (`loads`: 256 row counts)
            self.local_expert_offset = 0
        self.max_tokens = max_tokens
        self._exchange = None   # (symmetric buffer, handle, peer pointers, bytes), made on first fused run
        self._epoch = 0
        self._host_stage = None   # device staging of the host entry points (two sets)
        self._host_seq = 0

    def _ensure_exchange(self):
        """Allocate and exchange the receive buffers (torch symmetric memory: plumbing only;
        every byte that crosses NVLink is moved by this package's own kernels)."""
        if self._exchange is not None:
            return self._exchange
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib
        nbytes = int(_lib.load().moe_fp8_b200_exchange_bytes(self.max_tokens, self.world))
        dev = torch.device("cuda", self.layer.device)
        group = self.group if self.group is not None else dist.group.WORLD
        buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
        hdl = symm_mem.rendezvous(buf, group=group)
        buf.zero_()
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)   # nobody pushes before every buffer has been zeroed
        self._exchange = (buf, hdl, [int(p) for p in hdl.buffer_ptrs], nbytes)
        return self._exchange

    def run_fused(self, routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                  gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, routed_scaling_factor,
                  scatter_out: Optional[torch.Tensor] = None):
        """The layer with combine and reduce-scatter in one step; returns this rank's
        [ceil(T / world), 7168] slice of the summed output."""
        T = int(routing_logits.shape[0])
        per = (T + self.world - 1) // self.world
        if scatter_out is None:
            scatter_out = torch.empty((per, 7168), dtype=torch.bfloat16, device=routing_logits.device)
        if T == 0:
            return scatter_out
        _, _, ptrs, nbytes = self._ensure_exchange()
        self._epoch += 1
        return self.layer.run_reduce_scatter(
            routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights, gemm1_weights_scale,
            gemm2_weights, gemm2_weights_scale, self.local_expert_offset, routed_scaling_factor, scatter_out,
            ptrs, nbytes, self.rank, self.world, self._epoch, capacity_tokens=self.max_tokens)

    def _host_stage_set(self, T: int, which: int):
        """Device staging of the host entry points: two sets, so that a call's copies can overlap
        the neighbouring calls' compute."""
        W = self.world
        per = T // W
        dev = torch.device("cuda", self.layer.device)
        if self._host_stage is None or self._host_stage[0]["T"] != T:
            def one():
                return dict(T=T,
                            logits=torch.empty((T, NE), dtype=torch.float32, device=dev),
                            hidden=torch.empty((T, 7168), dtype=torch.float8_e4m3fn, device=dev),
                            scale_parts=torch.empty((W, 56, per), dtype=torch.float32, device=dev),
                            scale=torch.empty((56, T), dtype=torch.float32, device=dev),
                            out=torch.empty((per, 7168), dtype=torch.bfloat16, device=dev),
                            full=torch.empty((T, 7168), dtype=torch.bfloat16, device=dev),
                            ev_in=torch.cuda.Event(), ev_compute=torch.cuda.Event(), ev_out=torch.cuda.Event())
            torch.cuda.synchronize(dev)
            self._host_stage = [one(), one()]
            self._host_seq = 0
            self._s_in = torch.cuda.Stream(dev)
            self._s_out = torch.cuda.Stream(dev)
        return self._host_stage[which]

    def run_host_async(self, routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                       gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, routed_scaling_factor, output,
                       mode: str = "fused") -> int:
        """The per-call tensors live in HOST memory (every rank sees the same pinned `routing_logits`
        [T,256], `hidden_states` [T,7168], `hidden_states_scale` [56,T] and `output` [T,7168]).  A rank
        copies only ITS token slice over PCIe, the slices are all-gathered over NVLink (every rank
        routes all tokens), the layer runs with the reduce-scatter fused in, and the rank writes its
        slice of the summed output back to `output[lo:hi]` (`all_reduce`: all of `output`).  T must be
        a multiple of the group size.  Returns a ticket at once; the host tensors must stay untouched
        until `host_wait(ticket)`, and at most two calls may be in flight.  Copy-in, compute and
        copy-out run on three streams, so consecutive calls overlap them."""
        T = int(routing_logits.shape[0])
        W = self.world
        if T % W:
            raise ValueError(f"T = {T} must be a multiple of the group size {W}")
        per = T // W
        lo = self.rank * per
        dev = torch.device("cuda", self.layer.device)
        self._host_stage_set(T, 0)
        seq = self._host_seq
        self._host_seq += 1
        st = self._host_stage[seq & 1]
        cur = torch.cuda.current_stream(dev)
        with torch.cuda.stream(self._s_in):
            if seq >= 2:
                self._s_in.wait_event(st["ev_compute"])   # the set's inputs were read two calls ago
            # this rank's slice, straight into its place in the gathered tensors: two contiguous runs of
            # rows, and the rank's columns of the [56, T] scale matrix as ONE strided copy (a plain
            # tensor copy of that view would pack it through pageable memory and block the host)
            st["logits"][lo:lo + per].copy_(routing_logits[lo:lo + per], non_blocking=True)
            st["hidden"][lo:lo + per].view(torch.uint8).copy_(hidden_states[lo:lo + per].view(torch.uint8), non_blocking=True)
            part = st["scale_parts"][self.rank]
            rc = self.layer._lib.moe_fp8_b200_copy_rows_h2d(
                part.data_ptr(), per * 4, hidden_states_scale.data_ptr() + lo * 4, T * 4, per * 4, 56,
                self._s_in.cuda_stream)
            if rc != 0:
                raise RuntimeError(f"moe_fp8_b200_copy_rows_h2d failed: {rc}")
            # the all-gather that replicates the inputs runs behind the copies on the copy-in stream, so
            # that it overlaps the previous call's compute instead of standing in front of this call's
            gather_token_slices(st["logits"], st["hidden"].view(torch.uint8), st["scale_parts"], st["scale"],
                                self.rank, W, self.group)
            st["ev_in"].record(self._s_in)
        cur.wait_event(st["ev_in"])
        if seq >= 2:
            cur.wait_event(st["ev_out"])                  # the set's output was copied out two calls ago
        if mode == "fused" and W > 1:
            res = self.run_fused(st["logits"], routing_bias, st["hidden"], st["scale"], gemm1_weights, gemm1_weights_scale,
                                 gemm2_weights, gemm2_weights_scale, routed_scaling_factor, scatter_out=st["out"])
        else:
            res = self.run(st["logits"], routing_bias, st["hidden"], st["scale"], gemm1_weights, gemm1_weights_scale,
                           gemm2_weights, gemm2_weights_scale, routed_scaling_factor, st["full"],
                           mode="reduce_scatter" if mode == "fused" else mode, scatter_out=st["out"])
        st["ev_compute"].record(cur)
        with torch.cuda.stream(self._s_out):
            self._s_out.wait_event(st["ev_compute"])
            if mode == "all_reduce":
                output.copy_(res, non_blocking=True)
            else:
                output[lo:lo + per].copy_(res[:per], non_blocking=True)
            st["ev_out"].record(self._s_out)
        return seq

    def host_wait(self, ticket: int) -> None:
        """Blocks until the output of call `ticket` is in host memory."""
        if self._host_stage is None or not 0 <= ticket < self._host_seq:
            raise ValueError(f"ticket {ticket} was never issued")
        # the set's event is re-recorded by every later call on the set, in the stream of the ticket's own
        # copy-out: its latest record also covers the older ticket
        self._host_stage[ticket & 1]["ev_out"].synchronize()

    def run_host(self, *args, **kwargs):
        """Blocking form of run_host_async."""
        ticket = self.run_host_async(*args, **kwargs)
        self.host_wait(ticket)
        return args[9] if len(args) > 9 else kwargs.get("output")

    def run(self, routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
            gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, routed_scaling_factor, output,
            mode: str = "all_reduce", scatter_out: Optional[torch.Tensor] = None):
        if mode == "fused":
            return self.run_fused(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                                  gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, routed_scaling_factor,
                                  scatter_out)
        self.layer.run(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                       gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, self.local_expert_offset,
                       routed_scaling_factor, output)
        return combine_partials(output, mode, self.group, scatter_out)
