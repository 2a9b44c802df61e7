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
        self.trace = None         # diagnostics: a list makes run_host_async append its per-phase CUDA events
        self.copy_engine_gather = True   # host entry points: replicate the inputs with peer copies (False: NCCL)
        self._symm_stage = None

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

    def _symmetric_input_staging(self, T: int, dev):
        """Both sets' gathered inputs (logits [T,256], hidden [T,7168], scales [56,T]) in ONE peer-mapped buffer
        behind a 256-byte flag array, so that every rank can store its token slice straight into every peer's
        staging with copy engines.  Returns (views of set 0, views of set 1, byte offsets of the three tensors
        inside a set, set stride, peer base pointers, keep-alive objects)."""
        import torch.distributed._symmetric_memory as symm_mem
        W, per = self.world, T // self.world
        al = lambda n: (n + 255) // 256 * 256
        b_logits, b_hidden, b_parts = T * NE * 4, T * 7168, 56 * T * 4
        offs = (0, al(b_logits), al(b_logits) + al(b_hidden))
        set_bytes = offs[2] + al(b_parts)
        group = self.group if self.group is not None else dist.group.WORLD
        buf = symm_mem.empty(256 + 2 * set_bytes, dtype=torch.uint8, device=dev)
        hdl = symm_mem.rendezvous(buf, group=group)
        buf.zero_()
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)          # nobody signals before every flag array has been zeroed
        sets = []
        for s in range(2):
            base = 256 + s * set_bytes
            sets.append(dict(
                logits=buf[base + offs[0]: base + offs[0] + b_logits].view(torch.float32).view(T, NE),
                hidden=buf[base + offs[1]: base + offs[1] + b_hidden].view(torch.float8_e4m3fn).view(T, 7168),
                scale=buf[base + offs[2]: base + offs[2] + b_parts].view(torch.float32).view(56, T)))
        return sets, offs, set_bytes, [int(p) for p in hdl.buffer_ptrs], (buf, hdl)

    def _host_stage_set(self, T: int, which: int):
        """Device staging of the host entry points: two sets, so that a call's copies can overlap
        the neighbouring calls' compute."""
        W = self.world
        per = T // W
        dev = torch.device("cuda", self.layer.device)
        if self._host_stage is None or self._host_stage[0]["T"] != T:
            torch.cuda.synchronize(dev)
            self._symm_stage = None
            shared = [dict(), dict()]
            if W > 1 and self.copy_engine_gather:
                sets, offs, set_bytes, ptrs, keep = self._symmetric_input_staging(T, dev)
                shared = sets
                self._symm_stage = dict(offs=offs, set_bytes=set_bytes, ptrs=ptrs, keep=keep)

            def one(sh):
                st = dict(T=T, out=torch.empty((per, 7168), dtype=torch.bfloat16, device=dev),
                          full=torch.empty((T, 7168), dtype=torch.bfloat16, device=dev),
                          ev_in=torch.cuda.Event(), ev_compute=torch.cuda.Event(), ev_out=torch.cuda.Event())
                if sh:       # peer-mapped: the slices arrive in place, scales included
                    st.update(sh)
                else:        # NCCL: contiguous per-rank scale pieces are gathered, then re-laid as [56, T]
                    st.update(logits=torch.empty((T, NE), dtype=torch.float32, device=dev),
                              hidden=torch.empty((T, 7168), dtype=torch.float8_e4m3fn, device=dev),
                              scale_parts=torch.empty((W, 56, per), dtype=torch.float32, device=dev),
                              scale=torch.empty((56, T), dtype=torch.float32, device=dev))
                return st
            self._host_stage = [one(shared[0]), one(shared[1])]
            # one "output is in host memory" event per call in flight (three may be: one copying in, one
            # computing, one copying out), so that waiting for a call never waits for a later one
            self._done_events = [torch.cuda.Event() for _ in range(4)]
            self._waited_upto = -1
            # flag values for the peers, one pinned word per call (a 4-byte copy delivers it: no SM needed)
            self._flag_ring = torch.zeros(1024, dtype=torch.int32).pin_memory()
            self._host_seq = 0
            self._s_in = torch.cuda.Stream(dev)
            self._s_out = torch.cuda.Stream(dev)
        return self._host_stage[which]

    def _push_slices_to_peers(self, T: int, seq: int):
        """Copy-engine form of the all-gather that replicates the inputs: this rank's rows of logits and hidden
        and its columns of the scale matrix go from its own staging into the same place of every peer's staging
        (peer copies on the copy-in stream), followed by this call's number into this rank's word of every
        peer's flag array (a 4-byte copy from pinned host memory).  Nothing here needs an SM: the persistent
        GEMM CTAs of the call that is computing meanwhile leave none free, and an NCCL all-gather (or any
        kernel) on this stream would wait for them.  The consumer side is `_wait_for_peer_slices`.  Safe to
        overwrite a peer's set: this rank's compute of two calls ago has finished, and the cross-rank sum inside
        it completed only after every peer had finished the kernels that read that set."""
        sg, lib = self._symm_stage, self.layer._lib
        W, per, s = self.world, T // self.world, seq & 1
        lo = self.rank * per
        base = 256 + s * sg["set_bytes"]
        # (offset of the piece, dst/src pitch, bytes per row, rows)
        pieces = ((sg["offs"][0] + lo * NE * 4, per * NE * 4, per * NE * 4, 1),
                  (sg["offs"][1] + lo * 7168, per * 7168, per * 7168, 1),
                  (sg["offs"][2] + lo * 4, T * 4, per * 4, 56))
        stream = self._s_in.cuda_stream
        mine = sg["ptrs"][self.rank]
        slot = seq % self._flag_ring.numel()
        self._flag_ring[slot] = (seq + 1) & 0x7FFFFFFF
        flag_src = self._flag_ring.data_ptr() + 4 * slot
        for d in range(W):
            p = (self.rank + 1 + d) % W        # every rank starts on another destination; itself last (flag only)
            if p != self.rank:
                for off, pitch, row_bytes, rows in pieces:
                    if lib.moe_fp8_b200_copy_device(sg["ptrs"][p] + base + off, pitch, mine + base + off, pitch,
                                                    row_bytes, rows, stream) != 0:
                        raise RuntimeError("moe_fp8_b200_copy_device failed")
            if lib.moe_fp8_b200_copy_rows_h2d(sg["ptrs"][p] + 4 * self.rank, 4, flag_src, 4, 4, 1, stream) != 0:
                raise RuntimeError("flag copy failed")

    def _wait_for_peer_slices(self, seq: int, stream: int):
        """On the compute stream, in front of the layer: bounded wait until every rank's word of the local
        flag array has reached this call's number (a peer that never delivers shows up in layer.check())."""
        import ctypes as C
        sg, W = self._symm_stage, self.world
        arr = (C.c_void_p * W)(*sg["ptrs"])
        h = self.layer._h
        if self.layer._lib.moe_fp8_b200_wait_peers(h, arr, W, self.rank, 0, (seq + 1) & 0x7FFFFFFF, C.c_void_p(stream)) != 0:
            raise RuntimeError("peer wait launch failed: " + self.layer._lib.moe_fp8_b200_last_error(h).decode())

    def run_host_async(self, routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                       gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, routed_scaling_factor, output,
                       mode: str = "fused") -> int:
        """The per-call tensors live in HOST memory (every rank sees the same pinned `routing_logits`
        [T,256], `hidden_states` [T,7168], `hidden_states_scale` [56,T] and `output` [T,7168]).  A rank
        copies only ITS token slice over PCIe, the slices are all-gathered over NVLink (every rank
        routes all tokens), the layer runs with the reduce-scatter fused in, and the rank writes its
        slice of the summed output back to `output[lo:hi]` (`all_reduce`: all of `output`).  T must be
        a multiple of the group size.  Returns a ticket at once; the host tensors must stay untouched
        until `host_wait(ticket)`.  Up to three calls may be outstanding (one copying in, one computing,
        one copying out, on three streams): issue call i, then wait for call i-2 -- with three rotating host
        output buffers -- and neither PCIe direction stands in front of the compute.  (Two device staging
        sets suffice: a set's inputs are free once its call has computed, its output once it is copied out,
        and those two conditions are waited for on the device.)"""
        T = int(routing_logits.shape[0])
        W = self.world
        if T % W:
            raise ValueError(f"T = {T} must be a multiple of the group size {W}")
        per = T // W
        lo = self.rank * per
        dev = torch.device("cuda", self.layer.device)
        self._host_stage_set(T, 0)
        seq = self._host_seq
        if seq - 3 > self._waited_upto:
            raise RuntimeError(f"call {seq}: at most three calls may be outstanding; host_wait({seq - 3}) first")
        self._host_seq += 1
        st = self._host_stage[seq & 1]
        cur = torch.cuda.current_stream(dev)
        tr = None
        if self.trace is not None:   # (seq, copy-in start, copied, gathered, compute start, compute end, copy-out end)
            tr = [seq] + [torch.cuda.Event(enable_timing=True) for _ in range(6)]
            self.trace.append(tr)
        with torch.cuda.stream(self._s_in):
            if seq >= 2:
                self._s_in.wait_event(st["ev_compute"])   # the set's inputs were read two calls ago
            if tr:
                tr[1].record(self._s_in)
            # this rank's slice, straight into its place in the gathered tensors: two contiguous runs of
            # rows, and the rank's columns of the [56, T] scale matrix as ONE strided copy (a plain
            # tensor copy of that view would pack it through pageable memory and block the host)
            st["logits"][lo:lo + per].copy_(routing_logits[lo:lo + per], non_blocking=True)
            st["hidden"][lo:lo + per].view(torch.uint8).copy_(hidden_states[lo:lo + per].view(torch.uint8), non_blocking=True)
            if self._symm_stage is not None:    # straight into the rank's columns of the [56, T] staging
                dst, dpitch = st["scale"].data_ptr() + lo * 4, T * 4
            else:                               # contiguous piece for the NCCL gather
                dst, dpitch = st["scale_parts"][self.rank].data_ptr(), per * 4
            rc = self.layer._lib.moe_fp8_b200_copy_rows_h2d(
                dst, dpitch, hidden_states_scale.data_ptr() + lo * 4, T * 4, per * 4, 56, self._s_in.cuda_stream)
            if rc != 0:
                raise RuntimeError(f"moe_fp8_b200_copy_rows_h2d failed: {rc}")
            if tr:
                tr[2].record(self._s_in)
            # the all-gather that replicates the inputs runs behind the copies on the copy-in stream, so
            # that it overlaps the previous call's compute instead of standing in front of this call's:
            # with copy engines into peer-mapped staging (no SM: an NCCL kernel would have to wait for the
            # persistent GEMM CTAs of the previous call to leave), or through NCCL
            if self._symm_stage is not None:
                self._push_slices_to_peers(T, seq)
            else:
                gather_token_slices(st["logits"], st["hidden"].view(torch.uint8), st["scale_parts"], st["scale"],
                                    self.rank, W, self.group)
            st["ev_in"].record(self._s_in)
            if tr:
                tr[3].record(self._s_in)
        cur.wait_event(st["ev_in"])
        if seq >= 2:
            cur.wait_event(st["ev_out"])                  # the set's output was copied out two calls ago
        if self._symm_stage is not None:
            self._wait_for_peer_slices(seq, cur.cuda_stream)
        if tr:
            tr[4].record(cur)
        if mode == "fused" and W > 1:
            res = self.run_fused(st["logits"], routing_bias, st["hidden"], st["scale"], gemm1_weights, gemm1_weights_scale,
                                 gemm2_weights, gemm2_weights_scale, routed_scaling_factor, scatter_out=st["out"])
        else:
            res = self.run(st["logits"], routing_bias, st["hidden"], st["scale"], gemm1_weights, gemm1_weights_scale,
                           gemm2_weights, gemm2_weights_scale, routed_scaling_factor, st["full"],
                           mode="reduce_scatter" if mode == "fused" else mode, scatter_out=st["out"])
        st["ev_compute"].record(cur)
        if tr:
            tr[5].record(cur)
        with torch.cuda.stream(self._s_out):
            self._s_out.wait_event(st["ev_compute"])
            if mode == "all_reduce":
                output.copy_(res, non_blocking=True)
            else:
                output[lo:lo + per].copy_(res[:per], non_blocking=True)
            st["ev_out"].record(self._s_out)
            self._done_events[seq % 4].record(self._s_out)
            if tr:
                tr[6].record(self._s_out)
        return seq

    def host_wait(self, ticket: int) -> None:
        """Blocks until the output of call `ticket` is in host memory."""
        if self._host_stage is None or not 0 <= ticket < self._host_seq:
            raise ValueError(f"ticket {ticket} was never issued")
        if ticket + 4 <= self._host_seq:
            return   # run_host_async only let call ticket + 3 start after this one had been waited for
        self._done_events[ticket % 4].synchronize()
        self._waited_upto = max(self._waited_upto, ticket)

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
