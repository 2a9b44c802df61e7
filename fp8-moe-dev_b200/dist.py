"""Expert-parallel form of the layer on one NVSwitch box: the 256 experts are split evenly
over the G ranks of a torch.distributed group (rank r holds experts [r*256/G, (r+1)*256/G),
i.e. local_expert_offset = 256/G * r), every rank routes all T tokens and computes its own
experts, and the bf16 partial outputs are summed over NVLink.  The reference has no
multi-GPU code; its `local_expert_offset` argument (kernel/moe_fp8.cu:2668, 462-463) is the
hook this builds on.

The reduction is the path's one exchange step.  `partial -> all_reduce` (every rank ends
with the full [T,7168] output) or `partial -> reduce_scatter` (rank r ends with tokens
[r*T/G, (r+1)*T/G)).  The host-side planning (who owns which experts / tokens) is plain
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


class ShardedMoe:
    """One rank's share of the 256-expert layer plus the cross-rank sum."""

    def __init__(self, max_tokens: int, rank: Optional[int] = None, world: Optional[int] = None,
                 device: Optional[int] = None, group=None):
        from .op import MoeLayer
        if rank is None:
            rank = dist.get_rank(group) if dist.is_initialized() else 0
        if world is None:
            world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank, self.world, self.group = rank, world, group
        self.local_expert_offset, self.num_local_experts = expert_range(rank, world)
        self.layer = MoeLayer(max_tokens, self.num_local_experts, device)

    def run(self, routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
            gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, routed_scaling_factor, output,
            mode: str = "all_reduce", scatter_out: Optional[torch.Tensor] = None):
        self.layer.run(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                       gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, self.local_expert_offset,
                       routed_scaling_factor, output)
        return combine_partials(output, mode, self.group, scatter_out)
