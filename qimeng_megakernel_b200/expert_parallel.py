"""Expert parallelism for the mixture-of-experts route: E / N experts per GPU, attention and router replicated.

The reference has no distributed code; the math that is split is its routed accumulate
(qimeng_megakernel/models/LLM/qwen/qwen1_5_moe_a2_7b/A100/single_batch/decode_schedule/fused/operations.py:220-268): the
weighted sum over a row's selected experts becomes a sum over ranks of the weighted sums over the selected experts each
rank holds.  Inside the kernel's expert down-projection every rank stores its partial tiles into the peers' exchange
buffers over NVLink and adds what it receives in rank order (csrc/qmk_batch_kernel.cuh, ep_exchange); this module is the
host side: which experts a rank holds, how to cut a full set of weights, and the one-time exchange of buffer handles over
torch.distributed (one process per GPU).
"""
from __future__ import annotations

import torch


def expert_range(rank: int, world: int, num_experts: int) -> tuple[int, int]:
    """Experts [lo, hi) held by `rank`: contiguous blocks of num_experts / world."""
    if world < 1 or num_experts % world != 0 or not 0 <= rank < world:
        raise ValueError(f"{num_experts} experts cannot be split over {world} ranks (rank {rank})")
    per = num_experts // world
    return rank * per, (rank + 1) * per


def shard_config(config: dict, rank: int, world: int) -> dict:
    """The model config of one rank: the same model, with ep_world / ep_rank set."""
    expert_range(rank, world, int(config["num_experts"]))
    return dict(config, ep_world=world, ep_rank=rank)


def shard_moe_weights(weights: dict, rank: int, world: int) -> dict:
    """A rank's view of a full set of weights: its block of expert_gate_up / expert_down ([L, E / world, ...], views of
    the full tensors made contiguous), everything else shared."""
    E = int(weights["expert_gate_up_proj_weights"].shape[1])
    lo, hi = expert_range(rank, world, E)
    out = dict(weights)
    out["expert_gate_up_proj_weights"] = weights["expert_gate_up_proj_weights"][:, lo:hi].contiguous()
    out["expert_down_proj_weights"] = weights["expert_down_proj_weights"][:, lo:hi].contiguous()
    return out


def connect(mk, globs, group=None) -> None:
    """One-time set-up after the process group exists: gathers the exchange-buffer handles of all ranks and maps them.
    `globs` is this rank's decode state (its expert tensors hold this rank's experts only)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    mine = torch.tensor(list(mk.ep_export(globs)), dtype=torch.uint8)
    if dist.get_backend(group) == "nccl":
        mine = mine.cuda()
    gathered = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine, group=group)
    mk.ep_connect([bytes(t.cpu().tolist()) for t in gathered])
    dist.barrier(group)
