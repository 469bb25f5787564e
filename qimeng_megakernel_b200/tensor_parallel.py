"""Tensor parallelism for the dense decode route: every GPU holds 1 / N of every projection.

The reference has no distributed code; what is split are its two residual projections
(qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/single_batch/decode_kernel/oproj_gemv_residual.cu:217-225 and
down_proj_gemv_residual.cu:225-234: hidden += W x) and what feeds them.  Rank r of N holds
  Q/K/V rows of heads [r, r + 1) * NH / N (and the matching KV heads), so attention is local to a rank;
  O-proj columns of those heads and down-proj columns of intermediate units [r, r + 1) * I / N: both projections then
    produce PARTIAL sums over the rank's slice of K, which the kernel's residual epilogue pushes to the peers' buffers
    over NVLink and adds in rank order (csrc/qmk_batch_kernel.cuh, ep_exchange) -- every rank ends a phase with the same
    residual stream, bit for bit;
  up/gate rows of its intermediate units;
  LM-head rows of vocabulary slice [r, r + 1) * V / N; the arg-max key carries the global row and the ranks exchange
    their keys at the end of the step (finalize).
Norm gains, the embedding table and the RoPE tables are whole on every rank.  `logits` of a rank is its [B, V / N] slice.

This module is the host side: the per-rank config and weight slices.  The buffer handles are exchanged once with
expert_parallel.connect (the same exchange buffers serve both kinds of model parallelism).
"""
from __future__ import annotations

import torch


def check(config: dict, world: int) -> None:
    if world not in (2, 4, 8):
        raise ValueError(f"tensor parallelism over {world} ranks (2, 4 or 8)")
    if config.get("num_experts"):
        raise ValueError("mixture-of-experts models are split by experts (expert_parallel), not by tensors")
    for key in ("num_attention_heads", "num_key_value_heads", "vocab_size"):
        if int(config[key]) % world:
            raise ValueError(f"{key} = {config[key]} does not divide over {world} ranks")
    if int(config["intermediate_size"]) % (64 * world):
        raise ValueError(f"intermediate_size = {config['intermediate_size']} must be a multiple of 64 per rank")


def shard_config(config: dict, rank: int, world: int) -> dict:
    """The config of one rank: heads, KV heads, intermediate units and LM-head rows divided by `world`."""
    check(config, world)
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    return dict(config, num_attention_heads=config["num_attention_heads"] // world,
                num_key_value_heads=config["num_key_value_heads"] // world,
                intermediate_size=config["intermediate_size"] // world, vocab_size=config["vocab_size"] // world,
                head_dim=config.get("head_dim") or config["hidden_size"] // config["num_attention_heads"],
                embed_rows=config["vocab_size"], tp_world=world, tp_rank=rank)


def shard_weights(config: dict, weights: dict, rank: int, world: int) -> dict:
    """A rank's slices of a full set of weights (`config` is the WHOLE model's).  Slices are made contiguous; whole
    tensors are shared with `weights`."""
    check(config, world)
    NH, NKV = config["num_attention_heads"], config["num_key_value_heads"]
    HD = config.get("head_dim") or config["hidden_size"] // NH
    I, V = config["intermediate_size"], config["vocab_size"]
    qd, kd = NH * HD, NKV * HD
    ql, kl, il, vl = qd // world, kd // world, I // world, V // world
    qkv = weights["qkv_weights"]
    out = dict(weights)
    out["qkv_weights"] = torch.cat([qkv[:, rank * ql:(rank + 1) * ql], qkv[:, qd + rank * kl:qd + (rank + 1) * kl],
                                    qkv[:, qd + kd + rank * kl:qd + kd + (rank + 1) * kl]], dim=1).contiguous()
    out["o_proj_weights"] = weights["o_proj_weights"][:, :, rank * ql:(rank + 1) * ql].contiguous()
    out["up_proj_weights"] = weights["up_proj_weights"][:, rank * il:(rank + 1) * il].contiguous()
    out["gate_proj_weights"] = weights["gate_proj_weights"][:, rank * il:(rank + 1) * il].contiguous()
    out["down_proj_weights"] = weights["down_proj_weights"][:, :, rank * il:(rank + 1) * il].contiguous()
    out["lm_head_weights"] = weights["lm_head_weights"][rank * vl:(rank + 1) * vl].contiguous()
    out["embed_tokens"] = weights["embed_tokens"]          # whole, on every rank
    return out
