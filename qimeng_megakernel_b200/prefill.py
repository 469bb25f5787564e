"""Prefill for the B200 route: produces what `decode()` starts from.

The reference's fused prefill is a PyTorch pass over the whole prompt that allocates the Globals, fills the KV cache and
yields the first generated token (qimeng_megakernel/models/LLM/prefill.py:14-34 PrefillOutput, 145-181 run_prefill_fused;
llama/llama3_2__1b/A100/fused_prefill.py:185-335).  Here the prompt goes through the batched decode kernel with the rows
of a step being CONSECUTIVE POSITIONS of a sequence (`Globals.kv_slots`): up to 64 prompt tokens per launch on the
tensor cores -- a row attends to every earlier position, also to those appended by other rows of the same launch -- so
a 16-token prompt is one launch instead of sixteen decode steps, and several short prompts share a launch.  Same math,
same cache layout, no CPU route; checkpoints are replaced by the seeded synthetic weights because none can be loaded
offline.  `fused=False` keeps the token-by-token path (one decode step per prompt position).
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any

import torch

from . import _lib, mk_kernel, synthetic
from .globs import Globals


@dataclass
class PrefillOutput:
    input_ids: torch.Tensor          # [B, prompt_len] int64
    first_gen_token: torch.Tensor    # [B, 1] int64
    logits: torch.Tensor             # [B, V] logits of the last prompt position
    past_key_values: Any = None
    globs: Globals | None = None
    mk: Any = None
    launches: int = 0                # kernel launches the prefill took


def prefill_plan(batch: int, prompt_len: int, rows: int = _lib.MAX_BATCH) -> list[list[tuple[int, int]]]:
    """The launches of a fused prefill: each is a list of (sequence, position) rows, at most `rows` long.  Positions of
    one sequence are consecutive inside a launch and ascending over the launches, so whatever a row attends to is either
    in the cache already or appended by an earlier row of the same launch."""
    per_seq = min(prompt_len, rows)              # positions of one sequence in one launch
    seqs_per_launch = max(1, rows // per_seq)
    plan = []
    for p0 in range(0, prompt_len, per_seq):
        p1 = min(prompt_len, p0 + per_seq)
        for s0 in range(0, batch, seqs_per_launch):
            plan.append([(s, p) for s in range(s0, min(batch, s0 + seqs_per_launch)) for p in range(p0, p1)])
    return plan


def _prefill_state(g: Globals, config: dict, rows: int) -> Globals:
    """State tensors with `rows` rows around the weights and the KV cache of the decode state `g`."""
    dev, bf = g.k_cache.device, torch.bfloat16
    H, I, V = config["hidden_size"], config["intermediate_size"], config["vocab_size"]
    QD = config["num_attention_heads"] * config["head_dim"]
    z = lambda *shape, dtype=bf: torch.zeros(*shape, dtype=dtype, device=dev)
    return dataclasses.replace(
        g, hidden_states=z(rows, H), q_post_rope=z(rows, QD), attn_out=z(rows, QD), silu_out=z(rows, I), logits=z(rows, V),
        next_token=z(rows, dtype=torch.int64), token_in=z(rows, dtype=torch.int64), out_tokens=None,
        position_ids=z(rows, dtype=torch.int32), active_mask=z(rows, dtype=torch.uint8), kv_slots=z(rows, dtype=torch.int32))


@torch.inference_mode()
def run_prefill_synthetic(config: dict, weights: dict, prompt_ids: torch.Tensor, max_new_tokens: int,
                          device: str | torch.device = "cuda:0", mk: Any = None, fused: bool = True) -> PrefillOutput:
    """prompt_ids: [B, prompt_len] (or [prompt_len]) int64 token ids; B > 1 gives [B, ...] decode state (all prompts of
    one length, like the reference's fused prefill for a padded batch)."""
    ids = (prompt_ids.view(1, -1) if prompt_ids.dim() == 1 else prompt_ids).to(torch.int64)
    B, prompt_len = int(ids.shape[0]), int(ids.shape[1])
    if prompt_len < 1:
        raise ValueError("empty prompt")
    dev = torch.device(device)
    g = synthetic.make_globals(config, weights, kv_seq_len=prompt_len + max(0, max_new_tokens), device=dev,
                               batch=B if B > 1 else None)
    mk = mk if mk is not None else mk_kernel.get_mk()
    ids_dev = ids.to(dev)
    if fused:
        plan = prefill_plan(B, prompt_len)
        rows = max(len(launch) for launch in plan)
        gp = _prefill_state(g, config, rows)
        first = torch.zeros(B, dtype=torch.int64, device=dev)
        logits = torch.zeros(B, config["vocab_size"], dtype=torch.bfloat16, device=dev)
        for launch in plan:
            n = len(launch)
            seq = torch.tensor([s for s, _ in launch], dtype=torch.int64)
            pos = torch.tensor([p for _, p in launch], dtype=torch.int64)
            gp.token_in.zero_(); gp.position_ids.zero_(); gp.kv_slots.zero_(); gp.active_mask.zero_()
            gp.token_in[:n].copy_(ids[seq, pos])
            gp.position_ids[:n].copy_(pos.to(torch.int32))
            gp.kv_slots[:n].copy_(seq.to(torch.int32))
            gp.active_mask[:n].fill_(1)
            gp.position_id = int(pos.max())
            mk(gp)
            last = [(r, s) for r, (s, p) in enumerate(launch) if p == prompt_len - 1]
            if last:
                r_idx = torch.tensor([r for r, _ in last], device=dev)
                s_idx = torch.tensor([s for _, s in last], device=dev)
                first[s_idx] = gp.next_token[r_idx]
                logits[s_idx] = gp.logits[r_idx]
        mk.check_status()
        return PrefillOutput(input_ids=ids_dev, first_gen_token=first.view(B, 1), logits=logits, globs=g, mk=mk,
                             launches=len(plan))
    if B > 1:
        g.token_in = torch.zeros(B, dtype=torch.int64, device=dev)
        for pos in range(prompt_len):      # one position of every prompt per launch: fills the KV cache
            g.token_in.copy_(ids_dev[:, pos])
            g.position_id = pos
            mk(g)
        mk.check_status()
        first = g.next_token.clone().view(B, 1)
        g.token_in = None
        return PrefillOutput(input_ids=ids_dev, first_gen_token=first, logits=g.logits.clone(), globs=g, mk=mk,
                             launches=prompt_len)
    host = ids[0].cpu().contiguous()
    out = torch.zeros(prompt_len, dtype=torch.int64)
    mk.generate_host(g, host, 0, prompt_len, teacher_forced=True, host_argmax=out)
    mk.check_status()
    first = out[-1:].view(1, 1).to(dev)
    return PrefillOutput(input_ids=ids_dev, first_gen_token=first, logits=g.logits.view(1, -1).clone(),
                         globs=g, mk=mk, launches=prompt_len)
