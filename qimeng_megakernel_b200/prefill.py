"""Prefill for the B200 route: produces what `decode()` starts from.

The reference's fused prefill is a PyTorch pass over the whole prompt that allocates the Globals, fills the
KV cache and yields the first generated token (qimeng_megakernel/models/LLM/prefill.py:14-34 PrefillOutput,
145-181 run_prefill_fused; llama/llama3_2__1b/A100/fused_prefill.py:185-335).  Here the prompt is fed through
the decode kernel one token at a time (same math, same cache layout, no CPU route); checkpoints are replaced
by the seeded synthetic weights because none can be loaded offline.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from . import mk_kernel, synthetic
from .globs import Globals


@dataclass
class PrefillOutput:
    input_ids: torch.Tensor          # [B, prompt_len] int64
    first_gen_token: torch.Tensor    # [B, 1] int64
    logits: torch.Tensor             # [B, V] logits of the last prompt position
    past_key_values: Any = None
    globs: Globals | None = None
    mk: Any = None


@torch.inference_mode()
def run_prefill_synthetic(config: dict, weights: dict, prompt_ids: torch.Tensor, max_new_tokens: int,
                          device: str | torch.device = "cuda:0", mk: Any = None) -> PrefillOutput:
    """prompt_ids: [B, prompt_len] (or [prompt_len]) int64 token ids; B > 1 gives [B, ...] state and runs the
    batched kernel (all prompts of one length, like the reference's fused prefill for a padded batch)."""
    ids = (prompt_ids.view(1, -1) if prompt_ids.dim() == 1 else prompt_ids).to(torch.int64)
    prompt_len = int(ids.shape[1])
    if prompt_len < 1:
        raise ValueError("empty prompt")
    dev = torch.device(device)
    if ids.shape[0] > 1:
        B = int(ids.shape[0])
        g = synthetic.make_globals(config, weights, kv_seq_len=prompt_len + max(0, max_new_tokens), device=dev, batch=B)
        mk = mk if mk is not None else mk_kernel.get_mk()
        ids_dev = ids.to(dev)
        g.token_in = torch.zeros(B, dtype=torch.int64, device=dev)
        for pos in range(prompt_len):      # one position of every prompt per launch: fills the KV cache
            g.token_in.copy_(ids_dev[:, pos])
            g.position_id = pos
            mk(g)
        mk.check_status()
        first = g.next_token.clone().view(B, 1)
        g.token_in = None
        return PrefillOutput(input_ids=ids_dev, first_gen_token=first, logits=g.logits.clone(), globs=g, mk=mk)
    g = synthetic.make_globals(config, weights, kv_seq_len=prompt_len + max(0, max_new_tokens), device=dev)
    mk = mk if mk is not None else mk_kernel.get_mk()
    host = ids[0].cpu().contiguous()
    out = torch.zeros(prompt_len, dtype=torch.int64)
    mk.generate_host(g, host, 0, prompt_len, teacher_forced=True, host_argmax=out)
    mk.check_status()
    first = out[-1:].view(1, 1).to(dev)
    return PrefillOutput(input_ids=ids.to(dev), first_gen_token=first, logits=g.logits.view(1, -1).clone(),
                         globs=g, mk=mk)
