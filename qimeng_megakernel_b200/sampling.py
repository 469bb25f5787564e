"""Token selection after the LM head: greedy, or temperature / min-p / top-k / top-p sampling with a presence penalty.

Same semantics and the same order of operations as the reference's `_sample_logits`
(qimeng_megakernel/models/LLM/decode.py:53-143): presence penalty on the fp32 logits of every token id already in the
row -> greedy when temperature <= 0 or no filter is active -> logits / max(temperature, 1e-8) -> softmax -> min-p
(probabilities below min_p dropped, renormalised; if nothing is left the unfiltered softmax is used) -> top-k
(renormalised) -> top-p over the descending-sorted probabilities (a token is kept while the mass before it is <= top_p;
renormalised, same fall-back) -> one multinomial draw from the probabilities clamped to >= 1e-9.

The reference loops over the rows of a batch in Python; here all rows are filtered together on the device (the filters
are row-wise operations), and `filtered_probs` exposes the distribution the draw is taken from so that it can be compared
with the reference's.  The logits come from the kernel's LM-head phase (bf16 [B, V] on the device).
"""
from __future__ import annotations

import torch


def is_greedy(temperature: float = 0.0, top_p: float = 1.0, top_k: int = 0, min_p: float = 0.0,
              vocab: int | None = None) -> bool:
    """The reference's greedy rule (decode.py:70-72, 96): no temperature, or no filter that could exclude a token."""
    k_off = top_k <= 0 or (vocab is not None and top_k >= vocab)
    return temperature <= 0 or (top_p >= 1.0 and k_off and min_p <= 0.0)


def apply_presence_penalty(logits: torch.Tensor, generated_ids: torch.Tensor | None, presence_penalty: float) -> torch.Tensor:
    """fp32 copy of `logits` [B, V] with `presence_penalty` subtracted once for every distinct id in generated_ids [B, n]."""
    out = logits.float().clone()
    if presence_penalty != 0.0 and generated_ids is not None and generated_ids.numel() > 0:
        seen = torch.zeros_like(out, dtype=torch.bool)
        seen.scatter_(1, generated_ids.to(torch.int64), True)
        out = torch.where(seen, out - presence_penalty, out)
    return out


def filtered_probs(logits: torch.Tensor, temperature: float, top_p: float = 1.0, top_k: int = 0,
                   min_p: float = 0.0) -> torch.Tensor:
    """[B, V] fp32 probabilities after the temperature and the three filters (rows sum to 1 unless a filter emptied
    the row, which falls back exactly as the reference does)."""
    scaled = logits.float() / max(temperature, 1e-8)
    base = torch.softmax(scaled, dim=-1)
    probs = base
    V = probs.shape[-1]
    if min_p > 0.0:
        kept = torch.where(probs >= min_p, probs, torch.zeros_like(probs))
        s = kept.sum(dim=-1, keepdim=True)
        probs = torch.where(s > 1e-9, kept / s.clamp(min=1e-30), base)
    if 0 < top_k < V:
        vals, idx = torch.topk(probs, top_k, dim=-1)
        kept = torch.zeros_like(probs).scatter_(-1, idx, vals)
        s = kept.sum(dim=-1, keepdim=True)
        probs = torch.where(s > 1e-9, kept / s.clamp(min=1e-30), kept)
    if top_p < 1.0:
        sp, si = torch.sort(probs, descending=True, dim=-1)
        before = torch.cumsum(sp, dim=-1) - sp
        sp = torch.where(before > top_p, torch.zeros_like(sp), sp)
        kept = torch.zeros_like(probs).scatter_(-1, si, sp)
        s = kept.sum(dim=-1, keepdim=True)
        probs = torch.where(s > 1e-9, kept / s.clamp(min=1e-30), base)
    return probs


def sample_logits(logits: torch.Tensor, temperature: float = 0.0, top_p: float = 1.0, top_k: int = 0, min_p: float = 0.0,
                  presence_penalty: float = 0.0, generated_ids: torch.Tensor | None = None,
                  generator: torch.Generator | None = None) -> torch.Tensor:
    """Next token id per row: int64 [B] for logits [B, V] ([V] is treated as one row and returns a 0-d tensor)."""
    one_row = logits.dim() == 1
    lg = logits.view(1, -1) if one_row else logits
    gen = None
    if generated_ids is not None and generated_ids.numel() > 0:
        gen = generated_ids.view(1, -1) if generated_ids.dim() == 1 else generated_ids
    penalised = presence_penalty != 0.0 and gen is not None
    greedy = is_greedy(temperature, top_p, top_k, min_p, vocab=lg.shape[-1])
    if greedy and not penalised:
        out = torch.argmax(lg, dim=-1)
    else:
        work = apply_presence_penalty(lg, gen, presence_penalty) if penalised else lg.float()
        if greedy:
            out = torch.argmax(work, dim=-1)
        else:
            probs = filtered_probs(work, temperature, top_p, top_k, min_p)
            out = torch.multinomial(probs.clamp(min=1e-9), num_samples=1, replacement=True, generator=generator).squeeze(-1)
    return out[0] if one_row else out
