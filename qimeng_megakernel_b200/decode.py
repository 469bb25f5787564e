"""`decode()` for the B200 megakernel route: the host token loop around the kernel.

Host-side counterpart of the reference's `decode(..., decode_route="mk")` -> `_decode_mk` ->
`FusedGenerator.generate_greedy_fast` / `generate_with_eos` (qimeng_megakernel/models/LLM/decode.py:1885-2063, 536-849,
1340-1435).  The argument names, the returned dictionary {"generated_ids", "new_tokens", "per_row_new_tokens",
"timing"} and the timing keys are that function's interface and are reproduced key for key (decode.py:755-794), as is
its post-hoc end-of-sequence scan (decode.py:1397-1430), so that callers and benchmark scripts written against the
reference read the same fields: the first generated token belongs to prefill, the decode window holds
max_new_tokens - 1 kernel steps and `kernel_tok_s` divides those tokens by the sum of the per-step CUDA event spans
around the kernel call.

Two loops are offered:
  host_loop=True   the reference's loop verbatim: embed the token with PyTorch, copy into hidden_states,
                   set position_id, call_mk, arg-max of globs.logits with PyTorch.
  host_loop=False  (default) the kernel embeds the token itself and feeds its own arg-max back
                   (globs.token_in / next_token / out_tokens), so a step is exactly one launch.
With sampling arguments (temperature > 0 together with top_p / top_k / min_p, or a presence penalty; decode.py:53-143)
the kernel still embeds the fed token itself and the next token is drawn from `globs.logits` on the device after every
step (sampling.py); `seed` makes the draws reproducible.
"""
from __future__ import annotations

import time
from typing import Any

import torch

from .prefill import PrefillOutput
from .registry import import_decode_schedule, resolve_hardware
from .sampling import is_greedy, sample_logits


def _is_greedy(kw: dict) -> bool:
    """Greedy by the reference's rule (no temperature, or no filter that could exclude a token) and no penalty."""
    return (is_greedy(float(kw.get("temperature", 0.0)), float(kw.get("top_p", 1.0)), int(kw.get("top_k", 0) or 0),
                      float(kw.get("min_p", 0.0))) and float(kw.get("presence_penalty", 0.0)) == 0.0)


@torch.inference_mode()
def decode(model_name: str, *, prefill: PrefillOutput, max_new_tokens: int, decode_route: str = "mk",
           hardware: str = "B200", decode_time: bool = False, ignore_eos: bool = False,
           eos_token_ids: list[int] | None = None, pad_token_id: int | None = None, mk_dir: str | None = None,
           host_loop: bool = False, **kwargs: Any) -> dict:
    if decode_route != "mk":
        raise NotImplementedError(f"route {decode_route!r}: this package implements the compiled 'mk' route only "
                                  "(the PyTorch routes live in the reference)")
    sampled = not _is_greedy(kwargs)
    hardware = resolve_hardware(hardware)
    ids = prefill.input_ids
    batch_size, prompt_len = int(ids.shape[0]), int(ids.shape[1])
    if max_new_tokens <= 0:
        return {"generated_ids": ids, "new_tokens": ids.new_empty((batch_size, 0)),
                "per_row_new_tokens": ids.new_zeros(batch_size, dtype=torch.long)}
    if ignore_eos:
        eos_token_ids = []
    globs = prefill.globs
    if globs is None:
        raise ValueError("prefill.globs is required (run_prefill_synthetic builds it)")
    if int(globs.k_cache.shape[2]) < prompt_len + max_new_tokens:
        raise ValueError("KV cache shorter than prompt_len + max_new_tokens")
    # Per-row positions (the reference's multi-batch state): the kernel reads them instead of position_id, so they are
    # advanced on the stream after every step as the reference's loop does (decode.py:1398-1400).
    pids = getattr(globs, "position_ids", None)
    if pids is not None and int(pids.max()) + max_new_tokens > int(globs.k_cache.shape[2]):
        raise ValueError("KV cache shorter than the largest row position + max_new_tokens")
    setup_t0 = time.perf_counter()
    schedule = import_decode_schedule(model_name, hardware, batch_size=batch_size)
    static_megakernel = bool(getattr(schedule.package, "STATIC_MEGAKERNEL", False))
    assert static_megakernel, "the B200 package owns its scheduler"
    mk = prefill.mk if prefill.mk is not None and mk_dir is None else schedule.get_mk(mk_dir)
    instruction_setup_wall_s = time.perf_counter() - setup_t0
    device = ids.device
    ntok = max_new_tokens - 1

    output_tokens = ids.new_zeros(batch_size, prompt_len + max_new_tokens)
    output_tokens[:, :prompt_len] = ids
    output_tokens[:, prompt_len] = prefill.first_gen_token.squeeze(-1)

    events = []
    if decode_time:
        events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(ntok)]
        loop_start, loop_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(device)
        start_wall = time.perf_counter()
        loop_start.record()

    if sampled:
        # FusedGenerator.generate (decode.py:1147-1170) with _sample_logits after every step: the drawn token is fed
        # back through token_in, so a step is still one kernel launch plus the device-side draw
        saved = (globs.token_in, globs.out_tokens, globs.next_token)
        globs.out_tokens = None
        globs.token_in = output_tokens[:, prompt_len].clone()
        penalty = float(kwargs.get("presence_penalty", 0.0))
        gen = None
        if kwargs.get("seed") is not None:
            gen = torch.Generator(device=device)
            gen.manual_seed(int(kwargs["seed"]))
        for i in range(ntok):
            pos = prompt_len + i
            globs.position_id = pos
            if events:
                events[i][0].record()
            schedule.call_mk(globs, mk)
            if events:
                events[i][1].record()
            if pids is not None:
                pids.add_(1)
            nxt = sample_logits(globs.logits.view(batch_size, -1), temperature=float(kwargs.get("temperature", 0.0)),
                                top_p=float(kwargs.get("top_p", 1.0)), top_k=int(kwargs.get("top_k", 0) or 0),
                                min_p=float(kwargs.get("min_p", 0.0)), presence_penalty=penalty,
                                generated_ids=output_tokens[:, :pos + 1] if penalty != 0.0 else None, generator=gen)
            output_tokens[:, pos + 1] = nxt
            globs.token_in.copy_(nxt)
        globs.token_in, globs.out_tokens, globs.next_token = saved
    elif host_loop:
        # FusedGenerator.generate_greedy_fast (decode.py:1373-1395): [H] state for one sequence, [B, H] for several
        saved = (globs.token_in, globs.out_tokens)
        globs.token_in = None
        globs.out_tokens = None
        embed, dtype = globs.embed_tokens, globs.hidden_states.dtype
        for i in range(ntok):
            pos = prompt_len + i
            emb = embed[output_tokens[:, pos]].to(dtype)
            globs.hidden_states.copy_(emb.reshape(globs.hidden_states.shape))
            globs.position_id = pos
            if events:
                events[i][0].record()
            schedule.call_mk(globs, mk)
            if events:
                events[i][1].record()
            if pids is not None:
                pids.add_(1)
            output_tokens[:, pos + 1] = globs.logits.view(batch_size, -1).argmax(dim=-1)
        globs.token_in, globs.out_tokens = saved
    else:
        saved = (globs.token_in, globs.out_tokens, globs.next_token)
        globs.out_tokens = output_tokens[0] if batch_size == 1 else output_tokens
        globs.token_in = output_tokens[:, prompt_len].clone()
        globs.next_token = globs.token_in
        for i in range(ntok):
            globs.position_id = prompt_len + i
            if events:
                events[i][0].record()
            schedule.call_mk(globs, mk)
            if events:
                events[i][1].record()
            if pids is not None:
                pids.add_(1)
        globs.token_in, globs.out_tokens, globs.next_token = saved

    timing = None
    if decode_time:
        loop_end.record()
        torch.cuda.synchronize(device)
        decode_wall_s = time.perf_counter() - start_wall
        decode_gpu_s = loop_start.elapsed_time(loop_end) / 1000.0
        mk_kernel_gpu_s = sum(a.elapsed_time(b) for a, b in events) / 1000.0
    if ntok > 0:
        mk.check_status()

    # post-hoc EOS scan (decode.py:1397-1430)
    num_new_after_first = ntok
    per_row = torch.full((batch_size,), ntok + 1, dtype=torch.long, device=device)
    if eos_token_ids:
        eos = torch.tensor(eos_token_ids, dtype=output_tokens.dtype, device=device)
        chunk = output_tokens[:, prompt_len:prompt_len + ntok + 1]
        hits = (chunk.unsqueeze(-1) == eos.view(1, 1, -1)).any(dim=-1)
        has = hits.any(dim=1)
        end_excl = torch.full((batch_size,), prompt_len + ntok + 1, dtype=torch.long, device=device)
        if bool(has.any()):
            first_rel = hits.to(torch.int32).argmax(dim=1).to(torch.long)
            end_excl[has] = prompt_len + first_rel[has] + 1
        slice_end = int(end_excl.max())
        num_new_after_first = slice_end - prompt_len - 1
        per_row = (end_excl - prompt_len).clamp(min=0)
        if pad_token_id is not None:
            idx = torch.arange(slice_end, device=device)
            mask = idx.unsqueeze(0) >= end_excl.unsqueeze(1)
            output_tokens[:, :slice_end] = torch.where(mask, torch.full_like(output_tokens[:, :slice_end], pad_token_id),
                                                       output_tokens[:, :slice_end])

    if decode_time:
        effective = int(per_row.sum())
        window = max(effective - batch_size, 0)
        step_bytes = sum(mk.step_bytes(prompt_len + i) for i in range(ntok)) / ntok if ntok > 0 else 0.0
        timing = {
            "instruction_setup_wall_s": instruction_setup_wall_s, "queue_build_wall_s": 0.0, "tensorize_wall_s": 0.0,
            "decode_wall_s": decode_wall_s, "decode_gpu_s": decode_gpu_s, "mk_kernel_gpu_s": mk_kernel_gpu_s,
            "non_kernel_gpu_s": max(decode_gpu_s - mk_kernel_gpu_s, 0.0),
            "non_kernel_wall_s": max(decode_wall_s - mk_kernel_gpu_s, 0.0),
            "effective_new_tokens": effective, "decode_window_new_tokens": window,
            "effective_tok_s_wall": window / decode_wall_s if decode_wall_s > 0 and window > 0 else 0.0,
            "effective_tok_s_gpu": window / decode_gpu_s if decode_gpu_s > 0 and window > 0 else 0.0,
            "kernel_tok_s": window / mk_kernel_gpu_s if mk_kernel_gpu_s > 0 and window > 0 else 0.0,
            "kernel_steps": ntok,
            "hbm_bytes_per_step": step_bytes,
            "achieved_hbm_gbs": step_bytes * ntok / mk_kernel_gpu_s / 1e9 if mk_kernel_gpu_s > 0 else 0.0,
        }
        print("[mk] decode_time_fast: wall=%.3f s, gpu=%.3f s, mk_kernel_gpu=%.3f s, effective_new_tokens=%d, "
              "tok/s[wall=%.2f gpu=%.2f kernel=%.2f], decode_window_new_tokens=%d (B200 %s loop)"
              % (decode_wall_s, decode_gpu_s, mk_kernel_gpu_s, effective, timing["effective_tok_s_wall"],
                 timing["effective_tok_s_gpu"], timing["kernel_tok_s"], window,
                 "sampling" if sampled else ("host" if host_loop else "device")),
              flush=True)
    total_new = num_new_after_first + 1
    return {"generated_ids": output_tokens[:, :prompt_len + total_new],
            "new_tokens": output_tokens[:, prompt_len:prompt_len + total_new],
            "per_row_new_tokens": per_row, "timing": timing}
