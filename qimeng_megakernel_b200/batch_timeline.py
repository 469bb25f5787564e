"""In-kernel timeline of one decode step of the batched kernel: time and achieved HBM GB/s per phase kind.

    python -m qimeng_megakernel_b200.batch_timeline [--batch 8] [--model llama-3.2-1b|qwen3-0.6b|olmoe-1b-7b]
                                                    [--pos 299]

Runs `--pos` + 1 persistent steps (the last one with `qmk_set_trace` attached) and reads the globaltimer stamps
every CTA leaves per phase: when the phase's dependency became visible, when the CTA's first accumulator was
complete, when it arrived at the phase's counter.  A phase's span is the time between the last arrival of the
phase before it and its own last arrival, so the spans add up to the step.  No profiler is involved.  The
reference's counterpart is its compile-time clock64 profiling buffer
(qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/multi_batch/decode_kernel/profiling.cuh:7-35).
"""
from __future__ import annotations

import argparse
import os

import torch

from . import mk_kernel, synthetic
from .model_config import LLAMA_3_2_1B, OLMOE_1B_7B, QWEN3_0_6B

MODELS = {"llama-3.2-1b": LLAMA_3_2_1B, "qwen3-0.6b": QWEN3_0_6B, "olmoe-1b-7b": OLMOE_1B_7B}
DENSE = ("qkv", "attn", "oproj", "upgate", "down")
MOE = ("qkv", "attn", "oproj", "router", "expert_upgate", "expert_down")


def phase_bytes(cfg: dict, kind: str, T: int, B: int, experts: int) -> float:
    """Algorithmic bytes of one phase: its weights once, for attention the K/V rows of every sequence."""
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    NH, NKV, HD, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["vocab_size"]
    Ie, E = cfg.get("moe_intermediate_size", 0), cfg.get("num_experts", 0)
    return {"qkv": 2 * (NH + 2 * NKV) * HD * H, "attn": B * 2 * 2 * NKV * HD * T, "oproj": 2 * H * NH * HD,
            "upgate": 2 * 2 * I * H, "down": 2 * H * I, "lm_head": 2 * V * H, "router": 2 * E * H,
            "expert_upgate": 2 * experts * 2 * Ie * H, "expert_down": 2 * experts * H * Ie}[kind]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--model", default="llama-3.2-1b", choices=sorted(MODELS))
    ap.add_argument("--pos", type=int, default=299)
    ap.add_argument("--detail", default="", help="phase kind whose per-CTA stamps (second layer) are listed for the CTAs that had work")
    args = ap.parse_args()
    cfg = dict(MODELS[args.model])
    B, dev = args.batch, torch.device("cuda")
    w = synthetic.make_weights(cfg, seed=0, device=dev, max_positions=max(2048, args.pos + 8))
    g = synthetic.make_globals(cfg, w, kv_seq_len=args.pos + 8, device=dev, batch=B)
    mk = mk_kernel.get_mk()
    mk.set_kernel_variant(1)
    g.token_in = torch.randint(0, cfg["vocab_size"], (B,), device=dev)
    g.next_token = g.token_in
    moe = bool(cfg.get("num_experts"))
    names = MOE if moe else DENSE
    ppl, L = len(names), cfg["num_hidden_layers"]
    nph = ppl * L + 1
    trace = None
    for pos in range(args.pos + 1):
        g.position_id = pos
        if pos == args.pos:
            trace = torch.zeros(mk.geometry()[0], nph, 16, dtype=torch.int64, device=dev)
            mk.set_trace(trace)
        mk(g)
    torch.cuda.synchronize()
    mk.check_status()
    experts = mk.last_expert_count() if moe else 0
    t = trace.cpu().double()
    try:                      # SM clock in GHz: turns the cycle sums into nanoseconds like the timer stamps
        ghz = float(torch.cuda.clock_rate()) / 1e3
    except Exception:
        ghz = 1.9
    start = t[:, 0, 2][t[:, 0, 2] > 0].min()
    rows: dict[str, list] = {}
    for ph in range(nph):
        kind = "lm_head" if ph == ppl * L else names[ph % ppl]
        arr, dep, first = t[:, ph, 5], t[:, ph, 0], t[:, ph, 1]
        prev = t[:, ph - 1, 5].max() if ph > 0 else start
        rows.setdefault(kind, []).append((
            float(arr.max() - prev), float(dep.max() - prev) if float(dep.max()) > 0 else 0.0,
            float(first[first > 0].min() - prev) if bool((first > 0).any()) else 0.0,
            float(arr.max() - arr[arr > 0].min()),
            float(t[:, ph, 3].mean()) / ghz, float(t[:, ph, 4].mean()) / ghz,
            float(t[:, ph, 6].mean()) / ghz, float(t[:, ph, 7].mean()) / ghz,
            float(t[:, ph, 8].mean()) / ghz, float(t[:, ph, 9].mean()) / ghz, float(t[:, ph, 10].mean()) / ghz))
    T = args.pos + 1
    print(f"# {args.model} shape, {B} sequences, KV length {T}" + (f", {experts} experts read in the last layer" if moe else ""))
    print("# per phase kind, mean over layers, microseconds: span | dependency visible | first accumulator | arrival spread |"
          " issuer (waits: weights, activations, accumulator; issuing MMAs; commits) | stager warp 0 (slot wait, fill)")
    total = 0.0
    for kind in names + ("lm_head",):
        a = torch.tensor(rows[kind])
        m = a.mean(0)
        nbytes = phase_bytes(cfg, kind, T, B, experts)
        total += float(a[:, 0].sum())
        if kind == "attn":     # no issuer, no stagers: words 3 and 4 of this phase are the key-loop figures printed below
            m[4:] = 0.0
        print(f"{kind:14s} n={len(rows[kind]):3d} span {m[0] / 1e3:7.2f}  dep {m[1] / 1e3:5.2f}  first-acc {m[2] / 1e3:5.2f}  "
              f"spread {m[3] / 1e3:6.2f}  issuer {m[4] / 1e3:6.2f} {m[5] / 1e3:6.2f} {m[8] / 1e3:6.2f} {m[9] / 1e3:6.2f} {m[10] / 1e3:6.2f}  "
              f"stager {m[6] / 1e3:6.2f} {m[7] / 1e3:6.2f}  "
              f"| {nbytes / 1e6:9.2f} MB -> {nbytes / float(m[0]) :8.1f} GB/s  (phase total {float(a[:, 0].sum()) / 1e3:8.1f} us)")
    print(f"step total {total / 1e3:.1f} us")
    print("# tail of a CTA's last tile part, mean over layers and over the CTAs that have the figure, microseconds: last accumulator"
          " to arrival | part read out of tensor memory | count released or all parts counted | sum read back | tile epilogue")
    for kind in names + ("lm_head",):
        if kind == "attn":
            continue
        phs = [ph for ph in range(nph) if ("lm_head" if ph == ppl * L else names[ph % ppl]) == kind]
        cols = []
        for k in (12, 13, 14, 15):
            x = torch.cat([t[:, ph, k] for ph in phs])
            cols.append(float(x[x > 0].mean()) / ghz / 1e3 if bool((x > 0).any()) else 0.0)
        la = torch.cat([(t[:, ph, 5] - t[:, ph, 11])[t[:, ph, 11] > 0] for ph in phs])
        print(f"{kind:14s} {float(la.mean()) / 1e3:6.2f} | " + " ".join(f"{x:6.2f}" for x in cols))
    k = names.index("attn")
    loop = torch.stack([t[:, l * ppl + k, 3] for l in range(L)]).mean(0) / ghz / 1e3     # us per CTA (warp 0's last item)
    keys = torch.stack([t[:, l * ppl + k, 4] for l in range(L)]).mean(0)
    busy = loop > 0
    if bool(busy.any()):
        print(f"# attention, warp 0 of every CTA with an item: key loop {float(loop[busy].mean()):.2f} us for {float(keys[busy].mean()):.0f} keys "
              f"(max {float(loop[busy].max()):.2f} us); the rest of the phase's span is the dependency, the records, the ticket and the merge")
    if args.detail:
        ph = ppl + names.index(args.detail) if args.detail != "lm_head" else ppl * L
        prev = float(t[:, ph - 1, 5].max())
        print(f"# {args.detail}, phase {ph}: per CTA with work, microseconds after the previous phase's last arrival: dependency |"
              " first accumulator | last accumulator | arrival; then durations of the last tile part: read out of tensor memory |"
              " count released or all parts counted | sum read back | tile epilogue")
        for cta in range(t.shape[0]):
            if float(t[cta, ph, 1]) > 0 or args.detail == "attn":
                v = [float(t[cta, ph, k]) for k in (0, 1, 11, 5)]
                d = [float(t[cta, ph, k]) / ghz / 1e3 for k in (12, 13, 14, 15)]
                print(f"  cta {cta:3d} " + " ".join(f"{(x - prev) / 1e3:8.2f}" if x > 0 else "       -" for x in v) + "   " +
                      " ".join(f"{x:6.2f}" if x > 0 else "     -" for x in d))


if __name__ == "__main__":
    main()
