"""Runs every phase of one decode step as its own launch and reports time and achieved HBM GB/s per phase.

    python -m qimeng_megakernel_b200.profile_phases [--pos 500] [--reps 20]
    python -m qimeng_megakernel_b200.profile_phases --one-each     # six launches, one per phase kind: for a profiler

The persistent kernel normally runs all phases in one launch; `qmk_run_phases(mode 0)` launches the same
device code one phase at a time (stream-ordered, no cross-SM waits), which is what `ncu` needs to attribute
DRAM traffic to a phase.  Weights are the seeded synthetic Llama-3.2-1B model (2.5 GB on the device).
The counterpart in the reference is its per-op verifier launch (decode_schedule/mk_kernel.py:97-111).
"""
from __future__ import annotations

import argparse

import torch

from . import mk_kernel, synthetic
from .model_config import LLAMA_3_2_1B

NAMES = ("qkv", "attn", "oproj", "upgate", "down")


def phase_bytes(cfg: dict, kind: str, pos: int) -> int:
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    NH, NKV, HD, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["vocab_size"]
    return {"qkv": 2 * (NH + 2 * NKV) * HD * H, "attn": 2 * 2 * NKV * HD * (pos + 1), "oproj": 2 * H * NH * HD,
            "upgate": 2 * 2 * I * H, "down": 2 * H * I, "lm_head": 2 * V * H}[kind]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--pos", type=int, default=500)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--warm-steps", type=int, default=2, help="full persistent steps before the phase launches")
    ap.add_argument("--one-each", action="store_true",
                    help="launch the five phases of layer 1 and the LM head once each, in order, and stop (launches 4..9 of "
                         "the process with the default two warm steps and the binding launch)")
    args = ap.parse_args()
    cfg = dict(LLAMA_3_2_1B)
    w = synthetic.make_weights(cfg, seed=0, device="cuda", max_positions=max(2048, args.pos + 8))
    g = synthetic.make_globals(cfg, w, kv_seq_len=args.pos + 8, device="cuda")
    mk = mk_kernel.get_mk()
    g.token_in = torch.zeros(1, dtype=torch.int64, device="cuda")
    g.next_token = g.token_in
    for pos in range(args.warm_steps):
        g.position_id = pos
        mk(g)
    g.position_id = args.pos
    L = cfg["num_hidden_layers"]
    # One event pair around the same phase kind of ALL layers, queued back to back: each layer has its
    # own weights (16 x 12.6 MB for the smallest phase), so no launch finds its weights in the 126 MB L2,
    # and the host's launch latency is hidden behind the queue.
    mk.run_phases(g, 0, 1, 0)            # binds the state
    if args.one_each:
        for ph in [5 + k for k in range(5)] + [5 * L]:
            mk.run_phases(g, ph, ph + 1, 0)
        torch.cuda.synchronize()
        mk.check_status()
        print("one launch per phase kind done")
        return
    for k, name in enumerate(NAMES + ("lm_head",)):
        phs = [5 * L] * 4 if name == "lm_head" else [l * 5 + k for l in range(L)]
        times = []
        for _ in range(args.reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for ph in phs:
                mk.run_phases_bound(args.pos, ph, ph + 1, 0)
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3 / len(phs))
        times.sort()
        med = times[len(times) // 2]
        nbytes = phase_bytes(cfg, name, args.pos)
        print(f"phase {name:8s}: median {med:8.2f} us per stand-alone launch (launch overhead included), "
              f"{nbytes / 1e6:9.3f} MB algorithmic, {nbytes / med / 1e3:8.1f} GB/s")
    mk.check_status()


if __name__ == "__main__":
    main()
