"""Fixed-length decode matrix for the B200 route: `python -m qimeng_megakernel_b200.llm_decode_bench`.

The counterpart of the reference's `python -m benchmarks.llm_decode --hardware ...`
(benchmarks/llm_decode.py:33-60 arguments, 76-165 one run, 168-305 matrix and JSON): same matrix
(batch sizes x output lengths, warm-up + measured iterations, continuation forced past EOS), same per-run
and per-cell keys (tok_s, tok_s_gpu, kernel_tok_s, ..., validation.length_complete / greedy_rerun_match).
Differences: there is no checkpoint or tokenizer offline, so the model is the seeded synthetic
Llama-3.2-1B (or Qwen3-0.6B) shape and the prompts are 16 seeded token ids per row (batch sizes up to 64); text quality checks (gibberish / repetition) do not
apply to token ids and are left out; weights are generated once, not re-read from disk every iteration
(llm_decode.py:99-104 does); each cell also reports the HBM roofline fraction.
"""
from __future__ import annotations

import argparse
import json
import time
from pathlib import Path
from statistics import fmean

import torch

from . import mk_kernel, synthetic
from .decode import decode as llm_decode
from .model_config import LLAMA_3_2_1B, QWEN3_0_6B
from .prefill import run_prefill_synthetic

HBM_PEAK_GBS = 8000.0      # the "~8 TB/s" of the target specification; the measured copy bandwidth is lower


def _parse_args() -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Benchmark the B200 decode megakernel over a batch/output matrix")
    p.add_argument("--model", default="llama-3.2-1b")
    p.add_argument("--prompt-len", type=int, default=16)
    p.add_argument("--prompt-seed", type=int, default=1)
    p.add_argument("--batch-sizes", default="1")
    p.add_argument("--output-lengths", default="128,256,512,1024")
    p.add_argument("--out", default=None)
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--hardware", default="B200")
    p.add_argument("--warmup-iters", type=int, default=2)
    p.add_argument("--bench-iters", type=int, default=5)
    p.add_argument("--host-loop", action="store_true", help="use the reference's host token loop instead of the device loop")
    p.add_argument("--peak-gbs", type=float, default=HBM_PEAK_GBS)
    return p.parse_args()


def _run_once(args, cfg, weights, mk, prompt, batch_size: int, output_len: int) -> dict:
    prompts = prompt.view(1, -1) if batch_size == 1 else synthetic.make_prompts(
        cfg["vocab_size"], batch_size, args.prompt_len, args.prompt_seed)   # row 0 is the single-sequence prompt
    prefill = run_prefill_synthetic(cfg, weights, prompts, output_len, device=args.device, mk=mk)
    wall_t0 = time.perf_counter()
    out = llm_decode(args.model, prefill=prefill, max_new_tokens=output_len, decode_route="mk",
                     hardware=args.hardware, decode_time=True, ignore_eos=True, host_loop=args.host_loop)
    elapsed = time.perf_counter() - wall_t0
    per_row = [int(x) for x in out["per_row_new_tokens"].tolist()]
    t = out["timing"] or {}
    return {
        "backend": "mk", "batch_size": batch_size, "max_new_tokens": output_len,
        "decode_time_s": float(t.get("decode_wall_s", elapsed)), "decode_gpu_s": float(t.get("decode_gpu_s", 0.0)),
        "effective_new_tokens": int(sum(per_row)),
        "tok_s": float(t.get("effective_tok_s_wall", 0.0)), "tok_s_gpu": float(t.get("effective_tok_s_gpu", 0.0)),
        "kernel_tok_s": float(t.get("kernel_tok_s", 0.0)), "mk_kernel_gpu_s": float(t.get("mk_kernel_gpu_s", 0.0)),
        "non_kernel_gpu_s": float(t.get("non_kernel_gpu_s", 0.0)), "non_kernel_wall_s": float(t.get("non_kernel_wall_s", 0.0)),
        "instruction_setup_wall_s": float(t.get("instruction_setup_wall_s", 0.0)),
        "queue_build_wall_s": 0.0, "tensorize_wall_s": 0.0, "clock_domain": "wall", "per_row_new_tokens": per_row,
        "achieved_hbm_gbs": float(t.get("achieved_hbm_gbs", 0.0)), "hbm_bytes_per_step": float(t.get("hbm_bytes_per_step", 0.0)),
        "new_token_ids": [[int(x) for x in row.tolist()] for row in out["new_tokens"].cpu()],
    }


def main() -> int:
    args = _parse_args()
    batch_sizes = [int(x) for x in args.batch_sizes.split(",") if x.strip()]
    output_lengths = [int(x) for x in args.output_lengths.split(",") if x.strip()]
    cfg = dict(QWEN3_0_6B if "qwen3" in args.model.lower() else LLAMA_3_2_1B)
    weights = synthetic.make_weights(cfg, seed=0, device=args.device, max_positions=max(2048, args.prompt_len + max(output_lengths) + 1))
    mk = mk_kernel.get_mk()
    prompt = synthetic.make_prompt(cfg["vocab_size"], args.prompt_len, args.prompt_seed)
    results = {}
    for batch_size in batch_sizes:
        for output_len in output_lengths:
            for _ in range(args.warmup_iters):
                _run_once(args, cfg, weights, mk, prompt, batch_size, output_len)
            samples = [_run_once(args, cfg, weights, mk, prompt, batch_size, output_len) for _ in range(args.bench_iters)]
            ids = [s["new_token_ids"] for s in samples]
            length_complete = all(s["per_row_new_tokens"] == [output_len] * batch_size for s in samples)
            mean_gbs = fmean(s["achieved_hbm_gbs"] for s in samples)
            results[f"b{batch_size}_t{output_len}"] = {
                "backend": "mk", "batch_size": batch_size, "max_new_tokens": output_len,
                "eos_policy": "forced_continuation",
                "tok_s": fmean(s["tok_s"] for s in samples), "tok_s_gpu": fmean(s["tok_s_gpu"] for s in samples),
                "kernel_tok_s": fmean(s["kernel_tok_s"] for s in samples),
                "achieved_hbm_gbs": mean_gbs, "hbm_roofline_fraction": mean_gbs / args.peak_gbs,
                "new_token_ids": ids[0],
                "validation": {"length_complete": length_complete, "greedy_rerun_match": all(x == ids[0] for x in ids[1:]),
                               "pass": length_complete},
                "samples": [{k: v for k, v in s.items() if k != "new_token_ids"} for s in samples],
            }
            r = results[f"b{batch_size}_t{output_len}"]
            print(f"backend=mk batch={batch_size} max_new_tokens={output_len} tok_s={r['tok_s']:.2f} "
                  f"tok_s_gpu={r['tok_s_gpu']:.2f} kernel_tok_s={r['kernel_tok_s']:.2f} hbm={mean_gbs:.0f} GB/s")
    out = {"backend": "mk", "model_path": f"synthetic:{args.model}", "prompt_token_count": args.prompt_len,
           "prompt_mode": "token ids", "eos_policy": "forced_continuation", "decode_strategy": "greedy",
           "hardware": args.hardware, "torch_dtype": "bfloat16", "batch_sizes": batch_sizes,
           "output_lengths": output_lengths, "warmup_iters": args.warmup_iters, "bench_iters": args.bench_iters,
           "hbm_peak_gbs": args.peak_gbs, "results": results}
    if args.out:
        path = Path(args.out).expanduser().resolve()
        path.parent.mkdir(parents=True, exist_ok=True)
        path.write_text(json.dumps(out, indent=2), encoding="utf-8")
        print(f"saved_results={path}")
    else:
        print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
