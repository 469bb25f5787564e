#!/usr/bin/env python
"""Benchmark of the B200 decode megakernel: decode kernel_tok_s at batch 1 on the Llama-3.2-1B shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step (one token through all layers and the LM head) of one sequence.  The
workload is BASELINE configuration 1/2: Llama-3.2-1B architecture, seeded N(0, 0.02) bf16 weights,
batch 1, a seeded 16-token prompt, then K greedy decode steps (K = 1024 walks the KV length from 17
to 1040).  With N > 1 (torchrun) every rank drives its own GPU with a full weight copy and its own
sequence: batch sharding, no data-path collective ("weak" scaling).

Metric definitions follow the reference (qimeng_megakernel/models/LLM/decode.py:755-794):
  value  = kernel_tok_s: tokens / sum of per-step CUDA-event spans around the kernel launch, inputs
           (the fed token) already on the device.
  e2e    = tokens / wall time of the same loop driven with HOST token buffers through the C ABI
           (qmk_generate_host): per step an 8-byte host->device copy of the token, the launch, an
           8-byte device->host copy of the arg-max, one stream synchronisation.
The reference arm (--impl reference) times the reference's CPU route on the host cores: the oracle's
restatement of its fused PyTorch ops (oracle/fused_oracle.py); the reference checkout itself does not
travel to the GPU box.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PROMPT_LEN = 16
WORKLOAD = ("Llama-3.2-1B shape (16 layers, hidden 2048, 32/8 heads x 64, SwiGLU 8192, vocab 128256 tied), bf16, "
            "batch 1, seeded 16-token prompt, greedy decode forced past EOS")


def measured_peak_gbs() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons during the timed region (its output goes to a file and the
    child is killed by PID, so it can never hold the caller's pipes open)."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=self.file, stderr=subprocess.DEVNULL, stdin=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.kill()
        self.proc.wait()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.file.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        self.file.close()
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_reference_run(weights_cpu: dict, config: dict, n_steps: int, warmup: int, budget_s: float = 150.0):
    """The reference's CPU route (oracle port of its fused PyTorch ops) on all host cores.
    Returns (tok_s, steps_timed, cores, sample description)."""
    from oracle import fused_oracle as fo
    torch.set_num_threads(os.cpu_count() or 1)
    cores = torch.get_num_threads()
    keys = ("num_hidden_layers", "hidden_size", "intermediate_size", "head_dim", "num_attention_heads",
            "num_key_value_heads", "vocab_size", "rms_norm_eps")
    cfg = fo.OracleConfig(**{k: config[k] for k in keys})
    st = fo.make_state(cfg, weights_cpu, PROMPT_LEN + warmup + n_steps + 1, torch.bfloat16)
    from qimeng_megakernel_b200 import synthetic
    tok = int(synthetic.make_prompt(config["vocab_size"], 1, seed=1)[0])
    pos = 0
    t_w = time.perf_counter()
    for _ in range(max(1, warmup)):
        tok = fo.feed_token(st, tok, pos); pos += 1
    per_step = (time.perf_counter() - t_w) / max(1, warmup)
    steps = max(1, min(n_steps, int(budget_s / max(per_step, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = fo.feed_token(st, tok, pos); pos += 1
    dt = time.perf_counter() - t0
    sample = (f"{steps} greedy decode steps of the full workload model at KV lengths {pos - steps + 1}..{pos} "
              f"(bf16, oracle port of the reference's fused PyTorch route, {cores} threads)")
    return steps / dt, steps, cores, sample, dt / steps


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1024)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg (rank 0, N = 1 only)")
    ap.add_argument("--batch", type=int, default=1, help="sequences per GPU (> 1, or any --model but llama: the batched kernel)")
    ap.add_argument("--model", default="llama-3.2-1b", choices=["llama-3.2-1b", "qwen3-0.6b", "olmoe-1b-7b"])
    ap.add_argument("--kernel", default="auto", choices=["auto", "batched"], help="batched: the batched kernel also at batch 1")
    ap.add_argument("--layers", type=int, default=0,
                    help="batched runs only: keep this many decoder layers (a small case for a profiler capture; the line says so)")
    args = ap.parse_args()
    K, W = args.steps, max(3, args.warmup)
    if args.batch != 1 or args.model != "llama-3.2-1b" or args.kernel == "batched":
        if args.impl == "reference":
            raise SystemExit("--impl reference times the headline workload (batch 1, Llama-3.2-1B shape) only")
        return main_batched(args, K, W)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    from qimeng_megakernel_b200 import synthetic
    from qimeng_megakernel_b200.model_config import LLAMA_3_2_1B
    config = dict(LLAMA_3_2_1B)
    kv_len = PROMPT_LEN + W + K + 1
    metric = "decode kernel_tok_s at batch 1 (Llama-1B shape)"

    # ------------------------------------------------------------------ reference arm: CPU route
    if args.impl == "reference":
        if rank != 0:
            return
        weights = synthetic.make_weights(config, seed=0, device="cpu", max_positions=max(2048, kv_len))
        tok_s, steps, cores, sample, sec = cpu_reference_run(weights, config, K, min(W, 3))
        line = {"impl": "reference", "metric": metric, "value": tok_s, "unit": "tokens/s", "n_gpus": args.gpus,
                "steps": steps, "warmup": min(W, 3), "ms_per_step": sec * 1e3, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": WORKLOAD, "decode_steps": steps, "note": "CPU route, bounded sample of the workload"},
                "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
                "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line), flush=True)
        return

    # ------------------------------------------------------------------ our arm: the CUDA megakernel
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    from qimeng_megakernel_b200 import mk_kernel

    weights = synthetic.make_weights(config, seed=0, device=dev, max_positions=max(2048, kv_len))
    g = synthetic.make_globals(config, weights, kv_seq_len=kv_len, device=dev)
    mk = mk_kernel.get_mk()
    prompt = synthetic.make_prompt(config["vocab_size"], PROMPT_LEN, seed=1 + rank)
    stream = torch.cuda.current_stream(dev).cuda_stream

    # prompt: fed through the decode kernel one token at a time (fills the KV cache), host token buffers
    host = torch.zeros(PROMPT_LEN + W + K + 1, dtype=torch.int64).pin_memory()
    host[:PROMPT_LEN] = prompt
    scratch = torch.zeros(PROMPT_LEN, dtype=torch.int64).pin_memory()
    mk.generate_host(g, host, 0, PROMPT_LEN - 1, teacher_forced=True, host_argmax=scratch)
    # device-resident greedy loop: the kernel embeds the token and feeds its arg-max back
    g.token_in = torch.zeros(1, dtype=torch.int64, device=dev)
    g.next_token = g.token_in
    g.token_in.copy_(host[PROMPT_LEN - 1:PROMPT_LEN].to(dev))
    pos = PROMPT_LEN - 1
    g.position_id = pos
    mk(g)                       # binds the state; first generated token
    pos += 1
    kv_snapshot = None
    for _ in range(W):          # warm-up steps
        mk._lib.qmk_decode_step(mk._handle, pos, stream); pos += 1
    torch.cuda.synchronize(dev)
    mk.check_status()
    first_timed_pos = pos
    launches0 = mk.launch_count

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- timed region 1: kernel_tok_s (inputs resident on the device)
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    sampler = ClockSampler(local_rank) if rank == 0 else None
    barrier()
    t_wall0 = time.perf_counter()
    for i in range(K):
        events[i][0].record()
        rc = mk._lib.qmk_decode_step(mk._handle, pos, stream)
        events[i][1].record()
        if rc != 0:
            raise SystemExit(f"qmk_decode_step failed: {rc}")
        pos += 1
    barrier()
    wall = time.perf_counter() - t_wall0
    clocks = sampler.stop() if sampler else None
    mk.check_status()
    kernel_s = sum(a.elapsed_time(b) for a, b in events) / 1e3
    launches = mk.launch_count - launches0
    step_bytes = sum(mk.step_bytes(first_timed_pos + i) for i in range(K)) / K
    last_token = int(g.next_token.item())

    # ---- timed region 2: end to end through the C ABI with host token buffers
    # restart from the same position so that both regions cover the same KV lengths
    host[first_timed_pos] = int(prompt[0])      # any valid token: throughput does not depend on its value
    barrier()
    t0 = time.perf_counter()
    mk.generate_host(g, host, first_timed_pos, K)
    torch.cuda.synchronize(dev)
    e2e_s = time.perf_counter() - t0
    barrier()
    mk.check_status()

    times = torch.tensor([kernel_s, wall, e2e_s], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    kernel_s, wall, e2e_s = (float(x) for x in times.tolist())

    if rank == 0:
        peak, peak_src = measured_peak_gbs()
        achieved = step_bytes / (kernel_s / K) / 1e9
        line = {
            "metric": metric, "value": world * K / kernel_s, "unit": "tokens/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": kernel_s / K * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "decode_steps": K, "kv_lengths": [first_timed_pos + 1, first_timed_pos + K],
                       "sequences_per_gpu": 1, "sharding": "one independent sequence per GPU, no collective",
                       "l2": "inputs larger than L2: every step streams 2.47 GB of weights through a 126 MB L2",
                       "tok_s_gpu_loop": world * K / wall},
            "e2e": {"value": world * K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8},
            "gpu_launches": launches + K,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": TRAFFIC_BYTES_PER_LAUNCH, "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": step_bytes,
                         "kernel": "qmk_decode_kernel (one persistent launch per decode step)"},
            "clocks": clocks,
            "last_token": last_token,
        }
        if world == 1 and not args.no_cpu_baseline:
            wcpu = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in weights.items()}
            tok_s, steps, cores, sample, _ = cpu_reference_run(wcpu, config, 8, 2, budget_s=25.0)
            line["cpu_baseline"] = {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main_batched(args, K: int, W: int) -> None:
    """BASELINE configurations 3 and 4: B independent seeded sequences per GPU (batch-sharded over the ranks, no
    collective), every step one launch of the batched kernel; the device feeds each row's arg-max back as its next
    token.  Same timing rules as the headline run; not the line the driver records."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    from qimeng_megakernel_b200 import mk_kernel, synthetic
    from qimeng_megakernel_b200.model_config import LLAMA_3_2_1B, OLMOE_1B_7B, QWEN3_0_6B
    config = dict({"llama-3.2-1b": LLAMA_3_2_1B, "qwen3-0.6b": QWEN3_0_6B, "olmoe-1b-7b": OLMOE_1B_7B}[args.model])
    if args.layers > 0:
        config["num_hidden_layers"] = min(args.layers, config["num_hidden_layers"])
    B = args.batch
    kv_len = PROMPT_LEN + W + K + 1
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    weights = synthetic.make_weights(config, seed=0, device=dev, max_positions=max(2048, kv_len))
    g = synthetic.make_globals(config, weights, kv_seq_len=kv_len, device=dev, batch=B)
    mk = mk_kernel.get_mk()
    mk.set_kernel_variant(1)
    prompts = synthetic.make_prompts(config["vocab_size"], B, PROMPT_LEN, seed=1 + rank * B).to(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    g.token_in = torch.zeros(B, dtype=torch.int64, device=dev)
    g.next_token = torch.zeros(B, dtype=torch.int64, device=dev)
    for pos in range(PROMPT_LEN):           # the prompts, one position per launch (fills the KV cache)
        g.token_in.copy_(prompts[:, pos]); g.position_id = pos
        mk(g)
    g.next_token = g.token_in               # from here on the kernel feeds its arg-max back
    g.position_id = PROMPT_LEN
    g.token_in.copy_(prompts[:, 0])
    mk(g)
    pos = PROMPT_LEN + 1
    for _ in range(W):
        mk._lib.qmk_decode_step(mk._handle, pos, stream); pos += 1
    torch.cuda.synchronize(dev)
    mk.check_status()
    first_timed_pos = pos
    launches0 = mk.launch_count

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    sampler = ClockSampler(local_rank) if rank == 0 else None
    barrier()
    for i in range(K):
        events[i][0].record()
        rc = mk._lib.qmk_decode_step(mk._handle, pos, stream)
        events[i][1].record()
        if rc != 0:
            raise SystemExit(f"qmk_decode_step failed: {rc}")
        pos += 1
    barrier()
    clocks = sampler.stop() if sampler else None
    mk.check_status()
    kernel_s = sum(a.elapsed_time(b) for a, b in events) / 1e3
    launches = mk.launch_count - launches0
    step_bytes = sum(mk.step_bytes(first_timed_pos + i) for i in range(K)) / K

    # end to end with host token buffers: per step B tokens host -> device, the launch, B arg-max values device -> host
    host_in = prompts[:, :1].cpu().repeat(1, K + 1).t().contiguous().pin_memory()      # [K + 1, B]
    host_out = torch.zeros(K, B, dtype=torch.int64).pin_memory()
    tok_dev = torch.zeros(B, dtype=torch.int64, device=dev)
    out_dev = torch.zeros(B, dtype=torch.int64, device=dev)
    g.token_in, g.next_token = tok_dev, out_dev
    g.position_id = first_timed_pos
    mk(g)                                   # re-binds the state (untimed)
    pos = first_timed_pos
    barrier()
    t0 = time.perf_counter()
    for i in range(K):
        tok_dev.copy_(host_in[i], non_blocking=True)
        rc = mk._lib.qmk_decode_step(mk._handle, pos, stream)
        host_out[i].copy_(out_dev, non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()
        host_in[i + 1].copy_(host_out[i])
        pos += 1
    e2e_s = time.perf_counter() - t0
    barrier()
    mk.check_status()
    times = torch.tensor([kernel_s, e2e_s], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    kernel_s, e2e_s = (float(x) for x in times.tolist())
    if rank == 0:
        peak, peak_src = measured_peak_gbs()
        achieved = step_bytes / (kernel_s / K) / 1e9
        ctas, threads, smem = mk.geometry()
        line = {
            "metric": f"decode kernel_tok_s at batch {B} per GPU ({args.model} shape)", "value": world * B * K / kernel_s,
            "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": kernel_s / K * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{args.model} shape, bf16, {B} independent seeded 16-token prompts per GPU, greedy decode "
                                   "forced past EOS", "decode_steps": K,
                       "kv_lengths": [first_timed_pos + 1, first_timed_pos + K], "sequences_per_gpu": B,
                       "decoder_layers": config["num_hidden_layers"],
                       "sharding": "sequences sharded over the GPUs, full weight copy each, no collective",
                       "l2": "inputs larger than L2: every step streams the weights through a 126 MB L2",
                       "launch": {"ctas": ctas, "threads": threads, "smem_bytes": smem}},
            "e2e": {"value": world * B * K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 8 * B, "d2h_bytes_per_step": 8 * B},
            "gpu_launches": launches + K,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": peak_src, "algorithmic_bytes_per_launch": step_bytes,
                         "kernel": "qmk_batch_kernel (one persistent launch per decode step)"},
            "clocks": clocks, "cpu_baseline": None,
        }
        if config.get("num_experts"):
            line["config"]["experts_touched_last_layer_last_step"] = mk.last_expert_count()
            line["config"]["bytes_note"] = ("algorithmic bytes count min(E, B * k) experts per layer (upper bound of the "
                                            "distinct experts a step reads)")
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one full-size launch (KV length 36), from the ncu capture
# summarised in profiles/qmk_decode_kernel_step_llama1b.md.
TRAFFIC_BYTES_PER_LAUNCH = 2.4787e9

if __name__ == "__main__":
    main()
