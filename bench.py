#!/usr/bin/env python
"""Benchmark of the B200 decode megakernel: decode kernel_tok_s at batch 1 on the Llama-3.2-1B shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --model {llama-3.2-1b,qwen3-0.6b,olmoe-1b-7b} --batch B [--kernel batched] [--layers n]

A step is one decode step (one token through all layers and the LM head) of every sequence a GPU holds.  The headline
workload: Llama-3.2-1B architecture, seeded N(0, 0.02) bf16 weights, batch 1, a seeded 16-token prompt, then K greedy
decode steps (K = 1024 walks the KV length from about 17 to 1040).  With N > 1 (torchrun) every rank drives its own GPU
with a full weight copy and its own sequences: batch sharding, no data-path collective ("weak" scaling).

Metric definitions follow the reference (qimeng_megakernel/models/LLM/decode.py:755-794; one run of
benchmarks/llm_decode.py:76-165):
  value  = kernel_tok_s: tokens / sum of per-step CUDA-event spans around the kernel launch, inputs (the fed token)
           already on the device.
  e2e    = tokens / wall time of the same loop driven with HOST token buffers through the C ABI: per step a
           host->device copy of the fed tokens (8 bytes per sequence), the launch, a device->host copy of the arg-max,
           one stream synchronisation.
The default line also carries `secondary`: short runs of the batched kernel on the other workload shapes (Llama shape
at 32 sequences, Qwen3-0.6B shape at 16, OLMoE-1B-7B shape at 32), each with its own ms_per_step, roofline and clocks.
The reference arm (--impl reference) times the reference's CPU route on the host cores: the oracle's restatement of its
fused PyTorch ops (oracle/fused_oracle.py); the reference checkout itself does not travel to the GPU box.
"""
from __future__ import annotations

import argparse
import gc
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
METRIC = "decode kernel_tok_s at batch 1 (Llama-1B shape)"
# dram__bytes_read.sum + dram__bytes_write.sum of one full-size launch of qmk_decode_kernel (KV length 36), from the ncu
# capture summarised in profiles/qmk_decode_kernel_step_llama1b.md.
TRAFFIC_BYTES_PER_LAUNCH = 2.4791e9   # dram__bytes_read + write of one decode step (profiles/qmk_decode_kernel_step_llama1b.md)


def measured_peak_gbs() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons (query only), every 20 ms, started BEFORE the warm-up steps so that even a
    timed region of a few milliseconds has samples under load.  Output goes to a file and the child is killed by PID."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=self.file, stderr=subprocess.DEVNULL, stdin=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        self.t0 = time.perf_counter()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        if time.perf_counter() - self.t0 < 0.25:      # the tool needs a moment before its first line
            time.sleep(0.25 - (time.perf_counter() - self.t0))
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
        if len(sm) < 3:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": len(sm), "reasons": ["clocks: unavailable (too few samples)"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "samples": len(sm), "reasons": sorted(reasons),
                "window": "warm-up and timed steps"}


def pin_host_thread(local_rank: int, world: int) -> list[int] | None:
    """One block of host cores per rank: with N processes on one box the per-token host work (a launch and a stream
    synchronisation) otherwise migrates between cores and the slowest rank sets the end-to-end figure."""
    try:
        cores = sorted(os.sched_getaffinity(0))
        per = len(cores) // max(world, 1)
        if world > 1 and per >= 1:
            mine = cores[local_rank * per:(local_rank + 1) * per]
            os.sched_setaffinity(0, set(mine))
            return mine
    except (AttributeError, OSError):
        pass
    return None


# ----------------------------------------------------------------------------------------------------------------
# reference arm: the reference's CPU route
# ----------------------------------------------------------------------------------------------------------------
def cpu_reference_run(weights_cpu: dict, config: dict, n_steps: int, warmup: int, budget_s: float = 150.0):
    """The reference's CPU route (oracle port of its fused PyTorch ops) on all host cores, driven like the GPU arm: the
    16-token prompt is fed first (its last token yields the first generated one), then `warmup` untimed greedy steps,
    then up to n_steps timed greedy steps (fewer when the time budget says so).  Returns (tok_s, steps_timed, cores, sample text, s/step, first KV, last KV)."""
    from oracle import fused_oracle as fo
    from qimeng_megakernel_b200 import synthetic
    torch.set_num_threads(os.cpu_count() or 1)
    cores = torch.get_num_threads()
    keys = ("num_hidden_layers", "hidden_size", "intermediate_size", "head_dim", "num_attention_heads",
            "num_key_value_heads", "vocab_size", "rms_norm_eps")
    cfg = fo.OracleConfig(**{k: config[k] for k in keys})
    st = fo.make_state(cfg, weights_cpu, PROMPT_LEN + warmup + n_steps + 2, torch.bfloat16)
    prompt = synthetic.make_prompt(config["vocab_size"], PROMPT_LEN, seed=1).tolist()
    t_w = time.perf_counter()
    tok, pos = prompt[0], 0
    for pos in range(PROMPT_LEN):                       # teacher-forced prompt
        tok = fo.feed_token(st, prompt[pos], pos)
    pos = PROMPT_LEN
    for _ in range(warmup):                             # warm-up, greedy
        tok = fo.feed_token(st, tok, pos); pos += 1
    per_step = (time.perf_counter() - t_w) / (PROMPT_LEN + warmup)
    steps = max(1, min(n_steps, int(budget_s / max(per_step, 1e-3))))
    first_pos = pos
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = fo.feed_token(st, tok, pos); pos += 1
    dt = time.perf_counter() - t0
    sample = (f"{steps} greedy decode steps of the full workload model at KV lengths {first_pos + 1}..{pos} after the "
              f"16-token prompt and {warmup} untimed steps (bf16, oracle port of the reference's fused PyTorch "
              f"route, {cores} threads)")
    return steps / dt, steps, cores, sample, dt / steps, first_pos + 1, pos


def headline_config(K: int, first_kv: int, last_kv: int) -> dict:
    return {"workload": WORKLOAD, "decode_steps": K, "kv_lengths": [first_kv, last_kv], "sequences_per_gpu": 1,
            "sharding": "one independent sequence per GPU, no collective",
            "l2": "inputs larger than L2: every step streams 2.47 GB of weights through a 126 MB L2"}


def run_reference_arm(args, K: int, W: int) -> None:
    from qimeng_megakernel_b200 import synthetic
    from qimeng_megakernel_b200.model_config import LLAMA_3_2_1B
    if int(os.environ.get("RANK", "0")) != 0:
        return
    config = dict(LLAMA_3_2_1B)
    weights = synthetic.make_weights(config, seed=0, device="cpu", max_positions=2048)
    tok_s, steps, cores, sample, sec, kv0, kv1 = cpu_reference_run(weights, config, K, W)
    cfg = headline_config(steps, kv0, kv1)
    note = ("CPU route on the host cores; one sequence on one host whatever --gpus says" +
            (f"; {steps} of the {K} requested steps timed (time budget)" if steps < K else ""))
    line = {"impl": "reference", "note": note, "metric": METRIC, "value": tok_s, "unit": "tokens/s", "n_gpus": 1,
            "steps": steps, "warmup": W, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------------------------------------
class Dist:
    def __init__(self, dev):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.dev = dev
        if self.world > 1:
            import torch.distributed as dist
            self.dist = dist
            if not dist.is_initialized():
                dist.init_process_group("nccl", device_id=dev)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize(self.dev)

    def max_over_ranks(self, values: list[float]) -> list[float]:
        t = torch.tensor(values, dtype=torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t.tolist()]

    def sum_over_ranks(self, values: list[float]) -> list[float]:
        t = torch.tensor(values, dtype=torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return [float(x) for x in t.tolist()]


def timed_steps(mk, K: int, pos: int, D: Dist):
    """K decode steps from position `pos`, each bracketed by CUDA events on the launching stream; barrier and
    synchronise on both sides.  Returns (sum of event spans in seconds, wall seconds, next position)."""
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    D.barrier()
    t0 = time.perf_counter()
    for i in range(K):
        events[i][0].record()
        mk.decode_step(pos)
        events[i][1].record()
        pos += 1
    D.barrier()
    wall = time.perf_counter() - t0
    return sum(a.elapsed_time(b) for a, b in events) / 1e3, wall, pos


def timed_multi_step(mk, g, K: int, pos: int, per_launch: int, D: Dist):
    """The same K steps as persistent launches of `per_launch` steps each (the last one takes the rest): events around
    every launch.  Returns (sum of event spans in seconds, wall seconds, next position, launches)."""
    chunks = [per_launch] * (K // per_launch) + ([K % per_launch] if K % per_launch else [])
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in chunks]
    D.barrier()
    t0 = time.perf_counter()
    for ev, n in zip(events, chunks):
        ev[0].record()
        mk.generate_device(g, pos, n)
        ev[1].record()
        pos += n
    D.barrier()
    wall = time.perf_counter() - t0
    return sum(a.elapsed_time(b) for a, b in events) / 1e3, wall, pos, len(chunks)


def run_batch1(args, K: int, W: int, D: Dist, local_rank: int) -> dict | None:
    from qimeng_megakernel_b200 import mk_kernel, synthetic
    from qimeng_megakernel_b200.model_config import LLAMA_3_2_1B
    dev = D.dev
    config = dict(LLAMA_3_2_1B)
    kv_len = PROMPT_LEN + W + K + 2
    weights = synthetic.make_weights(config, seed=0, device=dev, max_positions=max(2048, kv_len))
    g = synthetic.make_globals(config, weights, kv_seq_len=kv_len, device=dev)
    mk = mk_kernel.get_mk()
    prompt = synthetic.make_prompt(config["vocab_size"], PROMPT_LEN, seed=1 + D.rank)

    # prompt: fed through the decode kernel one token at a time (fills the KV cache), host token buffers
    host = torch.zeros(PROMPT_LEN + W + K + 2, dtype=torch.int64).pin_memory()
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
    sampler = ClockSampler(local_rank) if D.rank == 0 else None
    for _ in range(W):          # warm-up steps
        mk.decode_step(pos); pos += 1
    torch.cuda.synchronize(dev)
    mk.check_status()
    first_timed_pos = pos
    launches0 = mk.launch_count

    # ---- timed region 1: kernel_tok_s (inputs resident on the device)
    S = max(1, int(args.steps_per_launch))
    if S > 1:
        kernel_s, wall, pos, _ = timed_multi_step(mk, g, K, pos, S, D)
    else:
        kernel_s, wall, pos = timed_steps(mk, K, pos, D)
    clocks = sampler.stop() if sampler else None
    mk.check_status()
    launches = mk.launch_count - launches0
    step_bytes = sum(mk.step_bytes(first_timed_pos + i) for i in range(K)) / K
    last_token = int(g.next_token.item())

    # ---- timed region 2: end to end through the C ABI with host token buffers, over the same KV lengths
    host[first_timed_pos] = int(prompt[0])      # any valid token: throughput does not depend on its value
    D.barrier()
    t0 = time.perf_counter()
    mk.generate_host(g, host, first_timed_pos, K)
    torch.cuda.synchronize(dev)
    e2e_s = time.perf_counter() - t0
    D.barrier()
    mk.check_status()
    launches_e2e = mk.launch_count - launches0 - launches
    kernel_s, wall, e2e_s = D.max_over_ranks([kernel_s, wall, e2e_s])
    mk.close()
    line = None
    if D.rank == 0:
        world = D.world
        peak, peak_src = measured_peak_gbs()
        achieved = step_bytes / (kernel_s / K) / 1e9
        cfg = headline_config(K, first_timed_pos + 1, first_timed_pos + K)
        line = {
            "tok_s_gpu_loop": world * K / wall,
            "metric": METRIC, "value": world * K / kernel_s, "unit": "tokens/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": kernel_s / K * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg,
            "e2e": {"value": world * K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8},
            "gpu_launches": launches + launches_e2e,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": TRAFFIC_BYTES_PER_LAUNCH * min(S, K), "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": step_bytes * min(S, K),
                         "kernel": "qmk_decode_kernel (one persistent launch per decode step)" if S == 1 else
                                   f"qmk_decode_kernel (one persistent launch per {min(S, K)} decode steps)"},
            "clocks": clocks,
            "last_token": last_token,
        }
        if world == 1 and not args.no_cpu_baseline:
            wcpu = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in weights.items()}
            tok_s, steps, cores, sample, _, _, _ = cpu_reference_run(wcpu, config, 8, 1, budget_s=20.0)
            line["cpu_baseline"] = {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
        else:
            line["cpu_baseline"] = None
    del g, weights
    gc.collect()
    torch.cuda.empty_cache()
    return line


def run_batched(model: str, B: int, K: int, W: int, layers: int, D: Dist, local_rank: int, ep: int = 1, tp: int = 1) -> dict | None:
    """B independent seeded sequences per GPU (batch-sharded over the ranks, no collective), every step one launch of
    the batched kernel; the device feeds each row's arg-max back as its next token.  Same timing rules as the headline.
    ep > 1 (mixture-of-experts shapes, one rank per GPU, world == ep): every rank decodes the SAME B sequences and holds
    E / ep experts; the partial expert outputs cross NVLink inside the kernel.  Total work is fixed: strong scaling.
    tp > 1 (dense shapes, world == tp): the same, with every projection cut over the ranks (tensor parallelism)."""
    from qimeng_megakernel_b200 import expert_parallel, mk_kernel, synthetic, tensor_parallel
    from qimeng_megakernel_b200.model_config import LLAMA_3_2_1B, OLMOE_1B_7B, QWEN3_0_6B
    dev = D.dev
    config = dict({"llama-3.2-1b": LLAMA_3_2_1B, "qwen3-0.6b": QWEN3_0_6B, "olmoe-1b-7b": OLMOE_1B_7B}[model])
    if layers > 0:
        config["num_hidden_layers"] = min(layers, config["num_hidden_layers"])
    kv_len = PROMPT_LEN + W + K + 2
    weights = synthetic.make_weights(config, seed=0, device=dev, max_positions=max(2048, kv_len))
    if ep > 1:
        if D.world != ep or not config.get("num_experts"):
            raise SystemExit("--ep N needs a mixture-of-experts --model and exactly N ranks (torchrun --nproc-per-node N)")
        weights = expert_parallel.shard_moe_weights(weights, D.rank, ep)      # the full copies are dropped here
        config = expert_parallel.shard_config(config, D.rank, ep)
        torch.cuda.empty_cache()
    full_vocab = config["vocab_size"]
    if tp > 1:
        if D.world != tp or config.get("num_experts"):
            raise SystemExit("--tp N needs a dense --model and exactly N ranks (torchrun --nproc-per-node N)")
        weights = tensor_parallel.shard_weights(config, weights, D.rank, tp)
        config = tensor_parallel.shard_config(config, D.rank, tp)
        torch.cuda.empty_cache()
    g = synthetic.make_globals(config, weights, kv_seq_len=kv_len, device=dev, batch=B)
    mk = mk_kernel.get_mk()
    mk.set_kernel_variant(1)
    if ep > 1 or tp > 1:
        expert_parallel.connect(mk, g)
    par = max(ep, tp)                        # ranks that decode the same sequences together
    prompts = synthetic.make_prompts(full_vocab, B, PROMPT_LEN, seed=1 + (0 if par > 1 else D.rank * B)).to(dev)
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
    sampler = ClockSampler(local_rank) if D.rank == 0 else None
    for _ in range(W):
        mk.decode_step(pos); pos += 1
    torch.cuda.synchronize(dev)
    mk.check_status()
    first_timed_pos = pos
    launches0 = mk.launch_count
    moe = bool(config.get("num_experts"))
    if moe:
        mk.expert_reads(reset=True)
    kernel_s, _, pos = timed_steps(mk, K, pos, D)
    clocks = sampler.stop() if sampler else None
    mk.check_status()
    launches = mk.launch_count - launches0
    step_bytes = sum(mk.step_bytes(first_timed_pos + i) for i in range(K)) / K
    experts_per_layer_step = None
    if moe:     # bytes from the experts the steps really read (distinct per layer and step), not from an upper bound
        L, E, k = config["num_hidden_layers"], config["num_experts"], config["num_experts_per_tok"]
        reads = mk.expert_reads(reset=True)
        experts_per_layer_step = reads / (K * L)
        per_expert = 3 * config["hidden_size"] * config["moe_intermediate_size"] * 2
        step_bytes += (reads / K - L * min(E, B * k)) * per_expert

    # end to end with host token buffers: per step B tokens host -> device, the launch, B arg-max values device -> host
    host_in = prompts[:, :1].cpu().repeat(1, K + 1).t().contiguous().pin_memory()      # [K + 1, B]
    host_out = torch.zeros(K, B, dtype=torch.int64).pin_memory()
    tok_dev = torch.zeros(B, dtype=torch.int64, device=dev)
    out_dev = torch.zeros(B, dtype=torch.int64, device=dev)
    g.token_in, g.next_token = tok_dev, out_dev
    g.position_id = first_timed_pos
    mk(g)                                   # re-binds the state (untimed)
    pos = first_timed_pos
    D.barrier()
    t0 = time.perf_counter()
    for i in range(K):
        tok_dev.copy_(host_in[i], non_blocking=True)
        mk.decode_step(pos)
        host_out[i].copy_(out_dev, non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()
        host_in[i + 1].copy_(host_out[i])
        pos += 1
    e2e_s = time.perf_counter() - t0
    D.barrier()
    mk.check_status()
    kernel_s, e2e_s = D.max_over_ranks([kernel_s, e2e_s])
    ctas, threads, smem = mk.geometry()
    mk.close()
    line = None
    if D.rank == 0:
        world = 1 if par > 1 else D.world      # under model parallelism all ranks decode the same sequences
        peak, peak_src = measured_peak_gbs()
        achieved = step_bytes / (kernel_s / K) / 1e9
        line = {
            "metric": f"decode kernel_tok_s at batch {B} per GPU ({model} shape)", "value": world * B * K / kernel_s,
            "unit": "tokens/s", "n_gpus": D.world, "steps": K, "warmup": W, "ms_per_step": kernel_s / K * 1e3,
            "higher_is_better": True, "scaling": "strong" if par > 1 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{model} shape, bf16, {B} independent seeded 16-token prompts per GPU, greedy decode "
                                   "forced past EOS", "decode_steps": K,
                       "kv_lengths": [first_timed_pos + 1, first_timed_pos + K], "sequences_per_gpu": B,
                       "decoder_layers": config["num_hidden_layers"],
                       "sharding": (f"expert parallel over {ep} GPUs: the same sequences on every GPU, {config['num_experts'] // ep} of "
                                    f"{config['num_experts']} experts each, partial expert outputs pushed to the peers over NVLink "
                                    "inside the kernel and added in rank order; roofline figures are rank 0's own bytes"
                                    if ep > 1 else
                                    f"tensor parallel over {tp} GPUs: the same sequences on every GPU, 1 / {tp} of every projection "
                                    "each, partial O-proj and down-proj sums pushed to the peers over NVLink inside the kernel and "
                                    "added in rank order, arg-max over the ranks' vocabulary slices; roofline figures are rank 0's own bytes"
                                    if tp > 1 else "sequences sharded over the GPUs, full weight copy each, no collective"),
                       "l2": "inputs larger than L2: every step streams the weights through a 126 MB L2",
                       "launch": {"ctas": ctas, "threads": threads, "smem_bytes": smem}},
            "e2e": {"value": world * B * K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 8 * B, "d2h_bytes_per_step": 8 * B},
            "gpu_launches": launches + K + 1,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": (BATCHED_TRAFFIC_RATIO[(model, B)][0] * step_bytes
                                     if (model, B) in BATCHED_TRAFFIC_RATIO and ep == 1 and tp == 1 else None),
                         "traffic_source": BATCHED_TRAFFIC_RATIO.get((model, B), (None, None))[1] if ep == 1 and tp == 1 else None,
                         "peak_source": peak_src, "algorithmic_bytes_per_launch": step_bytes,
                         "kernel": "qmk_batch_kernel (one persistent launch per decode step)"},
            "clocks": clocks, "cpu_baseline": None,
        }
        if moe:
            line["config"]["distinct_experts_per_layer_and_step"] = experts_per_layer_step
            line["config"]["bytes_note"] = "algorithmic bytes count the distinct experts every layer of every timed step read (device counter)"
    del g, weights
    gc.collect()
    torch.cuda.empty_cache()
    return line


SECONDARY = (("llama-3.2-1b", 32), ("qwen3-0.6b", 16), ("olmoe-1b-7b", 32))
# DRAM traffic / algorithmic bytes of one qmk_batch_kernel launch where an ncu capture exists (profiles/): the capture of
# the OLMoE case held 3 of the 16 layers (a few GB on the device); traffic grows with the layers like the algorithmic
# bytes do, so the ratio is applied to the full step's bytes.
BATCHED_TRAFFIC_RATIO = {("llama-3.2-1b", 8): (1.012, "profiles/qmk_batch_kernel_step_llama1b_b8.md"),
                         ("olmoe-1b-7b", 32): (1.009, "profiles/qmk_batch_kernel_step_olmoe_b32_3layers.md (3-layer capture, scaled by bytes)")}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1024)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg (rank 0, N = 1 only)")
    ap.add_argument("--no-secondary", action="store_true", help="headline line only: skip the short runs of the other workload shapes")
    ap.add_argument("--steps-per-launch", type=int, default=1,
                    help="headline run: decode steps per persistent launch of the batch-1 kernel in the device-timed loop")
    ap.add_argument("--batch", type=int, default=1, help="sequences per GPU (> 1, or any --model but llama: the batched kernel)")
    ap.add_argument("--model", default="llama-3.2-1b", choices=["llama-3.2-1b", "qwen3-0.6b", "olmoe-1b-7b"])
    ap.add_argument("--kernel", default="auto", choices=["auto", "batched"], help="batched: the batched kernel also at batch 1")
    ap.add_argument("--ep", type=int, default=1, help="expert parallelism over this many GPUs (mixture-of-experts --model; equals the number of ranks)")
    ap.add_argument("--tp", type=int, default=1, help="tensor parallelism over this many GPUs (dense --model; equals the number of ranks; batched kernel)")
    ap.add_argument("--layers", type=int, default=0,
                    help="batched runs only: keep this many decoder layers (a small case for a profiler capture; the line says so)")
    args = ap.parse_args()
    K, W = args.steps, max(3, args.warmup)
    single = args.batch != 1 or args.model != "llama-3.2-1b" or args.kernel == "batched" or args.tp > 1
    if args.impl == "reference":
        if single:
            raise SystemExit("--impl reference times the headline workload (batch 1, Llama-3.2-1B shape) only")
        return run_reference_arm(args, K, W)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode path has no CPU fallback")
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    pinned = pin_host_thread(local_rank, world)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    D = Dist(dev)
    if single:
        line = run_batched(args.model, args.batch, K, W, args.layers, D, local_rank, ep=args.ep, tp=args.tp)
    else:
        line = run_batch1(args, K, W, D, local_rank)
        if not args.no_secondary:
            # the other workload shapes, short: 32 timed steps after 4 warm-up steps each (a few seconds per run)
            sec = []
            for model, B in SECONDARY:
                s = run_batched(model, B, 32, 4, 0, D, local_rank)
                if s is not None:
                    sec.append({k: s[k] for k in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step",
                                                   "e2e", "roofline", "clocks", "config")})
            if line is not None:
                line["secondary"] = sec
    if line is not None:
        if pinned is not None:
            line["host_cores_per_rank"] = len(pinned)
        print(json.dumps(line), flush=True)
    if D.world > 1:
        D.dist.destroy_process_group()


if __name__ == "__main__":
    main()
