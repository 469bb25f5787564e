"""Generates the golden fixtures in this directory by running the REAL reference on the CPU.

Run once, in a container that has the reference checkout (it is not needed to run the tests):

    PYTHONPATH=/path/to/QiMeng-MegaKernel python tests/golden/make_golden.py [--full]

What is executed is the reference's own fused-PyTorch decode route, unmodified:
    qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/single_batch/decode_schedule/fused/operations.py
    (fused_rms_qkvproj_gemv_rope, fused_decode_attention, fused_oproj_gemv_residual, fused_mlp_upgate,
     fused_mlp_down_residual, fused_rms_lmhead_gemv) on its Globals dataclass (decode_schedule/globs.py),
in bf16 (the reference path) and in fp32 (same functions, fp32 tensors: the high-precision yardstick),
on the seeded synthetic weights of qimeng_megakernel_b200.synthetic.  The token loop is the one of
FusedGenerator.generate_greedy_fast (qimeng_megakernel/models/LLM/decode.py:1373-1395): embed, step, argmax.

Fixtures:
  small_l2_v4096.npz   2 layers, vocabulary 4096, Llama-3.2-1B layer shape; every intermediate buffer of
                       12 teacher-forced steps.  Pins the CPU oracle bit for bit (tests/test_oracle_golden.py).
  llama1b_cfg1.npz     (--full) the BASELINE configuration 1: 16 layers, vocabulary 128256, 16 seeded prompt
                       tokens then greedy decode; greedy tokens, top-8 logits per step, per-layer hidden
                       states of selected steps (bf16 and fp32).  Compared with the CUDA kernel on the GPU.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from qimeng_megakernel_b200 import synthetic  # noqa: E402
from qimeng_megakernel_b200.model_config import LLAMA_3_2_1B  # noqa: E402

REF_PKG = "qimeng_megakernel.models.LLM.llama.llama3_2__1b.A100.single_batch.decode_schedule"


def ref_modules():
    import importlib
    pkg = importlib.import_module(REF_PKG)
    ops = importlib.import_module(REF_PKG + ".fused.operations")
    return pkg, ops


def ref_globals(pkg, config: dict, weights: dict, kv_seq_len: int, dtype: torch.dtype):
    """The buffers the reference's fused prefill allocates for B = 1
    (qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/fused_prefill.py:61-160)."""
    pkg.LlamaConfig.update_from_dict({k: config[k] for k in (
        "num_hidden_layers", "hidden_size", "intermediate_size", "head_dim", "num_attention_heads",
        "num_key_value_heads", "vocab_size", "rms_norm_eps")})
    L, H, I = config["num_hidden_layers"], config["hidden_size"], config["intermediate_size"]
    NH, NKV, HD, V = (config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"],
                      config["vocab_size"])
    cast = lambda t: t.to(dtype)
    g = pkg.Globals(
        position_id=0,
        attn_norm_weights=cast(weights["attn_norm_weights"]), qkv_weights=cast(weights["qkv_weights"]),
        o_proj_weights=cast(weights["o_proj_weights"]), mlp_norm_weights=cast(weights["mlp_norm_weights"]),
        up_proj_weights=cast(weights["up_proj_weights"]), gate_proj_weights=cast(weights["gate_proj_weights"]),
        down_proj_weights=cast(weights["down_proj_weights"]),
        lm_head_norm_weights=cast(weights["lm_head_norm_weights"]), lm_head_weights=cast(weights["lm_head_weights"]),
        rope_cos=weights["rope_cos"].float(), rope_sin=weights["rope_sin"].float(),
        k_cache=torch.zeros(L, 1, kv_seq_len, NKV, HD, dtype=dtype),
        v_cache=torch.zeros(L, 1, kv_seq_len, NKV, HD, dtype=dtype),
        hidden_states=torch.zeros(H, dtype=dtype), q_post_rope=torch.zeros(NH * HD, dtype=dtype),
        attn_out=torch.zeros(NH * HD, dtype=dtype), silu_out=torch.zeros(I, dtype=dtype),
        logits=torch.zeros(V, dtype=dtype))
    g.embed_tokens = cast(weights["embed_tokens"])
    return g


def step(ops, g, layers: int, token: int, pos: int, record: dict | None = None):
    """embed -> per layer the five fused ops -> LM head; optionally records every buffer."""
    g.hidden_states.copy_(g.embed_tokens[token].to(g.hidden_states.dtype))
    g.position_id = pos
    hid = []
    for layer in range(layers):
        ops.fused_rms_qkvproj_gemv_rope(g, layer)
        if record is not None and layer == layers - 1:
            record["q_post_rope"] = g.q_post_rope.clone()
            record["k_row"] = g.k_cache[layer, 0, pos].clone()
            record["v_row"] = g.v_cache[layer, 0, pos].clone()
        ops.fused_decode_attention(g, layer)
        if record is not None and layer == layers - 1:
            record["attn_out"] = g.attn_out.clone()
        ops.fused_oproj_gemv_residual(g, layer)
        if record is not None and layer == layers - 1:
            record["hidden_after_oproj"] = g.hidden_states.clone()
        ops.fused_mlp_upgate(g, layer)
        if record is not None and layer == layers - 1:
            record["silu_out"] = g.silu_out.clone()
        ops.fused_mlp_down_residual(g, layer)
        hid.append(g.hidden_states.clone())
    ops.fused_rms_lmhead_gemv(g)
    if record is not None:
        record["layer_hidden"] = torch.stack(hid)
        record["logits"] = g.logits.clone()
    return int(g.logits.argmax())


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensors are stored as their 16-bit patterns."""
    return t.contiguous().view(torch.int16).numpy() if t.dtype == torch.bfloat16 else t.contiguous().numpy()


def make_small(pkg, ops):
    cfg = dict(LLAMA_3_2_1B, num_hidden_layers=2, vocab_size=4096, max_position_embeddings=4096)
    w = synthetic.make_weights(cfg, seed=1234, device="cpu")
    n_steps, S = 12, 64
    tokens = synthetic.make_prompt(cfg["vocab_size"], n_steps, seed=99).tolist()
    out = {"tokens": np.array(tokens, dtype=np.int64), "weights_seed": np.int64(1234), "prompt_seed": np.int64(99)}
    for name, dtype in (("bf16", torch.bfloat16), ("fp32", torch.float32)):
        g = ref_globals(pkg, cfg, w, S, dtype)
        recs = []
        for pos, tok in enumerate(tokens):
            r = {}
            r["argmax"] = step(ops, g, cfg["num_hidden_layers"], tok, pos, r)
            recs.append(r)
        keys = ("layer_hidden", "logits") if name == "fp32" else (
            "q_post_rope", "k_row", "v_row", "attn_out", "hidden_after_oproj", "silu_out", "layer_hidden", "logits")
        for k in keys:
            out[f"{name}_{k}"] = np.stack([bits(r[k]) for r in recs])
        out[f"{name}_argmax"] = np.array([r["argmax"] for r in recs], dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "small_l2_v4096.npz"), **out)
    print("wrote small_l2_v4096.npz")


def make_full(pkg, ops, n_new: int):
    cfg = dict(LLAMA_3_2_1B)
    t0 = time.time()
    w = synthetic.make_weights(cfg, seed=0, device="cpu", max_positions=2048)
    print("weights %.1fs" % (time.time() - t0), flush=True)
    prompt = synthetic.make_prompt(cfg["vocab_size"], 16, seed=1).tolist()
    S = 16 + n_new + 1
    L = cfg["num_hidden_layers"]
    out = {"prompt": np.array(prompt, dtype=np.int64), "weights_seed": np.int64(0), "prompt_seed": np.int64(1)}
    hid_steps = (0, 15, 16, 16 + n_new - 1)
    tokens = None
    for name, dtype in (("bf16", torch.bfloat16), ("fp32", torch.float32)):
        g = ref_globals(pkg, cfg, w, S, dtype)
        seq = list(prompt) if tokens is None else list(tokens)   # fp32 run is teacher-forced with the bf16 tokens
        top_v, top_i, hid = [], [], {}
        for pos in range(16 + n_new):
            r = {}
            nxt = step(ops, g, L, seq[pos], pos, r)
            if tokens is None and pos + 1 >= len(seq):
                seq.append(nxt)
            tv, ti = r["logits"].float().topk(8)
            top_v.append(tv.numpy()); top_i.append(ti.numpy())
            if pos in hid_steps:
                hid[pos] = bits(r["layer_hidden"])
            print(name, pos, nxt, "%.0fs" % (time.time() - t0), flush=True)
        if tokens is None:
            tokens = seq
            out["tokens"] = np.array(seq, dtype=np.int64)
        out[f"{name}_top8_values"] = np.stack(top_v).astype(np.float32)
        out[f"{name}_top8_indices"] = np.stack(top_i).astype(np.int64)
        out["hidden_steps"] = np.array(hid_steps, dtype=np.int64)
        out[f"{name}_layer_hidden"] = np.stack([hid[s] for s in hid_steps])
    np.savez_compressed(os.path.join(HERE, "llama1b_cfg1.npz"), **out)
    print("wrote llama1b_cfg1.npz")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--full", action="store_true", help="also generate the full-size Llama-3.2-1B fixture (minutes of CPU)")
    ap.add_argument("--new-tokens", type=int, default=16)
    args = ap.parse_args()
    torch.manual_seed(0)
    pkg, ops = ref_modules()
    make_small(pkg, ops)
    if args.full:
        make_full(pkg, ops, args.new_tokens)
