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
  batch3_l2_v4096.npz  the same small Llama shape with THREE sequences in [B, H] state (the reference's multi-batch
                       Globals, multi_batch/decode_schedule/globs.py, driven through the same fused ops): ragged
                       positions, a row that starts late and a row that finishes early (active_mask), norm gains
                       drawn around 1.  Every buffer of 7 steps.
  qwen3_l2_v4096.npz   the Qwen3-0.6B layer shape (hidden 1024, 16 / 8 heads of 128, intermediate 3072), 2 layers,
                       vocabulary 4096, through the reference's Qwen3 fused ops (per-head Q/K RMSNorm):
                       qimeng_megakernel/models/LLM/qwen/qwen3__0_6b/A100/single_batch/decode_schedule/fused/operations.py
  moe_block.npz        the reference's fused MoE block (qwen1_5_moe_a2_7b/.../fused/operations.py:151-268) on a small
                       shape, once with a shared expert and 16 experts / top-4, once shaped like an OLMoE layer in
                       miniature (no shared expert: its weights are zero; 64 experts / top-8, router logits ~ N(0,1)).
                       Pins oracle/moe_oracle.py.
  moe_olmoe_layer.npz  the same block at the full OLMoE-1B-7B layer shape (hidden 2048, 64 experts, top-8, expert
                       intermediate 1024, no shared expert), 8 input rows: experts, router weights, routed output
                       and new hidden state in bf16 and fp32.  The weights are regenerated from the seed by
                       moe_weights(MOE_LAYER_CASE); the CUDA kernel's MoE phases are compared with it on the GPU.
  sampling.npz         the reference's _sample_logits (qimeng_megakernel/models/LLM/decode.py:53-143) on seeded logits
                       for a grid of temperature / top-k / top-p / min-p / presence-penalty settings: the probability
                       vector it hands to torch.multinomial (captured by wrapping that call) or its greedy token.
  llama1b_cfg1.npz     (--full) the full-size Llama-3.2-1B workload: 16 layers, vocabulary 128256, 16 seeded prompt
                       tokens then greedy decode; greedy tokens, top-8 logits per step, per-layer hidden
                       states of selected steps (bf16 and fp32).  Compared with the CUDA kernel on the GPU.
  llama1b_kv1040.npz   (--full) the same full-size model, ONE decode step at position 1039 on a KV cache whose first
                       1039 rows are seeded random rows (synthetic.random_kv_rows, seed 1040): top-8 logits, arg-max
                       and per-layer hidden states in bf16 and fp32.  Long-context evidence at full size.
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
from qimeng_megakernel_b200.model_config import LLAMA_3_2_1B, QWEN3_0_6B  # noqa: E402

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


BATCH_PLAN = dict(
    # per step: (position, active) of each of the three rows; row 2 starts two steps late, row 1 stops after step 3
    positions=[[0, 0, 0], [1, 1, 0], [2, 2, 0], [3, 3, 1], [4, 3, 2], [5, 3, 3], [6, 3, 4]],
    active=[[1, 1, 0], [1, 1, 0], [1, 1, 1], [1, 1, 1], [1, 0, 1], [1, 0, 1], [1, 0, 1]])


def make_batch(ops):
    """Three sequences through the reference's fused ops on its multi-batch Globals."""
    import importlib
    mb = importlib.import_module(
        "qimeng_megakernel.models.LLM.llama.llama3_2__1b.A100.multi_batch.decode_schedule.globs")
    pkg = importlib.import_module(REF_PKG)
    cfg = dict(LLAMA_3_2_1B, num_hidden_layers=2, vocab_size=4096, max_position_embeddings=4096)
    w = synthetic.make_weights(cfg, seed=4321, device="cpu", gain_jitter=0.1)
    B, S, L = 3, 16, cfg["num_hidden_layers"]
    prompts = synthetic.make_prompts(cfg["vocab_size"], B, 8, seed=77)
    out = {"prompts": prompts.numpy(), "weights_seed": np.int64(4321), "prompt_seed": np.int64(77),
           "positions": np.array(BATCH_PLAN["positions"], dtype=np.int64),
           "active": np.array(BATCH_PLAN["active"], dtype=np.int64)}
    for name, dtype in (("bf16", torch.bfloat16), ("fp32", torch.float32)):
        base = ref_globals(pkg, cfg, w, S, dtype)
        NH, NKV, HD, H, I, V = (cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                                cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"])
        g = mb.Globals(**{f: getattr(base, f) for f in (
            "attn_norm_weights", "qkv_weights", "o_proj_weights", "mlp_norm_weights", "up_proj_weights",
            "gate_proj_weights", "down_proj_weights", "lm_head_norm_weights", "lm_head_weights", "rope_cos", "rope_sin")})
        g.embed_tokens = base.embed_tokens
        g.k_cache = torch.zeros(L, B, S, NKV, HD, dtype=dtype)
        g.v_cache = torch.zeros(L, B, S, NKV, HD, dtype=dtype)
        g.hidden_states = torch.zeros(B, H, dtype=dtype)
        g.q_post_rope = torch.zeros(B, NH * HD, dtype=dtype)
        g.attn_out = torch.zeros(B, NH * HD, dtype=dtype)
        g.silu_out = torch.zeros(B, I, dtype=dtype)
        g.logits = torch.zeros(B, V, dtype=dtype)
        recs = []
        for positions, active in zip(BATCH_PLAN["positions"], BATCH_PLAN["active"]):
            toks = [int(prompts[b, positions[b]]) for b in range(B)]
            g.hidden_states.copy_(g.embed_tokens[torch.tensor(toks)].to(dtype))
            g.position_ids = torch.tensor(positions, dtype=torch.int32)
            g.active_mask = torch.tensor(active, dtype=torch.bool)
            g.position_id = None
            r, hid = {}, []
            for layer in range(L):
                ops.fused_rms_qkvproj_gemv_rope(g, layer)
                if layer == L - 1:
                    r["q_post_rope"] = g.q_post_rope.clone()
                    r["k_row"] = torch.stack([g.k_cache[layer, b, positions[b]] for b in range(B)])
                    r["v_row"] = torch.stack([g.v_cache[layer, b, positions[b]] for b in range(B)])
                ops.fused_decode_attention(g, layer)
                if layer == L - 1:
                    r["attn_out"] = g.attn_out.clone()
                ops.fused_oproj_gemv_residual(g, layer)
                if layer == L - 1:
                    r["hidden_after_oproj"] = g.hidden_states.clone()
                ops.fused_mlp_upgate(g, layer)
                if layer == L - 1:
                    r["silu_out"] = g.silu_out.clone()
                ops.fused_mlp_down_residual(g, layer)
                hid.append(g.hidden_states.clone())
            ops.fused_rms_lmhead_gemv(g)
            r["layer_hidden"] = torch.stack(hid)
            r["logits"] = g.logits.clone()
            r["argmax"] = g.logits.argmax(dim=-1).clone()
            recs.append(r)
        keys = ("layer_hidden", "logits") if name == "fp32" else (
            "q_post_rope", "k_row", "v_row", "attn_out", "hidden_after_oproj", "silu_out", "layer_hidden", "logits")
        for k in keys:
            out[f"{name}_{k}"] = np.stack([bits(r[k]) for r in recs])
        out[f"{name}_argmax"] = np.stack([r["argmax"].numpy() for r in recs]).astype(np.int64)
    np.savez_compressed(os.path.join(HERE, "batch3_l2_v4096.npz"), **out)
    print("wrote batch3_l2_v4096.npz")


def make_qwen3():
    """One sequence through the reference's Qwen3 fused ops (per-head Q/K norm before RoPE)."""
    import importlib
    qpkg = "qimeng_megakernel.models.LLM.qwen.qwen3__0_6b.A100.single_batch.decode_schedule"
    pkg = importlib.import_module(qpkg)
    ops = importlib.import_module(qpkg + ".fused.operations")
    cfg = dict(QWEN3_0_6B, num_hidden_layers=2, vocab_size=4096, max_position_embeddings=4096)
    pkg.Qwen3Config.update_from_dict({k: cfg[k] for k in (
        "num_hidden_layers", "hidden_size", "intermediate_size", "head_dim", "num_attention_heads",
        "num_key_value_heads", "vocab_size", "rms_norm_eps")})
    w = synthetic.make_weights(cfg, seed=2468, device="cpu", gain_jitter=0.1)
    n_steps, S, L = 10, 16, cfg["num_hidden_layers"]
    NH, NKV, HD, H, I, V = (cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                            cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"])
    tokens = synthetic.make_prompt(V, n_steps, seed=55).tolist()
    out = {"tokens": np.array(tokens, dtype=np.int64), "weights_seed": np.int64(2468), "prompt_seed": np.int64(55)}
    for name, dtype in (("bf16", torch.bfloat16), ("fp32", torch.float32)):
        cast = lambda t: t.to(dtype)
        g = pkg.Globals(
            position_id=0,
            attn_norm_weights=cast(w["attn_norm_weights"]), qkv_weights=cast(w["qkv_weights"]),
            q_norm_weights=cast(w["q_norm_weights"]), k_norm_weights=cast(w["k_norm_weights"]),
            o_proj_weights=cast(w["o_proj_weights"]), mlp_norm_weights=cast(w["mlp_norm_weights"]),
            up_proj_weights=cast(w["up_proj_weights"]), gate_proj_weights=cast(w["gate_proj_weights"]),
            down_proj_weights=cast(w["down_proj_weights"]), lm_head_norm_weights=cast(w["lm_head_norm_weights"]),
            lm_head_weights=cast(w["lm_head_weights"]), rope_cos=w["rope_cos"].float(), rope_sin=w["rope_sin"].float(),
            k_cache=torch.zeros(L, 1, S, NKV, HD, dtype=dtype), v_cache=torch.zeros(L, 1, S, NKV, HD, dtype=dtype),
            hidden_states=torch.zeros(H, dtype=dtype), qkv_raw=torch.zeros((NH + 2 * NKV) * HD, dtype=dtype),
            q_post_rope=torch.zeros(NH * HD, dtype=dtype), attn_out=torch.zeros(NH * HD, dtype=dtype),
            silu_out=torch.zeros(I, dtype=dtype), logits=torch.zeros(V, dtype=dtype))
        embed = cast(w["embed_tokens"])
        recs = []
        for pos, tok in enumerate(tokens):
            g.hidden_states.copy_(embed[tok])
            g.position_id = pos
            r, hid = {}, []
            for layer in range(L):
                ops.fused_rms_qkvproj_gemv_rope(g, layer)
                if layer == L - 1:
                    r["q_post_rope"] = g.q_post_rope.clone()
                    r["k_row"] = g.k_cache[layer, 0, pos].clone()
                    r["v_row"] = g.v_cache[layer, 0, pos].clone()
                ops.fused_decode_attention(g, layer)
                if layer == L - 1:
                    r["attn_out"] = g.attn_out.clone()
                ops.fused_oproj_gemv_residual(g, layer)
                ops.fused_mlp_upgate(g, layer)
                if layer == L - 1:
                    r["silu_out"] = g.silu_out.clone()
                ops.fused_mlp_down_residual(g, layer)
                hid.append(g.hidden_states.clone())
            ops.fused_rms_lmhead_gemv(g)
            r["layer_hidden"] = torch.stack(hid)
            r["logits"] = g.logits.clone()
            r["argmax"] = int(g.logits.argmax())
            recs.append(r)
        keys = ("layer_hidden", "logits") if name == "fp32" else (
            "q_post_rope", "k_row", "v_row", "attn_out", "silu_out", "layer_hidden", "logits")
        for k in keys:
            out[f"{name}_{k}"] = np.stack([bits(r[k]) for r in recs])
        out[f"{name}_argmax"] = np.array([r["argmax"] for r in recs], dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "qwen3_l2_v4096.npz"), **out)
    print("wrote qwen3_l2_v4096.npz")


MOE_CASES = (dict(name="shared", hidden_size=256, intermediate_size=512, moe_intermediate_size=128, num_experts=16,
                       num_experts_per_tok=4, shared=True, seed=11),
                  dict(name="olmoe_like", hidden_size=256, intermediate_size=64, moe_intermediate_size=128,
                       num_experts=64, num_experts_per_tok=8, shared=False, seed=12))


def moe_weights(case: dict) -> dict:
    """Seeded weights of one MoE layer (N(0, 0.02) like the dense models; router rows scaled so that the logits of a
    unit-RMS input are ~ N(0, 1); gains drawn around 1)."""
    gen = torch.Generator().manual_seed(case["seed"])
    H, I, Ie, E = case["hidden_size"], case["intermediate_size"], case["moe_intermediate_size"], case["num_experts"]
    r = lambda *shape, std=0.02: (torch.randn(*shape, generator=gen) * std).to(torch.bfloat16)
    w = {"mlp_norm": (1.0 + 0.1 * torch.randn(H, generator=gen)).to(torch.bfloat16),
         "shared_gate_proj": r(I, H), "shared_up_proj": r(I, H), "shared_down_proj": r(H, I),
         "shared_expert_gate": r(H, 1), "router": r(E, H, std=H ** -0.5),
         "expert_gate_up": r(E, 2 * Ie, H), "expert_down": r(E, H, Ie)}
    if not case["shared"]:
        for k in ("shared_gate_proj", "shared_up_proj", "shared_down_proj", "shared_expert_gate"):
            w[k].zero_()
    w["inputs"] = (torch.randn(6, H, generator=gen) * 0.7).to(torch.bfloat16)
    return w


def make_moe():
    import importlib
    mpkg = "qimeng_megakernel.models.LLM.qwen.qwen1_5_moe_a2_7b.A100.single_batch.decode_schedule"
    pkg = importlib.import_module(mpkg)
    ops = importlib.import_module(mpkg + ".fused.operations")
    out = {}
    for case in MOE_CASES:
        C = pkg.QwenMoeConfig
        for k in ("hidden_size", "intermediate_size", "moe_intermediate_size", "num_experts", "num_experts_per_tok"):
            setattr(C, k, case[k])
        C.rms_norm_eps = 1e-6
        w = moe_weights(case)
        H, Ie, K = case["hidden_size"], case["moe_intermediate_size"], case["num_experts_per_tok"]
        for name, dtype in (("bf16", torch.bfloat16), ("fp32", torch.float32)):
            c = lambda t: t.to(dtype).unsqueeze(0)       # one layer
            g = pkg.Globals(
                mlp_norm_weights=c(w["mlp_norm"]), shared_expert_gate_proj_weights=c(w["shared_gate_proj"]),
                shared_expert_up_proj_weights=c(w["shared_up_proj"]), shared_expert_down_proj_weights=c(w["shared_down_proj"]),
                shared_expert_gate_weights=c(w["shared_expert_gate"]), router_weights=c(w["router"]),
                expert_gate_up_proj_weights=c(w["expert_gate_up"]), expert_down_proj_weights=c(w["expert_down"]),
                hidden_states=torch.zeros(H, dtype=dtype), shared_out=torch.zeros(H, dtype=dtype),
                routed_out=torch.zeros(H, dtype=dtype), silu_out=torch.zeros(Ie, dtype=dtype),
                expert_indices=torch.zeros(K, dtype=torch.int64), expert_weights=torch.zeros(K, dtype=torch.float32))
            recs = {"hidden": [], "shared_out": [], "routed_out": [], "expert_indices": [], "expert_weights": []}
            for x in w["inputs"]:
                g.hidden_states.copy_(x.to(dtype))
                g.routed_out.zero_()
                ops.fused_moe_block(g, 0)
                recs["hidden"].append(bits(g.hidden_states.clone()))
                recs["shared_out"].append(bits(g.shared_out.clone()))
                recs["routed_out"].append(bits(g.routed_out.clone()))
                recs["expert_indices"].append(g.expert_indices.clone().numpy())
                recs["expert_weights"].append(g.expert_weights.clone().numpy())
            for k, v in recs.items():
                out[f"{case['name']}_{name}_{k}"] = np.stack(v)
    np.savez_compressed(os.path.join(HERE, "moe_block.npz"), **out)
    print("wrote moe_block.npz")


MOE_LAYER_CASE = dict(name="olmoe_layer", hidden_size=2048, intermediate_size=64, moe_intermediate_size=1024,
                      num_experts=64, num_experts_per_tok=8, shared=False, seed=13, rows=8)


def make_moe_layer():
    """fused_moe_block of the reference at the full OLMoE layer shape (one layer, MOE_LAYER_CASE)."""
    import importlib
    mpkg = "qimeng_megakernel.models.LLM.qwen.qwen1_5_moe_a2_7b.A100.single_batch.decode_schedule"
    pkg = importlib.import_module(mpkg)
    ops = importlib.import_module(mpkg + ".fused.operations")
    case = MOE_LAYER_CASE
    C = pkg.QwenMoeConfig
    for k in ("hidden_size", "intermediate_size", "moe_intermediate_size", "num_experts", "num_experts_per_tok"):
        setattr(C, k, case[k])
    C.rms_norm_eps = 1e-5
    w = moe_weights(case)
    gen = torch.Generator().manual_seed(case["seed"] + 100)
    inputs = (torch.randn(case["rows"], case["hidden_size"], generator=gen) * 0.7).to(torch.bfloat16)
    H, Ie, K = case["hidden_size"], case["moe_intermediate_size"], case["num_experts_per_tok"]
    out = {"inputs": bits(inputs)}
    for name, dtype in (("bf16", torch.bfloat16), ("fp32", torch.float32)):
        c = lambda t: t.to(dtype).unsqueeze(0)
        g = pkg.Globals(
            mlp_norm_weights=c(w["mlp_norm"]), shared_expert_gate_proj_weights=c(w["shared_gate_proj"]),
            shared_expert_up_proj_weights=c(w["shared_up_proj"]), shared_expert_down_proj_weights=c(w["shared_down_proj"]),
            shared_expert_gate_weights=c(w["shared_expert_gate"]), router_weights=c(w["router"]),
            expert_gate_up_proj_weights=c(w["expert_gate_up"]), expert_down_proj_weights=c(w["expert_down"]),
            hidden_states=torch.zeros(H, dtype=dtype), shared_out=torch.zeros(H, dtype=dtype),
            routed_out=torch.zeros(H, dtype=dtype), silu_out=torch.zeros(Ie, dtype=dtype),
            expert_indices=torch.zeros(K, dtype=torch.int64), expert_weights=torch.zeros(K, dtype=torch.float32))
        recs = {"hidden": [], "routed_out": [], "expert_indices": [], "expert_weights": []}
        for x in inputs:
            g.hidden_states.copy_(x.to(dtype))
            g.routed_out.zero_()
            ops.fused_moe_block(g, 0)
            recs["hidden"].append(bits(g.hidden_states.clone()))
            recs["routed_out"].append(bits(g.routed_out.clone()))
            recs["expert_indices"].append(g.expert_indices.clone().numpy())
            recs["expert_weights"].append(g.expert_weights.clone().numpy())
        for k, v in recs.items():
            out[f"{name}_{k}"] = np.stack(v)
    np.savez_compressed(os.path.join(HERE, "moe_olmoe_layer.npz"), **out)
    print("wrote moe_olmoe_layer.npz")


SAMPLING_CASES = (
    dict(temperature=0.0, top_p=1.0, top_k=0, min_p=0.0, presence_penalty=0.0),
    dict(temperature=0.0, top_p=1.0, top_k=0, min_p=0.0, presence_penalty=1.5),
    dict(temperature=0.7, top_p=1.0, top_k=0, min_p=0.0, presence_penalty=0.0),     # greedy by the reference's rule
    dict(temperature=0.7, top_p=0.9, top_k=0, min_p=0.0, presence_penalty=0.0),
    dict(temperature=1.3, top_p=1.0, top_k=40, min_p=0.0, presence_penalty=0.0),
    dict(temperature=1.0, top_p=1.0, top_k=0, min_p=0.02, presence_penalty=0.0),
    dict(temperature=0.8, top_p=0.95, top_k=50, min_p=0.01, presence_penalty=0.6),
    dict(temperature=1.0, top_p=1.0, top_k=0, min_p=0.9, presence_penalty=0.0),      # min-p leaves nothing: fall-back
    dict(temperature=0.5, top_p=0.0, top_k=5, min_p=0.0, presence_penalty=0.0),      # top-p keeps the first token only
)


def sampling_inputs():
    """Seeded logits [3, 1000] (bf16-representable, spread like LM-head logits) and already generated ids [3, 12]."""
    gen = torch.Generator().manual_seed(2024)
    logits = (torch.randn(3, 1000, generator=gen) * 2.5).to(torch.bfloat16)
    generated = torch.randint(0, 1000, (3, 12), generator=gen, dtype=torch.int64)
    # make sure the penalty matters: every row has already produced its current best token
    generated[:, 0] = logits.float().argmax(dim=-1)
    return logits, generated


def make_sampling():
    """Runs the reference's _sample_logits row by row with torch.multinomial wrapped, recording what it samples from."""
    import importlib
    dec = importlib.import_module("qimeng_megakernel.models.LLM.decode")
    logits, generated = sampling_inputs()
    out = {}
    real = torch.multinomial
    for ci, case in enumerate(SAMPLING_CASES):
        probs_rows, greedy_rows = [], []
        for b in range(logits.shape[0]):
            captured = []

            def spy(p, *a, **k):
                captured.append(p.clone())
                return real(p, *a, **k)

            torch.multinomial = spy
            try:
                tok = dec._sample_logits(logits[b], generated_ids=generated[b:b + 1], **case)
            finally:
                torch.multinomial = real
            if captured:
                probs_rows.append(captured[0].float().numpy())
                greedy_rows.append(-1)
            else:
                probs_rows.append(np.zeros(logits.shape[1], dtype=np.float32))
                greedy_rows.append(int(tok))
        out[f"case{ci}_probs"] = np.stack(probs_rows)
        out[f"case{ci}_greedy"] = np.array(greedy_rows, dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "sampling.npz"), **out)
    print("wrote sampling.npz")


LONG_POS, LONG_KV_SEED = 1039, 1040


def make_long(pkg, ops):
    """One full-size Llama-3.2-1B decode step at position LONG_POS over a seeded random KV cache."""
    cfg = dict(LLAMA_3_2_1B)
    t0 = time.time()
    w = synthetic.make_weights(cfg, seed=0, device="cpu", max_positions=2048)
    token = int(synthetic.make_prompt(cfg["vocab_size"], 1, seed=5)[0])
    k, v = synthetic.random_kv_rows(cfg, LONG_POS, LONG_KV_SEED)
    L = cfg["num_hidden_layers"]
    out = {"token": np.int64(token), "pos": np.int64(LONG_POS), "kv_seed": np.int64(LONG_KV_SEED)}
    for name, dtype in (("bf16", torch.bfloat16), ("fp32", torch.float32)):
        g = ref_globals(pkg, cfg, w, LONG_POS + 1, dtype)
        g.k_cache[:, :, :LONG_POS].copy_(k.to(dtype))
        g.v_cache[:, :, :LONG_POS].copy_(v.to(dtype))
        r = {}
        nxt = step(ops, g, L, token, LONG_POS, r)
        tv, ti = r["logits"].float().topk(8)
        out[f"{name}_top8_values"] = tv.numpy().astype(np.float32)
        out[f"{name}_top8_indices"] = ti.numpy().astype(np.int64)
        out[f"{name}_argmax"] = np.int64(nxt)
        out[f"{name}_layer_hidden"] = bits(r["layer_hidden"])
        out[f"{name}_attn_out_last_layer"] = bits(r["attn_out"])
        print(name, nxt, "%.0fs" % (time.time() - t0), flush=True)
    np.savez_compressed(os.path.join(HERE, "llama1b_kv1040.npz"), **out)
    print("wrote llama1b_kv1040.npz")


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
    ap_only = os.environ.get("QMK_GOLDEN_ONLY", "")
    pkg, ops = ref_modules()
    if ap_only in ("", "small"):
        make_small(pkg, ops)
    if ap_only in ("", "batch"):
        make_batch(ops)
    if ap_only in ("", "qwen3"):
        make_qwen3()
    if ap_only in ("", "moe"):
        make_moe()
    if ap_only in ("", "moe_layer"):
        make_moe_layer()
    if ap_only in ("", "sampling"):
        make_sampling()
    if args.full and ap_only in ("", "long"):
        make_long(pkg, ops)
    if args.full and ap_only in ("", "full"):
        make_full(pkg, ops, args.new_tokens)
