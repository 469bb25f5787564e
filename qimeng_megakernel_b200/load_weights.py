"""Checkpoint -> device weights in the layout the decode kernels read.

Does what the reference's disk loaders do -- `load_llama_weights_from_disk`
(qimeng_megakernel/models/LLM/llama/load_weights.py:101-216) and the Qwen3 loader
(qimeng_megakernel/models/LLM/qwen/load_weights.py:221-339): read `config.json` and the safetensors file(s) of a Hugging
Face checkpoint directory, stack the per-layer matrices, put Q and K rows (and the Qwen3 per-head norm gains) into the
interleaved RoPE order `[0, half, 1, half + 1, ...]` per head (llama/preprocess.py:57-83), tie the LM head to the
embedding when the config says so, and build the fp32 interleaved RoPE tables.  The result is a dict keyed by the
`Globals` field names, ready for `synthetic.make_globals`.

Differences, on purpose: tensors are copied shard by shard straight into preallocated device tensors (`safe_open`, one
tensor resident on the host at a time) instead of materialising the whole state dict first; and the RoPE tables honour a
`rope_scaling` entry of type llama3 (the reference's disk loader computes plain-theta tables).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any

import torch

from .rope import rope_tables_interleaved


def load_config(model_path: str | Path) -> dict[str, Any]:
    path = Path(model_path)
    cfg_file = path / "config.json"
    if not cfg_file.exists():
        raise FileNotFoundError(f"config.json not found in {model_path}")
    with open(cfg_file) as f:
        return json.load(f)


def one_head_interleave(head_dim: int) -> torch.Tensor:
    """Index of the source dimension of every interleaved dimension of one head: [0, half, 1, half + 1, ...]."""
    half = head_dim // 2
    return torch.stack([torch.arange(half), torch.arange(half) + half], dim=1).reshape(-1)


def interleave_rows(num_heads: int, head_dim: int) -> torch.Tensor:
    """Row permutation of a [num_heads * head_dim, K] projection into the interleaved order, head by head."""
    one = one_head_interleave(head_dim)
    return (torch.arange(num_heads).view(-1, 1) * head_dim + one.view(1, -1)).reshape(-1)


def model_config_from_hf(hf: dict[str, Any]) -> dict[str, Any]:
    """The runtime descriptor (the keys of model_config.LlamaConfig) from a Hugging Face config.json."""
    nh = int(hf["num_attention_heads"])
    hd = int(hf.get("head_dim") or hf["hidden_size"] // nh)
    rs = hf.get("rope_scaling")
    scaling = None
    if isinstance(rs, dict) and rs.get("rope_type", rs.get("type")) == "llama3":
        scaling = (float(rs["factor"]), float(rs["low_freq_factor"]), float(rs["high_freq_factor"]),
                   int(rs["original_max_position_embeddings"]))
    qk_norm = "qwen3" in str(hf.get("model_type", "")).lower()
    return dict(num_hidden_layers=int(hf["num_hidden_layers"]), hidden_size=int(hf["hidden_size"]),
                intermediate_size=int(hf["intermediate_size"]), head_dim=hd, num_attention_heads=nh,
                num_key_value_heads=int(hf.get("num_key_value_heads", nh)), vocab_size=int(hf["vocab_size"]),
                rms_norm_eps=float(hf.get("rms_norm_eps", 1e-5)), rope_theta=float(hf.get("rope_theta", 10000.0)),
                rope_scaling=scaling, max_position_embeddings=int(hf.get("max_position_embeddings", 2048)),
                qk_norm=qk_norm)


def _shards(path: Path) -> list[Path]:
    single = path / "model.safetensors"
    if single.exists():
        return [single]
    index = path / "model.safetensors.index.json"
    if not index.exists():
        raise FileNotFoundError(f"No model.safetensors or model.safetensors.index.json in {path}")
    with open(index) as f:
        names = sorted(set(json.load(f).get("weight_map", {}).values()))
    for n in names:
        if not (path / n).exists():
            raise FileNotFoundError(f"Shard not found: {path / n}")
    return [path / n for n in names]


def load_weights_from_disk(model_path: str | Path, device: str | torch.device = "cuda",
                           dtype: torch.dtype = torch.bfloat16, max_positions: int | None = None
                           ) -> tuple[dict[str, Any], dict[str, torch.Tensor]]:
    """Returns (runtime config, weights keyed by Globals field names) with every tensor on `device`."""
    from safetensors import safe_open
    path = Path(model_path)
    hf = load_config(path)
    cfg = model_config_from_hf(hf)
    dev = torch.device(device)
    L, H, I = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"]
    NH, NKV, HD, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["vocab_size"]
    qd, kd = NH * HD, NKV * HD
    new = lambda *shape: torch.empty(shape, device=dev, dtype=dtype)
    w = {"embed_tokens": new(V, H), "qkv_weights": new(L, qd + 2 * kd, H), "o_proj_weights": new(L, H, qd),
         "attn_norm_weights": new(L, H), "mlp_norm_weights": new(L, H), "up_proj_weights": new(L, I, H),
         "gate_proj_weights": new(L, I, H), "down_proj_weights": new(L, H, I), "lm_head_norm_weights": new(H)}
    tied = bool(hf.get("tie_word_embeddings", False))
    if not tied:
        w["lm_head_weights"] = new(V, H)
    if cfg["qk_norm"]:
        w["q_norm_weights"], w["k_norm_weights"] = new(L, HD), new(L, HD)
    q_rows, k_rows, one = interleave_rows(NH, HD), interleave_rows(NKV, HD), one_head_interleave(HD)

    # where every checkpoint tensor goes: name suffix -> (destination, row slice of the layer, row permutation)
    def place(name: str, t: torch.Tensor) -> bool:
        if name == "model.embed_tokens.weight":
            w["embed_tokens"].copy_(t); return True
        if name in ("lm_head.weight", "model.lm_head.weight"):
            if not tied:
                w["lm_head_weights"].copy_(t)
            return True
        if name == "model.norm.weight":
            w["lm_head_norm_weights"].copy_(t); return True
        if not name.startswith("model.layers."):
            return False
        _, _, idx, rest = name.split(".", 3)
        i = int(idx)
        if i >= L:
            return False
        if rest == "self_attn.q_proj.weight":
            w["qkv_weights"][i, :qd].copy_(t[q_rows])
        elif rest == "self_attn.k_proj.weight":
            w["qkv_weights"][i, qd:qd + kd].copy_(t[k_rows])
        elif rest == "self_attn.v_proj.weight":
            w["qkv_weights"][i, qd + kd:].copy_(t)
        elif rest == "self_attn.o_proj.weight":
            w["o_proj_weights"][i].copy_(t)
        elif rest == "input_layernorm.weight":
            w["attn_norm_weights"][i].copy_(t)
        elif rest == "post_attention_layernorm.weight":
            w["mlp_norm_weights"][i].copy_(t)
        elif rest == "mlp.up_proj.weight":
            w["up_proj_weights"][i].copy_(t)
        elif rest == "mlp.gate_proj.weight":
            w["gate_proj_weights"][i].copy_(t)
        elif rest == "mlp.down_proj.weight":
            w["down_proj_weights"][i].copy_(t)
        elif rest == "self_attn.q_norm.weight" and cfg["qk_norm"]:
            w["q_norm_weights"][i].copy_(t[one])
        elif rest == "self_attn.k_norm.weight" and cfg["qk_norm"]:
            w["k_norm_weights"][i].copy_(t[one])
        else:
            return False
        return True

    placed = 0
    for shard in _shards(path):
        with safe_open(str(shard), framework="pt", device="cpu") as f:
            for name in f.keys():
                if place(name, f.get_tensor(name).to(dtype)):
                    placed += 1
    need = 2 + (0 if tied else 1) + L * (9 + (2 if cfg["qk_norm"] else 0))
    if placed < need:
        raise KeyError(f"{model_path}: {placed} of the {need} tensors this model needs were found in the checkpoint")
    if tied:
        w["lm_head_weights"] = w["embed_tokens"]
    cos, sin = rope_tables_interleaved(HD, max_positions or cfg["max_position_embeddings"], cfg["rope_theta"],
                                       cfg["rope_scaling"])
    w["rope_cos"], w["rope_sin"] = cos.to(dev).contiguous(), sin.to(dev).contiguous()
    return cfg, w
