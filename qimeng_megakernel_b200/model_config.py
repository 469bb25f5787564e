"""Llama-family model config for the B200 decode schedule.

Same class-attribute interface as the reference's LlamaConfig
(qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/single_batch/decode_schedule/model_config.py:4-78),
so host code that reads `ModelConfig.head_dim` etc. works unchanged.  The CUDA side takes these
as a runtime descriptor checked against its compiled shapes instead of mirrored constexprs.
"""
from __future__ import annotations


class LlamaConfig:
    num_hidden_layers = 16
    hidden_size = 2048
    intermediate_size = 8192
    head_dim = 64
    num_attention_heads = 32
    num_key_value_heads = 8
    num_heads = num_attention_heads + num_key_value_heads * 2
    qkv_out_dim = num_heads * head_dim
    vocab_size = 128256
    rms_norm_eps = 1e-5
    rope_theta = 500000.0
    # llama3 rope scaling (factor, low_freq_factor, high_freq_factor, original context); None = plain theta
    rope_scaling = (32.0, 1.0, 4.0, 8192)
    max_position_embeddings = 8192
    # Qwen3: per-head RMSNorm on Q and K before RoPE (the reference's Qwen3Config,
    # qimeng_megakernel/models/LLM/qwen/qwen3__0_6b/A100/single_batch/decode_schedule/model_config.py:4-16)
    qk_norm = False
    # mixture of experts (the reference's QwenMoeConfig fields, qwen1_5_moe_a2_7b/.../model_config.py:20-24); 0 = dense
    num_experts = 0
    num_experts_per_tok = 0
    moe_intermediate_size = 0
    # expert parallelism (B200 addition): ranks that share the experts, and this process's rank; 0 / 1 = off
    ep_world = 0
    ep_rank = 0
    tp_world = 0         # tensor parallelism: the other fields then describe this rank's slice (tensor_parallel.shard_config)
    tp_rank = 0
    embed_rows = 0       # rows of embed_tokens when they differ from vocab_size (tensor parallelism)

    _KEYS = ("num_hidden_layers", "hidden_size", "intermediate_size", "head_dim", "num_attention_heads",
             "num_key_value_heads", "vocab_size", "rms_norm_eps", "rope_theta", "rope_scaling",
             "max_position_embeddings", "qk_norm", "num_experts", "num_experts_per_tok", "moe_intermediate_size",
             "ep_world", "ep_rank", "tp_world", "tp_rank", "embed_rows")

    @classmethod
    def update_from_dict(cls, config: dict) -> None:
        cls.num_hidden_layers = config["num_hidden_layers"]
        cls.hidden_size = config["hidden_size"]
        cls.intermediate_size = config["intermediate_size"]
        cls.num_attention_heads = config["num_attention_heads"]
        cls.head_dim = config.get("head_dim") or (config["hidden_size"] // config["num_attention_heads"])
        cls.num_key_value_heads = config.get("num_key_value_heads", cls.num_attention_heads)
        cls.num_heads = cls.num_attention_heads + cls.num_key_value_heads * 2
        cls.qkv_out_dim = cls.num_heads * cls.head_dim
        cls.vocab_size = config["vocab_size"]
        cls.rms_norm_eps = config.get("rms_norm_eps", 1e-5)
        cls.rope_theta = float(config.get("rope_theta", 10000.0))
        rs = config.get("rope_scaling")
        if isinstance(rs, dict):
            rs = (float(rs["factor"]), float(rs["low_freq_factor"]), float(rs["high_freq_factor"]),
                  int(rs["original_max_position_embeddings"]))
        cls.rope_scaling = tuple(rs) if rs else None
        cls.max_position_embeddings = int(config.get("max_position_embeddings", 8192))
        cls.qk_norm = bool(config.get("qk_norm", False))
        cls.num_experts = int(config.get("num_experts", 0) or 0)
        cls.num_experts_per_tok = int(config.get("num_experts_per_tok", 0) or 0)
        cls.moe_intermediate_size = int(config.get("moe_intermediate_size", 0) or 0)
        cls.ep_world = int(config.get("ep_world", 0) or 0)
        cls.ep_rank = int(config.get("ep_rank", 0) or 0)
        cls.tp_world = int(config.get("tp_world", 0) or 0)
        cls.tp_rank = int(config.get("tp_rank", 0) or 0)
        cls.embed_rows = int(config.get("embed_rows", 0) or 0)

    @classmethod
    def update_from_hf(cls, config) -> None:
        d = {k: getattr(config, k) for k in ("num_hidden_layers", "hidden_size", "intermediate_size",
                                             "num_attention_heads", "vocab_size")}
        for k in ("head_dim", "num_key_value_heads", "rms_norm_eps", "rope_theta", "rope_scaling",
                  "max_position_embeddings"):
            if getattr(config, k, None) is not None:
                d[k] = getattr(config, k)
        cls.update_from_dict(d)

    @classmethod
    def as_dict(cls) -> dict:
        d = {k: getattr(cls, k) for k in cls._KEYS}
        d["num_heads"] = cls.num_heads
        d["qkv_out_dim"] = cls.qkv_out_dim
        return d


LLAMA_3_2_1B = dict(num_hidden_layers=16, hidden_size=2048, intermediate_size=8192, head_dim=64,
                    num_attention_heads=32, num_key_value_heads=8, vocab_size=128256, rms_norm_eps=1e-5,
                    rope_theta=500000.0, rope_scaling=(32.0, 1.0, 4.0, 8192), max_position_embeddings=8192)

# Qwen3-0.6B (qimeng_megakernel/models/LLM/qwen/qwen3__0_6b/A100/single_batch/decode_schedule/model_config.py:4-16)
QWEN3_0_6B = dict(num_hidden_layers=28, hidden_size=1024, intermediate_size=3072, head_dim=128,
                  num_attention_heads=16, num_key_value_heads=8, vocab_size=151936, rms_norm_eps=1e-6,
                  rope_theta=1000000.0, rope_scaling=None, max_position_embeddings=40960, qk_norm=True)

# OLMoE-1B-7B shape (the mixture-of-experts workload of the benchmark): MHA 16 x 128, 64 experts, top-8, expert intermediate 1024, no shared expert
OLMOE_1B_7B = dict(num_hidden_layers=16, hidden_size=2048, intermediate_size=1024, head_dim=128,
                   num_attention_heads=16, num_key_value_heads=16, vocab_size=50304, rms_norm_eps=1e-5,
                   rope_theta=10000.0, rope_scaling=None, max_position_embeddings=4096, qk_norm=False,
                   num_experts=64, num_experts_per_tok=8, moe_intermediate_size=1024)

# The reference keeps one config class per model package; here one runtime descriptor serves every shape.
Qwen3Config = LlamaConfig
QwenMoeConfig = LlamaConfig
