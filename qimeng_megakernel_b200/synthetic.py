"""Seeded synthetic model and prompt: the stand-in for the checkpoints the reference loads.

Every matrix ~ N(0, 0.02) in bf16, RMSNorm gains 1, embeddings tied to the LM head, prompt ids
uniform over the vocabulary.  Q/K rows are generated directly in the interleaved layout (the
distribution is invariant under the row permutation the reference applies at load,
qimeng_megakernel/models/LLM/llama/load_weights.py:175-178).
"""
from __future__ import annotations

import torch

from .globs import Globals
from .model_config import LlamaConfig
from .rope import rope_tables_interleaved

WEIGHT_NAMES = ("attn_norm_weights", "qkv_weights", "o_proj_weights", "mlp_norm_weights", "up_proj_weights",
                "gate_proj_weights", "down_proj_weights", "lm_head_norm_weights", "lm_head_weights",
                "embed_tokens", "rope_cos", "rope_sin")
QK_NORM_NAMES = ("q_norm_weights", "k_norm_weights")
MOE_NAMES = ("router_weights", "expert_gate_up_proj_weights", "expert_down_proj_weights")


def make_weights(config: dict, seed: int = 0, device: str | torch.device = "cpu", std: float = 0.02,
                 max_positions: int | None = None, gain_jitter: float = 0.0) -> dict:
    """Seeded weights as a dict of tensors on `device` (generator lives on that device).
    gain_jitter > 0 draws the RMSNorm gains from N(1, gain_jitter) instead of 1 (tests only: with gains of
    exactly 1 a kernel that ignored them would still pass)."""
    L, H, I = config["num_hidden_layers"], config["hidden_size"], config["intermediate_size"]
    NH, NKV, HD, V = (config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"],
                      config["vocab_size"])
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)

    def mat(*shape):
        out = torch.empty(shape, dtype=torch.bfloat16, device=dev)
        # generate per leading slice in fp32 to bound the temporary
        flat = out.view(shape[0], -1)
        for i in range(shape[0]):
            flat[i].copy_(torch.randn(flat.shape[1], generator=gen, device=dev, dtype=torch.float32) * std)
        return out

    E, Ie = int(config.get("num_experts", 0) or 0), int(config.get("moe_intermediate_size", 0) or 0)
    w = {
        "qkv_weights": mat(L, (NH + 2 * NKV) * HD, H),
        "o_proj_weights": mat(L, H, NH * HD),
    }
    if E:   # experts instead of the dense MLP; router rows scaled so that its logits are ~ N(0, 1): near-uniform load
        w["router_weights"] = (mat(L, E, H).float() * (H ** -0.5 / std)).to(torch.bfloat16)
        w["expert_gate_up_proj_weights"] = mat(L * E, 2 * Ie, H).view(L, E, 2 * Ie, H)
        w["expert_down_proj_weights"] = mat(L * E, H, Ie).view(L, E, H, Ie)
        for name in ("up_proj_weights", "gate_proj_weights", "down_proj_weights"):   # placeholders (never read)
            w[name] = torch.zeros(1, dtype=torch.bfloat16, device=dev)
    else:
        w.update({
            "up_proj_weights": mat(L, I, H),
            "gate_proj_weights": mat(L, I, H),
            "down_proj_weights": mat(L, H, I)})
    w.update({
        "attn_norm_weights": torch.ones(L, H, dtype=torch.bfloat16, device=dev),
        "mlp_norm_weights": torch.ones(L, H, dtype=torch.bfloat16, device=dev),
        "lm_head_norm_weights": torch.ones(H, dtype=torch.bfloat16, device=dev),
    })
    lm = torch.empty(V, H, dtype=torch.bfloat16, device=dev)
    rows = 8192
    for r0 in range(0, V, rows):
        r1 = min(V, r0 + rows)
        lm[r0:r1].copy_(torch.randn(r1 - r0, H, generator=gen, device=dev, dtype=torch.float32) * std)
    w["lm_head_weights"] = lm
    w["embed_tokens"] = lm                      # tied
    if config.get("qk_norm"):
        w["q_norm_weights"] = torch.ones(L, HD, dtype=torch.bfloat16, device=dev)
        w["k_norm_weights"] = torch.ones(L, HD, dtype=torch.bfloat16, device=dev)
    if gain_jitter > 0.0:
        for name in ("attn_norm_weights", "mlp_norm_weights", "lm_head_norm_weights", "q_norm_weights", "k_norm_weights"):
            if name in w:
                w[name] = (1.0 + gain_jitter * torch.randn(w[name].shape, generator=gen, device=dev)).to(torch.bfloat16)
    cos, sin = rope_tables_interleaved(HD, max_positions or config.get("max_position_embeddings", 8192),
                                       config.get("rope_theta", 10000.0), config.get("rope_scaling"))
    w["rope_cos"], w["rope_sin"] = cos.to(dev), sin.to(dev)
    return w


def make_prompt(vocab_size: int, length: int = 16, seed: int = 1) -> torch.Tensor:
    gen = torch.Generator()
    gen.manual_seed(seed)
    return torch.randint(0, vocab_size, (length,), generator=gen, dtype=torch.int64)


def make_prompts(vocab_size: int, batch: int, length: int = 16, seed: int = 1) -> torch.Tensor:
    """[batch, length] prompts, row b drawn with seed + b (independent seeded prompts per sequence)."""
    return torch.stack([make_prompt(vocab_size, length, seed + b) for b in range(batch)])


def random_kv_rows(config: dict, rows: int, seed: int, batch: int = 1, std: float = 0.9):
    """Seeded stand-in for a KV cache that `rows` earlier tokens have filled: (k, v) bf16 CPU tensors
    [L, batch, rows, NKV, HD] ~ N(0, std) (the spread K and V rows have with N(0, 0.02) weights and a normalised
    2048-wide input).  The same seed gives the same rows on every machine (CPU generator), so a fixture made with
    them can be checked elsewhere without shipping the cache."""
    L, NKV, HD = config["num_hidden_layers"], config["num_key_value_heads"], config["head_dim"]
    gen = torch.Generator()
    gen.manual_seed(seed)
    k = torch.empty(L, batch, rows, NKV, HD, dtype=torch.bfloat16)
    v = torch.empty(L, batch, rows, NKV, HD, dtype=torch.bfloat16)
    for layer in range(L):
        k[layer].copy_(torch.randn(batch, rows, NKV, HD, generator=gen) * std)
        v[layer].copy_(torch.randn(batch, rows, NKV, HD, generator=gen) * std)
    return k, v


def make_globals(config: dict, weights: dict, kv_seq_len: int, device: str | torch.device = "cuda",
                 batch: int | None = None) -> Globals:
    """Allocate the buffers the reference's fused prefill allocates
    (qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/fused_prefill.py:61-160) around `weights`:
    batch=None gives the single-batch shapes ([H], ...), batch=B the multi-batch ones ([B, H], ...)."""
    LlamaConfig.update_from_dict(config)
    dev = torch.device(device)
    L, H, I = config["num_hidden_layers"], config["hidden_size"], config["intermediate_size"]
    NH, NKV, HD, V = (config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"],
                      config["vocab_size"])
    bf = torch.bfloat16
    moved = {}
    names = WEIGHT_NAMES + tuple(n for n in QK_NORM_NAMES + MOE_NAMES if n in weights)
    for name in names:
        t = weights[name]
        key = (t.data_ptr(), tuple(t.shape))     # (a slice that starts a tensor shares its address)
        if key not in moved:
            moved[key] = t.to(dev).contiguous()
        weights_dev = moved[key]
        moved[name] = weights_dev
    g = Globals(position_id=0, **{n: moved[n] for n in names})
    B = batch or 1
    lead = () if batch is None else (B,)
    g.k_cache = torch.zeros(L, B, kv_seq_len, NKV, HD, dtype=bf, device=dev)
    g.v_cache = torch.zeros(L, B, kv_seq_len, NKV, HD, dtype=bf, device=dev)
    g.hidden_states = torch.zeros(*lead, H, dtype=bf, device=dev)
    g.q_post_rope = torch.zeros(*lead, NH * HD, dtype=bf, device=dev)
    g.attn_out = torch.zeros(*lead, NH * HD, dtype=bf, device=dev)
    g.silu_out = torch.zeros(*lead, I, dtype=bf, device=dev)
    g.logits = torch.zeros(*lead, V, dtype=bf, device=dev)
    g.next_token = torch.zeros(B, dtype=torch.int64, device=dev)
    return g
