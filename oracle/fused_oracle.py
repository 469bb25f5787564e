"""CPU oracle for the decode step -- TEST INFRASTRUCTURE, not part of the product.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may import this
module.  It restates, in plain PyTorch on the CPU, the reference's "fused" decode route: one
function per fused op, a whole layer at a time, with the reference's dtype behaviour (bf16 tensors
in, bf16 rounding after every einsum / norm; or fp32 throughout when given fp32 tensors).

Reference being restated (paths inside the QiMeng-MegaKernel project):
  qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/single_batch/decode_schedule/fused/operations.py
      _rms_norm                      126-131
      _rotate_half_interleaved       134-140
      fused_rms_qkvproj_gemv_rope    151-215
      fused_decode_attention         218-248
      fused_oproj_gemv_residual      251-262
      fused_mlp_upgate               265-282
      fused_mlp_down_residual        285-295
      fused_rms_lmhead_gemv          303-321
  .../decode_schedule/fused/layer_scheduler.py   run_fused_decode_step 45-56
  qimeng_megakernel/models/LLM/decode.py         generate_greedy_fast 1340-1435 (token loop)

Parity pin: tests/golden/ holds outputs of the real reference functions (imported from the
reference checkout by tests/golden/make_golden.py); tests/test_oracle_golden.py checks this
restatement against them bit for bit.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn.functional as F


@dataclass
class OracleConfig:
    num_hidden_layers: int = 16
    hidden_size: int = 2048
    intermediate_size: int = 8192
    head_dim: int = 64
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    vocab_size: int = 128256
    rms_norm_eps: float = 1e-5


@dataclass
class OracleState:
    """The tensors of the reference's Globals that the decode step touches (globs.py:8-41)."""
    cfg: OracleConfig
    attn_norm_weights: torch.Tensor = None
    qkv_weights: torch.Tensor = None
    o_proj_weights: torch.Tensor = None
    mlp_norm_weights: torch.Tensor = None
    up_proj_weights: torch.Tensor = None
    gate_proj_weights: torch.Tensor = None
    down_proj_weights: torch.Tensor = None
    lm_head_norm_weights: torch.Tensor = None
    lm_head_weights: torch.Tensor = None
    embed_tokens: torch.Tensor = None
    rope_cos: torch.Tensor = None
    rope_sin: torch.Tensor = None
    k_cache: torch.Tensor = None       # [L, 1, S, NKV, HD]
    v_cache: torch.Tensor = None
    hidden_states: torch.Tensor = None  # [H]
    q_post_rope: torch.Tensor = None
    attn_out: torch.Tensor = None
    silu_out: torch.Tensor = None
    logits: torch.Tensor = None
    position_id: int = 0
    layer_hidden: list = field(default_factory=list)   # hidden_states after each layer (last step)


def rms_norm(inp: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """operations.py:126-131 -- fp32 statistics, round to the input dtype, then scale."""
    input_dtype = inp.dtype
    x = inp.to(torch.float32)
    variance = x.pow(2).mean(-1, keepdim=True)
    x = x * torch.rsqrt(variance + eps)
    return weight * x.to(input_dtype)


def rotate_half_interleaved(x: torch.Tensor) -> torch.Tensor:
    """operations.py:134-140 -- pairs (2i, 2i+1): (a, b) -> (-b, a)."""
    x1 = x[..., ::2]
    x2 = x[..., 1::2]
    return torch.stack((-x2, x1), dim=-1).view_as(x)


def qkv_rope(st: OracleState, layer: int) -> None:
    """operations.py:151-215 (B = 1 branch)."""
    c = st.cfg
    k_start = c.num_attention_heads * c.head_dim
    v_start = k_start + c.num_key_value_heads * c.head_dim
    post_ln = rms_norm(st.hidden_states, st.attn_norm_weights[layer], c.rms_norm_eps)
    qkv = torch.einsum("oi,bi->bo", st.qkv_weights[layer], post_ln.unsqueeze(0))
    q = qkv[:, :k_start].view(1, c.num_attention_heads, c.head_dim)
    k = qkv[:, k_start:v_start].view(1, c.num_key_value_heads, c.head_dim)
    v = qkv[:, v_start:].view(1, c.num_key_value_heads, c.head_dim)
    pos = st.position_id
    cos = st.rope_cos[pos].view(1, 1, -1)
    sin = st.rope_sin[pos].view(1, 1, -1)
    q_rope = (q * cos) + (rotate_half_interleaved(q) * sin)
    k_rope = (k * cos) + (rotate_half_interleaved(k) * sin)
    st.q_post_rope.copy_(q_rope.reshape(-1).to(st.q_post_rope.dtype))
    st.k_cache[layer, 0, pos].copy_(k_rope[0].to(st.k_cache.dtype))
    st.v_cache[layer, 0, pos].copy_(v[0].to(st.v_cache.dtype))


def decode_attention(st: OracleState, layer: int) -> None:
    """operations.py:218-248 -- fp32 softmax attention over keys 0..pos, GQA by head repetition."""
    c = st.cfg
    gqa = c.num_attention_heads // c.num_key_value_heads
    seq_len = st.position_id + 1
    q = st.q_post_rope.view(c.num_attention_heads, c.head_dim).float()
    k = st.k_cache[layer, 0, :seq_len].float()
    v = st.v_cache[layer, 0, :seq_len].float()
    k = k.unsqueeze(2).expand(-1, -1, gqa, -1).reshape(seq_len, c.num_attention_heads, c.head_dim)
    v = v.unsqueeze(2).expand(-1, -1, gqa, -1).reshape(seq_len, c.num_attention_heads, c.head_dim)
    qk = torch.einsum("hi,shi->hs", q, k)
    softmax = torch.softmax(qk * (1 / math.sqrt(c.head_dim)), dim=-1)
    out = torch.einsum("hs,sho->ho", softmax, v)
    st.attn_out.copy_(out.reshape(-1).to(st.attn_out.dtype))


def oproj_residual(st: OracleState, layer: int) -> None:
    """operations.py:251-262."""
    out = torch.einsum("oi,bi->bo", st.o_proj_weights[layer], st.attn_out.unsqueeze(0))
    st.hidden_states.add_(out.squeeze(0).to(st.hidden_states.dtype))


def mlp_upgate(st: OracleState, layer: int) -> None:
    """operations.py:265-282."""
    post_ln = rms_norm(st.hidden_states, st.mlp_norm_weights[layer], st.cfg.rms_norm_eps).unsqueeze(0)
    up = torch.einsum("oi,bi->bo", st.up_proj_weights[layer], post_ln)
    gate = torch.einsum("oi,bi->bo", st.gate_proj_weights[layer], post_ln)
    st.silu_out.copy_((F.silu(gate) * up).reshape(-1).to(st.silu_out.dtype))


def mlp_down_residual(st: OracleState, layer: int) -> None:
    """operations.py:285-295."""
    down = torch.einsum("oi,bi->bo", st.down_proj_weights[layer], st.silu_out.unsqueeze(0))
    st.hidden_states.add_(down.squeeze(0).to(st.hidden_states.dtype))


def lm_head(st: OracleState) -> None:
    """operations.py:303-321."""
    post_ln = rms_norm(st.hidden_states, st.lm_head_norm_weights, st.cfg.rms_norm_eps).unsqueeze(0)
    logits = torch.einsum("oi,bi->bo", st.lm_head_weights, post_ln).to(st.logits.dtype)
    st.logits.copy_(logits.squeeze(0))


def decode_step(st: OracleState, num_layers: Optional[int] = None, record_layers: bool = False) -> None:
    """layer_scheduler.py:32-56 -- per layer: qkv+rope, attention, o-proj, mlp; LM head at the end."""
    layers = st.cfg.num_hidden_layers if num_layers is None else num_layers
    if record_layers:
        st.layer_hidden = []
    for layer in range(layers):
        qkv_rope(st, layer)
        decode_attention(st, layer)
        oproj_residual(st, layer)
        mlp_upgate(st, layer)
        mlp_down_residual(st, layer)
        if record_layers:
            st.layer_hidden.append(st.hidden_states.clone())
    if layers == st.cfg.num_hidden_layers:
        lm_head(st)


def feed_token(st: OracleState, token: int, pos: int, record_layers: bool = False) -> int:
    """One iteration of generate_greedy_fast (decode.py:1373-1395): embed, step, argmax."""
    st.hidden_states.copy_(st.embed_tokens[token].to(st.hidden_states.dtype))
    st.position_id = pos
    decode_step(st, record_layers=record_layers)
    return int(st.logits.argmax())


def make_state(cfg: OracleConfig, weights: dict, kv_seq_len: int, dtype: torch.dtype) -> OracleState:
    """Allocate the buffers the reference's fused prefill allocates for B = 1
    (qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/fused_prefill.py:61-160); weights are cast
    to `dtype` (bf16 = the reference path, fp32 = the high-precision yardstick)."""
    st = OracleState(cfg=cfg)
    for name in ("attn_norm_weights", "qkv_weights", "o_proj_weights", "mlp_norm_weights", "up_proj_weights",
                 "gate_proj_weights", "down_proj_weights", "lm_head_norm_weights", "lm_head_weights", "embed_tokens"):
        setattr(st, name, weights[name].to(dtype))
    st.rope_cos = weights["rope_cos"].float()
    st.rope_sin = weights["rope_sin"].float()
    L, nkv, hd = cfg.num_hidden_layers, cfg.num_key_value_heads, cfg.head_dim
    st.k_cache = torch.zeros(L, 1, kv_seq_len, nkv, hd, dtype=dtype)
    st.v_cache = torch.zeros(L, 1, kv_seq_len, nkv, hd, dtype=dtype)
    st.hidden_states = torch.zeros(cfg.hidden_size, dtype=dtype)
    st.q_post_rope = torch.zeros(cfg.num_attention_heads * hd, dtype=dtype)
    st.attn_out = torch.zeros(cfg.num_attention_heads * hd, dtype=dtype)
    st.silu_out = torch.zeros(cfg.intermediate_size, dtype=dtype)
    st.logits = torch.zeros(cfg.vocab_size, dtype=dtype)
    return st
