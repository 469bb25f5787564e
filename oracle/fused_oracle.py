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
The same functions serve [B, H] state (their `_as_decode_BH` / `decode_pos_id` / `row_active` branches:
per-row positions from position_ids, inactive rows write nothing, get zero projections and -1e9 logits).
Qwen3 (per-head RMSNorm on Q and K before RoPE):
  qimeng_megakernel/models/LLM/qwen/qwen3__0_6b/A100/single_batch/decode_schedule/fused/operations.py
      _per_head_rms_norm             52-63
      fused_rms_qkvproj_gemv         66-73
      fused_qknorm_rope_writecache   76-120
  (that package is batch-1 only: it flattens its state with .view(-1); for B > 1 the rows are looped.)

Parity pin: tests/golden/ holds outputs of the real reference functions (imported from the
reference checkout by tests/golden/make_golden.py) for batch 1, for a ragged batch with an inactive
row, and for the Qwen3 variant; tests/test_oracle_golden.py checks this restatement against them bit
for bit.
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
    qk_norm: bool = False


@dataclass
class OracleState:
    """The tensors of the reference's Globals that the decode step touches (globs.py:8-41; multi-batch
    additions multi_batch/decode_schedule/globs.py:13-26).  State tensors are [H]-shaped for one sequence
    (batch=None) or [B, H]-shaped."""
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
    q_norm_weights: torch.Tensor = None
    k_norm_weights: torch.Tensor = None
    rope_cos: torch.Tensor = None
    rope_sin: torch.Tensor = None
    k_cache: torch.Tensor = None       # [L, B, S, NKV, HD]
    v_cache: torch.Tensor = None
    hidden_states: torch.Tensor = None  # [H] or [B, H]
    q_post_rope: torch.Tensor = None
    attn_out: torch.Tensor = None
    silu_out: torch.Tensor = None
    logits: torch.Tensor = None
    position_id: int = 0
    position_ids: Optional[list] = None    # per-row positions (multi-batch); None = every row at position_id
    active_mask: Optional[list] = None     # per-row bool; None = all active
    layer_hidden: list = field(default_factory=list)   # hidden_states after each layer (last step)

    @property
    def batch(self) -> int:
        return int(self.k_cache.shape[1])

    def pos(self, b: int) -> int:
        """decode_pos_id (operations.py:60-73)."""
        return int(self.position_id) if self.position_ids is None else int(self.position_ids[b])

    def active(self, b: int) -> bool:
        """row_active (operations.py:76-84)."""
        return True if self.active_mask is None else bool(self.active_mask[b])


def _bh(t: torch.Tensor) -> torch.Tensor:
    """_as_decode_BH (operations.py:35-42): [H] -> [1, H]."""
    return t.unsqueeze(0) if t.dim() == 1 else t


def rms_norm(inp: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """operations.py:126-131 -- fp32 statistics, round to the input dtype, then scale."""
    input_dtype = inp.dtype
    x = inp.to(torch.float32)
    variance = x.pow(2).mean(-1, keepdim=True)
    x = x * torch.rsqrt(variance + eps)
    return weight * x.to(input_dtype)


def per_head_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Qwen3 operations.py:52-63 -- x [heads, head_dim]; fp32 throughout, one rounding at the end."""
    x32 = x.to(torch.float32)
    variance = x32.pow(2).mean(-1, keepdim=True)
    return (weight.to(torch.float32) * (x32 * torch.rsqrt(variance + eps))).to(x.dtype)


def rotate_half_interleaved(x: torch.Tensor) -> torch.Tensor:
    """operations.py:134-140 -- pairs (2i, 2i+1): (a, b) -> (-b, a)."""
    x1 = x[..., ::2]
    x2 = x[..., 1::2]
    return torch.stack((-x2, x1), dim=-1).view_as(x)


def qkv_rope(st: OracleState, layer: int) -> None:
    """operations.py:151-215; with cfg.qk_norm the Qwen3 sequence (operations.py:66-120): GEMV rounded to the
    state dtype (qkv_raw), per-head norm of Q and K, then RoPE."""
    c = st.cfg
    k_start = c.num_attention_heads * c.head_dim
    v_start = k_start + c.num_key_value_heads * c.head_dim
    post_ln = _bh(rms_norm(st.hidden_states, st.attn_norm_weights[layer], c.rms_norm_eps))
    B = post_ln.shape[0]
    qkv = torch.einsum("oi,bi->bo", st.qkv_weights[layer], post_ln)
    q = qkv[:, :k_start].view(B, c.num_attention_heads, c.head_dim)
    k = qkv[:, k_start:v_start].view(B, c.num_key_value_heads, c.head_dim)
    v = qkv[:, v_start:].view(B, c.num_key_value_heads, c.head_dim)
    for b in range(B):
        if not st.active(b):
            continue
        pos = st.pos(b)
        qb, kb = q[b:b + 1], k[b:b + 1]
        if c.qk_norm:
            qb = per_head_rms_norm(qb[0], st.q_norm_weights[layer], c.rms_norm_eps).unsqueeze(0)
            kb = per_head_rms_norm(kb[0], st.k_norm_weights[layer], c.rms_norm_eps).unsqueeze(0)
        cos = st.rope_cos[pos].view(1, 1, -1)
        sin = st.rope_sin[pos].view(1, 1, -1)
        q_rope = (qb * cos) + (rotate_half_interleaved(qb) * sin)
        k_rope = (kb * cos) + (rotate_half_interleaved(kb) * sin)
        _bh(st.q_post_rope)[b].copy_(q_rope.reshape(-1).to(st.q_post_rope.dtype))
        st.k_cache[layer, b, pos].copy_(k_rope[0].to(st.k_cache.dtype))
        st.v_cache[layer, b, pos].copy_(v[b].to(st.v_cache.dtype))


def decode_attention(st: OracleState, layer: int) -> None:
    """operations.py:218-248 -- fp32 softmax attention over keys 0..pos, GQA by head repetition; an inactive
    row's output is zeroed."""
    c = st.cfg
    gqa = c.num_attention_heads // c.num_key_value_heads
    for b in range(st.batch):
        out_row = _bh(st.attn_out)[b]
        if not st.active(b):
            out_row.zero_()
            continue
        seq_len = st.pos(b) + 1
        q = _bh(st.q_post_rope)[b].view(c.num_attention_heads, c.head_dim).float()
        k = st.k_cache[layer, b, :seq_len].float()
        v = st.v_cache[layer, b, :seq_len].float()
        k = k.unsqueeze(2).expand(-1, -1, gqa, -1).reshape(seq_len, c.num_attention_heads, c.head_dim)
        v = v.unsqueeze(2).expand(-1, -1, gqa, -1).reshape(seq_len, c.num_attention_heads, c.head_dim)
        qk = torch.einsum("hi,shi->hs", q, k)
        softmax = torch.softmax(qk * (1 / math.sqrt(c.head_dim)), dim=-1)
        out = torch.einsum("hs,sho->ho", softmax, v)
        out_row.copy_(out.reshape(-1).to(st.attn_out.dtype))


def _zero_inactive(st: OracleState, out: torch.Tensor, value: float = 0.0) -> None:
    for b in range(out.shape[0]):
        if not st.active(b):
            out[b] = value


def oproj_residual(st: OracleState, layer: int) -> None:
    """operations.py:251-262."""
    out = torch.einsum("oi,bi->bo", st.o_proj_weights[layer], _bh(st.attn_out))
    _zero_inactive(st, out)
    _bh(st.hidden_states).add_(out.to(st.hidden_states.dtype))


def mlp_upgate(st: OracleState, layer: int) -> None:
    """operations.py:265-282."""
    post_ln = _bh(rms_norm(st.hidden_states, st.mlp_norm_weights[layer], st.cfg.rms_norm_eps))
    up = torch.einsum("oi,bi->bo", st.up_proj_weights[layer], post_ln)
    gate = torch.einsum("oi,bi->bo", st.gate_proj_weights[layer], post_ln)
    silu_out = F.silu(gate) * up
    _zero_inactive(st, silu_out)
    _bh(st.silu_out).copy_(silu_out.to(st.silu_out.dtype))


def mlp_down_residual(st: OracleState, layer: int) -> None:
    """operations.py:285-295."""
    down = torch.einsum("oi,bi->bo", st.down_proj_weights[layer], _bh(st.silu_out))
    _zero_inactive(st, down)
    _bh(st.hidden_states).add_(down.to(st.hidden_states.dtype))


def lm_head(st: OracleState) -> None:
    """operations.py:303-321."""
    post_ln = _bh(rms_norm(st.hidden_states, st.lm_head_norm_weights, st.cfg.rms_norm_eps))
    logits = torch.einsum("oi,bi->bo", st.lm_head_weights, post_ln).to(st.logits.dtype)
    _zero_inactive(st, logits, -1e9)
    _bh(st.logits).copy_(logits)


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


def feed_tokens(st: OracleState, tokens, positions, active=None, record_layers: bool = False) -> list:
    """The multi-batch iteration: row b embeds tokens[b] at positions[b]; returns the per-row argmax."""
    st.hidden_states.copy_(st.embed_tokens[torch.as_tensor(tokens)].to(st.hidden_states.dtype))
    st.position_ids = [int(p) for p in positions]
    st.active_mask = None if active is None else [bool(a) for a in active]
    decode_step(st, record_layers=record_layers)
    return [int(t) for t in st.logits.argmax(dim=-1)]


def make_state(cfg: OracleConfig, weights: dict, kv_seq_len: int, dtype: torch.dtype,
               batch: Optional[int] = None) -> OracleState:
    """Allocate the buffers the reference's fused prefill allocates
    (qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/fused_prefill.py:61-160); weights are cast
    to `dtype` (bf16 = the reference path, fp32 = the high-precision yardstick).  batch=None: the
    single-batch shapes; batch=B: [B, ...] state."""
    st = OracleState(cfg=cfg)
    names = ["attn_norm_weights", "qkv_weights", "o_proj_weights", "mlp_norm_weights", "up_proj_weights",
             "gate_proj_weights", "down_proj_weights", "lm_head_norm_weights", "lm_head_weights", "embed_tokens"]
    if cfg.qk_norm:
        names += ["q_norm_weights", "k_norm_weights"]
    for name in names:
        setattr(st, name, weights[name].to(dtype))
    st.rope_cos = weights["rope_cos"].float()
    st.rope_sin = weights["rope_sin"].float()
    L, nkv, hd = cfg.num_hidden_layers, cfg.num_key_value_heads, cfg.head_dim
    B = batch or 1
    lead = () if batch is None else (B,)
    st.k_cache = torch.zeros(L, B, kv_seq_len, nkv, hd, dtype=dtype)
    st.v_cache = torch.zeros(L, B, kv_seq_len, nkv, hd, dtype=dtype)
    st.hidden_states = torch.zeros(*lead, cfg.hidden_size, dtype=dtype)
    st.q_post_rope = torch.zeros(*lead, cfg.num_attention_heads * hd, dtype=dtype)
    st.attn_out = torch.zeros(*lead, cfg.num_attention_heads * hd, dtype=dtype)
    st.silu_out = torch.zeros(*lead, cfg.intermediate_size, dtype=dtype)
    st.logits = torch.zeros(*lead, cfg.vocab_size, dtype=dtype)
    return st
